"""The allocation-free scoring entry point (collected last on purpose: if it fails, every
other test has already run).

``pqhsa_scan_scores_static`` is for callers that cannot allocate device memory - an attention
backend inside a server that has given all free memory to the KV cache, or a C host that only
owns the buffers it was passed.  It keeps its per-query tables in an array built into the
library instead of a caller-supplied workspace.  The test drives it through the C ABI twice in a
row with different queries and requires exactly the logits of the existing path
(pqhsa_lut_build + pqhsa_scan_scores with a workspace): both run the same kernels, so the
tolerance is zero.  The array keeps the previous call's contents, which is why two calls are made.
"""

import ctypes as C

import pytest
import torch

from helpers import make_case, pool_from_case

pytestmark = pytest.mark.gpu


def test_static_scratch_scores_equal_workspace_scores_twice_in_a_row():
    from pqhsa_release_b200 import _lib

    fn = _lib.lib.pqhsa_scan_scores_static
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(_lib.Params), C.c_void_p, C.c_void_p]

    case = make_case(B=2, Hkv=2, G=4, S=5200, L=96, dtype=torch.bfloat16, seed=31)
    pool, _, _ = pool_from_case(case)
    stream = torch.cuda.current_stream().cuda_stream
    base = case.queries.cuda().reshape(case.num_streams, case.G, 128).contiguous()
    n = int(pool.h_sorted.max())
    for call in range(2):
        q = (base.float() * (1.0 + 0.25 * call) + 0.1 * call).to(torch.bfloat16).contiguous()
        want = pool.scan_scores(q)                       # existing entry points, caller-owned workspace
        got = torch.full_like(want, float("nan"))
        ws, ws_bytes = pool.p.workspace, pool.p.workspace_bytes
        pool.p.workspace, pool.p.workspace_bytes = None, 0   # the new entry point must not need it
        try:
            rc = fn(C.byref(pool.p), got.data_ptr(), stream)
        finally:
            pool.p.workspace, pool.p.workspace_bytes = ws, ws_bytes
        assert rc == 0, _lib.lib.pqhsa_last_error_string().decode()
        torch.cuda.synchronize()
        assert torch.equal(got[:, :n], want[:, :n]), f"call {call}: logits differ from the workspace path"
        assert bool(torch.isfinite(got[:, :n]).all())


def test_static_scratch_rejects_more_rows_than_it_holds():
    from pqhsa_release_b200 import _lib

    fn = _lib.lib.pqhsa_scan_scores_static
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(_lib.Params), C.c_void_p, C.c_void_p]
    case = make_case(B=1, Hkv=1, G=4, S=400, L=16, dtype=torch.bfloat16, seed=32)
    pool, _, _ = pool_from_case(case)
    out = torch.zeros(4, pool.cap, device="cuda")
    q = case.queries.cuda().reshape(1, 4, 128).contiguous()
    pool.p.q = q.data_ptr()
    saved = pool.p.num_streams
    pool.p.num_streams = 65          # 65 * 4 = 260 rows > 256: refused before anything is launched
    try:
        rc = fn(C.byref(pool.p), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    finally:
        pool.p.num_streams = saved
    assert rc == -6 and "256" in _lib.lib.pqhsa_last_error_string().decode()
