"""ctypes binding of ``libpqhsa_b200.so`` (the C ABI declared in ``include/pqhsa.h``).

The library is the product: there is no Python or CPU fallback.  If it has not
been built, importing this module raises with the build command.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

ABI_VERSION = 4
SUBSPACES, CODES, HEAD_DIM, MAX_LISTS, UNIT_KEYS, SAMPLE_KEYS, HIST_BINS = 8, 16, 128, 512, 128, 4096, 2048
COMPACT_MAX_TAIL = 4096
STATE_INTS, ROW_INFO_INTS = 8, 8
ST_N_SORTED, ST_N_TAIL, ST_SEQ_LEN, ST_N_UNITS, ST_N_LISTS, ST_REQ, ST_KV_HEAD = range(7)
RI_K, RI_N, RI_NCAND, RI_NSEL, RI_FALLBACK, RI_TIES = range(6)
F32, BF16, F16 = 0, 1, 2
STAGE_LUT, STAGE_SCAN, STAGE_SELECT, STAGE_ATTEND, STAGE_MERGE = range(5)

import os

# PQHSA_LIBRARY names another build of the same ABI (a debug build, a build kept outside the package)
_LIB_PATH = Path(os.environ.get("PQHSA_LIBRARY") or Path(__file__).resolve().parent / "libpqhsa_b200.so")


class Params(C.Structure):
    """``pqhsa_params`` of include/pqhsa.h, field for field."""

    _fields_ = [
        ("abi_version", C.c_int32), ("dtype", C.c_int32), ("num_streams", C.c_int32), ("group", C.c_int32),
        ("head_dim", C.c_int32), ("num_lists", C.c_int32), ("slot_capacity", C.c_int32),
        ("unit_capacity", C.c_int32), ("sink_tokens", C.c_int32), ("local_window", C.c_int32),
        ("max_slots", C.c_int32), ("max_full", C.c_int32), ("topk_fixed", C.c_int32),
        ("tail_capacity", C.c_int32),
        ("top_fraction", C.c_double),
        ("scale", C.c_float), ("hist_lo", C.c_float), ("hist_inv_width", C.c_float), ("select_margin", C.c_float),
        ("codes", C.c_void_p), ("norms", C.c_void_p), ("list_ids", C.c_void_p), ("slot_pos", C.c_void_p),
        ("slot_unit", C.c_void_p), ("unit_off", C.c_void_p), ("unit_list", C.c_void_p),
        ("coarse", C.c_void_p), ("codebooks", C.c_void_p), ("vmeans", C.c_void_p),
        ("vsum", C.c_void_p), ("vcnt", C.c_void_p), ("state", C.c_void_p), ("norm_max", C.c_void_p),
        ("sample", C.c_void_p),
        ("k_base", C.c_void_p), ("v_base", C.c_void_p), ("block_table", C.c_void_p),
        ("max_blocks", C.c_int32), ("block_size", C.c_int32),
        ("stride_block", C.c_int64), ("stride_head", C.c_int64), ("stride_row", C.c_int64),
        ("peer_out", C.c_void_p), ("peer_gather", C.c_void_p), ("peer_seq", C.c_void_p),
        ("peer_world", C.c_int32), ("peer_rank", C.c_int32), ("peer_wait_polls", C.c_int32), ("external_append", C.c_int32),
        ("q", C.c_void_p), ("out", C.c_void_p), ("io_map", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class WsLayout(C.Structure):
    """``pqhsa_ws_layout`` of include/pqhsa.h."""

    _fields_ = [
        ("total_bytes", C.c_size_t), ("lut", C.c_size_t), ("list_scores", C.c_size_t), ("pair_tab", C.c_size_t),
        ("row_bin", C.c_size_t),
        ("row_tau", C.c_size_t), ("ticket", C.c_size_t), ("norm_pend", C.c_size_t), ("unit_max", C.c_size_t), ("unit_sum", C.c_size_t),
        ("tail_logit", C.c_size_t), ("row_info", C.c_size_t), ("hitmap", C.c_size_t),
        ("cand_key", C.c_size_t), ("cand_rec", C.c_size_t), ("cand_bin", C.c_size_t),
        ("part_hist", C.c_size_t), ("part_cnt", C.c_size_t),
        ("sel_slot", C.c_size_t), ("sel_off", C.c_size_t), ("partial", C.c_size_t), ("row_ticket", C.c_size_t), ("work_counter", C.c_size_t), ("combine_ticket", C.c_size_t),
        ("parts", C.c_int32), ("seg", C.c_int32), ("kcap", C.c_int32), ("tail_cap", C.c_int32), ("chunks", C.c_int32),
    ]


EXPORTS = {
    "pqhsa_abi_version": (C.c_int, []),
    "pqhsa_last_error_string": (C.c_char_p, []),
    "pqhsa_workspace_bytes": (C.c_size_t, [C.POINTER(Params)]),
    "pqhsa_workspace_layout": (C.c_int, [C.POINTER(Params), C.POINTER(WsLayout)]),
    "pqhsa_lut_build": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "pqhsa_scan_select": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "pqhsa_attend_merge": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "pqhsa_decode_step": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "pqhsa_copy_small": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "pqhsa_launch_empty": (C.c_int, [C.c_int32, C.c_void_p]),
    "pqhsa_wait_peers": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "pqhsa_decode_step_append": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "pqhsa_run_stage": (C.c_int, [C.POINTER(Params), C.c_int, C.c_void_p]),
    "pqhsa_compact": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_void_p]),
    "pqhsa_append_kv": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_void_p, C.c_void_p]),
    "pqhsa_append_encode": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_int32, C.c_void_p]),
    "pqhsa_encode_bulk": (
        C.c_int,
        [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p,
         C.c_void_p, C.c_void_p, C.c_void_p],
    ),
    "pqhsa_cluster_order": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "pqhsa_cluster_sums": (
        C.c_int,
        [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
         C.c_void_p, C.c_void_p, C.c_void_p],
    ),
    "pqhsa_subspace_assign": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "pqhsa_encode_bulk_assigned": (
        C.c_int,
        [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p,
         C.c_void_p, C.c_void_p, C.c_void_p],
    ),
    "pqhsa_scan_scores": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_void_p]),
    "pqhsa_scan_scores_static": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_void_p]),
    "pqhsa_topk_radix": (
        C.c_int,
        [C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p],
    ),
}


class PqhsaError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, call: str, code: int, text: str):
        super().__init__(f"{call} failed with status {code}: {text}")
        self.code = code


def library_path() -> Path:
    return _LIB_PATH


def _load() -> C.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m pqhsa_release_b200.build` (needs nvcc with sm_100a support). "
            "There is no CPU fallback."
        )
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    got = lib.pqhsa_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"{_LIB_PATH} speaks ABI {got}, this package needs {ABI_VERSION}: rebuild it")
    return lib


lib = _load()


def call(name: str, *args) -> None:
    """Invoke an int-returning entry point and raise :class:`PqhsaError` on failure."""
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise PqhsaError(name, rc, lib.pqhsa_last_error_string().decode("utf-8", "replace"))
