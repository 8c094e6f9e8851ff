"""Host-only checks of the C ABI: the library loads, exports every function that
include/pqhsa.h declares, lays out the workspace, and rejects bad arguments with a
status code and a message (no kernel is launched, no GPU is needed)."""

import ctypes as C
import re
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from pqhsa_release_b200 import _lib  # noqa: E402
from pqhsa_release_b200._lib import Params, WsLayout  # noqa: E402


def declared_functions():
    text = (ROOT / "include" / "pqhsa.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pqhsa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_function():
    names = declared_functions()
    assert "pqhsa_decode_step" in names and "pqhsa_append_encode" in names
    lib = C.CDLL(str(_lib.library_path()))
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/pqhsa.h but not exported"
    assert set(_lib.EXPORTS) <= set(names), "the ctypes binding names a function the header does not declare"


def test_abi_version_matches_header():
    text = (ROOT / "include" / "pqhsa.h").read_text()
    ver = int(re.search(r"#define PQHSA_ABI_VERSION (\d+)", text).group(1))
    assert _lib.lib.pqhsa_abi_version() == ver == _lib.ABI_VERSION
    for macro, val in (("PQHSA_UNIT_KEYS", _lib.UNIT_KEYS), ("PQHSA_SAMPLE_KEYS", _lib.SAMPLE_KEYS),
                       ("PQHSA_MAX_LISTS", _lib.MAX_LISTS), ("PQHSA_HEAD_DIM", _lib.HEAD_DIM)):
        assert int(re.search(rf"#define {macro} (\d+)", text).group(1)) == val


def _params(**over):
    p = Params()
    p.abi_version = _lib.ABI_VERSION
    p.dtype = _lib.BF16
    p.num_streams, p.group, p.head_dim = 8, 4, 128
    p.num_lists, p.slot_capacity = 512, 131072
    p.unit_capacity = 512 + 131072 // _lib.UNIT_KEYS + 1
    p.sink_tokens, p.local_window = 4, 128
    p.max_slots, p.max_full, p.topk_fixed, p.tail_capacity = 131000, 200, 100, 1024
    p.top_fraction, p.scale = 0.02, 128 ** -0.5
    for k, v in over.items():
        setattr(p, k, v)
    return p


def test_workspace_layout_is_ordered_and_aligned():
    p = _params()
    lay = WsLayout()
    _lib.call("pqhsa_workspace_layout", C.byref(p), C.byref(lay))
    assert _lib.lib.pqhsa_workspace_bytes(C.byref(p)) == lay.total_bytes
    offs = [getattr(lay, f) for f, _ in WsLayout._fields_[1:15]]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs) and offs[-1] < lay.total_bytes
    assert lay.kcap >= int(131072 * 0.02) and lay.kcap % 8 == 0
    assert lay.hitmap > lay.row_info and lay.chunks * 128 >= 200 + lay.kcap


@pytest.mark.parametrize(
    "over, code, text",
    [
        ({"abi_version": 1}, -2, "abi_version"),
        ({"dtype": 7}, -3, "dtype"),
        ({"group": 3}, -2, "group"),
        ({"head_dim": 64}, -2, "head_dim"),
        ({"num_lists": 1024}, -2, "num_lists"),
        ({"slot_capacity": 1001}, -2, "slot_capacity"),
        ({"unit_capacity": 10}, -2, "unit_capacity"),
        ({}, -1, "index pool pointer"),
    ],
)
def test_bad_arguments_are_rejected_with_a_message(over, code, text):
    p = _params(**over)
    with pytest.raises(_lib.PqhsaError) as e:
        _lib.call("pqhsa_decode_step", C.byref(p), None)
    assert e.value.code == code and text in str(e.value)


def test_null_params_and_topk_argument_checks():
    assert _lib.lib.pqhsa_workspace_bytes(None) == 0
    with pytest.raises(_lib.PqhsaError):
        _lib.call("pqhsa_decode_step", None, None)
    with pytest.raises(_lib.PqhsaError) as e:
        _lib.call("pqhsa_topk_radix", None, 1, 10, 10, 3, None, None, None)
    assert e.value.code == -1


def test_bulk_encode_argument_checks():
    """Validation happens before any CUDA call, so it can be exercised without a GPU."""
    a = 4096  # a non-null, 16-byte aligned address that is never dereferenced
    with pytest.raises(_lib.PqhsaError) as e:
        _lib.call("pqhsa_encode_bulk", None, 128, 1, 1, _lib.BF16, a, 4, a, a, a, a, None)
    assert e.value.code == -1
    with pytest.raises(_lib.PqhsaError) as e:  # stream stride shorter than a stream's keys
        _lib.call("pqhsa_encode_bulk", a, 64, 1, 1, _lib.BF16, a, 4, a, a, a, a, None)
    assert e.value.code == -2
    with pytest.raises(_lib.PqhsaError) as e:
        _lib.call("pqhsa_encode_bulk", a, 128, 1, 1, _lib.BF16, a, _lib.MAX_LISTS + 1, a, a, a, a, None)
    assert e.value.code == -2 and "num_lists" in str(e.value)
    with pytest.raises(_lib.PqhsaError) as e:
        _lib.call("pqhsa_encode_bulk", a + 2, 128, 1, 1, _lib.BF16, a, 4, a, a, a, a, None)
    assert e.value.code == -2 and "aligned" in str(e.value)
    with pytest.raises(_lib.PqhsaError) as e:
        _lib.call("pqhsa_encode_bulk", a, 128, 1, 1, 7, a, 4, a, a, a, a, None)
    assert e.value.code == -3
    _lib.call("pqhsa_encode_bulk", a, 128, 1, 0, _lib.BF16, a, 4, a, a, a, a, None)  # nothing to do
