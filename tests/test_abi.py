"""The C-ABI library builds, loads, and exports exactly what the header declares.
No compute calls: this runs without a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib_path():
    from catopt_b200 import build

    return build.build()


def _declared():
    text = (ROOT / "include" / "catopt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(cb2_[a-z0-9_]+)\s*\(", text))


def test_header_symbols_exported(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    declared = _declared()
    assert len(declared) >= 11
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_loader_signatures_cover_header(lib_path):
    from catopt_b200 import _lib

    assert set(_lib.SIGNATURES) == _declared()
    lib = _lib.load()
    assert lib.cb2_version() >= 100
    assert _lib.status_str(0) == "ok"
    assert "timed out" in _lib.status_str(_lib.CB2_WAIT_TIMEOUT)


def test_argument_errors_without_a_device(lib_path):
    """Argument validation happens before any CUDA call."""
    from catopt_b200 import _lib

    lib = _lib.load()
    assert lib.cb2_verify_reduce(None, None, 8, 1, 0, None, None) == 6      # NULL_PTR
    assert lib.cb2_verify_reduce(16, 16, 0, 1, 0, 16, None) == 1            # BAD_SHAPE
    assert lib.cb2_verify_reduce(16, 16, 8, 1, 7, 16, None) == 3            # UNSUPPORTED_DTYPE
    assert lib.cb2_decayed_chunk_fwd(16, 16, 16, 16, 16, 1, 1, 100, 8, 8, 64, 1.0, 0, None, 0, None, None) == 1
    assert lib.cb2_diag_scan_fwd(16, 16, 16, 16, None, 16, None, 1, 4, 8, 3, 0, 0, None, None) == 1
    assert lib.cb2_linear_f32_scratch_bytes(64, 512, 512) > 0
    assert lib.cb2_linear_f32_scratch_bytes(4096, 512, 512) == 2 * 512 * 512 * 4   # w split into hi + lo
    assert lib.cb2_decayed_chunk_on_tensor_cores(16, 32, 8192, 128, 128, 128, 1) == 1
    assert lib.cb2_decayed_chunk_on_tensor_cores(2, 4, 1024, 64, 64, 64, 0) == 0
    # fp32 with enough (batch, head) units and head dims up to 64: three-pass TF32, no scratch
    assert lib.cb2_decayed_chunk_on_tensor_cores(16, 32, 2048, 64, 64, 128, 0) == 1
    assert lib.cb2_decayed_chunk_on_tensor_cores(16, 32, 2048, 128, 128, 128, 0) == 0
    assert lib.cb2_decayed_chunk_scratch_bytes(16, 32, 2048, 64, 64, 128, 0) == 0
    # streaming step in the decode regime: partial carriers (m, l, a) of one wave of key splits — two
    # CTAs per SM for up to four query rows, one for eight
    assert lib.cb2_om_step_scratch_bytes(1, 32, 1, 65536, 128) == (2 * 148 // 32) * 32 * 1 * (128 + 2) * 4
    assert lib.cb2_om_step_scratch_bytes(1, 32, 8, 65536, 128) == (148 // 32) * 32 * 8 * (128 + 2) * 4
    assert lib.cb2_om_step_scratch_bytes(1, 32, 1, 512, 64) == 2 * 32 * 1 * (64 + 2) * 4      # at least 256 keys per split
    assert lib.cb2_om_step_scratch_bytes(0, 32, 1, 512, 64) == 0


def test_no_cpu_fallback():
    """Host wrappers refuse CPU tensors instead of computing on the host."""
    import torch

    from catopt_b200 import B200Error, ops, verify

    x = torch.zeros(4, 8)
    with pytest.raises(B200Error):
        ops.verify_reduce(x, x)
    with pytest.raises(B200Error):
        verify.verify_equiv(x, x)
    with pytest.raises(B200Error):
        ops.linear_f32(x, torch.zeros(8, 8))


def test_product_never_imports_oracle():
    for py in (ROOT / "catopt_b200").rglob("*.py"):
        src = py.read_text()
        assert "import oracle" not in src and "from oracle" not in src, py
