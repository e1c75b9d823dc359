"""The allocation-free chain fold (``cb2_chain_fold_f32_noalloc``).

Some users of this library fold weight chains at a point where they must not
allocate device memory (the allocator is frozen, or they only hold raw
pointers), so this entry point keeps its intermediates in a static device
array.  The test calls it through the C ABI twice in a row and expects the
bits of the ordinary entry point both times: the second call proves that what
the first call left in the shared array does no harm.  Collected last on
purpose, so a failure here cannot hide any other test's result.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _fold(lib, fn_name, weights, scratch=None):
    k = len(weights)
    dims = [weights[0].shape[1]] + [w.shape[0] for w in weights]
    dims_c = (C.c_int * (k + 1))(*dims)
    ptrs = (C.c_void_p * k)(*[w.data_ptr() for w in weights])
    out = torch.empty(dims[-1], dims[0], dtype=torch.float32, device=weights[0].device)
    stream = int(torch.cuda.current_stream().cuda_stream)
    if fn_name == "cb2_chain_fold_f32":
        rc = lib.cb2_chain_fold_f32(ptrs, dims_c, k, out.data_ptr(), scratch.data_ptr(),
                                    scratch.numel(), stream)
    else:
        rc = lib.cb2_chain_fold_f32_noalloc(ptrs, dims_c, k, out.data_ptr(), stream)
    return rc, out


def test_noalloc_fold_matches_regular_fold_twice():
    from catopt_b200 import _lib, build

    build.build()
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(99)
    limit = lib.cb2_chain_fold_f32_noalloc_max_bytes()
    assert limit == 2 * 512 * 512 * 4
    scratch = torch.empty(limit, dtype=torch.uint8, device=dev)
    for shapes in ([(512, 512)] * 8, [(96, 40), (512, 96), (33, 512), (7, 33)]):
        ws = [(torch.randn(o, i, generator=g) / i ** 0.5).to(dev) for o, i in shapes]
        rc, want = _fold(lib, "cb2_chain_fold_f32", ws, scratch)
        assert rc == 0
        for _ in range(2):  # two calls in a row share the static array
            rc, got = _fold(lib, "cb2_chain_fold_f32_noalloc", ws)
            assert rc == 0
            torch.cuda.synchronize()
            assert torch.equal(got, want)
    # beyond the static array: refused with a clear status, nothing launched
    big = [torch.zeros(1024, 1024, device=dev) for _ in range(3)]
    rc, _ = _fold(lib, "cb2_chain_fold_f32_noalloc", big)
    assert rc == 7 and "scratch" in _lib.status_str(rc)
