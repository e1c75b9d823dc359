"""ctypes binding of ``libcatopt_b200.so`` (the C ABI in ``include/catopt_b200.h``).

There is deliberately no fallback: if the shared library is missing or a call
returns a non-zero status, a :class:`B200Error` is raised.  The modules in this
package never compute on the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcatopt_b200.so"

CB2_OK = 0
CB2_WAIT_TIMEOUT = 5
CB2_F32 = 0
CB2_BF16 = 1

#: name -> (restype, argtypes); mirrors include/catopt_b200.h one to one.
SIGNATURES: dict[str, tuple] = {
    "cb2_version": (C.c_int, []),
    "cb2_status_str": (C.c_char_p, [C.c_int]),
    "cb2_wait_for_flag": (C.c_int, [C.c_void_p, C.c_uint, C.c_void_p, C.c_void_p]),
    "cb2_verify_reduce": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_linear_f32_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "cb2_linear_f32": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
         C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p],
    ),
    "cb2_linear_f32_split_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "cb2_linear_f32_split_weight": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "cb2_linear_f32_presplit": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_matmul_f32": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p],
    ),
    "cb2_chain_fold_f32_scratch_bytes": (C.c_size_t, [C.POINTER(C.c_int), C.c_int]),
    "cb2_chain_fold_f32": (
        C.c_int,
        [C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int, C.c_void_p, C.c_void_p,
         C.c_size_t, C.c_void_p],
    ),
    "cb2_chain_fold_f32_noalloc_max_bytes": (C.c_size_t, []),
    "cb2_chain_fold_f32_noalloc": (
        C.c_int,
        [C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_decayed_chunk_scratch_bytes": (
        C.c_size_t,
        [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int],
    ),
    "cb2_diag_compose_scratch_bytes": (C.c_size_t, [C.c_longlong, C.c_longlong, C.c_int]),
    "cb2_diag_compose_apply": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_int,
         C.c_void_p, C.c_size_t, C.c_void_p],
    ),
    "cb2_diag_fold_apply": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong,
         C.c_longlong, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p],
    ),
    "cb2_diag_prefix_maps_scratch_bytes": (C.c_size_t, [C.c_longlong, C.c_longlong, C.c_int]),
    "cb2_diag_prefix_maps": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong,
         C.c_longlong, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p],
    ),
    "cb2_diag_scan_states": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong,
         C.c_longlong, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p],
    ),
    "cb2_gated_contract_on_tensor_cores": (
        C.c_int, [C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int],
    ),
    "cb2_gated_contract_fwd": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_int,
         C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_decayed_chunk_plan": (
        C.c_int,
        [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int],
    ),
    "cb2_decayed_chunk_on_tensor_cores": (
        C.c_int,
        [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int],
    ),
    "cb2_decayed_chunk_fwd": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int,
         C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p],
    ),
    "cb2_om_causal_fwd": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
         C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_om_fwd": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
         C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_om_bias_fwd": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong,
         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_void_p],
    ),
    "cb2_om_step_scratch_bytes": (C.c_size_t, [C.c_int] * 5),
    "cb2_om_bias_step": (
        C.c_int,
        [C.c_void_p] * 4 + [C.c_longlong] * 3 + [C.c_void_p] * 6 + [C.c_int] * 6 +
        [C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p],
    ),
    "cb2_om_step": (
        C.c_int,
        [C.c_void_p] * 9 + [C.c_int] * 6 + [C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t,
                                            C.c_void_p, C.c_void_p],
    ),
    "cb2_diag_scan_seg_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "cb2_diag_scan_seg_starts": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
         C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p],
    ),
    "cb2_diag_scan_fwd": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p],
    ),
}


class B200Error(RuntimeError):
    """The native library is missing or an entry point reported an error."""


_lib: C.CDLL | None = None


def load() -> C.CDLL:
    """Load the shared library once and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise B200Error(
            f"{LIB_PATH} not found: build it with `python -m catopt_b200.build` "
            "(there is no CPU fallback)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:  # pragma: no cover - build/ABI mismatch
            raise B200Error(f"{LIB_PATH} does not export {name}") from exc
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_str(status: int) -> str:
    return load().cb2_status_str(int(status)).decode()


def check(status: int, what: str) -> None:
    """Raise :class:`B200Error` unless ``status`` is ``CB2_OK``."""
    if status != CB2_OK:
        raise B200Error(f"{what}: {status_str(status)} (status {status})")


def dtype_code(dtype) -> int:
    """Map a torch dtype to the ABI's element code."""
    import torch

    if dtype == torch.float32:
        return CB2_F32
    if dtype == torch.bfloat16:
        return CB2_BF16
    raise B200Error(f"unsupported dtype {dtype}: the kernels take float32 or bfloat16")


def stream_ptr() -> int:
    """Raw handle of torch's current CUDA stream."""
    import torch

    return int(torch.cuda.current_stream().cuda_stream)


def require_device(*tensors) -> None:
    """Every tensor must be a CUDA tensor on the current device (any layout): the check
    for operands that are made contiguous later.  A host tensor or one on another GPU
    would hand the kernel a pointer it cannot legally touch."""
    import torch

    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise B200Error("catopt_b200 executors take CUDA tensors only (no CPU fallback)")
        if t.device.index != torch.cuda.current_device():
            raise B200Error(
                f"tensor on {t.device} but the current device is cuda:{torch.cuda.current_device()}"
            )


def require_cuda(*tensors) -> None:
    """Every tensor must be a contiguous CUDA tensor on the current device."""
    import torch

    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise B200Error("catopt_b200 executors take CUDA tensors only (no CPU fallback)")
        if not t.is_contiguous():
            raise B200Error("catopt_b200 executors take contiguous tensors")
        if t.device.index != torch.cuda.current_device():
            raise B200Error(
                f"tensor on {t.device} but the current device is cuda:{torch.cuda.current_device()}"
            )
