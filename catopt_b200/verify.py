"""The verify gate on the GPU: same names and semantics as the reference's
``catopt_torch.report`` (``VerifyReport``, ``rel_diff``, ``verify_equiv``,
``verify_module``; report.py:43-202), with the four eager passes replaced by
one ``cb2_verify_reduce`` launch and, across ranks, one max all-reduce.

Gate semantics (NOT torch.allclose):
    max_abs = max|ref - out|           (difference formed in the tensor dtype)
    max_rel = max_abs / (max|ref| + 1e-8)
    passed  = max_rel < rtol and (atol is None or max_abs <= atol)
A NaN anywhere in the difference (or in ref) makes the maxima NaN and the
gate fail, as torch's ``max()`` propagates it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from . import ops
from ._lib import B200Error

_REL_FLOOR = 1e-8

__all__ = ["VerifyReport", "rel_diff", "verify_equiv", "verify_module", "verify_batched",
           "reports_from_result", "merge_across_ranks", "kernel_takes", "kernel_gate_calls"]

#: how many comparisons ``cb2_verify_reduce`` has served in this process (tests read it to
#: show that a gate ran on the kernel and not on a delegate)
kernel_gate_calls = 0


@dataclass(frozen=True)
class VerifyReport:
    """Result of one equivalence check (fields as in the reference)."""

    max_abs: float
    max_rel: float
    passed: bool
    per_output: tuple[float, ...] | None = None


def _report(max_abs: float, max_ref: float, rtol: float, atol: float | None) -> VerifyReport:
    max_rel = max_abs / (max_ref + _REL_FLOOR)
    passed = bool(max_rel < rtol) and (atol is None or bool(max_abs <= atol))
    return VerifyReport(max_abs=max_abs, max_rel=max_rel, passed=passed)


def reports_from_result(result: torch.Tensor, rtol: float = 1e-4,
                        atol: float | None = None) -> list[VerifyReport]:
    """Turn a ``[n_seg, 4]`` kernel result into one report per segment.

    This is the single device-to-host read of a verify step.
    """
    nan = float("nan")
    reps = []
    for max_abs, max_ref, nan_diff, nan_ref in result.tolist():
        reps.append(_report(nan if nan_diff else max_abs, nan if nan_ref else max_ref, rtol, atol))
    return reps


def _prepare(ref: torch.Tensor, out: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Mirror torch's promotion/broadcast of ``ref - out`` before the kernel."""
    if not (isinstance(ref, torch.Tensor) and isinstance(out, torch.Tensor)):
        raise B200Error("verify takes tensors (or tuples of tensors)")
    if not (ref.is_cuda and out.is_cuda):
        raise B200Error("catopt_b200.verify runs on CUDA tensors only (no CPU fallback)")
    dt = torch.result_type(ref, out)
    if dt not in (torch.float32, torch.bfloat16):
        raise B200Error(f"verify supports float32 and bfloat16 results, got {dt}")
    shape = torch.broadcast_shapes(ref.shape, out.shape)
    if ref.numel() == 0 or out.numel() == 0:
        raise RuntimeError("max(): Expected reduction dim to be specified for input.numel() == 0")
    ref2 = ref.to(dt).expand(shape).contiguous()
    out2 = out.to(dt).expand(shape).contiguous()
    return ref2, out2


def kernel_takes(ref: Any, out: Any) -> bool:
    """Whether ``cb2_verify_reduce`` can compare this pair: two non-empty CUDA tensors on
    one device whose difference is float32 or bfloat16."""
    if not (isinstance(ref, torch.Tensor) and isinstance(out, torch.Tensor)):
        return False
    if not (ref.is_cuda and out.is_cuda) or ref.device != out.device:
        return False
    if ref.numel() == 0 or out.numel() == 0:
        return False
    return torch.result_type(ref, out) in (torch.float32, torch.bfloat16)


def _verify_pair(ref: torch.Tensor, out: torch.Tensor, rtol: float, atol: float | None,
                 delegate: Any = None) -> VerifyReport:
    # max|ref| is taken over ref's own elements; broadcasting ref does not change it.
    global kernel_gate_calls
    if delegate is not None and not kernel_takes(ref, out):
        return delegate(ref, out, rtol=rtol, atol=atol)
    ref2, out2 = _prepare(ref, out)
    with torch.cuda.device(ref2.device):
        res = ops.verify_reduce(ref2, out2, 1)
        rep = reports_from_result(res, rtol, atol)[0]
        # the read-back above synchronised: a bounded wait that ran out in any kernel
        # launched before this gate on the device surfaces here
        ops.check_device_status(ref2.device)
    kernel_gate_calls += 1
    return rep


def _flatten_outputs(x: Any) -> list:
    if isinstance(x, (tuple, list)):
        flat: list = []
        for item in x:
            flat.extend(_flatten_outputs(item))
        return flat
    return [x]


def verify_equiv(ref_out: Any, out: Any, rtol: float = 1e-4, atol: float | None = None,
                 delegate: Any = None) -> VerifyReport:
    """Compare two already-computed outputs (tensor or tuple/list of tensors).

    Multi-output: both sides are flattened; a different number of outputs fails
    closed with ``inf``; the scalars are the worst case and ``per_output`` lists
    each output's ``max_abs``.

    ``delegate(ref, out, rtol=, atol=)``: who compares a pair the kernel does not take
    (fp64, integer or host tensors).  Without one such a pair raises ``B200Error``; the
    catopt-facing sink passes the reference's own gate, so a model the reference can
    verify is still gated.
    """
    if not isinstance(ref_out, (tuple, list)):
        return _verify_pair(ref_out, out, rtol, atol, delegate)
    ref_flat, out_flat = _flatten_outputs(ref_out), _flatten_outputs(out)
    if not isinstance(out, (tuple, list)) or len(out_flat) != len(ref_flat):
        return VerifyReport(max_abs=float("inf"), max_rel=float("inf"), passed=False)
    reports = [verify_equiv(r, o, rtol=rtol, atol=atol, delegate=delegate) for r, o in zip(ref_flat, out_flat)]
    return VerifyReport(
        max_abs=max(r.max_abs for r in reports),
        max_rel=max(r.max_rel for r in reports),
        passed=all(r.passed for r in reports),
        per_output=tuple(r.max_abs for r in reports),
    )


def rel_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    """``max|a-b| / (max|a| + 1e-8)`` (report.py:59-67)."""
    return _verify_pair(a, b, float("inf"), None).max_rel


def verify_module(ref_mod: torch.nn.Module, opt_mod: torch.nn.Module, inputs: Any,
                  rtol: float = 1e-4, atol: float | None = None, delegate: Any = None) -> VerifyReport:
    """Run both modules on (cloned) ``inputs`` under ``no_grad`` and compare
    (``delegate``: see ``verify_equiv``)."""
    args = inputs if isinstance(inputs, tuple) else (inputs,)
    ref_mod.eval()
    opt_mod.eval()
    with torch.no_grad():
        ref = ref_mod(*[a.clone() if isinstance(a, torch.Tensor) else a for a in args])
        out = opt_mod(*[a.clone() if isinstance(a, torch.Tensor) else a for a in args])
    return verify_equiv(ref, out, rtol=rtol, atol=atol, delegate=delegate)


def verify_batched(ref: torch.Tensor, out: torch.Tensor, n_checks: int, *, rtol: float = 1e-4,
                   atol: float | None = None, group: Any = None,
                   result: torch.Tensor | None = None) -> list[VerifyReport]:
    """Batched gate: ``n_checks`` comparisons stacked along dim 0.

    ``ref``/``out`` are ``[n_checks, ...]`` (all probes of one check contiguous);
    one launch reduces every check.  When ``torch.distributed`` is initialised
    (probes sharded over ranks) the per-rank ``[n_checks, 4]`` maxima and NaN
    flags are combined with a single ``all_reduce(MAX)``, so every rank returns
    the same reports.
    """
    if ref.shape != out.shape or ref.dtype != out.dtype or ref.shape[0] != n_checks:
        raise B200Error("verify_batched needs equal shapes [n_checks, ...] and dtypes")
    res = merge_across_ranks(ops.verify_reduce(ref, out, n_checks, result=result), group)
    return reports_from_result(res, rtol, atol)


def merge_across_ranks(result: torch.Tensor, group: Any = None) -> torch.Tensor:
    """Combine per-rank ``[n_checks, 4]`` results in place with ONE collective.

    All four fields (two maxima, two 0/1 NaN flags) are non-negative floats, so
    ``all_reduce(MAX)`` merges them exactly and every rank ends with the same
    tensor.  A no-op without an initialised process group.
    """
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(result, op=dist.ReduceOp.MAX, group=group)
    return result
