"""B200 bindings for catopt's generated-kernel tiers.

catopt's discovery game mints new ops (``scan_<i>_k``, ``decayed_<i>_k``) from
handler entries ``{"pattern": <spec tuple>, "kernel": <op name>, "args": <metavars>}``
and delivers them by generating a Triton kernel per handler
(``scan_triton_bindings`` / ``decayed_triton_bindings`` / ``hybrid_sink``,
catopt_discovery/genkernel.py:1277-1310, 1903-1925, 768-803).  This module is the
same seam with nothing generated: a handler whose spec is one of the two carrier
forms is bound to a hand-written kernel of ``libcatopt_b200.so``.

* scan tier — ``("applyd", ("aff_diag", a, b), h)``, the sequence form: the fold
  ``acc = a_t*acc + b_t`` along the step axis, one ``cb2_diag_fold_apply`` (rows
  in time order; an operand without a step axis is shared by every step);
  ``("applyd", <affd_compose tree of aff_diag leaves>, h)``, the unrolled form:
  the composed map of the leaves applied once, one ``cb2_diag_compose_apply``.
* decayed tier — ``("om_decayed", s, d, v)`` or the spelled
  ``("matmul", ("mul", s, d), v)``: ``(s*d) @ v`` on materialised scores, one
  ``cb2_gated_contract_fwd``.

Operand sub-specs (``("mul", "A", "B")`` in place of a metavar) are evaluated on the
device with the ambient torch bindings before the kernel call; they are
elementwise and small next to the fold or the contraction.  The semantics, the
positional calling convention (``fn(*vals)`` in the handler's ``args`` order) and
the decline rules follow the reference's bindings; what differs is the error
behaviour this package has everywhere: CPU tensors and dtypes other than
float32/bfloat16 raise ``B200Error`` instead of running somewhere else.

Only ``b200_hybrid_sink`` needs catopt importable; the binding builders take the
table of torch bindings as an argument.
"""
from __future__ import annotations

from typing import Any, Callable, Mapping

import torch

from . import ops
from ._lib import B200Error

__all__ = ["scan_site", "decayed_site", "b200_scan_bindings", "b200_decayed_bindings", "b200_gen_bindings",
           "b200_hybrid_sink"]


# --------------------------------------------------------------------------- spec helpers
def _split(spec: Any) -> tuple[list, dict | None]:
    """Children and the trailing attr dict (if any) of a spec node."""
    kids = [e for e in spec[1:] if not isinstance(e, dict)]
    attrs = next((e for e in spec[1:] if isinstance(e, dict)), None)
    return kids, attrs


def _is_node(spec: Any) -> bool:
    return isinstance(spec, (tuple, list)) and len(spec) >= 1 and isinstance(spec[0], str)


def _metas(spec: Any, out: list | None = None) -> list:
    """Ordered distinct metavar leaves (strings below the head position)."""
    out = [] if out is None else out
    if isinstance(spec, str):
        if spec not in out:
            out.append(spec)
    elif _is_node(spec):
        for e in spec[1:]:
            if not isinstance(e, dict):
                _metas(e, out)
    return out


def _spec_ops(spec: Any, out: set | None = None) -> set:
    out = set() if out is None else out
    if _is_node(spec):
        out.add(spec[0])
        for e in spec[1:]:
            if not isinstance(e, dict):
                _spec_ops(e, out)
    return out


def _eval(spec: Any, env: Mapping[str, Any], bindings: Mapping[str, Callable]) -> Any:
    """Value of a spec under a metavar environment (leaf numbers are constants)."""
    if isinstance(spec, str):
        return env[spec]
    if _is_node(spec):
        kids, attrs = _split(spec)
        return bindings[spec[0]](*[_eval(k, env, bindings) for k in kids], **(attrs or {}))
    return spec


def _leaves(f_spec: Any) -> list | None:
    """``(a, b)`` operand specs of an ``aff_diag`` / ``affd_compose`` tree in product
    order (leftmost = applied last), or ``None`` for anything else."""
    if not _is_node(f_spec):
        return None
    kids, attrs = _split(f_spec)
    if attrs is not None or len(kids) != 2:
        return None
    if f_spec[0] == "aff_diag":
        return [(kids[0], kids[1])]
    if f_spec[0] == "affd_compose":
        left, right = _leaves(kids[0]), _leaves(kids[1])
        return None if left is None or right is None else left + right
    return None


# --------------------------------------------------------------------------- recognisers
def scan_site(spec: Any) -> dict | None:
    """Descriptor of an ``applyd`` carrier spec, or ``None`` (decline).

    ``{"kind": "seq" | "unrolled", "leaves": [(a_spec, b_spec), ...], "h": meta,
    "axis": int | None (only when the spec declares one)}``.  One ``aff_diag`` leaf is
    the sequence form unless the ``applyd`` node pins ``{"kind": "unrolled"}``; a
    compose tree is unrolled (the rule of ``scan_spec``/``_scan_kind``,
    catopt_discovery/genkernel.py:947-985, 1012-1019).
    """
    if not (_is_node(spec) and spec[0] == "applyd"):
        return None
    kids, attrs = _split(spec)
    if len(kids) != 2 or not (isinstance(kids[1], str) and kids[1].isidentifier()):
        return None
    leaves = _leaves(kids[0])
    if leaves is None:
        return None
    kind = (attrs or {}).get("kind")
    if kind is None:
        kind = "seq" if len(leaves) == 1 else "unrolled"
    if kind not in ("seq", "unrolled") or (kind == "seq" and len(leaves) != 1):
        return None
    info: dict[str, Any] = {"kind": kind, "leaves": leaves, "h": kids[1]}
    if attrs is not None and "axis" in attrs:
        info["axis"] = attrs["axis"]
    return info


def decayed_site(spec: Any) -> dict | None:
    """``{"s": spec, "d": spec, "v": spec}`` for ``("om_decayed", s, d, v)`` or the spelled
    ``("matmul", ("mul", s, d), v)``, attr-free, with a tensor-valued ``v`` and a
    tensor-valued ``s`` or ``d`` (the rules of ``_decayed_operands`` / ``decayed_spec``,
    catopt_discovery/genkernel.py:1418-1437, 1480-1517); ``None`` otherwise."""
    if not _is_node(spec):
        return None
    kids, attrs = _split(spec)
    if attrs is not None:
        return None
    if spec[0] == "om_decayed" and len(kids) == 3:
        s, d, v = kids
    elif spec[0] == "matmul" and len(kids) == 2 and _is_node(kids[0]) and kids[0][0] == "mul":
        inner, inner_attrs = _split(kids[0])
        if inner_attrs is not None or len(inner) != 2:
            return None
        s, d, v = inner[0], inner[1], kids[1]
    else:
        return None
    if not _metas(v) or not (_metas(s) or _metas(d)):
        return None
    return {"s": s, "d": d, "v": v}


# --------------------------------------------------------------------------- bindings
def _ambient_bindings() -> Mapping[str, Callable]:
    import catopt_torch.torch_bridge as tb

    return tb._IR_TO_TORCH


def _tensor(x: Any, like: torch.Tensor) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x, dtype=like.dtype, device=like.device)


def _require_cuda(vals: Mapping[str, Any], what: str) -> None:
    for name, t in vals.items():
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise B200Error(f"{what}: operand {name} is not a CUDA tensor (no CPU fallback)")


def _step_axis(full: tuple, h_shape: tuple, axis: int | None) -> int:
    """The step axis of the common sequence shape: the declared one, or the only axis
    whose removal leaves a shape ``h`` broadcasts into (``_seq_axis``,
    catopt_discovery/genkernel.py:1136-1160)."""
    if axis is not None:
        return axis % len(full)
    cand = []
    for i in range(len(full)):
        rest = full[:i] + full[i + 1:]
        try:
            if tuple(torch.broadcast_shapes(tuple(h_shape), rest)) == tuple(rest):
                cand.append(i)
        except RuntimeError:
            pass
    if len(cand) != 1:
        raise ValueError(f"scan axis is not determined by the shapes: candidates={tuple(cand)} "
                         f"for full={tuple(full)} h={tuple(h_shape)}")
    return cand[0]


def _seq_binding(info: dict, args: tuple, axis: int | None, bindings: Mapping[str, Callable]) -> Callable:
    a_spec, b_spec = info["leaves"][0]

    def fn(*vals: Any, **_attrs: Any) -> torch.Tensor:
        env = dict(zip(args, vals, strict=True))
        _require_cuda(env, "generated scan binding")
        h = env[info["h"]]
        a = _tensor(_eval(a_spec, env, bindings), h)
        b = _tensor(_eval(b_spec, env, bindings), h)
        dt = torch.promote_types(torch.promote_types(a.dtype, b.dtype), h.dtype)
        full = tuple(torch.broadcast_shapes(a.shape, b.shape))
        if not full:
            raise ValueError("scan operands carry no step axis")
        ax = _step_axis(full, tuple(h.shape), axis)
        state = full[:ax] + full[ax + 1:]
        if tuple(torch.broadcast_shapes(tuple(h.shape), state)) != tuple(state):
            raise RuntimeError(f"state {tuple(h.shape)} does not broadcast into {tuple(state)}")

        def rows(x: torch.Tensor) -> torch.Tensor:
            x = x.to(dt).expand(full).movedim(ax, 0)
            # an operand that does not vary along the step axis is handed over as one row
            return x[0] if x.stride(0) == 0 and full[ax] > 1 else x

        return ops.diag_fold_apply(rows(a), rows(b), h.to(dt).expand(state).contiguous())

    return fn


def _unrolled_binding(info: dict, args: tuple, bindings: Mapping[str, Callable]) -> Callable:
    leaves = info["leaves"]

    def fn(*vals: Any, **_attrs: Any) -> torch.Tensor:
        env = dict(zip(args, vals, strict=True))
        _require_cuda(env, "generated scan binding")
        h = env[info["h"]]
        av = [_tensor(_eval(a, env, bindings), h) for a, _ in leaves]
        bv = [_tensor(_eval(b, env, bindings), h) for _, b in leaves]
        dt = h.dtype
        for t in av + bv:
            dt = torch.promote_types(dt, t.dtype)
        shape = tuple(torch.broadcast_shapes(h.shape, *[t.shape for t in av + bv]))
        a_seq = torch.stack([t.to(dt).expand(shape) for t in av])
        b_seq = torch.stack([t.to(dt).expand(shape) for t in bv])
        out = ops.diag_compose_apply(a_seq, b_seq, h.to(dt).expand(shape).contiguous())
        if out is None:
            raise B200Error(f"unsupported dtype {dt}: the kernels take float32 or bfloat16")
        return out

    return fn


def b200_scan_bindings(handlers: Mapping[str, dict], *, axis: int | None = -2,
                       bindings: Mapping[str, Callable] | None = None) -> dict:
    """One binding per handler whose pattern is an ``applyd`` carrier spec.

    Drop-in for ``scan_triton_bindings`` (catopt_discovery/genkernel.py:1277-1310): the
    step axis defaults to ``-2``, a handler may pin ``"axis"``, the spec may declare it
    as an ``applyd`` attr, ``None`` derives it from the state shape at call time.
    Unrecognised specs are skipped.
    """
    table = _ambient_bindings() if bindings is None else bindings
    out: dict[str, Callable] = {}
    for h in handlers.values():
        info = scan_site(h["pattern"])
        if info is None:
            continue
        operand_ops = set()
        for a, b in info["leaves"]:
            operand_ops |= _spec_ops(a) | _spec_ops(b)
        if not operand_ops <= set(table):
            continue   # an operand sub-spec nothing can evaluate: decline
        args = tuple(h.get("args") or _metas(h["pattern"]))
        if info["kind"] == "seq":
            out[h["kernel"]] = _seq_binding(info, args, h.get("axis", info.get("axis", axis)), table)
        else:
            out[h["kernel"]] = _unrolled_binding(info, args, table)
    return out


def b200_decayed_bindings(handlers: Mapping[str, dict], *,
                          bindings: Mapping[str, Callable] | None = None) -> dict:
    """One binding per handler whose pattern is a decayed-contraction spec.

    Drop-in for ``decayed_triton_bindings`` (catopt_discovery/genkernel.py:1903-1925):
    ``fn(*vals)`` binds the metavars in the handler's ``args`` order and returns
    ``(s*d) @ v`` with the usual broadcasting over leading dims; an empty output comes
    back empty and an empty contraction as zeros, without a launch.
    """
    table = _ambient_bindings() if bindings is None else bindings
    out: dict[str, Callable] = {}
    for h in handlers.values():
        site = decayed_site(h["pattern"])
        if site is None:
            continue
        if not (_spec_ops(site["s"]) | _spec_ops(site["d"]) | _spec_ops(site["v"])) <= set(table):
            continue
        args = tuple(h.get("args") or _metas(h["pattern"]))

        def fn(*vals: Any, _site=site, _args=args, **_attrs: Any) -> torch.Tensor:
            env = dict(zip(_args, vals, strict=True))
            _require_cuda(env, "generated decayed binding")
            v = _eval(_site["v"], env, table)
            s = _tensor(_eval(_site["s"], env, table), v)
            d = _tensor(_eval(_site["d"], env, table), v)
            if s.dim() < 2:   # a constant or vector score: let broadcasting give it the gate's shape
                s = s.expand(torch.broadcast_shapes(s.shape, d.shape))
            return ops.gated_contract(s, d, v)

        out[h["kernel"]] = fn
    return out


def b200_gen_bindings(handlers: Mapping[str, dict], *, axis: int | None = -2,
                      bindings: Mapping[str, Callable] | None = None) -> dict:
    """Both tiers' bindings in one table."""
    out = b200_scan_bindings(handlers, axis=axis, bindings=bindings)
    out.update(b200_decayed_bindings(handlers, bindings=bindings))
    return out


def b200_hybrid_sink(handlers: Mapping[str, dict], *, compile_kernels: bool = False) -> Any:
    """The probe-path sink of ``hybrid_sink`` (catopt_discovery/genkernel.py:768-803) with
    the carrier tiers on the B200 kernels.

    Elementwise handlers keep the reference's spelled-body binding (``gen_bindings``;
    ``compile_kernels`` is passed through and is off by default), sequence-form scan
    specs are left out of that fallback as in the reference (their spelled body is one
    map application, not the fold), and scan / decayed handlers get the bindings above.
    The result is a ``B200Sink``, so the B200 executors and the GPU verify gate come
    with it.
    """
    import catopt_discovery.genkernel as gk
    from catopt_core.ops import OpTable

    from .sink import B200Sink

    def is_seq(spec: Any) -> bool:
        info = scan_site(spec)
        return info is not None and info["kind"] == "seq"

    plain = {k: h for k, h in handlers.items() if not is_seq(h["pattern"])}
    table = dict(_ambient_bindings())
    table.update(gk.gen_bindings(plain, compile_kernels=compile_kernels))
    table.update(b200_gen_bindings(handlers, bindings=_ambient_bindings()))
    return B200Sink(ops=OpTable.core().register(torch_bindings=table))
