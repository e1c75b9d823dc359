"""Adapter into catopt's executor table (needs catopt importable).

catopt routes an extracted term to the first ``ExecutorSpec`` of
``Sink.executors`` whose ``carrier`` is not ``None`` and whose ``accepts(term)``
is true (catopt_orchestrator/optimize.py:485-495); mapping order is routing
order.  ``B200Sink`` puts three B200 specs in front of the torch ones:

* ``b200_om_decayed_chunked`` — the uniform K-chunk decayed term of
  ``om_decayed_kway_blocks`` (catopt_carriers/om.py:3076-3152).  ``accepts``
  reuses the reference's own parser (``build_decayed_plan``,
  decayed_lower.py:353-368) and then requires the exact state-carry shape:
  chunks ``split(q|k|v, dim=-2, sizes=[C]*K)`` of three shared bases, one shared
  ``decay(g, t=C)``, every pair ``i > j`` present once with row gate
  ``decay_vec(g, t=C, offset=(i-j)C)`` and column gate ``decay_vec(g, t=C,
  sign=-1)``, one constant scale.  Anything else is declined, so the reference's
  pairwise executor (or the generic module) still takes it.
* ``b200_scan`` — diagonal ``applyd(<aff_diag tree>, h)`` scan applications (the
  terms ``lift_scan_to_applyd`` creates); the reference's own plan builder and
  leaf stacking are reused, the composed-map reduction runs in
  ``cb2_diag_scan_fwd``.
* ``b200_linear_chain`` — ``linear(x, <matmul tree of weight Params>)``, the
  term ``assoc_linear`` leaves behind for a chain of bias-free Linear maps
  (catopt_core/laws/tensor.py:1293-1300) before ``_fold_weight_chains``
  (torch_bridge.py:2456-2510) folds it.

Both modules embed a plain ``IRModule`` (``eval_mod``) to evaluate operand
sub-terms, as every batched module of the reference does, and make one C-ABI
call for the hot part.  ``B200Sink.verify`` is the GPU verify gate.
"""
from __future__ import annotations

from typing import Any

import torch
from catopt_carriers.decayed_lower import build_decayed_plan
from catopt_carriers.om_lower import _slice_index
from catopt_core.ir import IR, Const, Op, Param
from catopt_core.ports import ExecutorSpec
from catopt_torch.adapters import TorchSink
from catopt_torch.torch_bridge import IRModule

from . import ops
from . import verify as b200_verify
from ._lib import B200Error
from .executors import _GraphMixin

__all__ = ["B200Sink", "b200_backend", "b200_target_profile", "decayed_state_carry_plan", "linear_chain_plan", "scan_diag_plan",
           "B200ChunkedDecayModule", "B200LinearChainModule"]


# --------------------------------------------------------------------------- decayed
def _chunk_of(term: Any, dim: int) -> tuple | None:
    """``split(base, dim, index=i, sizes=[C]*K)`` -> (base, i, K, C)."""
    p = _slice_index(term)
    if p is None:
        return None
    base, kind, d, idx, n, part = p
    if kind != "chunk" or part is None or d != dim:
        return None
    return base, idx, n, part


def _decay_vec_attrs(row: Any) -> tuple | None:
    """``unsqueeze(decay_vec(g, t, sign, offset), -1)`` -> (g, t, sign, offset)."""
    if not (isinstance(row, Op) and row.op == "unsqueeze" and row.attrs.get("dim") == -1):
        return None
    dv = row.args[0]
    if not (isinstance(dv, Op) and dv.op == "decay_vec"):
        return None
    a = dv.attrs
    return dv.args[0], int(a.get("t", 0) or 0), int(a["sign"]) if "sign" in a else 1, int(a.get("offset", 0) or 0)


def _const_value(t: Any) -> float | None:
    if isinstance(t, Const):
        return float(t.value)
    if isinstance(t, (int, float)):
        return float(t)
    return None


def decayed_state_carry_plan(root: Any) -> dict | None:
    """Recognise the uniform chunked decayed term and return what the kernel
    needs: ``{q, k, v (base terms), gamma (term), chunk, n, scale}``; ``None``
    for every other term."""
    plan = build_decayed_plan(root)
    if plan is None or plan["dim"] != -2 or plan["score_ab"] is None:
        return None
    K = plan["n"]
    if any(r is not None for r in plan["intra_row"]):
        return None
    dts = plan["decay_terms"]
    if not all(t == dts[0] for t in dts) or not (isinstance(dts[0], Op) and dts[0].op == "decay"):
        return None
    gamma, C = dts[0].args[0], int(dts[0].attrs.get("t", 0) or 0)
    scales = {_const_value(s) for s in plan["intra_scale"]} | {_const_value(p[3]) for p in plan["pairs"]}
    if len(scales) != 1 or None in scales:
        return None
    # intra operands: q_i, transpose(k) split on the last dim, v_i
    q = k = v = None
    for i, ((qa, kb), vi) in enumerate(zip(plan["score_ab"], plan["v_intra"])):
        cq, cv = _chunk_of(qa, -2), _chunk_of(vi, -2)
        ck = _chunk_of(kb, -1)
        if cq is None or cv is None or ck is None:
            return None
        kt = ck[0]
        if not (isinstance(kt, Op) and kt.op == "transpose"
                and {kt.attrs.get("dim0"), kt.attrs.get("dim1")} == {-1, -2}):
            return None
        if (cq[1:], cv[1:], ck[1:]) != ((i, K, C),) * 3:
            return None
        if i == 0:
            q, k, v = cq[0], kt.args[0], cv[0]
        elif (cq[0], kt.args[0], cv[0]) != (q, k, v):
            return None
    # cross operands: every pair i > j exactly once, gates g^((i-j)C + r) and g^(-r)
    seen = set()
    for qi, si, row, _ in plan["pairs"]:
        cq = _chunk_of(plan["q_terms"][qi], -2)
        kj, col, vj, d0, d1 = plan["states"][si]
        ck, cv = _chunk_of(kj, -2), _chunk_of(vj, -2)
        rg, cg = _decay_vec_attrs(row), _decay_vec_attrs(col)
        if None in (cq, ck, cv, rg, cg) or {d0, d1} != {-1, -2}:
            return None
        i, j = cq[1], ck[1]
        if (cq[0], ck[0], cv[0]) != (q, k, v) or cv[1] != j or not j < i < K:
            return None
        if rg != (gamma, C, 1, (i - j) * C) or cg != (gamma, C, -1, 0):
            return None
        seen.add((i, j))
    if len(seen) != K * (K - 1) // 2 or len(plan["pairs"]) != len(seen):
        return None
    return {"q": q, "k": k, "v": v, "gamma": gamma, "chunk": C, "n": K, "scale": scales.pop()}


class _EvalBase(_GraphMixin, torch.nn.Module):
    """Shared plumbing: embedded ``IRModule`` + operand evaluation."""

    def __init__(self, ir: IR, param_values: dict | None) -> None:
        super().__init__()
        self._inputs = ir.inputs
        self.eval_mod = IRModule(ir, param_values)
        self._init_graph_state()

    def _input_env(self, xs: tuple) -> tuple:
        """``(x, env)`` as the reference's batched modules build it
        (executors/base.py:227-241): ``"self"`` and every named IR input map to
        the matching positional argument, missing ones default to the first."""
        x = xs[0] if xs else None
        env: dict[str, Any] = {"self": x}
        for i, inp in enumerate(self._inputs):
            env[inp.name] = xs[i] if i < len(xs) else x
        return x, env

    def _ev(self, xs: tuple):
        x, env = self._input_env(xs)
        memo: dict = {None: None}
        return lambda t: self.eval_mod._eval(t, env, x, memo)


class B200ChunkedDecayModule(_EvalBase):
    """Drop-in for ``ChunkedDecayModule`` (decayed_lower.py:381-724): same
    constructor, ``_plan`` / ``is_batched`` / ``n_blocks`` / graph API; the
    forward evaluates the q, k, v bases through ``eval_mod`` and runs
    ``cb2_decayed_chunk_fwd``.  A non-matching IR degrades to ``eval_mod``."""

    def __init__(self, ir: IR, param_values: dict | None = None) -> None:
        super().__init__(ir, param_values)
        self._plan = decayed_state_carry_plan(self.eval_mod._root)

    @property
    def is_batched(self) -> bool:
        return self._plan is not None

    @property
    def n_blocks(self) -> int:
        return 0 if self._plan is None else self._plan["n"]

    def _forward_impl(self, *xs: torch.Tensor) -> Any:
        plan = self._plan
        if plan is None:
            return self.eval_mod(*xs)
        ev = self._ev(xs)
        q, k, v, g = ev(plan["q"]), ev(plan["k"]), ev(plan["v"]), ev(plan["gamma"])
        lead = q.shape[:-2]
        if len(lead) == 0:
            raise B200Error("decayed executor needs at least one leading (head) axis")
        H = lead[-1]
        g = torch.as_tensor(g, dtype=torch.float32, device=q.device).reshape(-1)
        g = (g.expand(H) if g.numel() == 1 else g).contiguous()
        q4, k4, v4 = (t.reshape(-1, H, t.shape[-2], t.shape[-1]).contiguous() for t in (q, k, v))
        out = ops.decayed_chunk_fwd(q4, k4, v4, g, plan["chunk"], plan["scale"])
        return out.reshape(*lead, out.shape[-2], out.shape[-1])


# --------------------------------------------------------------------------- linear chain
def _weight_tree(t: Any) -> bool:
    """A Var-free tree of ``matmul`` over Params."""
    if isinstance(t, Param):
        return True
    return isinstance(t, Op) and t.op == "matmul" and len(t.args) == 2 and all(_weight_tree(a) for a in t.args)


def linear_chain_plan(root: Any) -> dict | None:
    """``linear(x, W[, bias])`` with ``W`` a product tree of at least two weight
    Params -> ``{x, weight_tree, bias}``."""
    if not (isinstance(root, Op) and root.op == "linear" and len(root.args) in (2, 3)):
        return None
    w = root.args[1]
    if not (isinstance(w, Op) and _weight_tree(w)):
        return None
    bias = root.args[2] if len(root.args) == 3 else None
    if bias is not None and not isinstance(bias, Param):
        return None
    return {"x": root.args[0], "weight_tree": w, "bias": bias}


def _right_nested_chain(t: Any) -> list | None:
    """matmul(Wk-1, matmul(..., matmul(W1, W0))) -> [W0, W1, ..., Wk-1]."""
    chain = []
    while isinstance(t, Op):
        if not isinstance(t.args[0], Param):
            return None
        chain.append(t.args[0])
        t = t.args[1]
    chain.append(t)
    return chain[::-1]


class B200LinearChainModule(_EvalBase):
    """``linear(x, <weight product>)``: the product is folded once on the GPU at
    construction (``cb2_chain_fold_f32`` for the right-nested form the search
    extracts, ``cb2_matmul_f32`` node by node otherwise) and registered as
    ``fused_weight``; each forward is one ``cb2_linear_f32``."""

    def __init__(self, ir: IR, param_values: dict | None = None) -> None:
        # plan from the UN-folded root: IRModule folds the tree away at construction
        plan = linear_chain_plan(ir.root)
        super().__init__(ir, param_values)
        self._plan = plan
        if plan is None:
            return
        vals = param_values or {}

        def val(p: Param) -> torch.Tensor:
            t = vals.get(p.name)
            if t is None:
                raise B200Error(f"no value for weight {p.name}")
            return t.detach().to(device="cuda", dtype=torch.float32).contiguous()

        chain = _right_nested_chain(plan["weight_tree"])
        if chain is not None:
            fused = ops.chain_fold_f32([val(p) for p in chain])
        else:
            def fold(t):
                return val(t) if isinstance(t, Param) else ops.matmul_f32(fold(t.args[0]), fold(t.args[1]))
            fused = fold(plan["weight_tree"])
        self.fused_weight = torch.nn.Parameter(fused, requires_grad=False)
        self.bias = None if plan["bias"] is None else torch.nn.Parameter(val(plan["bias"]), requires_grad=False)

    @property
    def is_batched(self) -> bool:
        return self._plan is not None

    def _forward_impl(self, *xs: torch.Tensor) -> Any:
        if self._plan is None:
            return self.eval_mod(*xs)
        x = self._ev(xs)(self._plan["x"])
        return ops.linear_f32(x.contiguous(), self.fused_weight, self.bias)


# --------------------------------------------------------------------------- scan
def scan_diag_plan(root: Any) -> dict | None:
    """The reference's scan plan (``build_scan_plan``, scan_lower.py:339-424)
    when the term is a *diagonal* ``applyd(<aff_diag tree>, h)`` application."""
    from catopt_carriers.scan_lower import build_scan_plan

    plan = build_scan_plan(root)
    return plan if plan is not None and plan.get("diagonal") else None


def _make_scan_module():
    from catopt_carriers.scan_lower import BatchedScanModule

    class B200ScanModule(BatchedScanModule):
        """``BatchedScanModule`` (scan_lower.py:427-807) with the composed-map
        reduction replaced by ``cb2_diag_scan_fwd``.

        Term analysis, leaf stacking and the re-application of stripped output
        views stay the reference's own code; only the step that folds the leaf
        maps over the initial state is swapped (the hook the reference's
        ``fused=`` mode uses, ``_forward_fused``, scan_lower.py:785-807).  The
        leaves arrive in product order (latest step first); the kernel runs them
        chronologically as ``h <- a_t * h + u_t`` over the flattened state
        (channels = state elements, N = 1, b = c = 1) and returns the final state.
        fp64 tensors or state sizes the kernel cannot address degrade to the
        reference's own eager reduction on the same device.
        """

        def __init__(self, ir: IR, param_values: dict | None = None) -> None:
            super().__init__(ir, param_values, fused="eager")
            self.kernel_calls = 0

        def _forward_fused(self, a_vals, b_vals, ev):
            plan = self._plan
            if not plan["diagonal"]:
                return super()._forward_fused(a_vals, b_vals, ev)
            if not a_vals.is_cuda:
                raise B200Error("B200ScanModule runs on CUDA tensors only (no CPU fallback)")
            occ = self._occ_index(a_vals)
            if occ is not None:
                a_vals, b_vals = a_vals.index_select(0, occ), b_vals.index_select(0, occ)
            out = ops.diag_compose_apply(a_vals, b_vals, ev(plan["h"]))
            if out is None:   # fp64 / unaddressable state size: the reference's own reduction
                return super()._forward_fused(a_vals, b_vals, ev)
            self.kernel_calls += 1
            return out

    return B200ScanModule


# --------------------------------------------------------------------------- sink
def _engaged(m: Any) -> bool:
    return bool(getattr(m, "is_batched", False))


class B200Sink(TorchSink):
    """``TorchSink`` with the B200 executors routed first and the GPU verify gate."""

    @property
    def executors(self):
        if getattr(self, "_b200_executors", None) is None:
            table = {
                "b200_om_decayed_chunked": ExecutorSpec(
                    "b200_om_decayed_chunked",
                    lambda ir, p: B200ChunkedDecayModule(ir, param_values=p),
                    lambda term: decayed_state_carry_plan(term) is not None,
                    _engaged,
                    (frozenset({"concat"}), frozenset({"add", "mul", "div", "matmul"}),
                     frozenset({"om_decayed", "decay", "decay_vec"})),
                ),
                "b200_scan": ExecutorSpec(
                    "b200_scan",
                    lambda ir, p: _make_scan_module()(ir, param_values=p),
                    lambda term: scan_diag_plan(term) is not None,
                    _engaged,
                    (frozenset({"applyd"}), frozenset({"affd_compose"}), frozenset({"aff_diag"})),
                ),
                "b200_linear_chain": ExecutorSpec(
                    "b200_linear_chain",
                    lambda ir, p: B200LinearChainModule(ir, param_values=p),
                    lambda term: linear_chain_plan(term) is not None,
                    _engaged,
                    (frozenset({"linear"}), frozenset({"matmul"}), frozenset()),
                ),
            }
            table.update(super().executors)
            self._b200_executors = table
        return self._b200_executors

    def verify(self, ref: Any, opt: Any, inputs: Any, *, rtol: float = 1e-4, atol: float | None = None):
        return b200_verify.verify_module(ref, opt, inputs, rtol=rtol, atol=atol)


def b200_target_profile():
    """The measured B200 ``TargetProfile`` shipped with this package
    (catopt_core/profile.py:75-150), for catopt's roofline cost model:
    ``roofline_cost_for(b200_target_profile())``."""
    from pathlib import Path

    from catopt_core.profile import TargetProfile

    return TargetProfile.from_json((Path(__file__).with_name("target_profile_b200.json")).read_text())


def b200_backend():
    """``Backend`` value for ``Optimizer(backend=...)`` with the B200 sink."""
    from catopt_torch.backend import TorchBackend

    return TorchBackend(sink=B200Sink())
