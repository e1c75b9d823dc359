"""Adapter into catopt's executor table (needs catopt importable).

catopt routes an extracted term to the first ``ExecutorSpec`` of
``Sink.executors`` whose ``carrier`` is not ``None`` and whose ``accepts(term)``
is true (catopt_orchestrator/optimize.py:485-495); mapping order is routing
order.  ``B200Sink`` puts eight B200 specs in front of the torch ones:

* ``b200_om_decayed_chunked`` — the uniform K-chunk decayed term of
  ``om_decayed_kway_blocks`` (catopt_carriers/om.py:3076-3152).  ``accepts``
  reuses the reference's own parser (``build_decayed_plan``,
  decayed_lower.py:353-368) and then requires the exact state-carry shape:
  chunks ``split(q|k|v, dim=-2, sizes=[C]*K)`` of three shared bases, one shared
  ``decay(g, t=C)``, every pair ``i > j`` present once with row gate
  ``decay_vec(g, t=C, offset=(i-j)C)`` and column gate ``decay_vec(g, t=C,
  sign=-1)``, one constant scale.  Terms over a ragged partition — what
  extraction really returns when the K-way law fires at two levels, e.g. pieces
  of 32,32,32,32,128,128,128 rows, which the reference's executor declines — are
  recognised by ``decayed_ragged_plan``.  Anything else is declined and goes to
  the next spec.
* ``b200_om_decayed_pairwise`` — whatever else ``build_decayed_plan`` accepts: a
  decay-row gate on the intra element, a second rate in some arms' masks, a missing
  cross pair (tests/test_decayed_lower.py:440-482 there).  These are not decayed
  attention of one sequence at one rate and have no state-carry form; they run the
  reference's ``ChunkedDecayModule`` with the intra element ``(s * d) @ v`` of all
  arms in one ``cb2_gated_contract_fwd``.
* ``b200_om_causal`` — causal softmax attention over a sequence of key/value blocks in
  its online-softmax carrier form ``om_apply(<om_compose tree of om_elem(masked
  scores_i, v_i)>)`` (``om_causal_plan``), causal or unmasked; one ``cb2_om_fwd``.
  ``b200_om_streaming`` names the same module for callers that want the raw
  carrier (``forward_state``: one ``cb2_om_step`` per block), as the reference
  lists its batched and streaming om executors separately.
* ``b200_scan`` — diagonal ``applyd(<aff_diag tree>, h)`` scan applications (the
  terms ``lift_scan_to_applyd`` creates); the reference's own plan builder and
  leaf stacking are reused, the composed-map reduction runs in
  ``cb2_diag_compose_apply`` (one pass over the stacked leaves).
* ``b200_scan_all`` — every state of an unrolled diagonal scan in the stacked-map
  form ``applyd(aff_diag(stack(affd_a f_t), stack(affd_b f_t)), h)`` that
  ``gather_applyd_stack`` offers (xcarrier.py:2252-2275), one ``cb2_diag_scan_states``;
  with the per-step readout ``sum(mul(., c), -1)`` around it, one ``cb2_diag_scan_fwd``.
  Tried before ``b200_scan``, whose plan builder would take the form as a one-leaf tree.
* ``b200_omd`` — deferred-affine attention ``omd_apply(<omd tree>, h)``: the
  reference's ``BatchedOmdModule`` with its all-prefix scan of the diagonal step
  maps (``_prefix_scan``) running in ``cb2_diag_prefix_maps`` (one pass).
* ``b200_linear_chain`` — ``linear(x, <matmul tree of weight Params>)``, the
  term ``assoc_linear`` leaves behind for a chain of bias-free Linear maps
  (catopt_core/laws/tensor.py:1293-1300) before ``_fold_weight_chains``
  (torch_bridge.py:2456-2510) folds it.

The modules embed a plain ``IRModule`` (``eval_mod``) to evaluate operand
sub-terms, as every batched module of the reference does, and make one C-ABI
call for the hot part.  ``B200Sink.verify`` is the GPU verify gate.
"""
from __future__ import annotations

from typing import Any

import torch
from catopt_carriers.decayed_lower import build_decayed_plan
from catopt_carriers.om_lower import _slice_index
from catopt_core.ir import IR, Const, Op, Param, Var
from catopt_core.ports import ExecutorSpec
from catopt_core.typing import _shape_of
from catopt_torch.adapters import TorchSink
from catopt_torch.torch_bridge import IRModule

from . import ops
from . import verify as b200_verify
from ._lib import B200Error
from .executors import _GraphMixin, causal_softmax_blocks, decayed_whole_sequence, softmax_blocks_state

__all__ = ["B200Sink", "b200_backend", "b200_target_profile", "decayed_state_carry_plan", "decayed_ragged_plan",
           "decayed_plan", "uniform_decayed_term", "om_causal_plan", "linear_chain_plan", "scan_diag_plan",
           "scan_states_plan", "B200ChunkedDecayModule", "B200CausalSoftmaxModule", "B200LinearChainModule",
           "B200ScanStatesModule"]


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


# ---- ragged / hierarchical partitions: what the search really extracts -------------------
def _norm_dim(term: Any, dim: Any, memo: dict) -> int | None:
    """Axis as a negative index (needs the operand's rank when given as a positive one)."""
    if not isinstance(dim, int):
        return None
    if dim < 0:
        return dim
    shape = _shape_of(term, memo)
    return dim - len(shape) if isinstance(shape, tuple) and dim < len(shape) else None


def _split_piece(term: Any, memo: dict) -> tuple | None:
    """``split(x, dim, index, sizes)`` -> (x, negative dim, start, length, total)."""
    if not (isinstance(term, Op) and term.op == "split" and len(term.args) == 1):
        return None
    a = term.attrs
    sizes, idx = a.get("sizes"), a.get("index", 0)
    dim = _norm_dim(term.args[0], a.get("dim"), memo)
    if dim is None or not isinstance(idx, int) or not isinstance(sizes, (tuple, list)):
        return None
    if not all(isinstance(z, int) and z > 0 for z in sizes) or not 0 <= idx < len(sizes):
        return None
    return term.args[0], dim, sum(sizes[:idx]), sizes[idx], sum(sizes)


def _range_of(term: Any, dim: int, memo: dict | None = None) -> tuple | None:
    """Resolve (possibly nested) row/column slices of one base tensor to
    ``(base, start, length, total)`` along ``dim``; ``None`` for anything else."""
    memo = {} if memo is None else memo
    p = _split_piece(term, memo)
    if p is None or p[1] != dim:
        return None
    x, _, start, length, total = p
    inner = _range_of(x, dim, memo)
    if inner is None:
        return x, start, length, total
    base, s0, l0, t0 = inner
    return (base, s0 + start, length, t0) if total == l0 else None


def _is_swap_last_two(t: Any) -> bool:
    return (isinstance(t, Op) and t.op == "transpose" and len(t.args) == 1
            and {t.attrs.get("dim0"), t.attrs.get("dim1")} == {-1, -2})


def _gate(t: Any, dim: int) -> tuple | None:
    """``unsqueeze(decay_vec(g, t, sign, offset), dim)`` -> (g, t, sign, offset)."""
    if not (isinstance(t, Op) and t.op == "unsqueeze" and t.attrs.get("dim") == dim):
        return None
    dv = t.args[0]
    if not (isinstance(dv, Op) and dv.op == "decay_vec"):
        return None
    a = dv.attrs
    return dv.args[0], int(a.get("t", 0) or 0), int(a["sign"]) if "sign" in a else 1, int(a.get("offset", 0) or 0)


class _Coverage:
    """Abstract interpretation of a chunked decayed term.

    Every sub-term is read as a list of row pieces ``[a, s, cov]``: rows
    ``[a, a+s)`` of the output, with ``cov`` a list of ``(b, l, kind, scale)``
    saying which keys ``[b, b+l)`` those rows already attend to:

    * ``"diag"``: the causal decayed block of the rows with their own keys
      (``om_decayed(q_r k_r^T, decay(g, s), v_r)``; b = a, l = s);
    * ``"pend"``: an earlier key block weighted by ``g^(-c)`` (c the key's index in
      the block) — a cross product that still lacks its row gate;
    * ``"full"``: an earlier key block with the complete weight ``g^(t - s)``.

    ``add`` merges coverages on the common refinement of the row pieces,
    ``concat`` appends pieces, a row gate ``decay_vec(g, t, offset)`` completes
    pending blocks when ``offset`` is the distance from the key block's start to
    the gated rows' start, ``div`` by a constant multiplies the scale, a row
    ``split`` restricts pieces (cutting a diagonal block into an earlier full part
    and a smaller diagonal).  The term is decayed attention of the whole sequence
    iff at the end the pieces tile ``[0, T)`` and each piece holds its diagonal
    block plus full blocks tiling ``[0, a)``, all with one scale."""

    def __init__(self) -> None:
        self.q = self.k = self.v = self.gamma = None
        self.total: int | None = None
        self.memo: dict = {}
        self.cache: dict = {}

    def _same(self, name: str, val: Any) -> bool:
        cur = getattr(self, name)
        if cur is None:
            setattr(self, name, val)
            return True
        return cur == val

    def _rows(self, t: Any, dim: int, slot: str, transposed: bool = False) -> tuple | None:
        r = _range_of(t, dim, self.memo)
        if r is None:
            return None
        base, start, length, total = r
        if transposed:
            if not _is_swap_last_two(base):
                return None
            base = base.args[0]
        if not self._same(slot, base) or not self._same("total", total):
            return None
        return start, length

    # -- leaves ---------------------------------------------------------------------------
    def _om_decayed(self, t: Op) -> list | None:
        score, dec, vv = t.args
        if not (isinstance(score, Op) and score.op == "matmul" and len(score.args) == 2 and isinstance(dec, Op)):
            return None
        rq = self._rows(score.args[0], -2, "q")
        rk = self._rows(score.args[1], -1, "k", transposed=True)
        rv = self._rows(vv, -2, "v")
        if None in (rq, rk, rv) or rk != rv:
            return None
        (a, s), (b, l) = rq, rk
        if dec.op == "decay":
            if not self._same("gamma", dec.args[0]) or int(dec.attrs.get("t", 0) or 0) != s or (a, s) != (b, l):
                return None
            return [[a, s, [(a, s, "diag", 1.0)]]]
        col = _gate(dec, -2)          # (s_ij * g^(-c)[None, :]) @ v_j spelled as om_decayed
        if col is None or not self._same("gamma", col[0]) or col[1:] != (l, -1, 0) or b + l > a:
            return None
        return [[a, s, [(b, l, "pend", 1.0)]]]

    def _state_product(self, t: Op) -> list | None:
        """``q_r @ ((k_b * g^(-c)[:, None])^T @ v_b)``."""
        rq, state = self._rows(t.args[0], -2, "q"), t.args[1]
        if rq is None or not (isinstance(state, Op) and state.op == "matmul" and len(state.args) == 2):
            return None
        kt = state.args[0]
        if not _is_swap_last_two(kt):
            return None
        kg = kt.args[0]
        if not (isinstance(kg, Op) and kg.op == "mul" and len(kg.args) == 2):
            return None
        col, kk = _gate(kg.args[1], -1), kg.args[0]
        if col is None:
            col, kk = _gate(kg.args[0], -1), kg.args[1]
        if col is None or not self._same("gamma", col[0]):
            return None
        rk, rv = self._rows(kk, -2, "k"), self._rows(state.args[1], -2, "v")
        if rk is None or rk != rv or col[1:] != (rk[1], -1, 0) or rk[0] + rk[1] > rq[0]:
            return None
        return [[rq[0], rq[1], [(rk[0], rk[1], "pend", 1.0)]]]

    # -- combinators ----------------------------------------------------------------------
    @staticmethod
    def _restrict(pieces: list, lo: int, hi: int) -> list | None:
        """Rows [lo, hi) of a piece list that covers them."""
        out = []
        for a, s, cov in pieces:
            x, y = max(a, lo), min(a + s, hi)
            if x >= y:
                continue
            c2 = []
            for b, l, kind, sc in cov:
                if kind == "diag" and (x, y - x) != (b, l):
                    if x > b:
                        c2.append((b, x - b, "full", sc))
                    c2.append((x, y - x, "diag", sc))
                else:
                    c2.append((b, l, kind, sc))
            out.append([x, y - x, c2])
        if not out or out[0][0] != lo or out[-1][0] + out[-1][1] != hi:
            return None
        return out

    @staticmethod
    def _span(pieces: list) -> tuple:
        return pieces[0][0], pieces[-1][0] + pieces[-1][1]

    def _add(self, parts: list) -> list | None:
        span = self._span(parts[0])
        if any(self._span(p) != span for p in parts[1:]):
            return None
        cuts = sorted({span[0], span[1]} | {a for p in parts for a, _, _ in p})
        out = []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            cov = []
            for p in parts:
                r = self._restrict(p, lo, hi)
                if r is None or len(r) != 1:
                    return None
                cov.extend(r[0][2])
            out.append([lo, hi - lo, cov])
        return out

    def interp(self, t: Any) -> list | None:
        if not isinstance(t, Op):
            return None
        if t in self.cache:
            return self.cache[t]
        out = self._interp(t)
        self.cache[t] = out
        return out

    def _interp(self, t: Op) -> list | None:
        op, args = t.op, t.args
        if op == "div" and len(args) == 2 and _const_value(args[1]) is not None:
            x, c = self.interp(args[0]), _const_value(args[1])
            return None if x is None else [[a, s, [(b, l, kd, sc * c) for b, l, kd, sc in cov]] for a, s, cov in x]
        if op == "mul" and len(args) == 2:
            g, other = _gate(args[0], -1), args[1]
            if g is None:
                g, other = _gate(args[1], -1), args[0]
            if g is None or g[2] != 1 or not self._same("gamma", g[0]):
                return None
            x = self.interp(other)
            if x is None:
                return None
            lo, hi = self._span(x)
            if g[1] != hi - lo:
                return None
            out = []
            for a, s, cov in x:
                if any(kd != "pend" or lo - b != g[3] for b, _, kd, _ in cov):
                    return None
                out.append([a, s, [(b, l, "full", sc) for b, l, _, sc in cov]])
            return out
        if op == "add":
            parts = [self.interp(a) for a in args]
            return None if any(p is None for p in parts) else self._add(parts)
        if op == "concat" and _norm_dim(t, t.attrs.get("dim"), self.memo) == -2:
            out: list = []
            for a in args:
                p = self.interp(a)
                if p is None or (out and self._span(out)[1] != p[0][0]):
                    return None
                out = out + p
            return out or None
        if op == "om_decayed" and len(args) == 3:
            return self._om_decayed(t)
        if op == "matmul" and len(args) == 2:
            return self._state_product(t)
        if op == "split":
            p = _split_piece(t, self.memo)
            if p is None or p[1] != -2:
                return None
            x = self.interp(p[0])
            if x is None:
                return None
            lo, hi = self._span(x)
            if hi - lo != p[4]:
                return None
            return self._restrict(x, lo + p[2], lo + p[2] + p[3])
        return None


def decayed_ragged_plan(root: Any) -> dict | None:
    """Recognise chunked decayed attention over an ARBITRARY, possibly
    hierarchical partition of the sequence — what extraction returns when the
    K-way law (``om_decayed_kway_blocks``, catopt_carriers/om.py:3155-3201) fires
    at more than one level: nested ``concat``s over pieces such as
    (32,32,32,32,128,128,128) rows, cross terms that reach back to coarser source
    blocks, a coarse cross term added to a ``concat`` of finer arms or shared by
    several arms through row slices, cross products spelled either as
    ``q_i @ ((k_j * col)^T @ v_j)`` or as ``om_decayed(q_i k_j^T, col, v_j)``.  The
    reference's own executor declines all of these (non-uniform shapes,
    decayed_lower.py:198-207) and the generic module evaluates them op by op.

    The term is accepted iff its coverage (see ``_Coverage``) is exactly: every
    row attends to all earlier keys and itself with weight ``g^(t-s)``, under one
    constant scale — i.e. it equals decayed attention of the whole sequence,
    which is all the kernel needs: it picks its own chunking.  Returns
    ``{q, k, v, gamma, sizes, scale, n, chunk: None}`` or ``None``."""
    if not (isinstance(root, Op) and root.op == "concat"):
        return None
    cv = _Coverage()
    pieces = cv.interp(root)
    if pieces is None or cv.total is None or None in (cv.q, cv.k, cv.v, cv.gamma):
        return None
    if cv._span(pieces) != (0, cv.total) or len(pieces) < 2:
        return None
    scales = set()
    for a, s, cov in pieces:
        diag = [c for c in cov if c[2] == "diag"]
        if len(diag) != 1 or diag[0][:2] != (a, s) or any(c[2] == "pend" for c in cov):
            return None
        pos = 0
        for b, l, _, _ in sorted(c for c in cov if c[2] == "full"):
            if b != pos:
                return None
            pos = b + l
        if pos != a:
            return None
        scales.update(c[3] for c in cov)
    if len(scales) != 1:
        return None
    return {"q": cv.q, "k": cv.k, "v": cv.v, "gamma": cv.gamma, "sizes": tuple(s for _, s, _ in pieces),
            "n": len(pieces), "chunk": None, "scale": scales.pop()}


def uniform_decayed_term(B: int, H: int, T: int, d: int, chunk: int, per_head: bool = True, scale: float = 1.0,
                         dv: int | None = None) -> IR:
    """The uniform K-chunk decayed-attention term over inputs ``q, k, v`` ``[B,H,T,d]`` and a
    rate parameter ``g`` (``[H]`` or scalar), spelled exactly as the right-hand side of
    ``om_decayed_kway_blocks`` (catopt_carriers/om.py:3076-3152) with every summand divided by
    the constant ``scale`` — the form the reference's own executor tests build by hand
    (tests/test_decayed_lower.py:55-196 there).  ``B200Sink().executors`` routes it to
    ``b200_om_decayed_chunked``; benchmarks and examples use it to obtain the module a catopt
    user is handed for a decayed-attention block of these sizes."""
    from catopt_core.ir import TensorType

    K = T // chunk
    if K * chunk != T or K < 1:
        raise ValueError("T must be a multiple of chunk")
    dv = d if dv is None else dv
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    q, k = Var("q", tt(B, H, T, d)), Var("k", tt(B, H, T, d))
    v = Var("v", tt(B, H, T, dv))
    g = Param("g", tt(H)) if per_head else Param("g", tt())
    sc = Const(float(scale))
    sizes = [chunk] * K
    part = lambda t, i: Op.make("split", t, dim=-2, index=i, sizes=sizes)  # noqa: E731
    kt = Op.make("transpose", k, dim0=-1, dim1=-2)
    dec = Op.make("decay", g, t=chunk)
    col = Op.make("unsqueeze", Op.make("decay_vec", g, t=chunk, sign=-1, offset=0), dim=-1)
    states = [Op.make("matmul", Op.make("transpose", Op.make("mul", part(k, j), col), dim0=-1, dim1=-2), part(v, j))
              for j in range(K - 1)]
    arms = []
    for i in range(K):
        arm = Op.make("div", Op.make("om_decayed", Op.make("matmul", part(q, i),
                                                           Op.make("split", kt, dim=-1, index=i, sizes=sizes)),
                                     dec, part(v, i)), sc)
        for j in range(i):
            row = Op.make("unsqueeze", Op.make("decay_vec", g, t=chunk, sign=1, offset=(i - j) * chunk), dim=-1)
            arm = Op.make("add", arm, Op.make("mul", row, Op.make("div", Op.make("matmul", part(q, i), states[j]), sc)))
        arms.append(arm)
    root = arms[0] if K == 1 else Op.make("concat", *arms, dim=-2)
    return IR(root=root, inputs=[q, k, v], input_names={"q", "k", "v"}, params={"g": g})


def decayed_plan(root: Any) -> dict | None:
    """Uniform K-chunk term first (the reference's own parser), then any ragged partition."""
    plan = decayed_state_carry_plan(root)
    return plan if plan is not None else decayed_ragged_plan(root)


class _EvalBase(_GraphMixin, torch.nn.Module):
    """Shared plumbing: embedded ``IRModule`` + operand evaluation."""

    def __init__(self, ir: IR, param_values: dict | None) -> None:
        super().__init__()
        self._inputs = ir.inputs
        self.eval_mod = IRModule(ir, param_values)
        self._init_graph_state()

    # what catopt's autotuner reads off a delivered module to re-lower the same term through
    # another executor (``_recover_ir``, catopt_orchestrator/autotune.py:279-310); the reference's
    # batched executors delegate these to their embedded module in the same way
    @property
    def _root(self) -> Any:
        return self.eval_mod._root

    @property
    def _param_map(self) -> Any:
        return self.eval_mod._param_map

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


def _var_free(t: Any) -> bool:
    """No input variable below ``t``: its value depends on parameters and constants only."""
    if isinstance(t, Var):
        return False
    return all(_var_free(a) for a in t.args) if isinstance(t, Op) else True


class B200ChunkedDecayModule(_EvalBase):
    """Drop-in for ``ChunkedDecayModule`` (decayed_lower.py:381-724): same
    constructor, ``_plan`` / ``is_batched`` / ``n_blocks`` / graph API; the
    forward evaluates the q, k, v bases through ``eval_mod`` and runs
    ``cb2_decayed_chunk_fwd``.  A non-matching IR degrades to ``eval_mod``.
    A decay rate that depends on parameters only is evaluated once per device and
    kept as the kernel's per-head fp32 vector (the counterpart of the reference's
    ``_const`` cache, decayed_lower.py:449-468)."""

    def __init__(self, ir: IR, param_values: dict | None = None) -> None:
        super().__init__(ir, param_values)
        self._plan = decayed_plan(self.eval_mod._root)
        self._const_cache: dict = {}
        self._gamma_is_const = self._plan is not None and _var_free(self._plan["gamma"])

    def _const(self, term: Any, ev: Any, like: torch.Tensor, heads: int) -> torch.Tensor:
        """``term`` (Var-free) as a contiguous fp32 vector with one rate per head on
        ``like``'s device, evaluated once per (device, head count)."""
        key = ("gamma", term, like.device, heads)
        g = self._const_cache.get(key)
        if g is None:
            g = torch.as_tensor(ev(term), dtype=torch.float32, device=like.device).reshape(-1)
            g = (g.expand(heads) if g.numel() == 1 else g).contiguous()
            self._const_cache[key] = g
        return g

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
        q, k, v = ev(plan["q"]), ev(plan["k"]), ev(plan["v"])
        if self._gamma_is_const and isinstance(q, torch.Tensor) and q.dim() >= 3:
            g = self._const(plan["gamma"], ev, q, q.shape[-3])
        else:
            g = ev(plan["gamma"])
        out = decayed_whole_sequence(q, k, v, g, plan["chunk"], plan["scale"])
        return self.eval_mod(*xs) if out is None else out     # fp64 / awkward length: generic module, same device


def decayed_pairwise_plan(root: Any) -> dict | None:
    """The reference's pairwise plan (``build_decayed_plan``, decayed_lower.py:353-368) for
    the members that are NOT decayed attention of one sequence at one rate per head — a row
    gate on the intra element, another decay mask per arm, a missing cross pair — and so
    have no state-carry form."""
    return build_decayed_plan(root)


def _make_pairwise_decay_module():
    from catopt_carriers.decayed_lower import ChunkedDecayModule

    class B200PairwiseDecayModule(ChunkedDecayModule):
        """``ChunkedDecayModule`` (decayed_lower.py:381-724) with the intra-chunk element
        ``(s * d) @ v`` of every arm in ``cb2_gated_contract_fwd``: the stacked scores are
        gated and contracted in one kernel (the product lives in tensor memory as the MMA's
        A operand and is never written out), one decay mask shared by all arms indexed in
        place.  Plan, operand stacking, row gates, scales, the cross pairs and the assembly
        stay the reference's own code.  fp64 tensors take the reference's eager product on
        the same device; host tensors are refused."""

        def __init__(self, ir: IR, param_values: dict | None = None) -> None:
            super().__init__(ir, param_values)
            self.kernel_calls = 0

        def _forward_intra(self, plan, ev, env, x, like):
            if not like.is_cuda:
                raise B200Error("B200PairwiseDecayModule runs on CUDA tensors only (no CPU fallback)")
            if like.dtype not in (torch.float32, torch.bfloat16):
                return super()._forward_intra(plan, ev, env, x, like)
            ab = plan["score_ab"]
            if ab is None:
                scores = self._stack_terms(plan["score_terms"], ev)
            else:
                scores = torch.matmul(self._stack_terms([a for a, _ in ab], ev),
                                      self._stack_terms([b for _, b in ab], ev))
            masks = plan["decay_terms"]
            if all(m == masks[0] for m in masks):
                gate = self._const(masks[0], like)
            else:
                gate = self._pad_stacked(torch.stack([self._const(m, like) for m in masks]), scores.dim())
            out = ops.gated_contract(scores, gate.to(scores.dtype), self._stack_terms(plan["v_intra"], ev))
            self.kernel_calls += 1
            if any(r is not None for r in plan["intra_row"]):
                out = self._row_stack(plan["intra_row"], like, len(plan["chunk"])) * out
            div = self._scales("intra", plan["intra_scale"], env, x, like)
            return out / div.reshape(-1, *((1,) * (out.dim() - 1)))

    return B200PairwiseDecayModule


# --------------------------------------------------------------------------- om causal
def _scaled_scores(t: Any) -> tuple | None:
    """Scores of one key block -> (q, k, scale).  Spellings: ``matmul(q, k^T)``
    (scale 1) and the one the sdpa-over-concat laws leave behind,
    ``om_decayed(q, fill(q, value=scale), k^T)`` = ``(q * scale) @ k^T``."""
    if not isinstance(t, Op):
        return None
    if t.op == "matmul" and len(t.args) == 2 and _is_swap_last_two(t.args[1]):
        q = t.args[0]
        if isinstance(q, Op) and q.op == "mul" and len(q.args) == 2:
            # (q * fill(q, scale)) @ k^T: the spelling of the masked sdpa law (om.py:1325-1331)
            for a, f in (q.args, q.args[::-1]):
                if isinstance(f, Op) and f.op == "fill" and len(f.args) == 1 and f.args[0] == a \
                        and isinstance(f.attrs.get("value"), (int, float)):
                    return a, t.args[1].args[0], float(f.attrs["value"])
        return q, t.args[1].args[0], 1.0
    if t.op == "om_decayed" and len(t.args) == 3 and _is_swap_last_two(t.args[2]):
        q, f = t.args[0], t.args[1]
        if isinstance(f, Op) and f.op == "fill" and len(f.args) == 1 and f.args[0] == q \
                and isinstance(f.attrs.get("value"), (int, float)):
            return q, t.args[2].args[0], float(f.attrs["value"])
    return None


def _score_blocks(t: Any) -> list | None:
    """Scores over one or more key blocks: a single block or ``concat(..., dim=-1)`` of blocks ->
    ``[(q, k, scale), ...]`` in key order."""
    if isinstance(t, Op) and t.op == "concat" and t.attrs.get("dim") == -1 and len(t.args) >= 1:
        out = [_scaled_scores(a) for a in t.args]
        return None if any(b is None for b in out) else out
    one = _scaled_scores(t)
    return None if one is None else [one]


def _bias_piece(t: Any, memo: dict) -> tuple | None:
    """``attnbias(m)`` or a column range of one -> ``(base, start, length | None)`` (None: all columns)."""
    if isinstance(t, Op) and t.op == "attnbias" and len(t.args) == 1:
        return t, 0, None
    r = _range_of(t, -1, memo)
    if r is not None and isinstance(r[0], Op) and r[0].op == "attnbias" and len(r[0].args) == 1:
        return r[0], r[1], r[2]
    return None


def _split_bias(sterm: Any, memo: dict) -> tuple:
    """``add(scores, <attention bias>)`` in either order -> (scores, bias piece); else (sterm, None)."""
    if isinstance(sterm, Op) and sterm.op == "add" and len(sterm.args) == 2:
        for a, b in (sterm.args, sterm.args[::-1]):
            bp = _bias_piece(b, memo)
            if bp is not None:
                return a, bp
    return sterm, None


def om_causal_plan(root: Any) -> dict | None:
    """Recognise softmax attention over a sequence of key/value blocks in its
    online-softmax carrier form (the members the ``sdpa_cat`` /
    ``sdpa_cat_causal`` laws add, tests/test_om_causal.py:286-345 of the
    reference):

        om_apply(<om_compose tree of om_elem(masked_fill(S_i, M_i, -inf), v_i)>)     causal
        om_apply(<om_compose tree of om_elem(S_i, v_i)>)                             unmasked

    with ``S_i = (q * scale) @ k_i^T`` and ``M_i`` the columns ``[o_i, o_i + n_i)``
    of ``cmask(<any [.., Tq, sum n] tensor>)`` (bad where ``j > t``; o_i the keys
    before block i).  Leaves are read left to right = key order; every block must
    share q and the scale and appear once; all masks slice ONE ``cmask``, whose
    offset ``off`` (key j visible to query t iff ``j + off <= t``, om.py:1023-1029)
    is part of the plan.  An explicit attention mask in the form the masked sdpa law
    leaves (om.py:1313-1362) is taken too:

        om_apply(om_elem(add(concat(S_1, .., dim=-1), attnbias(m)), v))              one leaf
        om_apply(<om_compose tree of om_elem(add(S_i, <columns of attnbias(m)>), v_i)>)

    (the pieces must tile ONE ``attnbias(m)`` in key order; ``m`` is evaluated at run
    time: a bool keep-mask or a float bias).  Returns ``{q, k_blocks, v_blocks, sizes,
    scale, n, causal, off, bias}`` or ``None`` (a mask together with ``cmask``, mixed
    trees: the reference's own om executors keep them)."""
    if not (isinstance(root, Op) and root.op == "om_apply" and len(root.args) == 1):
        return None
    leaves = _flatten(root.args[0], "om_compose")
    if len(set(leaves)) != len(leaves):
        return None
    memo: dict = {}
    q = scale = None
    ks, vs, sizes, vsizes, pos, total = [], [], [], [], 0, None
    causal = None
    mask_base, off = None, 0
    bias_base, biased = None, None
    for leaf in leaves:
        if not (isinstance(leaf, Op) and leaf.op == "om_elem" and len(leaf.args) == 2):
            return None
        sterm, v = leaf.args
        masked = isinstance(sterm, Op) and sterm.op == "masked_fill"
        if causal is None:
            causal = masked
        elif causal != masked:
            return None
        if masked and not (len(sterm.args) == 3 and _const_value(sterm.args[2]) == float("-inf")):
            return None
        score_part, bp = _split_bias(sterm.args[0] if masked else sterm, memo)
        if biased is None:
            biased = bp is not None
        if biased != (bp is not None) or (biased and masked):
            return None
        blocks = _score_blocks(score_part)
        if blocks is None:
            return None
        leaf_pos = pos
        for sc in blocks:
            kshape = _shape_of(sc[1], memo)
            if not isinstance(kshape, tuple) or len(kshape) < 2 or not isinstance(kshape[-2], int):
                return None
            if q is None:
                q, scale = sc[0], sc[2]
            elif sc[0] != q or sc[2] != scale:
                return None
            ks.append(sc[1])
            sizes.append(kshape[-2])
            pos += kshape[-2]
        n_i = pos - leaf_pos
        if masked:
            # the mask: columns [leaf_pos, leaf_pos + n_i) of one cmask over the whole score tensor
            r = _range_of(sterm.args[1], -1, memo)
            if r is None:
                return None
            base, start, length, tot = r
            if not (isinstance(base, Op) and base.op == "cmask"):
                return None
            o_i = base.attrs.get("off", 0) or 0
            if not isinstance(o_i, int) or (mask_base is not None and base != mask_base):
                return None
            mask_base, off = base, o_i
            if (start, length) != (leaf_pos, n_i) or (total is not None and tot != total):
                return None
            total = tot
        if bp is not None:
            base, start, length = bp
            if (bias_base is not None and base != bias_base) or start != leaf_pos or (length is not None and length != n_i):
                return None
            if length is None and len(leaves) != 1:
                return None                     # an unsliced bias belongs to a single leaf
            bias_base = base
        vs.append(v)
        vsizes.append(n_i)
    if len(leaves) < 2 and not biased:
        return None
    if not causal:
        total = pos
    if pos != total:
        return None

    def whole(blocks, sizes_):
        """The one tensor the blocks are consecutive row slices of, if they tile it: no join needed."""
        base, at = None, 0
        for t, n_i in zip(blocks, sizes_):
            r = _range_of(t, -2, memo)
            if r is None or (base is not None and r[0] != base) or r[1] != at or r[2] != n_i or r[3] != total:
                return None
            base, at = r[0], at + n_i
        return base

    kb, vb = whole(ks, sizes), whole(vs, vsizes)
    if kb is not None and vb is not None:
        ks, vs = [kb], [vb]
    return {"q": q, "k_blocks": ks, "v_blocks": vs, "sizes": tuple(sizes), "scale": scale, "n": len(sizes),
            "causal": bool(causal), "off": off, "bias": None if bias_base is None else bias_base.args[0]}


def _flatten(t: Any, op: str) -> list:
    """Leaves of a nested tree of ``op`` nodes, left to right."""
    if isinstance(t, Op) and t.op == op:
        out: list = []
        for a in t.args:
            out.extend(_flatten(a, op))
        return out
    return [t]


class B200CausalSoftmaxModule(_EvalBase):
    """Drop-in for ``BatchedOMModule`` / ``StreamingOMModule``
    (catopt_carriers/om_lower.py:729-835, 996-1040) on the causal carrier: the
    key/value blocks are joined along the key axis (they are the pieces of a
    ``concat`` in the source program) and one ``cb2_om_causal_fwd`` replaces the
    per-block softmax triples and their pairwise merges.  A non-matching IR
    degrades to ``eval_mod``."""

    def __init__(self, ir: IR, param_values: dict | None = None) -> None:
        super().__init__(ir, param_values)
        self._plan = om_causal_plan(self.eval_mod._root)

    @property
    def is_batched(self) -> bool:
        return self._plan is not None

    @property
    def n_blocks(self) -> int:
        return 0 if self._plan is None else self._plan["n"]

    @property
    def is_streaming(self) -> bool:
        return self._plan is not None

    def forward_state(self, *xs: torch.Tensor) -> Any:
        """The raw carrier ``(m, l, a)`` (fp32) after folding the blocks one kernel
        call at a time — ``StreamingOMModule.forward_state`` (om_lower.py:1003-1040);
        ``ops.om_apply_state`` reads it out, ``ops.om_step_qk`` extends it."""
        plan = self._plan
        if plan is None:
            return self.eval_mod(*xs)
        ev = self._ev(xs)
        ks, vs = [ev(t) for t in plan["k_blocks"]], [ev(t) for t in plan["v_blocks"]]
        if len(ks) != len(vs):                           # (one joined value tensor: cut it like the keys)
            vs = list(torch.split(vs[0] if len(vs) == 1 else torch.cat(vs, dim=-2), [k.shape[-2] for k in ks], dim=-2))
        return softmax_blocks_state(ev(plan["q"]), ks, vs, plan["scale"], plan["causal"], key_offset=plan["off"],
                                    mask=None if plan["bias"] is None else ev(plan["bias"]))

    def _forward_impl(self, *xs: torch.Tensor) -> Any:
        plan = self._plan
        if plan is None:
            return self.eval_mod(*xs)
        ev = self._ev(xs)
        q = ev(plan["q"])
        if plan["off"] and isinstance(q, torch.Tensor) and q.dtype in (torch.float32, torch.bfloat16):
            # a shifted causal mask: the streaming step carries the key offset (cb2_om_step);
            # rows that see no key come out NaN, as the reference's unclamped a / l does
            st = softmax_blocks_state(q, [ev(t) for t in plan["k_blocks"]], [ev(t) for t in plan["v_blocks"]],
                                      plan["scale"], True, key_offset=plan["off"])
            return ops.om_apply_state(st).to(q.dtype)
        out = causal_softmax_blocks(q, [ev(t) for t in plan["k_blocks"]],
                                    [ev(t) for t in plan["v_blocks"]], plan["scale"], plan["causal"],
                                    mask=None if plan["bias"] is None else ev(plan["bias"]))
        return self.eval_mod(*xs) if out is None else out     # fp64: generic module, same device


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
        self._unfolded_root, self._unfolded_params = ir.root, dict(param_values or {})
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
        # constant weight: its TF32 split for the tensor-core path is made once, here
        self.register_buffer("fused_split", ops.linear_split_weight(fused), persistent=False)
        self.bias = None if plan["bias"] is None else torch.nn.Parameter(val(plan["bias"]), requires_grad=False)

    @property
    def is_batched(self) -> bool:
        return self._plan is not None

    # the embedded module has folded the weight tree away; a re-lowering of "the same term"
    # (catopt's autotuner) must see the chain, or no chain executor could ever take it again
    @property
    def _root(self) -> Any:
        return self._unfolded_root

    @property
    def _param_map(self) -> Any:
        return self._unfolded_params

    def _forward_impl(self, *xs: torch.Tensor) -> Any:
        if self._plan is None:
            return self.eval_mod(*xs)
        x = self._ev(xs)(self._plan["x"])
        if not (isinstance(x, torch.Tensor) and x.is_cuda):
            raise B200Error("B200LinearChainModule runs on CUDA tensors only (no CPU fallback)")
        if x.dtype != torch.float32 or x.device != self.fused_weight.device:
            return self.eval_mod(*xs)       # bf16 / fp64 activations: generic module, same device
        with torch.cuda.device(x.device):
            return ops.linear_f32(x.contiguous(), self.fused_weight, self.bias, w_split=self.fused_split)


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
        leaves arrive in product order (latest step first) and are composed in
        that stored order in one pass (``cb2_diag_compose_apply``: B += A*b_j,
        A *= a_j per state element), then applied to the initial state.  fp64
        tensors degrade to the reference's own eager reduction on the same device.
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
            if out is None:   # fp64: the reference's own reduction
                return super()._forward_fused(a_vals, b_vals, ev)
            self.kernel_calls += 1
            return out

    return B200ScanModule


# --------------------------------------------------------------------------- scan, every state
def _prefix_chain_leaves(fs: list) -> list | None:
    """Maps ``f_t`` that are the running compositions of one leaf sequence —
    ``f_0 = leaf_0``, ``f_t = affd_compose(leaf_t, f_(t-1))`` (any nesting of the same
    product for short sequences) — to the leaves in time order; ``None`` otherwise."""
    leaves: list = []
    for t, f in enumerate(fs):
        if t == 0:
            if not (isinstance(f, Op) and f.op == "aff_diag" and len(f.args) == 2):
                return None
            leaves.append(f)
            continue
        if not (isinstance(f, Op) and f.op == "affd_compose" and len(f.args) == 2):
            return None
        new, rest = f.args
        if rest == fs[t - 1] and isinstance(new, Op) and new.op == "aff_diag" and len(new.args) == 2:
            leaves.append(new)
            continue
        if len(fs) > 256:
            return None
        flat = _flatten(f, "affd_compose")                 # product order: latest step first
        if len(flat) != t + 1 or flat[1:] != leaves[::-1]:
            return None
        if not (isinstance(flat[0], Op) and flat[0].op == "aff_diag" and len(flat[0].args) == 2):
            return None
        leaves.append(flat[0])
    return leaves


def _per_step_operand(terms: list, memo: dict) -> tuple | None:
    """How to hand T per-step operand terms to a kernel without T evaluations:
    ``("shared", term)`` when every step uses the same term, ``("gather", base, dim)``
    when step t is ``select(base, dim, t)`` of one tensor with T entries along ``dim``,
    else ``("stack", terms)``."""
    if all(t == terms[0] for t in terms[1:]) and len(terms) > 1:
        return ("shared", terms[0])
    base = dim = None
    for i, t in enumerate(terms):
        if not (isinstance(t, Op) and t.op == "select" and len(t.args) == 1 and t.attrs.get("index") == i):
            base = None
            break
        d = _norm_dim(t.args[0], t.attrs.get("dim"), memo)
        if d is None or (base is not None and (t.args[0] != base or d != dim)):
            base = None
            break
        base, dim = t.args[0], d
    if base is not None:
        shape = _shape_of(base, memo)
        if isinstance(shape, tuple) and shape[dim] == len(terms):
            return ("gather", base, dim)
    return ("stack", list(terms))


def scan_states_plan(root: Any) -> dict | None:
    """Recognise the stacked-map form of an unrolled diagonal scan,

        applyd(aff_diag(stack(affd_a f_0 .. f_(T-1), dim=D), stack(affd_b f_0 .. f_(T-1), dim=D)), h)

    with ``f_t`` the prefix maps of one leaf sequence ``aff_diag(a_t, b_t)`` — what
    ``gather_applyd_stack`` (catopt_carriers/xcarrier.py:2252-2275) offers for
    ``stack(h_1 .. h_T)`` once ``lift_scan_to_applyd`` has written every ``h_t`` as an
    application to the shared initial state.  Its value is every state of
    ``h_t = a_t*h_(t-1) + b_t``, stacked along ``D``.

    Also recognised, one level up: the per-step readout ``sum(mul(<that form>, c), dim=-1)``
    of a ``[B, D, N]`` state stacked along dim 1 whose offsets are ``b * unsqueeze(x_t, -1)``
    with ``x_t = select(x, 1, t)`` — benchmark config 3's recurrence
    ``y_t = sum_n c*h_t``, which is exactly ``cb2_diag_scan_fwd``.

    Returns ``{a, b, h, n, stack_dim, state_shape, readout}`` (``a``/``b`` as
    ``_per_step_operand`` tuples; ``readout`` ``None`` or ``{x, b, c}``), or ``None``."""
    memo: dict = {}
    readout_c = None
    states = root
    if isinstance(root, Op) and root.op == "sum" and len(root.args) == 1 and not root.attrs.get("keepdim"):
        body = root.args[0]
        rdim = root.attrs.get("dim")
        if isinstance(rdim, (tuple, list)) and len(rdim) == 1:
            rdim = rdim[0]
        rd = _norm_dim(body, rdim, memo)
        if rd != -1 or not (isinstance(body, Op) and body.op == "mul" and len(body.args) == 2):
            return None
        x0, x1 = body.args
        states, readout_c = (x0, x1) if isinstance(x0, Op) and x0.op == "applyd" else (x1, x0)
    if not (isinstance(states, Op) and states.op == "applyd" and len(states.args) == 2):
        return None
    fmap, h = states.args
    if not (isinstance(fmap, Op) and fmap.op == "aff_diag" and len(fmap.args) == 2):
        return None
    sa, sb = fmap.args
    if not all(isinstance(t, Op) and t.op == "stack" and len(t.args) >= 2 for t in (sa, sb)):
        return None
    if len(sa.args) != len(sb.args) or sa.attrs.get("dim", 0) != sb.attrs.get("dim", 0):
        return None
    fs = []
    for pa, pb in zip(sa.args, sb.args):
        if not (isinstance(pa, Op) and pa.op == "affd_a" and isinstance(pb, Op) and pb.op == "affd_b"
                and len(pa.args) == 1 and pa.args == pb.args):
            return None
        fs.append(pa.args[0])
    leaves = _prefix_chain_leaves(fs)
    if leaves is None:
        return None
    T = len(leaves)
    shapes = {_shape_of(lf.args[0], memo) for lf in leaves} | {_shape_of(lf.args[1], memo) for lf in leaves}
    if len(shapes) != 1:
        return None
    state_shape = shapes.pop()
    if not (isinstance(state_shape, tuple) and state_shape and all(isinstance(z, int) for z in state_shape)):
        return None
    hshape = _shape_of(h, memo)
    try:
        if not isinstance(hshape, tuple) or torch.broadcast_shapes(hshape, state_shape) != torch.Size(state_shape):
            return None
    except RuntimeError:
        return None
    sd = sa.attrs.get("dim", 0)
    if not isinstance(sd, int):
        return None
    sd = sd % (len(state_shape) + 1)
    plan = {"a": _per_step_operand([lf.args[0] for lf in leaves], memo),
            "b": _per_step_operand([lf.args[1] for lf in leaves], memo),
            "h": h, "n": T, "stack_dim": sd, "state_shape": state_shape, "readout": None}
    if readout_c is None:
        return plan
    # the readout form must be the kernel's own recurrence
    if len(state_shape) != 3 or sd != 1 or _shape_of(readout_c, memo) != state_shape[1:]:
        return None
    xs, bcoef = [], None
    for lf in leaves:
        u = lf.args[1]
        if not (isinstance(u, Op) and u.op == "mul" and len(u.args) == 2):
            return None
        for coef, xt in (u.args, u.args[::-1]):
            if isinstance(xt, Op) and xt.op == "unsqueeze" and _norm_dim(xt, xt.attrs.get("dim"), memo) == -1 \
                    and _shape_of(coef, memo) == state_shape[1:]:
                break
        else:
            return None
        if bcoef is not None and coef != bcoef:
            return None
        bcoef = coef
        xs.append(xt.args[0])
    xop = _per_step_operand(xs, memo)
    if xop[0] != "gather" or xop[2] != -2 or plan["a"][0] != "gather" or plan["a"][2] != -3:
        return None
    plan["readout"] = {"x": xop[1], "b": bcoef, "c": readout_c}
    return plan


class B200ScanStatesModule(_EvalBase):
    """Executor for ``scan_states_plan`` terms.  The reference has no batched module
    for them (its generic ``IRModule`` composes one prefix map per step, T launches);
    here the step operands are taken whole — a ``select`` sequence hands over its base
    tensor, a shared operand is read in place — and every state comes out of one
    ``cb2_diag_scan_states`` pass, or, for the readout form, every ``y_t`` out of one
    ``cb2_diag_scan_fwd`` pass (the kernel of benchmark config 3).  fp64 tensors and a
    non-matching IR degrade to ``eval_mod``."""

    def __init__(self, ir: IR, param_values: dict | None = None) -> None:
        super().__init__(ir, param_values)
        self._plan = scan_states_plan(self.eval_mod._root)
        self.kernel_calls = 0

    @property
    def is_batched(self) -> bool:
        return self._plan is not None

    @property
    def n_levels(self) -> int:
        return 0 if self._plan is None else 1

    @staticmethod
    def _rows(spec: tuple, ev: Any, T: int) -> torch.Tensor:
        """The step operand as a ``[T, ...]`` tensor (a view when it can be one)."""
        if spec[0] == "shared":
            v = ev(spec[1])
            return v.unsqueeze(0).expand(T, *v.shape)
        if spec[0] == "gather":
            return ev(spec[1]).movedim(spec[2], 0)
        return torch.stack([ev(t) for t in spec[1]])

    def _forward_impl(self, *xs: torch.Tensor) -> Any:
        plan = self._plan
        if plan is None:
            return self.eval_mod(*xs)
        ev = self._ev(xs)
        T = plan["n"]
        rd = plan["readout"]
        if rd is not None:
            a, x, b, c, h = ev(plan["a"][1]), ev(rd["x"]), ev(rd["b"]), ev(rd["c"]), ev(plan["h"])
            if not a.is_cuda:
                raise B200Error("B200ScanStatesModule runs on CUDA tensors only (no CPU fallback)")
            dt = a.dtype
            if dt not in (torch.float32, torch.bfloat16) or not (x.dtype == b.dtype == c.dtype == dt):
                return self.eval_mod(*xs)
            B_, D_, N_ = plan["state_shape"]
            h0 = torch.as_tensor(h, device=a.device).to(torch.float32).expand(B_, D_, N_).contiguous()
            out = ops.diag_scan_fwd(a.contiguous(), x.contiguous(), b.contiguous(), c.contiguous(), h0)
            self.kernel_calls += 1
            return out
        a_rows, b_rows, h = self._rows(plan["a"], ev, T), self._rows(plan["b"], ev, T), ev(plan["h"])
        if not b_rows.is_cuda:
            raise B200Error("B200ScanStatesModule runs on CUDA tensors only (no CPU fallback)")
        out = ops.diag_scan_states(a_rows, b_rows, torch.as_tensor(h, device=b_rows.device))
        if out is None:                    # fp64: the generic module on the same device
            return self.eval_mod(*xs)
        self.kernel_calls += 1
        return out.movedim(0, plan["stack_dim"])


# --------------------------------------------------------------------------- omd (deferred-affine attention)
def _make_omd_module():
    from catopt_carriers.omd_lower import BatchedOmdModule

    class B200OmdModule(BatchedOmdModule):
        """``BatchedOmdModule`` (omd_lower.py:560-1020) with the all-prefix scan of
        the scanned values' step maps (``_prefix_scan``, omd_lower.py:771-824: blocks
        of sqrt(T) compose steps) replaced by ``cb2_diag_prefix_maps``, which reads
        the step maps once and writes every prefix of both components.  Term analysis,
        the omd tree reduction and every other path stay the reference's own code;
        dense maps and fp64 tensors keep the reference's scan on the same device."""

        def __init__(self, ir: IR, param_values: dict | None = None) -> None:
            super().__init__(ir, param_values)
            self.kernel_calls = 0
            self._kernel_error: Exception | None = None

        def _forward_impl(self, *xs):
            # The reference's forward degrades to the generic module on ANY exception
            # (omd_lower.py:1015-1019); a kernel-path failure must not disappear that way.
            if self._plan is not None and any(isinstance(t, torch.Tensor) and not t.is_cuda for t in xs):
                raise B200Error("B200OmdModule runs on CUDA tensors only (no CPU fallback)")
            self._kernel_error = None
            out = super()._forward_impl(*xs)
            if self._kernel_error is not None:
                raise self._kernel_error
            return out

        def _prefix_scan(self, A, B, domain):
            if domain != "diag" or A.shape[0] < 2 or not A.is_cuda:
                return super()._prefix_scan(A, B, domain)
            try:
                out = ops.diag_prefix_maps(A, B)
            except B200Error as e:
                self._kernel_error = e
                raise
            if out is None:
                return super()._prefix_scan(A, B, domain)
            self.kernel_calls += 1
            return out

    return B200OmdModule


def omd_plan(root: Any) -> dict | None:
    """The reference's omd plan (``build_omd_plan``, omd_lower.py) for
    ``omd_apply[m](<omd tree>, h)`` terms, ``None`` otherwise."""
    from catopt_carriers.omd_lower import build_omd_plan, is_omd_apply_term

    return build_omd_plan(root) if is_omd_apply_term(root) else None


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
                    lambda term: decayed_plan(term) is not None,
                    _engaged,
                    (frozenset({"concat"}), frozenset({"add", "mul", "div", "matmul"}),
                     frozenset({"om_decayed", "decay", "decay_vec"})),
                ),
                "b200_om_decayed_pairwise": ExecutorSpec(
                    "b200_om_decayed_pairwise",
                    lambda ir, p: _make_pairwise_decay_module()(ir, param_values=p),
                    lambda term: decayed_pairwise_plan(term) is not None,
                    _engaged,
                    (frozenset({"concat"}), frozenset({"add", "mul", "div", "matmul"}),
                     frozenset({"om_decayed", "decay", "decay_vec"})),
                ),
                "b200_om_causal": ExecutorSpec(
                    "b200_om_causal",
                    lambda ir, p: B200CausalSoftmaxModule(ir, param_values=p),
                    lambda term: om_causal_plan(term) is not None,
                    _engaged,
                    (frozenset({"om_apply"}), frozenset({"om_compose"}), frozenset({"om", "om_elem"})),
                ),
                "b200_om_streaming": ExecutorSpec(
                    "b200_om_streaming",
                    lambda ir, p: B200CausalSoftmaxModule(ir, param_values=p),
                    lambda term: om_causal_plan(term) is not None,
                    lambda m: bool(getattr(m, "is_streaming", False)),
                    (frozenset({"om_apply"}), frozenset({"om_compose"}), frozenset({"om", "om_elem"})),
                ),
                "b200_scan_all": ExecutorSpec(
                    "b200_scan_all",
                    lambda ir, p: B200ScanStatesModule(ir, param_values=p),
                    lambda term: scan_states_plan(term) is not None,
                    _engaged,
                    (frozenset({"applyd", "sum"}), frozenset({"affd_compose", "stack", "affd_a", "affd_b"}),
                     frozenset({"aff_diag"})),
                ),
                "b200_scan": ExecutorSpec(
                    "b200_scan",
                    lambda ir, p: _make_scan_module()(ir, param_values=p),
                    lambda term: scan_diag_plan(term) is not None,
                    _engaged,
                    (frozenset({"applyd"}), frozenset({"affd_compose"}), frozenset({"aff_diag"})),
                ),
                "b200_omd": ExecutorSpec(
                    "b200_omd",
                    lambda ir, p: _make_omd_module()(ir, param_values=p),
                    lambda term: omd_plan(term) is not None,
                    _engaged,
                    (frozenset({"omd_apply", "omd_applym"}), frozenset({"omd_compose"}), frozenset({"omd", "omd_elem"})),
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
        """``TorchSink.verify`` (adapters.py:126-139) with the comparison of every
        float32 / bfloat16 CUDA output pair in ``cb2_verify_reduce``.  Pairs the kernel
        does not take (fp64, integer or host tensors) go to the reference's own gate
        (``report.verify_equiv``) on the device they live on, so whatever the
        reference verifies is still gated.  The gate's read-back is also where a
        bounded device wait that ran out in an earlier kernel raises ``B200Error``."""
        from catopt_torch.report import verify_equiv as reference_gate

        return b200_verify.verify_module(ref, opt, inputs, rtol=rtol, atol=atol, delegate=reference_gate)


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
