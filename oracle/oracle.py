"""CPU restatement of the reference's lowered-executor arithmetic.

TEST INFRASTRUCTURE ONLY.  Nothing under ``catopt_b200/`` imports this file;
it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU legs of
``bench.py`` as the checker / timed CPU baseline, never as the product path.

The reference (luisfuturist/catopt) computes this path with eager torch ops on
whatever device its tensors live on, so the restatement uses the same torch CPU
ops in the same order; every function cites the reference lines it follows
(paths relative to the reference's project root).

Parity is pinned: ``tests/golden/make_golden.py`` imports the real reference,
runs its own lowered modules / bindings on seeded inputs and stores the
outputs; ``tests/test_oracle_golden.py`` checks every function here against
those stored outputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch

_REL_FLOOR = 1e-8  # packages/catopt-torch/src/catopt_torch/report.py (module constant)


# --------------------------------------------------------------------------- (d) verify
@dataclass(frozen=True)
class OracleVerifyReport:
    """Fields of the reference's VerifyReport (report.py:43-56)."""

    max_abs: float
    max_rel: float
    passed: bool
    per_output: tuple | None = None


def verify_pair(ref: torch.Tensor, out: torch.Tensor, rtol: float = 1e-4,
                atol: float | None = None) -> OracleVerifyReport:
    """report.py:128-140 (`_verify_pair`), same expression order."""
    max_abs = (ref - out).abs().max().item()
    max_rel = max_abs / (ref.abs().max().item() + _REL_FLOOR)
    passed = bool(max_rel < rtol) and (atol is None or bool(max_abs <= atol))
    return OracleVerifyReport(max_abs, max_rel, passed)


def _flatten(x: Any) -> list:
    """report.py:70-87 (`_flatten_outputs`)."""
    if isinstance(x, (tuple, list)):
        out: list = []
        for item in x:
            out.extend(_flatten(item))
        return out
    return [x]


def verify_equiv(ref: Any, out: Any, rtol: float = 1e-4,
                 atol: float | None = None) -> OracleVerifyReport:
    """report.py:143-165 with the multi-output arm of 90-125."""
    if not isinstance(ref, (tuple, list)):
        return verify_pair(ref, out, rtol, atol)
    rf, of = _flatten(ref), _flatten(out)
    if not isinstance(out, (tuple, list)) or len(rf) != len(of):
        return OracleVerifyReport(float("inf"), float("inf"), False)
    reps = [verify_equiv(r, o, rtol, atol) for r, o in zip(rf, of)]
    return OracleVerifyReport(
        max(r.max_abs for r in reps),
        max(r.max_rel for r in reps),
        all(r.passed for r in reps),
        tuple(r.max_abs for r in reps),
    )


# --------------------------------------------------------------------------- (a) chain
def fold_chain(weights: list[torch.Tensor]) -> torch.Tensor:
    """Fold `linear(...linear(x, W0)..., Wk-1)` into one weight.

    `assoc_linear` (catopt_core/laws/tensor.py:1293-1300) rewrites
    linear(linear(x,A),B) to linear(x, matmul(B,A)); the extracted term is
    right-nested, and `_fold_weight_chains` (torch_bridge.py:2485-2510)
    evaluates it innermost-first with torch.matmul: W1@W0, W2@(.), ...
    """
    acc = weights[0]
    for w in weights[1:]:
        acc = torch.matmul(w, acc)
    return acc


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The `linear` binding (torch_bridge.py:1251-1253): F.linear."""
    return torch.nn.functional.linear(x, w, bias)


def chain_eager(x: torch.Tensor, weights: list[torch.Tensor]) -> torch.Tensor:
    """The unoptimised model: k Linear layers applied in sequence."""
    for w in weights:
        x = torch.nn.functional.linear(x, w)
    return x


# --------------------------------------------------------------------------- (b) decayed
def decay_matrix(g: torch.Tensor, t: int) -> torch.Tensor:
    """`_decay_torch` (catopt_carriers/om.py:1060-1072): tril(g^(i-j))."""
    g = torch.as_tensor(g)
    pos = torch.arange(t, dtype=g.dtype, device=g.device)
    diff = pos.unsqueeze(-1) - pos.unsqueeze(-2)
    return torch.tril(g[..., None, None] ** diff.clamp_min(0))


def decay_vec(g: torch.Tensor, t: int, sign: int = 1, offset: int = 0) -> torch.Tensor:
    """`_decay_vec_torch` (om.py:1075-1088): g^(sign*k + offset), k in [0,t)."""
    g = torch.as_tensor(g)
    pos = torch.arange(t, dtype=g.dtype, device=g.device)
    return g[..., None] ** (pos * sign + offset)


def decayed_quadratic(q, k, v, gamma, scale: float = 1.0) -> torch.Tensor:
    """The spelled form `om_decayed(q@k^T, decay(g,T), v) / scale`
    (`_om_decayed_torch`, om.py:1053-1057: (s*d)@v).

    q,k: [B,H,T,dk], v: [B,H,T,dv], gamma: [H] (or scalar) in q's dtype.
    """
    T = q.shape[-2]
    s = torch.matmul(q, k.transpose(-1, -2))
    d = decay_matrix(gamma, T)  # (H,T,T) or (T,T): broadcasts over B
    return torch.matmul(s * d, v) / scale


def om_decayed(s: torch.Tensor, d: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """`_om_decayed_torch` (catopt_carriers/om.py:1053-1057): `(s * d) @ v` on
    materialised scores — the element the reference's generated fused-contraction
    kernel computes (catopt_discovery/genkernel.py:1582-1631)."""
    return torch.matmul(s * d, v)


def decayed_chunked_pairwise(q, k, v, gamma, chunk: int, scale: float = 1.0) -> torch.Tensor:
    """`ChunkedDecayModule._forward_impl` (decayed_lower.py:702-724) on the
    uniform K-chunk term of `om_decayed_kway_blocks` (om.py:3076-3152):

      intra (609-639): matmul(stack q_i, stack k_i^T) * decay(g,C) @ stack v_i / S
      cross (671-700): states M_j = (k_j * g^(-r))^T @ v_j; every pair i>j:
                       q_i @ M_j * g^((i-j)C + r) / S; per-chunk segment sums.
    """
    B, H, T, dk = q.shape
    K = T // chunk
    qs = q.reshape(B, H, K, chunk, dk).movedim(2, 0)       # (K,B,H,C,dk)
    ks = k.reshape(B, H, K, chunk, dk).movedim(2, 0)
    vs = v.reshape(B, H, K, chunk, -1).movedim(2, 0)
    g = torch.as_tensor(gamma, dtype=q.dtype)
    s = torch.matmul(qs, ks.transpose(-1, -2))
    d = decay_matrix(g, chunk)
    out = torch.matmul(s * d, vs) / scale
    if K > 1:
        col = decay_vec(g, chunk, sign=-1).unsqueeze(-1)    # (H,C,1) or (C,1)
        m = torch.matmul((ks[: K - 1] * col).transpose(-1, -2), vs[: K - 1])  # (K-1,B,H,dk,dv)
        pi = [i for i in range(K) for j in range(i)]
        pj = [j for i in range(K) for j in range(i)]
        prod = torch.matmul(qs.index_select(0, torch.tensor(pi)), m.index_select(0, torch.tensor(pj)))
        rows = torch.stack([decay_vec(g, chunk, offset=(i - j) * chunk).unsqueeze(-1)
                            for i, j in zip(pi, pj)])       # (P,[H],C,1)
        # pad to the chunk's rank the way `_row_stack` does: (P,1,H,C,1) / (P,1,1,C,1)
        rows = rows.unsqueeze(1) if rows.dim() == 4 else rows.reshape(-1, 1, 1, chunk, 1)
        prod = prod * (rows / scale)
        parts = prod.split([i for i in range(K)][1:])
        cross = torch.stack([torch.zeros_like(out[0])] + [p.sum(0) for p in parts])
        out = out + cross
    return out.movedim(0, 2).flatten(2, 3)


def decayed_state_carry(q, k, v, gamma, chunk: int, scale: float = 1.0) -> torch.Tensor:
    """The state-carry recurrence of `_paper_eqn`
    (lab/probes/retnet_baseline_probe.py:77-110), per-head gamma."""
    B, H, T, dk = q.shape
    dv = v.shape[-1]
    nc = T // chunk
    g = torch.as_tensor(gamma, dtype=q.dtype).reshape(-1, 1)           # (H|1, 1)
    pos = torch.arange(chunk, dtype=q.dtype)
    decay = decay_matrix(g.reshape(-1), chunk)                          # (H|1,C,C)
    q_dec = (g ** (pos + 1)).unsqueeze(-1)                              # (H|1,C,1)
    v_dec = (g ** (chunk - 1 - pos)).unsqueeze(-1)
    cross_decay = (g ** chunk).unsqueeze(-1)                            # (H|1,1,1)
    qc = q.reshape(B, H, nc, chunk, dk)
    kc = k.reshape(B, H, nc, chunk, dk)
    vc = v.reshape(B, H, nc, chunk, dv)
    inner = ((qc @ kc.transpose(-1, -2)) * decay.unsqueeze(1)) @ vc
    kv = kc.transpose(-1, -2) @ (vc * v_dec.unsqueeze(1))
    state = torch.zeros(B, H, dk, dv, dtype=q.dtype)
    cross = torch.zeros_like(inner)
    for i in range(nc):
        cross[:, :, i] = (qc[:, :, i] * q_dec) @ state
        state = state * cross_decay + kv[:, :, i]
    return ((inner + cross) / scale).reshape(B, H, T, dv)


# --------------------------------------------------------------------------- (b') om causal
def om_elem(s, v):
    """`_om_elem` (torch_bridge.py:1974-1981): (rowmax s, sum exp(s-m), exp(s-m) @ v)."""
    m = s.amax(dim=-1, keepdim=True)
    e = torch.exp(s - m)
    return (m, e.sum(dim=-1, keepdim=True), e @ v)


def om_compose(f, g):
    """`_om_compose` (torch_bridge.py:1984-2006): the FlashAttention combine with
    the isfinite guard for entirely masked blocks."""
    m1, l1, a1 = f
    m2, l2, a2 = g
    mx = torch.maximum(m1, m2)
    fin1, fin2 = torch.isfinite(m1), torch.isfinite(m2)
    e1 = torch.where(fin1, torch.exp(m1 - mx), torch.zeros_like(mx))
    e2 = torch.where(fin2, torch.exp(m2 - mx), torch.zeros_like(mx))
    lv = torch.where(fin1, l1 * e1, torch.zeros_like(l1)) + torch.where(fin2, l2 * e2, torch.zeros_like(l2))
    a = torch.where(fin1, a1 * e1, torch.zeros_like(a1)) + torch.where(fin2, a2 * e2, torch.zeros_like(a2))
    return (mx, lv, a)


def cmask(x: torch.Tensor, off: int = 0) -> torch.Tensor:
    """`_cmask_torch` (catopt_carriers/om.py:1023-1029): True where key j+off > query t."""
    t, k = x.shape[-2], x.shape[-1]
    keep = torch.ones(t, k, dtype=torch.bool).tril(-off)
    return keep.logical_not().expand(x.shape)


def om_causal_chunked(q, k, v, sizes, scale: float | None = None):
    """`om_apply` over a left fold of `om_elem` key blocks of the given sizes
    (the streaming schedule of om_lower.py:996-1040): scale folded into q, each
    block's scores masked with the causal mask shifted by the block offset,
    read-out a / l (torch_bridge.py:1887-1890)."""
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    qs = q * sc
    state, off = None, 0
    for n in sizes:
        kb, vb = k[..., off:off + n, :], v[..., off:off + n, :]
        s = qs @ kb.transpose(-1, -2)
        s = s.masked_fill(cmask(s, off), float("-inf"))
        el = om_elem(s, vb)
        state = el if state is None else om_compose(state, el)
        off += n
    return state[2] / state[1]


# --------------------------------------------------------------------------- (c) scan
def affd_compose(f, g):
    """`affd_compose` binding (torch_bridge.py:1896-1899): f after g."""
    return (f[0] * g[0], f[0] * g[1] + f[1])


def applyd(f, h):
    """`applyd` binding (torch_bridge.py:1900)."""
    return f[0] * h + f[1]


def diag_scan_serial(a, x, b, c, h0=None):
    """Serial fold of `applyd(aff_diag(a_t, b*x_t), h)` with readout.

    All operands are widened to fp32 before any arithmetic; y is returned in
    fp32 (the caller rounds once if it wants the storage dtype).
    a: [B,T,D,N] or [B,T,D]; x: [B,T,D]; b,c: [D,N]; h0: [B,D,N] or None.
    Returns (y [B,T,D] fp32, h_T [B,D,N] fp32).
    """
    a, x, b, c = a.float(), x.float(), b.float(), c.float()
    if a.dim() == 3:
        a = a.unsqueeze(-1)
    B, T, D = x.shape
    N = b.shape[1]
    h = torch.zeros(B, D, N) if h0 is None else h0.float().clone()
    y = torch.empty(B, T, D)
    for t in range(T):
        u = b * x[:, t].unsqueeze(-1)          # aff_diag's second component
        h = applyd((a[:, t], u), h)
        y[:, t] = (h * c).sum(-1)
    return y, h


def seq_fold(a_rows, b_rows, h, axis: int = 0):
    """The sequence form `applyd(aff_diag(a, b), h)` folded along the step axis:
    `acc = a_t * acc + b_t` for t in time order, the loop of the reference's
    generated scan kernel (`_seq_triton_source`, catopt_discovery/genkernel.py:
    1031-1060) with its right-aligned broadcasting (`_seq_args`, 1173-1205): an
    operand without a step axis is shared by every step."""
    full = torch.broadcast_shapes(a_rows.shape, b_rows.shape)
    a_rows, b_rows = a_rows.expand(full), b_rows.expand(full)
    acc = h
    for t in range(full[axis]):
        acc = applyd((a_rows.select(axis, t), b_rows.select(axis, t)), acc)
    return acc


def scan_states(a_rows, b_rows, h):
    """Every state of the sequence form: `h_t = applyd(aff_diag(a_t, b_t), h_(t-1))`
    stacked along dim 0 — the value of the stacked-map member
    `applyd(aff_diag(stack(affd_a f_t), stack(affd_b f_t)), h)` that
    `gather_applyd_stack` offers (catopt_carriers/xcarrier.py:2252-2275), whose
    prefix maps f_t the reference composes with `affd_compose`
    (torch_bridge.py:1896-1899: `(f0*g0, f0*g1 + f1)`, g applied first)."""
    full = torch.broadcast_shapes(a_rows.shape, b_rows.shape, (1, *h.shape))
    a_rows, b_rows = a_rows.expand(full), b_rows.expand(full)
    fa, fb = a_rows[0], b_rows[0]
    out = [applyd((fa, fb), h)]
    for t in range(1, full[0]):
        fa, fb = affd_compose((a_rows[t], b_rows[t]), (fa, fb))
        out.append(applyd((fa, fb), h))
    return torch.stack(out)


def fused_diag_levels(a_seq, b_seq, h):
    """`fused_diag_levels` (catopt_carriers/scan_fused.py:100-120): leaves in
    product order (latest step first), identity padding to a power of two,
    adjacent-pair reduction, final `addcmul`."""
    def pad(t, fill):
        n = t.shape[0]
        p = (1 << max(n - 1, 0).bit_length()) - n
        return t if not p else torch.cat([t, t.new_full((p, *t.shape[1:]), fill)])

    a, b = pad(a_seq, 1.0), pad(b_seq, 0.0)
    while a.shape[0] > 1:
        fa, ga = a[0::2], a[1::2]
        fb, gb = b[0::2], b[1::2]
        a = fa * ga
        b = torch.addcmul(fb, fa, gb)
    return torch.addcmul(b[0], a[0], h)


def prefix_scan_diag(A, Bv):
    """`BatchedOmdModule._prefix_scan` (omd_lower.py:771-824), diagonal domain:
    all prefix maps (P_a[t], P_b[t]) with h_t = P_a[t]*h_0 + P_b[t]."""
    T = A.shape[0]
    if T == 1:
        return A, Bv
    blk = math.ceil(math.sqrt(T))
    C = (T + blk - 1) // blk
    padn = C * blk - T
    sa, sb = A.shape[1:], Bv.shape[1:]
    ida, idb = torch.ones(*sa, dtype=A.dtype), torch.zeros(*sb, dtype=A.dtype)
    if padn:
        A = torch.cat([A, ida.unsqueeze(0).expand(padn, *sa)])
        Bv = torch.cat([Bv, idb.unsqueeze(0).expand(padn, *sb)])
    A, Bv = A.reshape(C, blk, *sa), Bv.reshape(C, blk, *sb)
    las, lbs = [A[:, 0]], [Bv[:, 0]]
    for kk in range(1, blk):
        na, nb = affd_compose((A[:, kk], Bv[:, kk]), (las[-1], lbs[-1]))
        las.append(na)
        lbs.append(nb)
    La, Lb = torch.stack(las, 1), torch.stack(lbs, 1)
    cpa, cpb = [ida], [idb]
    for cc in range(1, C):
        na, nb = affd_compose((La[cc - 1, -1], Lb[cc - 1, -1]), (cpa[-1], cpb[-1]))
        cpa.append(na)
        cpb.append(nb)
    CPa, CPb = torch.stack(cpa).unsqueeze(1), torch.stack(cpb).unsqueeze(1)
    Pa, Pb = affd_compose((La, Lb), (CPa, CPb))
    n = C * blk
    return Pa.reshape(n, *sa)[:T], Pb.reshape(n, *sb)[:T]
