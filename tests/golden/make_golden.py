"""Generate the golden fixtures by running the REAL reference (catopt) on CPU.

Usage (in a checkout that has the reference's source tree next to it):

    PYTHONHASHSEED=0 python tests/golden/make_golden.py /path/to/catopt

The script puts ``<catopt>/packages/*/src`` on ``sys.path``, builds each case's
seeded inputs (``cases.py``), runs the reference's own lowered modules /
bindings / verify gate, and writes the outputs to ``tests/golden/*.npz``.  The
fixtures are what pins ``oracle/oracle.py`` (see ``tests/test_oracle_golden.py``);
the parity tests then compare the CUDA path with the oracle and with these files.
Nothing else in the repository imports the reference.
"""
from __future__ import annotations

import glob
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402


def _add_reference(root: str) -> None:
    srcs = sorted(glob.glob(os.path.join(root, "packages", "*", "src")))
    if not srcs:
        raise SystemExit(f"no packages/*/src under {root}")
    for p in srcs:
        sys.path.insert(0, p)


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.detach().numpy()


# --------------------------------------------------------------------------- decayed
def _decayed_terms(B, H, T, d, C, per_head, scale):
    """The uniform K-chunk term of om_decayed_kway_blocks and the spelled
    quadratic term, over three inputs q, k, v and a rate parameter g."""
    from catopt_core.ir import IR, Const, Op, Param, TensorType, Var

    K = T // C
    tt = lambda *s: TensorType(tuple(s))  # noqa: E731
    q, k, v = (Var(n, tt(B, H, T, d)) for n in "qkv")
    g = Param("g", tt(H)) if per_head else Param("g", tt())
    sc = Const(scale)
    sizes = [C] * K
    part = lambda t, i: Op.make("split", t, dim=-2, index=i, sizes=sizes)  # noqa: E731
    kt = Op.make("transpose", k, dim0=-1, dim1=-2)
    kti = lambda i: Op.make("split", kt, dim=-1, index=i, sizes=sizes)  # noqa: E731
    dvec = lambda **kw: Op.make("decay_vec", g, t=C, **kw)  # noqa: E731
    dec = Op.make("decay", g, t=C)

    def cross(i, j):
        a = Op.make("transpose",
                    Op.make("mul", part(k, j), Op.make("unsqueeze", dvec(sign=-1, offset=0), dim=-1)),
                    dim0=-1, dim1=-2)
        body = Op.make("matmul", part(q, i), Op.make("matmul", a, part(v, j)))
        row = Op.make("unsqueeze", dvec(sign=1, offset=(i - j) * C), dim=-1)
        return Op.make("mul", row, Op.make("div", body, sc))

    def arm(i):
        t = Op.make("div", Op.make("om_decayed", Op.make("matmul", part(q, i), kti(i)), dec, part(v, i)), sc)
        for j in range(i):
            t = Op.make("add", t, cross(i, j))
        return t

    names = {"q", "k", "v"}
    chunked = IR(root=Op.make("concat", *[arm(i) for i in range(K)], dim=-2),
                 inputs=[q, k, v], input_names=names, params={"g": g})
    quad = IR(root=Op.make("div", Op.make("om_decayed", Op.make("matmul", q, kt),
                                          Op.make("decay", g, t=T), v), sc),
              inputs=[q, k, v], input_names=names, params={"g": g})
    return chunked, quad


def gen_decayed() -> None:
    from catopt_torch.adapters import TorchSink
    from catopt_torch.torch_bridge import IRModule

    out = {}
    for name, (B, H, T, d, C, dtype, per_head, scale) in cases.DECAYED_CASES.items():
        q, k, v, gamma, C, scale = cases.decayed_inputs(name)
        chunked, quad = _decayed_terms(B, H, T, d, C, gamma.dim() == 1, scale)
        sink = TorchSink()
        spec = next(s for s in sink.executors.values()
                    if s.carrier is not None and s.accepts(chunked.root))
        assert spec.name == "om_decayed_chunked", spec.name
        mod = spec.lower(chunked, {"g": gamma})
        assert spec.engaged(mod)
        with torch.no_grad():
            o_chunk = mod(q, k, v)
            o_quad = IRModule(quad, {"g": gamma})(q, k, v)
        if name in cases.ROW_STRIDE:
            o_chunk = o_chunk[:, :, :: cases.ROW_STRIDE[name]].contiguous()
            o_quad = o_quad[:, :, :: cases.ROW_STRIDE[name]].contiguous()
        out[f"{name}.chunked"] = _np(o_chunk)
        out[f"{name}.quadratic"] = _np(o_quad)
        print(f"decayed {name}: chunked-vs-quadratic max abs {(o_chunk - o_quad).abs().max().item():.3e}")
    np.savez_compressed(HERE / "decayed.npz", **out)


# --------------------------------------------------------------------------- chain
def gen_chain() -> None:
    from catopt_orchestrator.optimize import Optimizer
    from catopt_torch.backend import TorchBackend

    out = {}
    for name in cases.CHAIN_CASES:
        ws, x = cases.chain_inputs(name)
        d = ws[0].shape[0]
        seq = torch.nn.Sequential(*[torch.nn.Linear(d, d, bias=False) for _ in ws])
        with torch.no_grad():
            for lin, w in zip(seq, ws):
                lin.weight.copy_(w)
        res = Optimizer(backend=TorchBackend()).optimize(seq, x)
        mod = res.module if hasattr(res, "module") else res[0]
        root = mod._root
        fused = [n for n, _ in mod.named_parameters() if n.startswith("fused_")] or \
                [n for n in getattr(mod, "_param_map", {}) if str(n).startswith("fused_")]
        print(f"chain {name}: folded root = {root}  fused params: {fused[-1:]}")
        assert str(root).startswith("linear(input, fused_"), str(root)
        with torch.no_grad():
            y_opt = mod(x)
            y_eager = seq(x)
        wf = dict(mod.named_parameters()).get(str(root.args[1].name))
        if wf is None:
            wf = mod._param_map[root.args[1].name]
        out[f"{name}.y_folded"] = _np(y_opt)
        out[f"{name}.y_eager"] = _np(y_eager)
        if name == "small":
            out[f"{name}.w_folded"] = _np(wf.detach())
        else:  # 1 MiB is too large for a fixture: keep a strided sample
            out[f"{name}.w_folded_sample"] = _np(wf.detach()[::16, ::16].contiguous())
    np.savez_compressed(HERE / "chain.npz", **out)


# --------------------------------------------------------------------------- scan
def gen_scan() -> None:
    from catopt_carriers.omd_lower import BatchedOmdModule
    from catopt_carriers.scan_fused import fused_diag_levels
    from catopt_torch.torch_bridge import _IR_TO_TORCH as BIND

    out = {}
    for name in cases.SCAN_CASES:
        a, x, b, c, h0 = cases.scan_inputs(name)
        af, xf, bf, cf = a.float(), x.float(), b.float(), c.float()
        if af.dim() == 3:
            af = af.unsqueeze(-1).expand(*af.shape, bf.shape[1])
        B, T, D = xf.shape
        N = bf.shape[1]
        h = torch.zeros(B, D, N) if h0 is None else h0.clone()
        ys, leaves_a, leaves_u = [], [], []
        for t in range(T):
            u = bf * xf[:, t].unsqueeze(-1)
            f = BIND["aff_diag"](af[:, t], u)
            h = BIND["applyd"](f, h)
            ys.append((h * cf).sum(-1))
            leaves_a.append(af[:, t])
            leaves_u.append(u)
        y = torch.stack(ys, 1)
        A, U = torch.stack(leaves_a), torch.stack(leaves_u)
        h_init = torch.zeros(B, D, N) if h0 is None else h0
        # final state through the reference's level-batched reduction (latest leaf first)
        hT_tree = fused_diag_levels(A.flip(0), U.flip(0), h_init)
        # all prefixes through the reference's blocked scan
        omd = BatchedOmdModule.__new__(BatchedOmdModule)
        Pa, Pb = omd._prefix_scan(A, U, "diag")
        y_prefix = ((Pa * h_init + Pb) * cf).sum(-1).movedim(0, 1)
        out[f"{name}.y"] = _np(y)
        out[f"{name}.hT"] = _np(h)
        out[f"{name}.hT_tree"] = _np(hT_tree)
        out[f"{name}.y_prefix"] = _np(y_prefix.contiguous())
        print(f"scan {name}: serial-vs-prefix {(y - y_prefix).abs().max().item():.3e} "
              f"serial-vs-tree {(h - hT_tree).abs().max().item():.3e}")
    np.savez_compressed(HERE / "scan.npz", **out)


# --------------------------------------------------------------------------- om causal
def gen_om_causal() -> None:
    """Left fold of the reference's own `om_elem` / `om_compose` bindings over key
    blocks masked with its `cmask` binding, read out as a / l; also dense sdpa."""
    import math

    from catopt_carriers.om import TORCH_BINDINGS as OMB
    from catopt_torch.torch_bridge import _IR_TO_TORCH as BIND

    out = {}
    for name in cases.OM_CAUSAL_CASES:
        q, k, v, sizes, scale = cases.om_causal_inputs(name)
        sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        qs = q * sc
        state, off = None, 0
        for n in sizes:
            s = qs @ k[..., off:off + n, :].transpose(-1, -2)
            s = s.masked_fill(OMB["cmask"](s, off=off), float("-inf"))
            el = BIND["om_elem"](s, v[..., off:off + n, :])
            state = el if state is None else BIND["om_compose"](state, el)
            off += n
        o = BIND["om_apply"](state)
        st = cases.OM_ROW_STRIDE.get(name, 1)
        out[f"{name}.chunked"] = _np(o[..., ::st, :].contiguous())
        if q.shape[-2] == k.shape[-2]:
            dense = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=sc)
            out[f"{name}.sdpa"] = _np(dense[..., ::st, :].contiguous())
            print(f"om_causal {name}: chunked-vs-sdpa {(o - dense).abs().max().item():.3e}")
    np.savez_compressed(HERE / "om_causal.npz", **out)


# --------------------------------------------------------------------------- generated-kernel tier
def gen_gated() -> None:
    """The `om_decayed` binding `(s*d)@v` on materialised scores, and the sequence
    form `applyd(aff_diag(a_t, b_t), h)` folded in time order with the reference's
    own bindings — the two functions its generated kernels compute."""
    from catopt_carriers.om import TORCH_BINDINGS as OMB
    from catopt_torch.torch_bridge import _IR_TO_TORCH as BIND

    out = {}
    for name in cases.GATED_CASES:
        s, gate, v = cases.gated_inputs(name)
        o = OMB["om_decayed"](s, gate, v)
        out[f"gated.{name}"] = _np(o.contiguous())
        print(f"gated {name}: {tuple(o.shape)} {o.dtype}")
    for name in cases.FOLD_CASES:
        a, b, h = cases.fold_inputs(name)
        n = cases.FOLD_CASES[name][0]
        acc = h
        for t in range(n):
            at = a[t] if a.dim() == h.dim() + 1 else a
            bt = b[t] if b.dim() == h.dim() + 1 else b
            acc = BIND["applyd"](BIND["aff_diag"](at, bt), acc)
        out[f"fold.{name}"] = _np(acc.contiguous())
        print(f"fold {name}: {tuple(acc.shape)} {acc.dtype}")
    np.savez_compressed(HERE / "gated.npz", **out)


# --------------------------------------------------------------------------- verify
def gen_verify() -> None:
    from catopt_torch.report import verify_equiv

    out = {}
    for name, ref, o, rtol, atol in cases.verify_cases():
        rep = verify_equiv(ref, o, rtol=rtol, atol=atol)
        out[name] = np.array([rep.max_abs, rep.max_rel, float(rep.passed)], dtype=np.float64)
        print(f"verify {name}: {rep}")
    # multi-output: worst case over outputs, per_output in order; length mismatch fails closed
    cs = cases.verify_cases()
    rep = verify_equiv((cs[0][1], cs[3][1]), (cs[0][2], cs[3][2]), rtol=2e-2)
    out["tuple"] = np.array([rep.max_abs, rep.max_rel, float(rep.passed), *rep.per_output])
    rep = verify_equiv((cs[0][1], cs[3][1]), (cs[0][2],), rtol=2e-2)
    out["tuple_mismatch"] = np.array([rep.max_abs, rep.max_rel, float(rep.passed)])
    np.savez_compressed(HERE / "verify.npz", **out)


def gen_states() -> None:
    """The stacked-map member `applyd(aff_diag(stack(affd_a f_t), stack(affd_b f_t)), h)` over the
    prefix chain f_t = affd_compose(leaf_t, f_(t-1)) — the form `gather_applyd_stack` offers
    (catopt_carriers/xcarrier.py:2252-2275) — evaluated by the reference's generic module."""
    from catopt_core.ir import IR, Op, TensorType, Var
    from catopt_torch.torch_bridge import IRModule

    out = {}
    for name in ("per_step_f32", "shared_decay_f32", "per_step_bf16"):
        a, b, h = cases.fold_inputs(name)
        n, state = cases.FOLD_CASES[name][:2]
        tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
        av, bv, hv = Var("a", tt(*a.shape)), Var("b", tt(*b.shape)), Var("h", tt(*state))
        step = lambda v, full, t: Op.make("select", v, dim=0, index=t) if full else v  # noqa: E731
        leaves = [Op.make("aff_diag", step(av, a.dim() == len(state) + 1, t), step(bv, b.dim() == len(state) + 1, t))
                  for t in range(n)]
        fs = [leaves[0]]
        for lf in leaves[1:]:
            fs.append(Op.make("affd_compose", lf, fs[-1]))
        root = Op.make("applyd", Op.make("aff_diag", Op.make("stack", *(Op.make("affd_a", f) for f in fs), dim=0),
                                         Op.make("stack", *(Op.make("affd_b", f) for f in fs), dim=0)), hv)
        ir = IR(root=root, inputs=[av, bv, hv], input_names={"a", "b", "h"}, params={})
        with torch.no_grad():
            val = IRModule(ir, None)(a, b, h)
        out[f"states.{name}"] = _np(val)
        print(f"states {name}: {tuple(val.shape)} {val.dtype}")
    np.savez_compressed(HERE / "states.npz", **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    if os.environ.get("PYTHONHASHSEED") != "0":
        raise SystemExit("run with PYTHONHASHSEED=0: the reference's search order depends on it")
    _add_reference(sys.argv[1])
    torch.manual_seed(0)
    only = set(sys.argv[2:])
    for nm, fn in (("verify", gen_verify), ("scan", gen_scan), ("states", gen_states), ("om_causal", gen_om_causal),
                   ("gated", gen_gated), ("decayed", gen_decayed), ("chain", gen_chain)):
        if not only or nm in only:
            fn()
