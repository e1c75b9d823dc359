"""The catopt-facing layer on a B200: catopt's own optimizer, executor routing,
runner and verify gate driving the modules of ``catopt_b200.sink`` with CUDA
tensors, so every kernel call below is made by catopt's code paths and not by a
test harness (the pattern of the reference's tests/test_pluggable_sink.py:124-165
and tests/test_batched_scan_lift.py:1089-1135).

Needs catopt importable (see ``_catopt_path``); the module is skipped with an
explicit reason when it is not.  Tolerances: fp32 ``max|d|/max|ref| <= 1e-5``,
bf16 ``<= 2e-2`` (the reference's own verify metric).
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(__file__))
import _catopt_path  # noqa: E402

pytestmark = pytest.mark.gpu

_LAYOUT = _catopt_path.add_catopt_to_path()
if _LAYOUT is None:
    pytest.skip(_catopt_path.SKIP_REASON, allow_module_level=True)

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402
import make_golden  # noqa: E402
from catopt_core.ir import IR, Const, Op, Param, TensorType, Var  # noqa: E402
from catopt_core.ports import BatchedExecutor  # noqa: E402
from decoder_model import decoder  # noqa: E402

from catopt_b200 import ops, verify  # noqa: E402
from catopt_b200 import sink as b200  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DEV = torch.device("cuda", 0)


def _rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return ((got - want).abs().max() / (want.abs().max() + 1e-8)).item()


def _route(sink, term):
    from catopt_orchestrator.optimize import _route_spec

    return _route_spec(term, sink)


def _tt(*sh):
    return TensorType(tuple(sh))


# --------------------------------------------------------------------------- (a) config 1 end to end
def test_config1_chain_through_the_optimizer_lowers_to_the_b200_module_and_is_gated_by_the_kernel():
    from catopt_orchestrator.optimize import Optimizer

    ws, x = cases.chain_inputs("c1")
    seq = torch.nn.Sequential(*[torch.nn.Linear(512, 512, bias=False) for _ in ws])
    with torch.no_grad():
        for lin, w in zip(seq, ws):
            lin.weight.copy_(w)
    seq, xc = seq.to(DEV), x.to(DEV)
    gates0 = verify.kernel_gate_calls
    res = Optimizer(backend=b200.b200_backend()).optimize(seq, xc, verbose=False)
    mod, stats = res.module, res.stats
    assert stats["lowering"] == "batched", stats.get("lowering")
    assert isinstance(mod, b200.B200LinearChainModule) and mod.is_batched
    assert isinstance(mod, BatchedExecutor)
    # the optimizer's own gate (Optimizer.lower -> sink.verify) ran on cb2_verify_reduce and passed
    assert verify.kernel_gate_calls > gates0
    assert res.verified is not None and res.verified.passed and res.verified.max_rel < 1e-5
    z = np.load(os.path.join(GOLDEN, "chain.npz"))
    with torch.no_grad():
        y = mod(xc)
    assert _rel(y, torch.from_numpy(z["c1.y_folded"])) <= 1e-5
    assert _rel(y, torch.from_numpy(z["c1.y_eager"])) <= 1e-5
    # the fold happened on the GPU at construction: one [512, 512] weight is all that is left
    assert tuple(mod.fused_weight.shape) == (512, 512) and mod.fused_weight.is_cuda
    ops.check_device_status(DEV)


def test_cuda_graph_runner_captures_and_replays_b200_modules():
    """``CudaGraphRunner.apply`` (catopt_cuda/runners.py:54-89) on two B200 modules:
    capture through the reference's runner, then replay on new inputs."""
    from catopt_cuda.runners import CudaGraphRunner

    # folded chain
    ws, x = cases.chain_inputs("small")
    x_in = Var("input", _tt(*x.shape))
    ps = [Param(f"p_{i}_weight", _tt(*w.shape)) for i, w in enumerate(ws)]
    tree = ps[0]
    for p in ps[1:]:
        tree = Op.make("matmul", p, tree)
    ir = IR(root=Op.make("linear", x_in, tree), inputs=[x_in], input_names={"input"},
            params={p.name: p for p in ps})
    sink = b200.B200Sink()
    spec = _route(sink, ir.root)
    assert spec.name == "b200_linear_chain"
    mod = spec.lower(ir, {p.name: w.to(DEV) for p, w in zip(ps, ws)})
    xc = x.to(DEV)
    with torch.no_grad():
        eager = mod(xc).clone()
    stats: dict = {}
    out_mod = CudaGraphRunner().apply(mod, xc, stats)
    assert out_mod is mod and stats["cuda_graph"] is True, stats
    assert mod.is_graph_captured
    z = np.load(os.path.join(GOLDEN, "chain.npz"))
    with torch.no_grad():
        assert torch.equal(mod(xc), eager)
        assert _rel(mod(xc), torch.from_numpy(z["small.y_folded"])) <= 1e-5
        x2 = torch.randn_like(xc)
        got = mod(x2).clone()
    mod.drop_cuda_graph()
    with torch.no_grad():
        assert torch.equal(got, mod(x2))

    # decayed attention, config 2's shape
    q, k, v, gamma, C, scale = cases.decayed_inputs("c2_f32")
    chunked, _ = make_golden._decayed_terms(2, 4, 1024, 64, C, False, scale)
    dmod = _route(sink, chunked.root).lower(chunked, {"g": gamma.to(DEV)})
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    with torch.no_grad():
        eager = dmod(qc, kc, vc).clone()
    stats = {}
    CudaGraphRunner().apply(dmod, (qc, kc, vc), stats)
    assert stats["cuda_graph"] is True and dmod.is_graph_captured, stats
    with torch.no_grad():
        assert torch.equal(dmod(qc, kc, vc), eager)
        got = dmod(kc, qc, vc).clone()          # other values, same shapes: replayed
    dmod.drop_cuda_graph()
    with torch.no_grad():
        assert torch.equal(got, dmod(kc, qc, vc))
    ops.check_device_status(DEV)


# --------------------------------------------------------------------------- (b) decayed terms
@pytest.mark.parametrize("name", ["c2_f32", "tiny_f32_scalar", "odd_f32", "c4_slice"])
def test_hand_built_decayed_term_routed_by_the_sink_matches_the_reference_executor(name):
    B, H, T, d, C, dtype, per_head, scale = cases.DECAYED_CASES[name]
    q, k, v, gamma, C, scale = cases.decayed_inputs(name)
    chunked, _ = make_golden._decayed_terms(B, H, T, d, C, gamma.dim() == 1, scale)
    sink = b200.B200Sink()
    spec = _route(sink, chunked.root)
    assert spec.name == "b200_om_decayed_chunked"
    mod = spec.lower(chunked, {"g": gamma.to(DEV)})
    assert spec.engaged(mod) and mod.n_blocks == T // C and mod._gamma_is_const
    with torch.no_grad():
        got = mod(q.to(DEV), k.to(DEV), v.to(DEV))
        again = mod(q.to(DEV), k.to(DEV), v.to(DEV))       # second call: rate vector from the const cache
    assert torch.equal(got, again) and len(mod._const_cache) == 1
    z = np.load(os.path.join(GOLDEN, "decayed.npz"))
    stride = cases.ROW_STRIDE.get(name, 1)
    want = torch.from_numpy(z[f"{name}.chunked"])
    assert _rel(got[:, :, ::stride], want) <= 1e-5
    assert _rel(got[:, :, ::stride], torch.from_numpy(z[f"{name}.quadratic"])) <= 1e-5
    ops.check_device_status(DEV)


def test_really_extracted_ragged_decayed_term_runs_on_the_kernel_and_matches_the_source_model():
    """Saturate a decay-masked attention module with the K-way law as the reference's
    delivery test does (tests/test_om_decayed_kway_deliver.py:72-103), route what
    extraction returns, and run the delivered module on the GPU against the source model."""
    from catopt_carriers.om import OM_CHUNKIFY, OM_LAWS, om_kway_laws
    from catopt_core.cost import flops_cost
    from catopt_core.egraph import EGraph
    from catopt_core.laws import tensor as tl
    from catopt_torch.adapters import TorchSource

    class Retention(torch.nn.Module):
        def __init__(self, d):
            super().__init__()
            self.q, self.k, self.v = (torch.nn.Linear(d, d) for _ in range(3))

        def forward(self, x):
            t = x.shape[-2]
            pos = torch.arange(t, dtype=x.dtype, device=x.device)
            decay = torch.tril(torch.pow(torch.tensor(0.9, dtype=x.dtype, device=x.device),
                                         (pos.unsqueeze(1) - pos.unsqueeze(0)).clamp_min(0)))
            return ((self.q(x) @ self.k(x).transpose(-1, -2) / (t ** 0.5)) * decay) @ self.v(x)

    torch.manual_seed(0)
    kk, T = 2, 256
    rules = (list(OM_LAWS) + list(OM_CHUNKIFY) + list(tl.SPLIT_SCALAR_RULES)
             + [tl.MUL_DIV_SWAP, tl.MATMUL_DIV_DISTRIBUTE, tl.ASSOC_MATMUL_REV, tl.FACTOR_MUL, tl.FACTOR_MUL_ADD,
                tl.DIV_ADD_FACTOR] + om_kway_laws(kk))
    model = Retention(16)
    x = torch.randn(2, T, 16)
    ir, leaves = TorchSource().to_ir(model, x)
    eg = EGraph()
    root = eg.add_term(ir.root)
    eg.run(rules, root, max_iterations=16, max_nodes=200_000, patience=8,
           rule_budgets={"om_decayed_chunkify_rows": 60, "om_decayed_chunkify_keys": 60,
                         f"om_decayed_kway_blocks_{kk}": 200})
    best = eg.extract_best(eg.find(root), flops_cost)
    sink = b200.B200Sink()
    spec = _route(sink, best)
    assert spec is not None and spec.name == "b200_om_decayed_chunked"
    ex_ir = IR(root=best, inputs=list(ir.inputs), input_names=set(ir.input_names), params=dict(ir.params))
    mod = spec.lower(ex_ir, {n: (t.to(DEV) if isinstance(t, torch.Tensor) else t) for n, t in leaves.items()})
    assert spec.engaged(mod)
    with torch.no_grad():
        got = mod(x.to(DEV))
        want = model.double()(x.double())
    assert _rel(got, want) <= 1e-5
    ops.check_device_status(DEV)


@pytest.mark.parametrize("kw", [dict(intra_row=True), dict(second_rate=True), dict(drop_pair=True),
                                dict(intra_row=True, second_rate=True)])
@pytest.mark.parametrize("dtype,shape,tol", [(torch.float32, (2, 3, 48, 8, 16), 1e-5),
                                             (torch.float32, (1, 4, 256, 64, 64), 1e-5),
                                             (torch.bfloat16, (2, 4, 256, 64, 64), 2e-2)])
def test_row_gated_and_two_rate_decayed_arms_on_the_pairwise_module_match_the_reference_executor(kw, dtype, shape, tol):
    """The members of the decayed family that have no state-carry form (a decay-row gate on the intra
    element, a second rate in the later arms, a missing cross pair): routed to `b200_om_decayed_pairwise`,
    the intra products of all arms run in one `cb2_gated_contract_fwd`, and the result equals the
    reference's own pairwise executor and its generic evaluation on the same device."""
    from catopt_torch.adapters import TorchSink
    from catopt_torch.torch_bridge import IRModule
    from decayed_variants import variant_term

    B, H, T, d, C = shape
    ir = variant_term(B, H, T, d, C, 4.0, **kw)
    gen = torch.Generator().manual_seed(T + d)
    q, k, v = (torch.randn(B, H, T, d, generator=gen).div(d ** 0.25).to(dtype).to(DEV) for _ in range(3))
    rates = {"g": torch.linspace(0.85, 0.98, H).to(dtype).to(DEV), "g2": torch.linspace(0.6, 0.9, H).to(dtype).to(DEV)}
    vals = {n: rates[n] for n in ir.params}
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_om_decayed_pairwise"
    mod = spec.lower(ir, vals)
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod) and mod.n_blocks == T // C
    rspec = _route(TorchSink(), ir.root)
    assert rspec.name == "om_decayed_chunked"
    ref = rspec.lower(ir, vals)
    with torch.no_grad():
        got = mod(q, k, v)
        want = ref(q, k, v)
        plain = IRModule(ir, vals)(q, k, v)
    assert mod.kernel_calls == 1
    assert got.dtype == want.dtype and got.shape == want.shape
    assert _rel(got, want) <= tol
    assert _rel(got, plain) <= tol
    ops.check_device_status(DEV)


# --------------------------------------------------------------------------- (c) scan, omd, om causal
def _scan_term(T, d):
    """applyd(affd_compose(... aff_diag(a_t, select(u, 0, t)) ...), h) over T steps, per-step decays."""
    u, a = Var("u", _tt(T, d)), Var("a", _tt(T, d))
    h = Param("h0", _tt(d))
    leaf = lambda t: Op.make("aff_diag", Op.make("select", a, dim=0, index=t),  # noqa: E731
                             Op.make("select", u, dim=0, index=t))
    tree = leaf(T - 1)
    for t in range(T - 2, -1, -1):
        tree = Op.make("affd_compose", tree, leaf(t))
    return IR(root=Op.make("applyd", tree, h), inputs=[u, a], input_names={"u", "a"}, params={"h0": h})


def test_scan_term_on_the_b200_module_matches_the_reference_executor_on_the_same_device():
    from catopt_torch.adapters import TorchSink

    T, d = 96, 4096
    ir = _scan_term(T, d)
    g = torch.Generator().manual_seed(11)
    u = torch.randn(T, d, generator=g).to(DEV)
    a = torch.sigmoid(3 + torch.randn(T, d, generator=g)).to(DEV)
    vals = {"h0": torch.randn(d, generator=g).to(DEV)}
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_scan"
    mod = spec.lower(ir, vals)
    assert spec.engaged(mod) and mod._plan["diagonal"]
    rspec = _route(TorchSink(), ir.root)
    ref = rspec.lower(ir, vals)
    assert rspec.engaged(ref)
    with torch.no_grad():
        got, want = mod(u, a), ref(u, a)
    assert mod.kernel_calls == 1
    assert _rel(got, want) <= 1e-5
    # the serial recurrence in fp64
    h = vals["h0"].double()
    for t in range(T):
        h = a[t].double() * h + u[t].double()
    assert _rel(got, h) <= 1e-5
    ops.check_device_status(DEV)


def test_omd_term_on_the_b200_module_matches_the_reference_executor_on_the_same_device():
    from catopt_torch.adapters import TorchSink

    T, Tq, d = 64, 8, 2048
    a_p, x_v = Param("p_a", _tt(T, d)), Var("x", _tt(T, d))
    s, h = Param("s", _tt(Tq, T)), Param("h", _tt(d))
    leaves = [Op.make("aff_diag", Op.make("select", a_p, dim=0, index=t), Op.make("select", x_v, dim=0, index=t))
              for t in range(T)]
    fs = [leaves[0]]
    for t in range(1, T):
        fs.append(Op.make("affd_compose", leaves[t], fs[-1]))
    root = Op.make("omd_apply", Op.make("omd_elem", s, Op.make("stack", *(Op.make("affd_a", f) for f in fs), dim=0),
                                        Op.make("stack", *(Op.make("affd_b", f) for f in fs), dim=0)), h)
    ir = IR(root=root, inputs=[x_v], input_names={"x"}, params={"p_a": a_p, "s": s, "h": h})
    g = torch.Generator().manual_seed(12)
    vals = {"p_a": (torch.rand(T, d, generator=g) * 0.5 + 0.5).to(DEV), "s": torch.randn(Tq, T, generator=g).to(DEV),
            "h": torch.randn(d, generator=g).to(DEV)}
    x = torch.randn(T, d, generator=g).to(DEV)
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_omd"
    mod = spec.lower(ir, vals)
    rspec = _route(TorchSink(), ir.root)
    ref = rspec.lower(ir, vals)
    assert spec.engaged(mod) and rspec.engaged(ref)
    with torch.no_grad():
        got, want = mod(x), ref(x)
    assert mod.kernel_calls >= 1
    assert _rel(got, want) <= 1e-5
    ops.check_device_status(DEV)


def _om_causal_term(ksizes, Tq, d, dv, batch, scale):
    q = Var("q", _tt(*batch, Tq, d))
    ks = [Var(f"k{i}", _tt(*batch, n, d)) for i, n in enumerate(ksizes)]
    vs = [Var(f"v{i}", _tt(*batch, n, dv)) for i, n in enumerate(ksizes)]

    def scores(k):
        return Op.make("om_decayed", q, Op.make("fill", q, value=scale), Op.make("transpose", k, dim0=-2, dim1=-1))

    kall = ks[0]
    for k in ks[1:]:
        kall = Op.make("concat", kall, k, dim=-2)
    cm = Op.make("cmask", scores(kall))
    rank = len(batch) + 2
    leaves = [Op.make("om_elem", Op.make("masked_fill", scores(k), Op.make("split", cm, dim=rank - 1, index=i,
                                                                         sizes=tuple(ksizes)), Const(float("-inf"))), v)
              for i, (k, v) in enumerate(zip(ks, vs))]
    tree = leaves[-1]
    for lf in reversed(leaves[:-1]):
        tree = Op.make("om_compose", lf, tree)
    inputs = [q, *ks, *vs]
    return IR(root=Op.make("om_apply", tree), inputs=inputs, input_names={v.name for v in inputs}, params={})


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_om_causal_term_on_the_b200_module_matches_the_reference_executor_on_the_same_device(dtype, tol):
    from catopt_torch.adapters import TorchSink

    ksizes, Tq, d, dv, batch, scale = (128, 64, 192), 384, 64, 64, (2, 4), 0.125
    ir = _om_causal_term(ksizes, Tq, d, dv, batch, scale)
    g = torch.Generator().manual_seed(13)
    q = torch.randn(*batch, Tq, d, generator=g).to(dtype).to(DEV)
    ks = [torch.randn(*batch, n, d, generator=g).to(dtype).to(DEV) for n in ksizes]
    vs = [torch.randn(*batch, n, dv, generator=g).to(dtype).to(DEV) for n in ksizes]
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_om_causal"
    mod = spec.lower(ir, None)
    rspec = _route(TorchSink(), ir.root)
    ref = rspec.lower(ir, None)
    assert spec.engaged(mod) and rspec is not None
    with torch.no_grad():
        got = mod(q, *ks, *vs)
        want = ref(*(t.float() for t in (q, *ks, *vs)))          # the reference in fp32 on the rounded inputs
        state = mod.forward_state(q, *ks, *vs)
    assert got.dtype == dtype and _rel(got, want) <= tol
    assert _rel(ops.om_apply_state(state), want) <= tol
    ops.check_device_status(DEV)


# --------------------------------------------------------------------------- (e) config 5's caller
class _Fp32GraphAsBf16(torch.nn.Module):
    """An fp32 module seen through bf16 tensors: input widened, output rounded once."""

    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, x):
        return self.m(x.float()).bfloat16()


def test_compositional_on_the_config5_decoder_gates_every_block_and_the_whole_model_with_the_kernel():
    """``Optimizer.optimize(model, x, strategy=Compositional())`` with the B200 backend
    on the decoder of benchmark config 5.  The search runs in fp32 (the reference's
    search cannot take bf16 parameters) on weights that are bf16-representable, so the
    original model has an exact bf16 twin.  Then config 5's pairs: for every block the
    bf16 original against the optimized graph (delivered in fp32, seen through bf16
    tensors) on the input the ORIGINAL model's forward hands that block, as
    ``_block_gate`` does (optimize.py:1334-1368, 3555), plus the end-to-end pair — all
    through ``B200Sink.verify`` at rtol 2e-2 and float-identical with the CPU
    restatement of the gate."""
    import copy

    from catopt_orchestrator.optimize import Compositional, Optimizer

    from oracle import oracle

    n_blocks = int(os.environ.get("CB2_TEST_DECODER_BLOCKS", "12"))
    model = decoder(n_blocks)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(p.bfloat16().float())
    model = model.to(DEV)
    x = torch.randn(4, 512, 1024, generator=torch.Generator().manual_seed(1)).bfloat16().float().to(DEV)
    gates0 = verify.kernel_gate_calls
    res = Optimizer(backend=b200.b200_backend()).optimize(model, x, strategy=Compositional(), verbose=False)
    opt, stats = res.module, res.stats
    assert stats["n_optimized"] == n_blocks and stats["n_failed"] == 0, {k: stats[k] for k in
                                                                        ("n_optimized", "n_failed", "n_skipped")}
    assert "rolled_back" not in stats["end_to_end"] and stats["end_to_end"]["max_rel_diff"] < 1e-4
    # the block gates and the end-to-end gate of the run itself went through cb2_verify_reduce
    assert verify.kernel_gate_calls - gates0 >= n_blocks + 1
    assert stats["cache"]["hits"] == n_blocks - 1

    sink = b200.B200Sink()
    mb = copy.deepcopy(model).bfloat16()          # exact: the weights are bf16-representable
    xb = x.bfloat16()
    captured = []
    hooks = [blk.register_forward_pre_hook(lambda m, args: captured.append(args[0].detach().clone())) for blk in mb]
    with torch.no_grad():
        mb(xb)
    for h in hooks:
        h.remove()
    assert len(captured) == n_blocks
    gates1 = verify.kernel_gate_calls
    for i, (blk, oblk) in enumerate(zip(mb, opt)):
        oblk = _Fp32GraphAsBf16(oblk)
        rep = sink.verify(blk, oblk, captured[i], rtol=2e-2)
        with torch.no_grad():
            want = oracle.verify_pair(blk(captured[i]).cpu(), oblk(captured[i]).cpu(), rtol=2e-2)
        assert (rep.max_abs, rep.max_rel, rep.passed) == (want.max_abs, want.max_rel, want.passed), i
        assert rep.passed and rep.max_abs > 0.0, (i, rep)      # a real pair: equivalent graphs, different rounding
    whole = _Fp32GraphAsBf16(opt)
    rep = sink.verify(mb, whole, xb, rtol=2e-2)
    with torch.no_grad():
        want = oracle.verify_pair(mb(xb).cpu(), whole(xb).cpu(), rtol=2e-2)
    assert (rep.max_abs, rep.max_rel, rep.passed) == (want.max_abs, want.max_rel, want.passed)
    assert 0.0 < rep.max_rel < 0.1, rep                 # bf16 rounding accumulated over the whole stack
    assert verify.kernel_gate_calls - gates1 == n_blocks + 1
    ops.check_device_status(DEV)


def test_sink_verify_delegates_what_the_kernel_does_not_take():
    """fp64 and host outputs go to the reference's own gate instead of failing the run."""
    sink = b200.B200Sink()
    lin = torch.nn.Linear(8, 8).double().to(DEV)
    x = torch.randn(4, 8, dtype=torch.float64, device=DEV)
    n0 = verify.kernel_gate_calls
    rep = sink.verify(lin, lin, x)
    assert rep.passed and rep.max_abs == 0.0 and verify.kernel_gate_calls == n0
    cpu = torch.nn.Linear(8, 8)
    rep = sink.verify(cpu, cpu, torch.randn(4, 8))
    assert rep.passed and verify.kernel_gate_calls == n0
    lin32 = torch.nn.Linear(8, 8).to(DEV)
    rep = sink.verify(lin32, lin32, x.float())
    assert rep.passed and verify.kernel_gate_calls == n0 + 1


# --------------------------------------------------------------------------- scan, every state (stacked-map form)
def _stacked_map_term(leaves, h, dim):
    """applyd(aff_diag(stack(affd_a f_t), stack(affd_b f_t)), h) over the prefix chain of ``leaves``
    — the member ``gather_applyd_stack`` offers (catopt_carriers/xcarrier.py:2252-2275)."""
    fs = [leaves[0]]
    for lf in leaves[1:]:
        fs.append(Op.make("affd_compose", lf, fs[-1]))
    sa = Op.make("stack", *(Op.make("affd_a", f) for f in fs), dim=dim)
    sb = Op.make("stack", *(Op.make("affd_b", f) for f in fs), dim=dim)
    return Op.make("applyd", Op.make("aff_diag", sa, sb), h)


def test_every_state_of_a_scan_through_b200_scan_all_matches_the_reference_evaluation():
    from catopt_torch.torch_bridge import IRModule

    T, d = 128, 8192
    a_p, x_v, h = Param("p_a", _tt(T, d)), Var("x", _tt(T, d)), Param("h0", _tt(d))
    leaves = [Op.make("aff_diag", Op.make("select", a_p, dim=0, index=t), Op.make("select", x_v, dim=0, index=t))
              for t in range(T)]
    ir = IR(root=_stacked_map_term(leaves, h, 0), inputs=[x_v], input_names={"x"}, params={"p_a": a_p, "h0": h})
    g = torch.Generator().manual_seed(21)
    vals = {"p_a": torch.sigmoid(3 + torch.randn(T, d, generator=g)).to(DEV), "h0": torch.randn(d, generator=g).to(DEV)}
    x = torch.randn(T, d, generator=g).to(DEV)
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_scan_all"
    mod = spec.lower(ir, vals)
    assert spec.engaged(mod) and mod._plan["a"][0] == "gather" and mod._plan["b"][0] == "gather"
    with torch.no_grad():
        got = mod(x)
        want = IRModule(ir, vals)(x)            # the reference's eager evaluation of the same term, same device
    assert mod.kernel_calls == 1 and got.shape == want.shape == (T, d)
    assert _rel(got, want) <= 1e-5
    hh, rows = vals["h0"].double(), []
    for t in range(T):
        hh = vals["p_a"][t].double() * hh + x[t].double()
        rows.append(hh)
    assert _rel(got, torch.stack(rows)) <= 1e-5
    ops.check_device_status(DEV)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_config3_recurrence_as_a_term_runs_on_the_scan_kernel(dtype, tol):
    """``y_t = sum_n c*h_t``, ``h_t = a_t*h_(t-1) + b*x_t`` spelled as the readout of the
    stacked-map form: routed to ``b200_scan_all`` and run by ``cb2_diag_scan_fwd``."""
    from catopt_torch.torch_bridge import IRModule

    from oracle import oracle

    B, T, D, N = 2, 48, 64, 16
    a_v, x_v = Var("a", _tt(B, T, D, N)), Var("x", _tt(B, T, D))
    b_p, c_p, h_p = Param("p_b", _tt(D, N)), Param("p_c", _tt(D, N)), Param("p_h0", _tt(N))
    leaves = [Op.make("aff_diag", Op.make("select", a_v, dim=1, index=t),
                      Op.make("mul", b_p, Op.make("unsqueeze", Op.make("select", x_v, dim=1, index=t), dim=-1)))
              for t in range(T)]
    states = _stacked_map_term(leaves, h_p, 1)
    root = Op.make("sum", Op.make("mul", states, c_p), dim=(-1,))
    ir = IR(root=root, inputs=[a_v, x_v], input_names={"a", "x"}, params={"p_b": b_p, "p_c": c_p, "p_h0": h_p})
    g = torch.Generator().manual_seed(22)
    a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, N, generator=g)).to(dtype)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    vals = {"p_b": (torch.randn(D, N, generator=g) / 4).to(dtype), "p_c": (torch.randn(D, N, generator=g) / 4).to(dtype),
            "p_h0": torch.zeros(N, dtype=dtype)}
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_scan_all"
    mod = spec.lower(ir, {k: v.to(DEV) for k, v in vals.items()})
    assert spec.engaged(mod) and mod._plan["readout"] is not None
    with torch.no_grad():
        got = mod(a.to(DEV), x.to(DEV))
        # the reference's eager evaluation of the same term in fp32 on the (rounded) inputs
        want = IRModule(ir, {k: v.float().to(DEV) for k, v in vals.items()})(a.float().to(DEV), x.float().to(DEV))
    assert mod.kernel_calls == 1 and got.dtype == dtype and got.shape == (B, T, D)
    assert _rel(got, want) <= tol
    wy, _ = oracle.diag_scan_serial(a, x, vals["p_b"], vals["p_c"])
    assert _rel(got, wy) <= tol
    ops.check_device_status(DEV)


def test_an_expired_device_wait_fails_the_sink_gate_as_a_timeout():
    """A bounded wait that ran out in some earlier kernel is reported where the
    catopt-facing layer next synchronises — the verify gate's read-back — as a
    ``B200Error`` that ``catopt_core.failures.classify`` buckets as TIMEOUT
    (failures.py:74-112); the gate after it is clean."""
    from catopt_core.failures import FailureClass, classify

    from catopt_b200 import B200Error

    sink = b200.B200Sink()
    lin = torch.nn.Linear(8, 8).to(DEV)
    x = torch.randn(4, 8, device=DEV)
    assert sink.verify(lin, lin, x).passed
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.wait_for_flag(flag, budget_us=500)            # nobody sets the flag: the wait gives up
    with pytest.raises(B200Error) as err:
        sink.verify(lin, lin, x)
    assert classify(err.value) == FailureClass.TIMEOUT
    assert sink.verify(lin, lin, x).passed            # status consumed, stream and context intact


# --------------------------------------------------------------------------- autotuner and measured profile
def test_autotuned_verifies_times_and_ships_the_b200_candidate_and_feeds_the_profile():
    """``Autotuned`` (optimize.py:2543-2621, autotune.py) on config 1 with the B200 executor as a
    named candidate: one search, every candidate re-lowered from the delivered module's term,
    gated by ``B200Sink.verify`` and timed by the backend's ``Meter``; the winner ships.  With
    ``profile=`` the medians land in ``TargetProfile.measured_ns`` through the reference's own
    ``record_measured`` under this input's shape bucket."""
    from catopt_core.profile import measured_price_ns, record_measured, shape_bucket
    from catopt_orchestrator.optimize import Autotuned, Optimizer

    ws, x = cases.chain_inputs("c1")
    seq = torch.nn.Sequential(*[torch.nn.Linear(512, 512, bias=False) for _ in ws])
    with torch.no_grad():
        for lin, w in zip(seq, ws):
            lin.weight.copy_(w)
    seq, xc = seq.to(DEV).eval(), x.to(DEV)
    prof = b200.b200_target_profile()
    assert prof.op_kernel_ns.get("matmul") and prof.measured_ns     # shipped with measured entries
    gates0 = verify.kernel_gate_calls
    res = Optimizer(backend=b200.b200_backend()).optimize(
        seq, xc, strategy=Autotuned(candidates=("eager", "generic", "b200_linear_chain"), n_calls=20, warmup=5,
                                    profile=prof))
    at = res.stats["autotune"]
    recs = at["candidates"]
    rec = recs["b200_linear_chain"]
    assert rec["status"] == "timed" and rec["verified"] and rec["max_rel"] < 1e-5, rec
    assert rec["median_s"] > 0 and rec["n_calls"] == 20
    assert verify.kernel_gate_calls - gates0 >= 3             # every candidate went through the kernel gate
    timed = {n: r["median_s"] for n, r in recs.items() if r.get("status") == "timed"}
    assert set(timed) == {"eager", "generic", "b200_linear_chain"}
    assert at["winner"] == min(timed, key=timed.get) and not at.get("fallback")
    bucket = shape_bucket(xc)
    new_prof = at["profile"]
    assert new_prof.measured_ns["b200_linear_chain"][bucket]["median_ns"] == pytest.approx(rec["median_s"] * 1e9)
    # against the unlowered model alone the B200 module wins and is what ships
    res2 = Optimizer(backend=b200.b200_backend()).optimize(
        seq, xc, strategy=Autotuned(candidates=("eager", "b200_linear_chain"), n_calls=20, warmup=5))
    at2 = res2.stats["autotune"]
    assert at2["winner"] == "b200_linear_chain", {n: r.get("median_s") for n, r in at2["candidates"].items()}
    assert isinstance(res2.module, b200.B200LinearChainModule) and res2.module.is_batched
    z = np.load(os.path.join(GOLDEN, "chain.npz"))
    with torch.no_grad():
        assert _rel(res2.module(xc), torch.from_numpy(z["c1.y_folded"])) <= 1e-5

    # config 2's term: the B200 executor and the reference's own, both timed by the backend's meter;
    # the measurement goes into the profile the same way and prices the candidate afterwards
    from catopt_torch.adapters import TorchSink
    from catopt_torch.meter import TorchMeter

    q, k, v, gamma, C, scale = cases.decayed_inputs("c2_f32")
    ir = b200.uniform_decayed_term(2, 4, 1024, 64, C, per_head=False, scale=scale)
    ins = (q.to(DEV), k.to(DEV), v.to(DEV))
    ours = _route(b200.B200Sink(), ir.root).lower(ir, {"g": gamma.to(DEV)})
    theirs = _route(TorchSink(), ir.root).lower(ir, {"g": gamma.to(DEV)})
    meter = TorchMeter()
    t_ours = meter.time(ours, ins, warmup=5, n_calls=20)
    t_theirs = meter.time(theirs, ins, warmup=5, n_calls=20)
    assert t_ours.failure == "ok" and t_theirs.failure == "ok"
    assert t_ours.median_s < t_theirs.median_s                 # one launch against the all-pairs schedule
    b2 = shape_bucket(ins)
    p2 = record_measured(new_prof, "b200_om_decayed_chunked", b2, t_ours.median_s * 1e9)
    assert measured_price_ns(p2, "b200_om_decayed_chunked", b2, None) == pytest.approx(t_ours.median_s * 1e9)
    ops.check_device_status(DEV)


@pytest.mark.parametrize("off", [1, -3])
def test_om_causal_term_with_a_shifted_mask_matches_the_reference_executor(off):
    """``cmask(x, off)`` hides key j from query t when ``j + off > t`` (om.py:1023-1029); the
    offset travels to ``cb2_om_step`` as its key offset.  With off > 0 the first rows see no key
    at all and are NaN in the reference (unclamped a / l) and here."""
    from catopt_torch.adapters import TorchSink

    ksizes, Tq, d, dv, batch, scale = (96, 160), 256, 64, 64, (2, 2), 0.125
    q = Var("q", _tt(*batch, Tq, d))
    ks = [Var(f"k{i}", _tt(*batch, n, d)) for i, n in enumerate(ksizes)]
    vs = [Var(f"v{i}", _tt(*batch, n, dv)) for i, n in enumerate(ksizes)]

    def scores(k):
        return Op.make("om_decayed", q, Op.make("fill", q, value=scale), Op.make("transpose", k, dim0=-2, dim1=-1))

    cm = Op.make("cmask", scores(Op.make("concat", *ks, dim=-2)), off=off)
    leaves = [Op.make("om_elem", Op.make("masked_fill", scores(k), Op.make("split", cm, dim=3, index=i, sizes=ksizes),
                                         Const(float("-inf"))), v) for i, (k, v) in enumerate(zip(ks, vs))]
    ins = [q, *ks, *vs]
    ir = IR(root=Op.make("om_apply", Op.make("om_compose", *leaves)), inputs=ins,
            input_names={t.name for t in ins}, params={})
    g = torch.Generator().manual_seed(14 + off)
    tq = torch.randn(*batch, Tq, d, generator=g).to(DEV)
    tks = [torch.randn(*batch, n, d, generator=g).to(DEV) for n in ksizes]
    tvs = [torch.randn(*batch, n, dv, generator=g).to(DEV) for n in ksizes]
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_om_causal"
    mod = spec.lower(ir, None)
    assert mod._plan["off"] == off
    ref = _route(TorchSink(), ir.root).lower(ir, None)
    with torch.no_grad():
        got, want = mod(tq, *tks, *tvs), ref(tq, *tks, *tvs)
    assert torch.equal(torch.isnan(got), torch.isnan(want))
    if off > 0:
        assert torch.isnan(want[..., :off, :]).all() and not torch.isnan(want[..., off:, :]).any()
    ok = ~torch.isnan(want)
    assert _rel(got[ok], want[ok]) <= 1e-5
    ops.check_device_status(DEV)


# --------------------------------------------------------------------------- explicit attention masks
def _om_masked_term(ksizes, Tq, d, dv, batch, scale, mask_shape, one_leaf):
    q = Var("q", _tt(*batch, Tq, d))
    ks = [Var(f"k{i}", _tt(*batch, n, d)) for i, n in enumerate(ksizes)]
    vs = [Var(f"v{i}", _tt(*batch, n, dv)) for i, n in enumerate(ksizes)]
    m = Var("m", _tt(*mask_shape))
    bias = Op.make("attnbias", m)
    if one_leaf:
        qs = Op.make("mul", q, Op.make("fill", q, value=scale))
        sc = Op.make("concat", *(Op.make("matmul", qs, Op.make("transpose", k, dim0=-2, dim1=-1)) for k in ks), dim=-1)
        tree = Op.make("om_elem", Op.make("add", sc, bias), Op.make("concat", *vs, dim=-2))
    else:
        def scores(k):
            return Op.make("om_decayed", q, Op.make("fill", q, value=scale), Op.make("transpose", k, dim0=-2, dim1=-1))

        leaves = [Op.make("om_elem", Op.make("add", scores(k), Op.make("split", bias, dim=len(mask_shape) - 1, index=i,
                                                                       sizes=tuple(ksizes))), v)
                  for i, (k, v) in enumerate(zip(ks, vs))]
        tree = leaves[-1]
        for lf in reversed(leaves[:-1]):
            tree = Op.make("om_compose", lf, tree)
    ins = [q, *ks, *vs, m]
    return IR(root=Op.make("om_apply", tree), inputs=ins, input_names={t.name for t in ins}, params={})


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("kind", ["bool", "additive", "finite", "per_batch", "per_head"])
@pytest.mark.parametrize("one_leaf", [False, True])
def test_om_term_with_an_explicit_mask_on_the_b200_module_matches_the_reference_executor(dtype, tol, kind, one_leaf):
    """The carrier of sdpa with an attn_mask (``add(scores, attnbias(m))``, om.py:1313-1362) through the
    routed B200 module against the reference's own executor for the same term on the same device: bool
    keep-masks, additive 0/-inf masks, finite biases, masks with a batch or a head axis.  Rows whose keys
    are all hidden are NaN in both."""
    from catopt_torch.adapters import TorchSink

    ksizes, Tq, d, dv, batch, scale = (128, 64, 192), 320, 64, 64, (2, 4), 0.125
    Tk = sum(ksizes)
    g = torch.Generator().manual_seed(21)
    if kind == "bool":
        shape, m = (Tq, Tk), torch.rand(Tq, Tk, generator=g) < 0.6
        m[5] = False                                   # one row sees no key at all
    elif kind == "additive":
        shape = (Tq, Tk)
        m = torch.where(torch.rand(Tq, Tk, generator=g) < 0.35, torch.tensor(float("-inf")), torch.zeros(()))
    elif kind == "finite":
        shape, m = (Tq, Tk), torch.randn(Tq, Tk, generator=g)
    elif kind == "per_batch":
        shape = (2, 1, Tq, Tk)
        m = torch.where(torch.rand(*shape, generator=g) < 0.35, torch.tensor(float("-inf")), torch.zeros(()))
    else:
        shape, m = (1, 4, Tq, Tk), torch.randn(1, 4, Tq, Tk, generator=g)
    ir = _om_masked_term(ksizes, Tq, d, dv, batch, scale, shape, one_leaf)
    q = torch.randn(*batch, Tq, d, generator=g).to(dtype).to(DEV)
    ks = [torch.randn(*batch, n, d, generator=g).to(dtype).to(DEV) for n in ksizes]
    vs = [torch.randn(*batch, n, dv, generator=g).to(dtype).to(DEV) for n in ksizes]
    m = m.to(DEV)
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_om_causal"
    mod = spec.lower(ir, None)
    assert mod.is_batched and mod._plan["bias"] is not None
    from catopt_torch.torch_bridge import IRModule

    rspec = _route(TorchSink(), ir.root)
    ref = rspec.lower(ir, None) if rspec is not None else IRModule(ir, None).to(DEV)
    with torch.no_grad():
        got = mod(q, *ks, *vs, m)
        want = ref(*(t.float() for t in (q, *ks, *vs)), m if m.dtype == torch.bool else m.float())
        state = mod.forward_state(q, *ks, *vs, m)     # the streaming fold: one cb2_om_bias_step per key block
    assert got.dtype == dtype
    assert torch.equal(torch.isnan(got), torch.isnan(want))
    streamed = ops.om_apply_state(state)
    assert torch.equal(torch.isnan(streamed), torch.isnan(want))
    assert _rel(streamed[~torch.isnan(want)], want[~torch.isnan(want)]) <= tol
    if kind == "bool":
        assert torch.isnan(want[..., 5, :]).all()
    ok = ~torch.isnan(want)
    assert _rel(got[ok], want[ok]) <= tol
    ops.check_device_status(DEV)
