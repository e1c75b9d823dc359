"""Routing and plan extraction of catopt_b200.sink against the real catopt
package.  CPU only (no kernel runs); skipped when catopt is not importable."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(__file__))
import _catopt_path  # noqa: E402

if _catopt_path.add_catopt_to_path() is None:
    pytest.skip(_catopt_path.SKIP_REASON, allow_module_level=True)

# a source checkout (not just an install) also carries the reference's own test helpers
_REF = os.environ.get("CATOPT_SRC") or os.path.join(os.path.dirname(__file__), "..", "..", "reference")

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402
from catopt_core.ir import IR, Op, Param, TensorType, Var  # noqa: E402
from catopt_core.ports import BatchedExecutor, ExecutorSpec  # noqa: E402

from catopt_b200 import sink as b200  # noqa: E402


def _route(sink, term):
    for spec in sink.executors.values():
        if spec.carrier is not None and spec.accepts(term):
            return spec
    return None


def test_b200_specs_come_first_and_are_executor_specs():
    s = b200.B200Sink()
    names = list(s.executors)
    assert names[:8] == ["b200_om_decayed_chunked", "b200_om_decayed_pairwise", "b200_om_causal",
                         "b200_om_streaming", "b200_scan_all", "b200_scan", "b200_omd", "b200_linear_chain"]
    assert "om_decayed_chunked" in names and names[-1] == "generic"
    assert all(isinstance(v, ExecutorSpec) for v in s.executors.values())


@pytest.mark.parametrize("per_head", [True, False])
def test_uniform_chunked_term_routes_to_b200(per_head):
    chunked, quad = make_golden._decayed_terms(2, 4, 64, 16, 16, per_head, 2.0)
    s = b200.B200Sink()
    assert _route(s, chunked.root).name == "b200_om_decayed_chunked"
    plan = b200.decayed_state_carry_plan(chunked.root)
    assert plan["chunk"] == 16 and plan["n"] == 4 and plan["scale"] == 2.0
    assert [getattr(plan[k], "name", None) for k in "qkv"] == ["q", "k", "v"]
    assert getattr(plan["gamma"], "name", None) == "g"
    # the spelled quadratic term is not ours (and not the reference executor's either)
    assert b200.decayed_state_carry_plan(quad.root) is None


def test_non_state_carry_variants_go_to_the_pairwise_spec():
    """Terms the reference's pairwise executor accepts but that are not the
    uniform state-carry form are declined by the state-carry spec and taken by
    the pairwise one (the reference's module with its intra element in the
    gated-contraction kernel), ahead of the reference's own spec."""
    chunked, _ = make_golden._decayed_terms(1, 2, 48, 8, 16, True, 1.0)
    arms = list(chunked.root.args)
    # drop one cross summand from the last arm: pair (2,0) is missing
    last = arms[-1]
    assert last.op == "add"
    broken = Op.make("concat", *arms[:-1], last.args[0], dim=-2)
    s = b200.B200Sink()
    assert b200.decayed_state_carry_plan(broken) is None
    assert _route(s, broken).name == "b200_om_decayed_pairwise"
    assert s.executors["om_decayed_chunked"].accepts(broken)


@pytest.mark.parametrize("kw", [dict(intra_row=True), dict(second_rate=True), dict(drop_pair=True),
                                dict(intra_row=True, second_rate=True)])
def test_row_gated_and_two_rate_arms_route_to_the_pairwise_spec(kw):
    """The variants of the reference's own executor tests (tests/test_decayed_lower.py:440-482
    there): a decay-row gate on the intra element, a second rate in the later arms' masks, a
    missing cross pair.  None is decayed attention at one rate, so the state-carry plans decline
    them; the pairwise spec lowers them to the reference's module with the B200 intra element,
    which refuses host tensors like every other B200 module."""
    from catopt_b200 import B200Error
    from decayed_variants import variant_term

    ir = variant_term(2, 3, 48, 8, 16, 2.0, **kw)
    s = b200.B200Sink()
    assert b200.decayed_plan(ir.root) is None
    spec = _route(s, ir.root)
    assert spec.name == "b200_om_decayed_pairwise"
    pv = {"g": torch.tensor([0.9, 0.95, 0.8]), "g2": torch.tensor([0.7, 0.85, 0.99])}
    mod = spec.lower(ir, {n: pv[n] for n in ir.params})
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod) and mod.n_blocks == 3
    q, k, v = (torch.randn(2, 3, 48, 8) for _ in range(3))
    with pytest.raises(B200Error):
        mod(q, k, v)
    # the plain uniform term and the gate written inside the division keep the state-carry spec
    assert _route(s, variant_term(2, 3, 48, 8, 16, 2.0).root).name == "b200_om_decayed_chunked"
    assert _route(s, variant_term(2, 3, 48, 8, 16, 2.0, gate_inside=True).root).name == "b200_om_decayed_chunked"


def test_lowered_module_conforms_to_ports_and_refuses_cpu():
    chunked, _ = make_golden._decayed_terms(1, 2, 32, 8, 16, True, 1.0)
    s = b200.B200Sink()
    spec = s.executors["b200_om_decayed_chunked"]
    mod = spec.lower(chunked, {"g": torch.tensor([0.9, 0.95])})
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod)
    assert mod.n_blocks == 2 and not mod.is_graph_captured
    q = torch.randn(1, 2, 32, 8)
    from catopt_b200 import B200Error

    with pytest.raises(B200Error):  # no CPU fallback: the kernel path refuses host tensors
        mod(q, q, q)
    with pytest.raises(ValueError):
        mod.capture_cuda_graph(q, q, q)


def test_linear_chain_plan_on_the_extracted_form():
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    x = Var("input", tt(4, 8))
    ws = [Param(f"p_{i}_weight", tt(8, 8)) for i in range(4)]
    tree = ws[0]
    for w in ws[1:]:
        tree = Op.make("matmul", w, tree)          # W3 @ (W2 @ (W1 @ W0))
    root = Op.make("linear", x, tree)
    plan = b200.linear_chain_plan(root)
    assert plan is not None and plan["bias"] is None
    assert [p.name for p in b200._right_nested_chain(plan["weight_tree"])] == [w.name for w in ws]
    s = b200.B200Sink()
    assert _route(s, root).name == "b200_linear_chain"
    # a plain linear with a single weight is left to the generic module
    assert b200.linear_chain_plan(Op.make("linear", x, ws[0])) is None
    assert b200.linear_chain_plan(Op.make("linear", x, Op.make("matmul", x, ws[0]))) is None


def test_non_matching_ir_degrades_to_eval_mod():
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    x = Var("x", tt(2, 3))
    ir = IR(root=Op.make("add", x, x), inputs=[x], input_names={"x"}, params={})
    mod = b200.B200ChunkedDecayModule(ir, None)
    assert not mod.is_batched and mod.n_blocks == 0
    t = torch.ones(2, 3)
    assert torch.equal(mod(t), t + t)


def _scan_term(T=6, d=8):
    """applyd(affd_compose(... aff_diag(a_t, select(u, 0, t)) ...), h) over T steps."""
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    u = Var("u", tt(T, d))
    a = Param("a", tt(d))
    h = Param("h0", tt(d))
    leaf = lambda t: Op.make("aff_diag", a, Op.make("select", u, dim=0, index=t))  # noqa: E731
    tree = leaf(T - 1)                      # latest step outermost
    for t in range(T - 2, -1, -1):
        tree = Op.make("affd_compose", tree, leaf(t))
    root = Op.make("applyd", tree, h)
    ir = IR(root=root, inputs=[u], input_names={"u"}, params={"a": a, "h0": h})
    return ir


def test_scan_term_routes_to_b200_scan_and_keeps_reference_plan():
    ir = _scan_term()
    s = b200.B200Sink()
    assert "b200_scan" in list(s.executors)[:6]
    spec = _route(s, ir.root)
    assert spec.name == "b200_scan"
    vals = {"a": torch.full((8,), 0.9), "h0": torch.ones(8)}
    mod = spec.lower(ir, vals)
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod) and mod._plan["diagonal"]
    from catopt_b200 import B200Error

    with pytest.raises(B200Error):      # the kernel path refuses host tensors
        mod(torch.randn(6, 8))


def test_b200_target_profile_prices_with_the_reference_cost_model():
    prof = b200.b200_target_profile()
    assert prof.gbps > 6000 and prof.tflops > 50 and prof.name.startswith("b200")
    cost = prof.cost_fn()
    assert callable(cost)


def test_b200_target_profile_carries_measurements_where_the_cost_model_reads_them():
    """The executor times sit in ``op_kernel_ns`` / ``measured_ns`` (not in free-form notes):
    the roofline's measured-kernel floor finds config 1's GEMM, and the autotuner's price lookup
    finds every B200 executor under its shape bucket."""
    from catopt_core.cost.roofline import _kernel_lookup
    from catopt_core.profile import corrected_price_ns, measured_price_ns, shape_bucket

    prof = b200.b200_target_profile()
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    lin = Op.make("linear", Var("input", tt(64, 512)), Param("fused_14", tt(512, 512)))
    kns = _kernel_lookup(prof.op_kernel_ns)
    assert kns is not None and kns(lin, {}) == prof.op_kernel_ns["matmul"]["64x512x512"] > 0
    names = set(prof.measured_ns)
    assert {"b200_om_decayed_chunked", "b200_linear_chain", "b200_scan_all", "b200_scan", "b200_omd",
            "b200_om_causal", "b200_om_streaming"} <= names
    assert names <= set(b200.B200Sink().executors)           # every candidate name is a spec of the sink
    bucket = shape_bucket(torch.empty(64, 512))
    assert bucket.endswith("2^15")
    cuda_bucket = "cuda:0:2^15"
    want = prof.measured_ns["b200_linear_chain"][cuda_bucket]["median_ns"]
    assert measured_price_ns(prof, "b200_linear_chain", cuda_bucket, None) == want
    assert corrected_price_ns(prof, "b200_linear_chain", cuda_bucket, None) == want
    assert not prof.meta.get("executors_us")                 # nothing left in free-form notes


# --------------------------------------------------------------------------- ragged partitions
def _ragged_term(T, d, arms, sources, scale=2.0, nested=False, per_head=False, B=2, H=2):
    """Hand-built chunked decayed term over a non-uniform partition.

    ``arms``: row counts of the output pieces; ``sources[i]``: row counts of the
    source blocks arm i reaches back to (they must add up to the arm's start).
    Slices are written as ``split`` with whichever size tuple names the range —
    the fine partition for arms, a coarse (start, len, rest) one for sources — and
    optionally as a split of a split, as saturation leaves them."""
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    q, k, v = (Var(n, tt(B, H, T, d)) for n in "qkv")
    g = Param("g", tt(H)) if per_head else Param("g", tt())
    kT = Op.make("transpose", k, dim0=-1, dim1=-2)

    def piece(base, dim, start, length):
        sizes = tuple(z for z in (start, length, T - start - length) if z > 0)
        idx = 1 if start > 0 else 0
        if nested and length % 2 == 0 and start == 0 and length < T:
            # first half-open range expressed as split(split(base, [2*length, rest]), [length, length])
            outer = tuple(z for z in (2 * length, T - 2 * length) if z > 0)
            if sum(outer) == T and 2 * length <= T:
                return Op.make("split", Op.make("split", base, dim=dim, index=0, sizes=outer),
                               dim=dim, index=0, sizes=(length, length))
        return Op.make("split", base, dim=dim, index=idx, sizes=sizes)

    def fine(base, dim, i):
        return Op.make("split", base, dim=dim, index=i, sizes=tuple(arms))

    c = Const(scale)
    out, a = [], 0
    for i, s in enumerate(arms):
        qi = fine(q, -2, i)
        t = Op.make("div", Op.make("om_decayed", Op.make("matmul", qi, fine(kT, -1, i)),
                                   Op.make("decay", g, t=s), fine(v, -2, i)), c)
        b = 0
        for l in sources[i]:
            col = Op.make("unsqueeze", Op.make("decay_vec", g, t=l, sign=-1), dim=-1)
            row = Op.make("unsqueeze", Op.make("decay_vec", g, t=s, offset=a - b), dim=-1)
            state = Op.make("matmul", Op.make("transpose", Op.make("mul", piece(k, -2, b, l), col), dim0=-1, dim1=-2),
                            piece(v, -2, b, l))
            t = Op.make("add", t, Op.make("mul", row, Op.make("div", Op.make("matmul", qi, state), c)))
            b += l
        assert b == a
        out.append(t)
        a += s
    root = out[-1]
    for t in reversed(out[:-1]):                       # right-nested concat, as extracted
        root = Op.make("concat", t, root, dim=-2)
    ir = IR(root=root, inputs=[q, k, v], input_names={"q", "k", "v"}, params={"g": g})
    return ir


from catopt_core.ir import Const  # noqa: E402

_RAGGED = [
    ((8, 8, 16, 32), [(), (8,), (8, 8), (16, 16)]),           # sources coarser than the arms
    ((32, 32, 32, 32, 128, 128, 128), [(), (32,), (32, 32), (32, 32, 32), (128,), (128, 128), (128, 128, 128)]),
    ((24, 40), [(), (24,)]),
    ((16, 16, 16), [(), (16,), (16, 16)]),                    # uniform: also legal for the ragged parser
]


@pytest.mark.parametrize("arms,sources", _RAGGED, ids=lambda z: "-".join(map(str, z)) if z and isinstance(z[0], int) else None)
@pytest.mark.parametrize("nested", [False, True])
def test_ragged_partition_is_recognised_and_equals_whole_sequence_attention(arms, sources, nested):
    from catopt_torch.torch_bridge import IRModule
    from oracle import oracle

    T, d = sum(arms), 8
    ir = _ragged_term(T, d, arms, sources, scale=2.0, nested=nested)
    plan = b200.decayed_ragged_plan(ir.root)
    assert plan is not None and plan["sizes"] == tuple(arms) and plan["scale"] == 2.0
    assert [getattr(plan[n], "name", None) for n in "qkv"] == ["q", "k", "v"] and plan["gamma"].name == "g"
    s = b200.B200Sink()
    assert _route(s, ir.root).name == "b200_om_decayed_chunked"
    # the recognised term really is decayed attention of the whole sequence (reference bindings, fp64)
    gen = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(2, 2, T, d, dtype=torch.float64, generator=gen) / 3 for _ in range(3))
    g = torch.tensor(0.93, dtype=torch.float64)
    with torch.no_grad():
        want = IRModule(ir, {"g": g})(q, k, v)
    got = oracle.decayed_quadratic(q, k, v, g, 2.0)
    assert (want - got).abs().max().item() < 1e-12


def _mutate(ir, fn):
    """Rebuild the term bottom-up, letting ``fn(op_node)`` replace nodes."""
    def walk(t):
        if not isinstance(t, Op):
            return t
        new = Op.make(t.op, *[walk(a) for a in t.args], **dict(t.attrs))
        return fn(new)
    return walk(ir.root)


def test_ragged_lookalikes_are_declined():
    arms, sources = _RAGGED[0]
    ir = _ragged_term(sum(arms), 8, arms, sources)
    assert b200.decayed_ragged_plan(ir.root) is not None

    def bump_offset(n):   # one row gate off by one
        if n.op == "decay_vec" and n.attrs.get("offset") == 16 and n.attrs.get("t") == 16:
            return Op.make("decay_vec", *n.args, t=16, offset=17)
        return n

    def flip_sign(n):     # a column gate with the wrong sign
        if n.op == "decay_vec" and n.attrs.get("sign") == -1 and n.attrs.get("t") == 16:
            return Op.make("decay_vec", *n.args, t=16, sign=1)
        return n

    def other_scale(n):   # one summand divided by a different constant
        if n.op == "div" and isinstance(n.args[0], Op) and n.args[0].op == "om_decayed" \
                and n.args[0].args[1].attrs.get("t") == 32:
            return Op.make("div", n.args[0], Const(3.0))
        return n

    def wrong_decay_len(n):
        if n.op == "decay" and n.attrs.get("t") == 32:
            return Op.make("decay", *n.args, t=16)
        return n

    for fn in (bump_offset, flip_sign, other_scale, wrong_decay_len):
        bad = _mutate(ir, fn)
        assert bad != ir.root
        assert b200.decayed_ragged_plan(bad) is None, fn.__name__
    # a source block missing (gap in [0, a)) and arms in the wrong order
    gap = _ragged_term(64, 8, arms, [(), (8,), (8, 8), (16, 16)]).root
    last_arm = gap.args[1].args[1].args[1]
    assert last_arm.op == "add"
    broken = Op.make("concat", gap.args[0], Op.make("concat", gap.args[1].args[0],
                     Op.make("concat", gap.args[1].args[1].args[0], last_arm.args[0], dim=-2), dim=-2), dim=-2)
    assert b200.decayed_ragged_plan(broken) is None
    swapped = Op.make("concat", gap.args[1].args[0], Op.make("concat", gap.args[0], gap.args[1].args[1], dim=-2), dim=-2)
    assert b200.decayed_ragged_plan(swapped) is None


def test_kernel_chunk_choice():
    from catopt_b200.executors import kernel_chunk

    assert kernel_chunk(512, None) == 128 and kernel_chunk(512, 64) == 64
    assert kernel_chunk(96, None) == 96 and kernel_chunk(320, None) == 80
    assert kernel_chunk(1021, None) is None and kernel_chunk(61, None) == 61


def test_real_extraction_of_the_kway_carrier_routes_to_b200():
    """Saturate the export of a decay-masked attention module with the K-way law
    the way the reference's own delivery test does
    (tests/test_om_decayed_kway_deliver.py:72-103) and check that what extraction
    returns — a nested concat over a ragged partition, declined by the
    reference's executor — is routed to the B200 executor."""
    from catopt_carriers.decayed_lower import build_decayed_plan
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
            pos = torch.arange(t, dtype=x.dtype)
            decay = torch.tril(torch.pow(torch.tensor(0.9, dtype=x.dtype),
                                         (pos.unsqueeze(1) - pos.unsqueeze(0)).clamp_min(0)))
            return ((self.q(x) @ self.k(x).transpose(-1, -2) / (t ** 0.5)) * decay) @ self.v(x)

    torch.manual_seed(0)
    kk, T = 2, 256
    rules = (list(OM_LAWS) + list(OM_CHUNKIFY) + list(tl.SPLIT_SCALAR_RULES)
             + [tl.MUL_DIV_SWAP, tl.MATMUL_DIV_DISTRIBUTE, tl.ASSOC_MATMUL_REV, tl.FACTOR_MUL, tl.FACTOR_MUL_ADD,
                tl.DIV_ADD_FACTOR] + om_kway_laws(kk))
    model = Retention(16).double()
    x = torch.randn(2, T, 16, dtype=torch.float64)
    ir, leaves = TorchSource().to_ir(model, x)
    eg = EGraph()
    root = eg.add_term(ir.root)
    eg.run(rules, root, max_iterations=16, max_nodes=200_000, patience=8,
           rule_budgets={"om_decayed_chunkify_rows": 60, "om_decayed_chunkify_keys": 60,
                         f"om_decayed_kway_blocks_{kk}": 200})
    best = eg.extract_best(eg.find(root), flops_cost)
    assert best.op == "concat"
    plan = b200.decayed_plan(best)
    assert plan is not None and sum(plan["sizes"] if "sizes" in plan else [plan["chunk"]] * plan["n"]) == T
    assert _route(b200.B200Sink(), best).name == "b200_om_decayed_chunked"
    if build_decayed_plan(best) is None:       # the partition was ragged: only the B200 spec takes it
        assert len(set(plan["sizes"])) > 1
    # the three bases are the projections of the one input, gamma the lifted constant
    assert all(getattr(plan[n], "op", None) == "linear" for n in "qkv")
    # what the module would hand to the kernel reproduces the source model (fp64, CPU oracle)
    from oracle import oracle

    ex_ir = IR(root=best, inputs=list(ir.inputs), input_names=set(ir.input_names), params=dict(ir.params))
    mod = b200.B200ChunkedDecayModule(ex_ir, leaves)
    assert mod.is_batched and mod.n_blocks == plan["n"]
    with torch.no_grad():
        ev = mod._ev((x,))
        mp = mod._plan          # built from the module's own (constant-folded) root
        q, k, v, g = (ev(mp[n]) for n in ("q", "k", "v", "gamma"))
        want = model(x)
    got = oracle.decayed_quadratic(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), g.reshape(()), plan["scale"])[0]
    assert (got - want).abs().max().item() < 1e-10


# --------------------------------------------------------------------------- om causal carrier
def _om_causal_term(ksizes, Tq, d=4, dv=6, batch=(2, 3), scale=0.5, right_nested=True, off=None):
    """Hand-built carrier of causal attention over key blocks, in the form the
    sdpa-over-concat laws produce."""
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    q = Var("q", tt(*batch, Tq, d))
    ks = [Var(f"k{i}", tt(*batch, n, d)) for i, n in enumerate(ksizes)]
    vs = [Var(f"v{i}", tt(*batch, n, dv)) for i, n in enumerate(ksizes)]

    def scores(k):
        return Op.make("om_decayed", q, Op.make("fill", q, value=scale), Op.make("transpose", k, dim0=-2, dim1=-1))

    kall = ks[0]
    for k in ks[1:]:
        kall = Op.make("concat", kall, k, dim=-2)
    cm = Op.make("cmask", scores(kall)) if off is None else Op.make("cmask", scores(kall), off=off)
    rank = len(batch) + 2
    leaves = [Op.make("om_elem", Op.make("masked_fill", scores(k), Op.make("split", cm, dim=rank - 1, index=i,
                                                                         sizes=tuple(ksizes)), Const(float("-inf"))), v)
              for i, (k, v) in enumerate(zip(ks, vs))]
    if right_nested:
        tree = leaves[-1]
        for lf in reversed(leaves[:-1]):
            tree = Op.make("om_compose", lf, tree)
    else:
        tree = leaves[0]
        for lf in leaves[1:]:
            tree = Op.make("om_compose", tree, lf)
    inputs = [q, *ks, *vs]
    return IR(root=Op.make("om_apply", tree), inputs=inputs, input_names={v.name for v in inputs}, params={}), leaves


@pytest.mark.parametrize("ksizes,Tq", [((4, 4, 4), 12), ((3, 6), 5), ((1, 8), 9), ((2, 3, 4), 1)])
@pytest.mark.parametrize("right_nested", [True, False])
def test_om_causal_carrier_is_recognised_and_means_causal_attention(ksizes, Tq, right_nested):
    import torch.nn.functional as F
    from catopt_torch.torch_bridge import IRModule

    ir, _ = _om_causal_term(ksizes, Tq, right_nested=right_nested)
    plan = b200.om_causal_plan(ir.root)
    assert plan is not None and plan["sizes"] == tuple(ksizes) and plan["scale"] == 0.5 and plan["causal"]
    assert plan["q"].name == "q" and [k.name for k in plan["k_blocks"]] == [f"k{i}" for i in range(len(ksizes))]
    assert [v.name for v in plan["v_blocks"]] == [f"v{i}" for i in range(len(ksizes))]
    assert _route(b200.B200Sink(), ir.root).name == "b200_om_causal"
    # the hand-built term evaluates (reference bindings, fp64) to torch's causal attention
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(2, 3, Tq, 4, dtype=torch.float64, generator=gen)
    ks = [torch.randn(2, 3, n, 4, dtype=torch.float64, generator=gen) for n in ksizes]
    vs = [torch.randn(2, 3, n, 6, dtype=torch.float64, generator=gen) for n in ksizes]
    with torch.no_grad():
        got = IRModule(ir, None)(q, *ks, *vs)
    want = F.scaled_dot_product_attention(q, torch.cat(ks, -2), torch.cat(vs, -2), is_causal=True, scale=0.5)
    assert (got - want).abs().max().item() < 1e-12
    # and the oracle the GPU kernel is tested against agrees on the joined blocks
    from oracle import oracle

    o = oracle.om_causal_chunked(q, torch.cat(ks, -2), torch.cat(vs, -2), list(ksizes), 0.5)
    assert (o - want).abs().max().item() < 1e-12


def test_om_causal_lookalikes_are_declined():
    ir, leaves = _om_causal_term((4, 4, 4), 12)
    s = b200.B200Sink()
    # masks in the wrong order, a duplicated block, an offset mask, an unmasked carrier
    a, b_, c = leaves
    assert b200.om_causal_plan(Op.make("om_apply", Op.make("om_compose", b_, Op.make("om_compose", a, c)))) is None
    assert b200.om_causal_plan(Op.make("om_apply", Op.make("om_compose", a, Op.make("om_compose", a, c)))) is None
    assert b200.om_causal_plan(Op.make("om_apply", Op.make("om_compose", a, b_))) is None      # keys 8..12 missing
    shifted, _ = _om_causal_term((4, 4, 4), 12, off=1)
    ps = b200.om_causal_plan(shifted.root)       # a shifted causal mask is taken, with its offset
    assert ps is not None and ps["off"] == 1 and ps["causal"]
    assert b200.om_causal_plan(_om_causal_term((4, 4, 4), 12)[0].root)["off"] == 0
    plain = Op.make("om_apply", Op.make("om_compose", *[Op.make("om_elem", lf.args[0].args[0], lf.args[1])
                                                         for lf in leaves[:2]]))
    pp = b200.om_causal_plan(plain)              # the unmasked carrier is plain softmax attention
    assert pp is not None and pp["causal"] is False and pp["sizes"] == (4, 4)
    mixed = Op.make("om_apply", Op.make("om_compose", a, Op.make("om_elem", b_.args[0].args[0], b_.args[1])))
    assert b200.om_causal_plan(mixed) is None    # one masked and one unmasked leaf: not ours
    assert _route(s, mixed).name in ("om_batched", "om_streaming")
    # different scale on one block
    other, ol = _om_causal_term((4, 4, 4), 12, scale=0.25)
    assert b200.om_causal_plan(Op.make("om_apply", Op.make("om_compose", a, Op.make("om_compose", ol[1], c)))) is None


def test_om_causal_module_conforms_and_refuses_cpu():
    ir, _ = _om_causal_term((4, 4), 8)
    spec = b200.B200Sink().executors["b200_om_causal"]
    mod = spec.lower(ir, None)
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod) and mod.n_blocks == 2
    sspec = b200.B200Sink().executors["b200_om_streaming"]
    assert sspec.engaged(sspec.lower(ir, None)) and mod.is_streaming
    from catopt_b200 import B200Error

    q = torch.randn(2, 3, 8, 4)
    ks = [torch.randn(2, 3, 4, 4) for _ in range(2)]
    vs = [torch.randn(2, 3, 4, 6) for _ in range(2)]
    with pytest.raises(B200Error):
        mod(q, *ks, *vs)


def test_om_causal_real_saturation_member_is_accepted():
    """Saturate sdpa(q, cat k, cat v, is_causal) with the reference's om laws
    and force-extract the chunked carrier with the reference's own test helper
    (tests/test_om_causal.py:128-160 there); the B200 spec must take it."""
    import importlib.util

    path = os.path.join(_REF, "tests", "test_om_causal.py")
    if not os.path.exists(path):
        pytest.skip("reference test helpers not available")
    spec = importlib.util.spec_from_file_location("_ref_test_om_causal", path)
    helper = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(helper)
    for ksizes, kw in (((3, 6), {}), ((2, 3, 4), {}), ((2, 5), {"batch": (2, 3)}), ((3, 6), {"scale": 0.25})):
        _, term, _, _, _ = helper._causal_chunked_ok(list(ksizes), **kw)
        plan = b200.om_causal_plan(term)
        assert plan is not None and plan["sizes"] == tuple(ksizes), (ksizes, kw)
        assert _route(b200.B200Sink(), term).name == "b200_om_causal"
    # the unmasked companion carrier is taken as plain softmax attention
    _, term, _, _, _ = helper._causal_chunked_ok([3, 6], causal=False)
    plan = b200.om_causal_plan(term)
    assert plan is not None and plan["causal"] is False and plan["sizes"] == (3, 6)


def _om_masked_term(ksizes, Tq, d=4, dv=6, batch=(2, 3), scale=0.5, one_leaf=False, mask_shape=None):
    """The carrier the reference's masked sdpa law leaves (catopt_carriers/om.py:1313-1362): one
    ``om_elem`` over the concatenated scores plus ``attnbias(m)``, or its chunked form with the
    bias sliced per key block."""
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    q = Var("q", tt(*batch, Tq, d))
    ks = [Var(f"k{i}", tt(*batch, n, d)) for i, n in enumerate(ksizes)]
    vs = [Var(f"v{i}", tt(*batch, n, dv)) for i, n in enumerate(ksizes)]
    mask_shape = mask_shape or (Tq, sum(ksizes))
    m = Var("m", tt(*mask_shape))
    bias = Op.make("attnbias", m)
    rank = len(mask_shape)                     # the mask is sliced along ITS key axis
    if one_leaf:
        qs = Op.make("mul", q, Op.make("fill", q, value=scale))
        sc = Op.make("concat", *(Op.make("matmul", qs, Op.make("transpose", k, dim0=-2, dim1=-1)) for k in ks), dim=-1)
        tree = Op.make("om_elem", Op.make("add", sc, bias), Op.make("concat", *vs, dim=-2))
    else:
        def scores(k):
            return Op.make("om_decayed", q, Op.make("fill", q, value=scale), Op.make("transpose", k, dim0=-2, dim1=-1))

        leaves = [Op.make("om_elem", Op.make("add", scores(k), Op.make("split", bias, dim=rank - 1, index=i,
                                                                       sizes=tuple(ksizes))), v)
                  for i, (k, v) in enumerate(zip(ks, vs))]
        tree = leaves[-1]
        for lf in reversed(leaves[:-1]):
            tree = Op.make("om_compose", lf, tree)
    inputs = [q, *ks, *vs, m]
    return IR(root=Op.make("om_apply", tree), inputs=inputs, input_names={v.name for v in inputs}, params={})


@pytest.mark.parametrize("one_leaf", [False, True])
def test_om_carrier_with_an_explicit_mask_is_recognised_and_means_masked_attention(one_leaf):
    import torch.nn.functional as F
    from catopt_torch.torch_bridge import IRModule

    ksizes, Tq = (3, 6), 5
    ir = _om_masked_term(ksizes, Tq, one_leaf=one_leaf)
    plan = b200.om_causal_plan(ir.root)
    assert plan is not None and plan["sizes"] == ksizes and plan["scale"] == 0.5 and not plan["causal"]
    assert plan["bias"].name == "m" and [k.name for k in plan["k_blocks"]] == ["k0", "k1"]
    spec = _route(b200.B200Sink(), ir.root)
    assert spec.name == "b200_om_causal"
    mod = spec.lower(ir, None)
    assert mod.is_batched and mod.is_streaming
    # the term evaluates (reference bindings, fp64) to torch's masked attention, bool and float masks alike
    gen = torch.Generator().manual_seed(4)
    q = torch.randn(2, 3, Tq, 4, dtype=torch.float64, generator=gen)
    ks = [torch.randn(2, 3, n, 4, dtype=torch.float64, generator=gen) for n in ksizes]
    vs = [torch.randn(2, 3, n, 6, dtype=torch.float64, generator=gen) for n in ksizes]
    keep = torch.rand(Tq, 9, generator=gen) < 0.6
    keep[:, 0] = True
    for m in (keep, torch.randn(Tq, 9, dtype=torch.float64, generator=gen)):
        with torch.no_grad():
            got = IRModule(ir, None)(q, *ks, *vs, m)
        want = F.scaled_dot_product_attention(q, torch.cat(ks, -2), torch.cat(vs, -2), attn_mask=m, scale=0.5)
        assert (got - want).abs().max().item() < 1e-12
    with pytest.raises(b200.B200Error):                   # no CPU fallback inside the executor
        mod(q.float(), *(t.float() for t in ks), *(t.float() for t in vs), keep)


def test_om_masked_lookalikes_are_declined():
    ir = _om_masked_term((4, 4, 4), 12)
    a, b_, c = b200._flatten(ir.root.args[0], "om_compose")
    mk = lambda *ls: Op.make("om_apply", Op.make("om_compose", ls[0], Op.make("om_compose", *ls[1:])))  # noqa: E731
    assert b200.om_causal_plan(mk(a, b_, c)) is not None
    assert b200.om_causal_plan(mk(b_, a, c)) is None                    # mask columns out of key order
    other = _om_masked_term((4, 4, 4), 12, mask_shape=(1, 12))
    o_leaves = b200._flatten(other.root.args[0], "om_compose")
    # (same spelling, so the pieces are equal terms; a second mask needs another variable)
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    m2 = Op.make("attnbias", Var("m2", tt(12, 12)))
    sterm = o_leaves[1].args[0]
    swapped = Op.make("om_elem", Op.make("add", sterm.args[0], Op.make("split", m2, dim=1, index=1, sizes=(4, 4, 4))),
                      o_leaves[1].args[1])
    assert b200.om_causal_plan(mk(a, swapped, c)) is None               # two different masks
    plain = _om_causal_term((4, 4, 4), 12)[1]
    assert b200.om_causal_plan(mk(a, plain[1], c)) is None              # a masked and a causal leaf
    both = Op.make("om_elem", Op.make("masked_fill", a.args[0], plain[0].args[0].args[1], Const(float("-inf"))), a.args[1])
    assert b200.om_causal_plan(mk(both, b_, c)) is None                 # cmask and an explicit mask together


def test_om_masked_real_saturation_members_are_accepted():
    """Saturate sdpa(q, cat k, cat v, attn_mask) with the reference's om laws and extract the chunked
    carrier with the reference's own test helper (tests/test_mask_chunk.py there): additive 0/-inf
    masks, finite biases, bool keep-masks, three uneven blocks, a (B,1,T,K) mask over heads."""
    import importlib.util

    path = os.path.join(_REF, "tests", "test_mask_chunk.py")
    if not os.path.exists(path):
        pytest.skip("reference test helpers not available")
    spec = importlib.util.spec_from_file_location("_ref_test_mask_chunk", path)
    helper = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(helper)

    def head_mask(T, K):
        return torch.where(torch.rand(2, 1, T, K) < 0.35, torch.tensor(float("-inf"), dtype=torch.float64),
                           torch.zeros(2, 1, T, K, dtype=torch.float64))

    for ksizes, fn, kw in (((3, 6), helper._addmask_fn(), {}), ((2, 3, 4), helper._boolmask_fn, {}),
                           ((3, 6), helper._finite_bias_fn, {"spelling": "kwarg", "scale": 0.5}),
                           ((1, 8), helper._addmask_fn(), {}), ((2, 5), head_mask, {"batch": (2, 3)})):
        _, term, _, _, _ = helper._mask_chunked_ok(list(ksizes), fn, **kw)
        plan = b200.om_causal_plan(term)
        assert plan is not None and plan["sizes"] == tuple(ksizes) and not plan["causal"], (ksizes, kw)
        assert plan["bias"] is not None and plan["bias"].name == "m"
        assert _route(b200.B200Sink(), term).name == "b200_om_causal"


# --------------------------------------------------------------------------- omd: prefix-scan hook
def _omd_chain_term(T=8, Tq=3, d=4):
    """omd_apply(omd_elem(s, stack(affd_a f_i), stack(affd_b f_i)), h) over the shared
    prefix chain f_i = affd_compose(aff_diag(a[i], x[i]), f_{i-1}) — the form an
    unrolled scan under softmax attention extracts to (reference tests/test_omd_lower.py:52-75)."""
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    a_p, x_v = Param("p_a", tt(T, d)), Var("x", tt(T, d))
    s, h = Param("s", tt(Tq, T)), Param("h", tt(d))
    leaves = [Op.make("aff_diag", Op.make("select", a_p, dim=0, index=t), Op.make("select", x_v, dim=0, index=t))
              for t in range(T)]
    fs = [leaves[0]]
    for t in range(1, T):
        fs.append(Op.make("affd_compose", leaves[t], fs[-1]))
    a_map = Op.make("stack", *(Op.make("affd_a", f) for f in fs), dim=0)
    b_map = Op.make("stack", *(Op.make("affd_b", f) for f in fs), dim=0)
    root = Op.make("omd_apply", Op.make("omd_elem", s, a_map, b_map), h)
    return IR(root=root, inputs=[x_v], input_names={"x"}, params={"p_a": a_p, "s": s, "h": h})


def test_omd_term_routes_to_b200_omd_and_keeps_reference_plan():
    ir = _omd_chain_term()
    s = b200.B200Sink()
    spec = _route(s, ir.root)
    assert spec.name == "b200_omd"
    vals = {"p_a": torch.rand(8, 4) * 0.5 + 0.5, "s": torch.randn(3, 8), "h": torch.randn(4)}
    mod = spec.lower(ir, vals)
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod)
    assert mod._plan["map_mode"] == "chain"          # the all-prefix scan is what runs
    from catopt_b200 import B200Error

    with pytest.raises(B200Error):                   # the prefix scan refuses host tensors
        mod(torch.randn(8, 4))
    # dense maps and single-step sequences stay with the reference's own scan
    A, B = torch.rand(5, 3, 3), torch.rand(5, 3)
    pa, pb = mod._prefix_scan(A, B, "dense")
    assert pa.shape == (5, 3, 3) and pb.shape == (5, 3) and mod.kernel_calls == 0


def test_om_causal_blocks_that_slice_one_tensor_are_not_joined():
    """Key/value blocks written as consecutive row slices of one K and one V (a
    chunked attention over resident tensors): the plan hands the whole tensors to
    the kernel instead of re-joining the slices."""
    tt = lambda *sh: TensorType(tuple(sh))  # noqa: E731
    sizes, T, d = (4, 8, 4), 16, 4
    q, k, v = Var("q", tt(2, T, d)), Var("k", tt(2, T, d)), Var("v", tt(2, T, d))
    kall = k

    def scores(kk):
        return Op.make("om_decayed", q, Op.make("fill", q, value=0.5), Op.make("transpose", kk, dim0=-2, dim1=-1))

    cm = Op.make("cmask", scores(kall))
    leaves = [Op.make("om_elem",
                      Op.make("masked_fill", scores(Op.make("split", k, dim=-2, index=i, sizes=sizes)),
                              Op.make("split", cm, dim=2, index=i, sizes=sizes), Const(float("-inf"))),
                      Op.make("split", v, dim=-2, index=i, sizes=sizes)) for i in range(3)]
    root = Op.make("om_apply", Op.make("om_compose", leaves[0], Op.make("om_compose", leaves[1], leaves[2])))
    plan = b200.om_causal_plan(root)
    assert plan is not None and plan["n"] == 3 and plan["sizes"] == sizes
    assert plan["k_blocks"] == [k] and plan["v_blocks"] == [v]


def test_ragged_recogniser_on_random_partitions():
    """Seeded random partitions: arms of random sizes, each reaching back to a random
    coarsening of the rows before it.  Every such term is decayed attention of the whole
    sequence and must be accepted with the arms' sizes; shifting any one row gate must
    be declined."""
    import random

    rnd = random.Random(20240607)
    for _ in range(25):
        n_arms = rnd.randint(2, 6)
        arms = tuple(rnd.choice((4, 8, 12, 16, 24)) for _ in range(n_arms))
        sources, start = [], 0
        for i, s in enumerate(arms):
            # random coarsening of the previous arms' boundaries
            cuts = [0]
            acc = 0
            for prev in arms[:i]:
                acc += prev
                if acc < start and rnd.random() < 0.5:
                    cuts.append(acc)
            cuts.append(start)
            sources.append(tuple(b - a for a, b in zip(cuts[:-1], cuts[1:]) if b > a))
            start += s
        ir = _ragged_term(sum(arms), 4, arms, sources, scale=1.0, nested=rnd.random() < 0.5)
        plan = b200.decayed_ragged_plan(ir.root)
        assert plan is not None and plan["sizes"] == arms, (arms, sources)
        # break it: one row gate off by one (wherever that gate occurs)
        gates = []

        def collect(n):
            if n.op == "decay_vec" and int(n.attrs.get("offset", 0) or 0) > 0:
                gates.append((n.attrs.get("t"), n.attrs.get("offset")))
            return n

        _mutate(ir, collect)
        t_bad, off_bad = rnd.choice(sorted(set(gates)))

        def bump(n):
            if n.op == "decay_vec" and n.attrs.get("t") == t_bad and n.attrs.get("offset") == off_bad:
                return Op.make("decay_vec", *n.args, t=t_bad, offset=off_bad + 1)
            return n

        bad = _mutate(ir, bump)
        assert bad != ir.root and b200.decayed_ragged_plan(bad) is None


def test_equivalent_spellings_of_the_cross_gate_are_accepted_and_other_functions_declined():
    """The spellings the reference's own executor tests vary (tests/test_decayed_lower.py:
    139-166 there): the row gate on either side of the product, or inside the division,
    is the same function and is taken; a missing gate, a row-gated intra arm or a
    second decay rate is a different function and is left to the reference's executor."""
    chunked, _ = make_golden._decayed_terms(1, 2, 48, 8, 16, True, 2.0)
    base = b200.decayed_plan(chunked.root)
    assert base is not None

    def is_gate(t):
        return isinstance(t, Op) and t.op == "unsqueeze" and isinstance(t.args[0], Op) and t.args[0].op == "decay_vec" \
            and int(t.args[0].attrs.get("sign", 1)) == 1

    def swap(n):       # mul(row, x) -> mul(x, row)
        if n.op == "mul" and len(n.args) == 2 and is_gate(n.args[0]):
            return Op.make("mul", n.args[1], n.args[0])
        return n

    def gate_inside(n):   # mul(row, div(body, c)) -> div(mul(row, body), c)
        if n.op == "mul" and len(n.args) == 2 and is_gate(n.args[0]) and isinstance(n.args[1], Op) \
                and n.args[1].op == "div":
            body, c = n.args[1].args
            return Op.make("div", Op.make("mul", n.args[0], body), c)
        return n

    for fn in (swap, gate_inside):
        variant = _mutate(chunked, fn)
        assert variant != chunked.root
        plan = b200.decayed_plan(variant)
        assert plan is not None, fn.__name__
        assert (plan["q"], plan["k"], plan["v"], plan["gamma"], plan["scale"]) == \
            (base["q"], base["k"], base["v"], base["gamma"], base["scale"])

    def drop_gate(n):     # mul(row, x) -> x : gateless cross terms are another function
        if n.op == "mul" and len(n.args) == 2 and is_gate(n.args[0]):
            return n.args[1]
        return n

    def second_rate(n):   # decay(g, t) of the later arms replaced by another parameter's
        if n.op == "decay":
            return Op.make("decay", Param("g2", n.args[0].typ), **dict(n.attrs))
        return n

    for fn in (drop_gate, second_rate):
        other = _mutate(chunked, fn)
        assert other != chunked.root and b200.decayed_plan(other) is None, fn.__name__


# --------------------------------------------------------------------------- scan, every state (stacked-map form)
def _gathered_scan_terms(readout: bool, T=5, B=2, D=8, N=4):
    """Export an unrolled diagonal scan that returns every state (or the per-step readout
    of the stacked states), saturate, and run the reference's own non-local lifts
    (machinery.py:73-103: lift_scan_to_applyd + gather_applyd_stack); returns the model,
    its inputs, the export and the term with the offered stacked-map member in place."""
    from catopt_carriers.trace_lift import lift_scan_to_applyd
    from catopt_carriers.xcarrier import gather_applyd_stack
    from catopt_core.egraph import EGraph
    from catopt_torch.regime import default_rules
    from catopt_torch.torch_bridge import export_to_ir

    class States(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Parameter(torch.rand(T, D) * 0.5 + 0.5)
            self.h0 = torch.nn.Parameter(torch.randn(D) * 0.1)

        def forward(self, x):
            h, outs = self.h0, []
            for t in range(x.shape[0]):
                h = self.a[t] * h + x[t]
                outs.append(h)
            return torch.stack(outs)

    class Readout(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.b = torch.nn.Parameter(torch.randn(D, N) / 4)
            self.c = torch.nn.Parameter(torch.randn(D, N) / 4)
            self.h0 = torch.nn.Parameter(torch.zeros(N))

        def forward(self, a, x):
            h, hs = self.h0, []
            for t in range(x.shape[1]):
                h = a[:, t] * h + self.b * x[:, t].unsqueeze(-1)
                hs.append(h)
            return (torch.stack(hs, 1) * self.c).sum(-1)

    torch.manual_seed(0)
    if readout:
        model, xs = Readout().eval().double(), (torch.rand(B, T, D, N, dtype=torch.float64) * 0.5 + 0.5,
                                                torch.randn(B, T, D, dtype=torch.float64))
    else:
        model, xs = States().eval().double(), (torch.randn(T, D, dtype=torch.float64),)
    ir, leaves = export_to_ir(model, xs if len(xs) > 1 else xs[0])
    eg = EGraph()
    root = eg.add_term(ir.root)
    eg.run(default_rules(), root, max_iterations=4, max_nodes=200_000)
    lift_scan_to_applyd(eg)
    eg.rebuild()
    offers = gather_applyd_stack(eg)
    assert len(offers) == 1
    member = offers[0]["term"]
    if readout:   # the source root with the offered member in the stack's place
        body = ir.root.args[0]
        member = Op.make("sum", Op.make("mul", *[member if getattr(z, "op", None) == "stack" else z
                                                 for z in body.args]), **dict(ir.root.attrs))
    return model, xs, ir, leaves, member


@pytest.mark.parametrize("readout", [False, True])
def test_stacked_map_form_from_the_reference_machinery_routes_to_b200_scan_all(readout):
    from catopt_torch.torch_bridge import IRModule

    from oracle import oracle

    model, xs, ir, leaves, term = _gathered_scan_terms(readout)
    s = b200.B200Sink()
    spec = _route(s, term)
    assert spec.name == "b200_scan_all"
    plan = b200.scan_states_plan(term)
    assert plan["n"] == 5 and plan["a"][0] == "gather"
    assert (plan["readout"] is not None) == readout
    ex_ir = IR(root=term, inputs=list(ir.inputs), input_names=set(ir.input_names), params=dict(ir.params))
    mod = spec.lower(ex_ir, leaves)
    assert isinstance(mod, BatchedExecutor) and spec.engaged(mod)
    from catopt_b200 import B200Error

    with pytest.raises(B200Error):
        mod(*xs)
    # the term means the source model (reference bindings), and what the module would hand to
    # the kernel reproduces it through the serial oracle
    with torch.no_grad():
        want = model(*xs)
        assert (IRModule(ex_ir, leaves)(*xs) - want).abs().max().item() < 1e-12
        ev = mod._ev(xs)
        if readout:
            a, x, b, c = ev(plan["a"][1]), ev(plan["readout"]["x"]), ev(plan["readout"]["b"]), ev(plan["readout"]["c"])
            y, _ = oracle.diag_scan_serial(a, x, b, c, ev(plan["h"]).expand(plan["state_shape"]))
            assert (y.double() - want).abs().max().item() < 1e-5        # the oracle folds in fp32
        else:
            a_rows, b_rows = mod._rows(plan["a"], ev, 5), mod._rows(plan["b"], ev, 5)
            h, hs = ev(plan["h"]), []
            for t in range(5):
                h = a_rows[t] * h + b_rows[t]
                hs.append(h)
            assert (torch.stack(hs).movedim(0, plan["stack_dim"]) - want).abs().max().item() < 1e-12


def test_stacked_map_lookalikes_are_declined():
    _, _, _, _, term = _gathered_scan_terms(False)
    fmap, h = term.args
    sa, sb = fmap.args
    # the two stacks list different maps, a step is missing from the chain, independent maps (no scan)
    swapped = Op.make("stack", *sb.args[::-1], **dict(sb.attrs))
    assert b200.scan_states_plan(Op.make("applyd", Op.make("aff_diag", sa, swapped), h)) is None
    fs = [p.args[0] for p in sa.args]
    gap = fs[:2] + fs[3:]
    mk = lambda proj: Op.make("stack", *(Op.make(proj, f) for f in gap), **dict(sa.attrs))  # noqa: E731
    assert b200.scan_states_plan(Op.make("applyd", Op.make("aff_diag", mk("affd_a"), mk("affd_b")), h)) is None
    leaves = [fs[0]] + [f.args[0] for f in fs[1:]]
    mk = lambda proj: Op.make("stack", *(Op.make(proj, f) for f in leaves), **dict(sa.attrs))  # noqa: E731
    indep = Op.make("applyd", Op.make("aff_diag", mk("affd_a"), mk("affd_b")), h)
    assert b200.scan_states_plan(indep) is None
    # and a plain scan application still goes to b200_scan
    ir = _scan_term()
    assert _route(b200.B200Sink(), ir.root).name == "b200_scan"
    assert b200.scan_states_plan(ir.root) is None
