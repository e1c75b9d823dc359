"""Routing and plan extraction of catopt_b200.sink against the real catopt
package.  CPU only (no kernel runs); skipped when catopt is not importable."""
import glob
import os
import sys

import pytest
import torch

# catopt's source tree: $CATOPT_SRC, else a "reference" checkout next to this repository
_REF = os.environ.get("CATOPT_SRC") or os.path.join(os.path.dirname(__file__), "..", "..", "reference")
for _p in glob.glob(os.path.join(_REF, "packages", "*", "src")):
    if _p not in sys.path:
        sys.path.insert(0, _p)
pytest.importorskip("catopt_core", reason="catopt source tree not available")
pytest.importorskip("catopt_carriers")

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
    assert names[:3] == ["b200_om_decayed_chunked", "b200_scan", "b200_linear_chain"]
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


def test_non_state_carry_variants_are_declined():
    """Terms the reference's pairwise executor accepts but that are not the
    uniform state-carry form fall through to the reference's own spec."""
    chunked, _ = make_golden._decayed_terms(1, 2, 48, 8, 16, True, 1.0)
    arms = list(chunked.root.args)
    # drop one cross summand from the last arm: pair (2,0) is missing
    last = arms[-1]
    assert last.op == "add"
    broken = Op.make("concat", *arms[:-1], last.args[0], dim=-2)
    s = b200.B200Sink()
    assert b200.decayed_state_carry_plan(broken) is None
    assert _route(s, broken).name == "om_decayed_chunked"


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
    assert list(s.executors)[:3] == ["b200_om_decayed_chunked", "b200_scan", "b200_linear_chain"]
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
