"""The generated-kernel seam (catopt_b200.gen).

CPU: the recognisers agree with the reference's own (``scan_spec`` / ``decayed_spec``,
read from the catopt source tree when it is there), handlers minted by the reference
get a binding, and a CPU tensor is refused loudly.  GPU (``-m gpu``): the bindings,
called the way catopt calls them (positionally, in the handler's ``args`` order),
against the spelled torch expressions; these need no catopt, the table of operand
bindings is passed in.
"""
import glob
import os
import sys

import pytest
import torch

from catopt_b200 import gen
from catopt_b200._lib import B200Error

_REF = os.environ.get("CATOPT_SRC") or os.path.join(os.path.dirname(__file__), "..", "..", "reference")
for _p in glob.glob(os.path.join(_REF, "packages", "*", "src")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

TORCH_OPS = {"mul": torch.mul, "add": torch.add, "sigmoid": torch.sigmoid, "neg": torch.neg, "exp": torch.exp}

SCAN_SPECS = [
    ("applyd", ("aff_diag", "A", "B"), "H"),
    ("applyd", ("aff_diag", ("sigmoid", "A"), ("mul", "B", "X")), "H"),
    ("applyd", ("aff_diag", "A", "B"), "H", {"axis": 0}),
    ("applyd", ("aff_diag", "A", "B"), "H", {"kind": "unrolled"}),
    ("applyd", ("affd_compose", ("aff_diag", "A2", "B2"), ("aff_diag", "A1", "B1")), "H"),
    ("applyd", ("affd_compose", ("affd_compose", ("aff_diag", "A3", "B3"), ("aff_diag", "A2", "B2")),
                ("aff_diag", "A1", "B1")), "H"),
]
NOT_SCAN = [
    ("mul", "X", "Y"),
    ("applyd", ("aff", "A", "B"), "H"),                       # dense map, not the diagonal carrier
    ("applyd", ("aff_diag", "A", "B"), ("mul", "H", "H")),    # the state must be a metavar
    ("applyd", ("aff_diag", "A", "B"), "H", {"kind": "other"}),
    ("apply", ("aff_diag", "A", "B"), "H"),
]
DECAYED_SPECS = [
    ("om_decayed", "S", "D", "V"),
    ("matmul", ("mul", "S", "D"), "V"),
    ("om_decayed", ("mul", "A", "B"), "D", "V"),
    ("om_decayed", "S", 0.5, "V"),
]
NOT_DECAYED = [
    ("add", "A", "B"),
    ("om_decayed", "S", "D"),
    ("matmul", ("add", "S", "D"), "V"),
    ("om_decayed", "S", "D", 2.0),                   # a constant value operand
    ("om_decayed", 1.0, 2.0, "V"),                   # neither scores nor gate is a tensor
    ("om_decayed", "S", "D", "V", {"scale": 2.0}),   # attrs this tier does not model
]


# --------------------------------------------------------------------------- CPU
def test_recognisers_accept_and_decline():
    for spec in SCAN_SPECS:
        assert gen.scan_site(spec) is not None, spec
    for spec in NOT_SCAN:
        assert gen.scan_site(spec) is None, spec
    for spec in DECAYED_SPECS:
        assert gen.decayed_site(spec) is not None, spec
    for spec in NOT_DECAYED:
        assert gen.decayed_site(spec) is None, spec
    seq = gen.scan_site(SCAN_SPECS[0])
    assert seq["kind"] == "seq" and seq["h"] == "H" and seq["leaves"] == [("A", "B")]
    assert gen.scan_site(SCAN_SPECS[2])["axis"] == 0
    assert gen.scan_site(SCAN_SPECS[3])["kind"] == "unrolled"
    tree = gen.scan_site(SCAN_SPECS[5])
    assert tree["kind"] == "unrolled"
    assert tree["leaves"] == [("A3", "B3"), ("A2", "B2"), ("A1", "B1")]     # product order: latest first
    spelled = gen.decayed_site(DECAYED_SPECS[1])
    assert (spelled["s"], spelled["d"], spelled["v"]) == ("S", "D", "V")


def test_recognisers_agree_with_the_reference():
    gk = pytest.importorskip("catopt_discovery.genkernel", reason="catopt source tree not available")
    for spec in SCAN_SPECS + NOT_SCAN:
        ref = gk.scan_spec(spec)
        got = gen.scan_site(spec)
        assert (ref is None) == (got is None), spec
        if ref is not None:
            assert ref["kind"] == got["kind"] and ref["h"] == got["h"], spec
            assert ref.get("axis") == got.get("axis"), spec
    for spec in DECAYED_SPECS + NOT_DECAYED:
        assert (gk.decayed_spec(spec) is None) == (gen.decayed_site(spec) is None), spec


def test_handlers_minted_by_the_reference_get_bindings():
    gk = pytest.importorskip("catopt_discovery.genkernel", reason="catopt source tree not available")
    from catopt_core.ir import Op, TensorType, Var

    def v(name, *shape):
        return Var(name, TensorType(tuple(shape)))

    a, x, h = v("a", 8, 4), v("x", 8, 4), v("h", 4)
    hs = gk.scan_handlers([Op.make("applyd", Op.make("aff_diag", a, x), h)])
    assert hs["scan_0"]["pattern"] == ("applyd", ("aff_diag", "X1", "X2"), "X3")
    assert set(gen.b200_scan_bindings(hs)) == {"scan_0_k"}
    s, d, vv = v("s", 8, 8), v("d", 8, 8), v("v", 8, 4)
    hd = gk.decayed_handlers([Op.make("om_decayed", s, d, vv), Op.make("matmul", Op.make("mul", s, d), vv)])
    assert set(gen.b200_decayed_bindings(hd)) == {h_["kernel"] for h_ in hd.values()}
    assert gen.b200_decayed_bindings({"x": {"pattern": ("add", "A", "B"), "kernel": "no", "args": ("A", "B")}}) == {}


def test_hybrid_sink_supports_the_minted_ops_and_refuses_cpu_tensors():
    pytest.importorskip("catopt_discovery.genkernel", reason="catopt source tree not available")
    from catopt_core.ir import IR, Op, TensorType, Var

    from catopt_b200.sink import B200Sink

    hs = {
        "s": {"pattern": ("applyd", ("aff_diag", "A", "B"), "H"), "kernel": "sc_hyb", "args": ("A", "B", "H")},
        "d": {"pattern": ("om_decayed", "S", "D", "V"), "kernel": "dc_hyb", "args": ("S", "D", "V")},
        "e": {"pattern": ("mul", "X1", ("relu", "X1")), "kernel": "gk_hyb", "args": ("X1",)},
    }
    sink = gen.b200_hybrid_sink(hs)
    assert isinstance(sink, B200Sink)
    assert {"sc_hyb", "dc_hyb", "gk_hyb"} <= set(sink.supported_ops)
    assert list(sink.executors)[0] == "b200_om_decayed_chunked"

    def v(name, *shape):
        return Var(name, TensorType(tuple(shape)))

    # the elementwise handler keeps the reference's spelled body (runs anywhere)
    x1 = v("x1", 5)
    mod = sink.lower(IR(root=Op.make("gk_hyb", x1), inputs=[x1], input_names={"x1"}, params={}), params={})
    xv = torch.randn(5)
    assert torch.equal(mod(xv), xv * torch.relu(xv))
    # the carrier handlers are bound to the CUDA kernels: a CPU tensor is an error, not a detour
    s, d, vv = v("s", 8, 8), v("d", 8, 8), v("v", 8, 4)
    mod = sink.lower(IR(root=Op.make("dc_hyb", s, d, vv), inputs=[s, d, vv], input_names={"s", "d", "v"},
                        params={}), params={})
    with pytest.raises(B200Error):
        mod(torch.randn(8, 8), torch.rand(8, 8), torch.randn(8, 4))


def test_bindings_refuse_cpu_tensors_without_catopt():
    b = gen.b200_gen_bindings({
        "s": {"pattern": SCAN_SPECS[0], "kernel": "k_scan", "args": ("A", "B", "H")},
        "d": {"pattern": DECAYED_SPECS[0], "kernel": "k_dec", "args": ("S", "D", "V")},
    }, bindings=TORCH_OPS)
    assert set(b) == {"k_scan", "k_dec"}
    with pytest.raises(B200Error):
        b["k_scan"](torch.rand(4, 3), torch.rand(4, 3), torch.rand(3))
    with pytest.raises(B200Error):
        b["k_dec"](torch.rand(4, 4), torch.rand(4, 4), torch.rand(4, 2))
    # a sub-spec no binding can evaluate is declined at build time
    assert gen.b200_scan_bindings({"s": {"pattern": ("applyd", ("aff_diag", ("mystery", "A"), "B"), "H"),
                                         "kernel": "k", "args": ("A", "B", "H")}}, bindings=TORCH_OPS) == {}


# --------------------------------------------------------------------------- GPU
def _spelled_scan(a, b, h, axis):
    acc = h
    for t in range(a.shape[axis]):
        acc = a.select(axis, t) * acc + b.select(axis, t)
    return acc


@pytest.mark.gpu
def test_scan_bindings_on_the_device():
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    hs = {
        "plain": {"pattern": SCAN_SPECS[0], "kernel": "k_plain", "args": ("A", "B", "H")},
        "fused": {"pattern": SCAN_SPECS[1], "kernel": "k_fused", "args": ("A", "B", "X", "H")},
        "axis0": {"pattern": SCAN_SPECS[2], "kernel": "k_axis0", "args": ("A", "B", "H")},
        "derive": {"pattern": SCAN_SPECS[0], "kernel": "k_derive", "args": ("A", "B", "H"), "axis": None},
        "tree": {"pattern": SCAN_SPECS[5], "kernel": "k_tree", "args": ("A3", "B3", "A2", "B2", "A1", "B1", "H")},
        "once": {"pattern": SCAN_SPECS[3], "kernel": "k_once", "args": ("A", "B", "H")},
    }
    b = gen.b200_scan_bindings(hs, bindings=TORCH_OPS)
    assert set(b) == {h["kernel"] for h in hs.values()}
    a = (torch.rand(3, 40, 8, generator=g) * 0.5 + 0.4).to(dev)      # (B, T, d): step axis -2
    x = torch.randn(3, 40, 8, generator=g).to(dev)
    h = torch.randn(3, 8, generator=g).to(dev)
    torch.testing.assert_close(b["k_plain"](a, x, h), _spelled_scan(a, x, h, 1), rtol=1e-5, atol=1e-5)
    # a decay shared by every step: (d,) under (B, T, d) inputs broadcasts over steps
    shared = (torch.rand(8, generator=g) * 0.5 + 0.4).to(dev)
    torch.testing.assert_close(b["k_plain"](shared, x, h), _spelled_scan(shared.expand(3, 40, 8), x, h, 1),
                               rtol=1e-5, atol=1e-5)
    # operand sub-specs are evaluated first: a = sigmoid(A), b = B*X
    raw = torch.randn(3, 40, 8, generator=g).to(dev)
    gate = torch.randn(3, 40, 8, generator=g).to(dev)
    torch.testing.assert_close(b["k_fused"](raw, gate, x, h), _spelled_scan(torch.sigmoid(raw), gate * x, h, 1),
                               rtol=1e-5, atol=1e-5)
    # declared and derived step axes: (T, d) rows with a (d,) state
    a2, x2, h2 = a[0].contiguous(), x[0].contiguous(), h[0].contiguous()
    want = _spelled_scan(a2, x2, h2, 0)
    torch.testing.assert_close(b["k_axis0"](a2, x2, h2), want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(b["k_derive"](a2, x2, h2), want, rtol=1e-5, atol=1e-5)
    with pytest.raises(RuntimeError):
        b["k_plain"](a2, a2, torch.rand(3, device=dev))             # state shape violation surfaces
    # compose tree (unrolled): f3 . f2 . f1 applied once, and the pinned single step
    leaves = [(torch.rand(8, generator=g).to(dev), torch.randn(8, generator=g).to(dev)) for _ in range(3)]
    (a3, b3), (a2_, b2_), (a1, b1) = leaves
    want = a3 * (a2_ * (a1 * h2 + b1) + b2_) + b3
    torch.testing.assert_close(b["k_tree"](a3, b3, a2_, b2_, a1, b1, h2), want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(b["k_once"](a2, x2, h2.expand(40, 8).contiguous()), a2 * h2 + x2,
                               rtol=1e-5, atol=1e-5)
    with pytest.raises(B200Error):
        b["k_plain"](a.double(), x.double(), h.double())            # fp64 is refused, not detoured


@pytest.mark.gpu
def test_decayed_bindings_on_the_device():
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(4)
    hs = {
        "el": {"pattern": DECAYED_SPECS[0], "kernel": "k_el", "args": ("S", "D", "V")},
        "sp": {"pattern": DECAYED_SPECS[1], "kernel": "k_sp", "args": ("S", "D", "V")},
        "fu": {"pattern": DECAYED_SPECS[2], "kernel": "k_fu", "args": ("A", "B", "D", "V")},
        "co": {"pattern": DECAYED_SPECS[3], "kernel": "k_co", "args": ("S", "V")},
    }
    b = gen.b200_decayed_bindings(hs, bindings=TORCH_OPS)
    assert set(b) == {"k_el", "k_sp", "k_fu", "k_co"}
    B, T, DV = 2, 24, 16
    s = torch.randn(B, T, T, generator=g).to(dev)
    d = torch.rand(T, T, generator=g).to(dev)
    v = torch.randn(B, T, DV, generator=g).to(dev)
    want = (s * d) @ v
    torch.testing.assert_close(b["k_el"](s, d, v), want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(b["k_sp"](s, d, v), want, rtol=1e-5, atol=1e-5)
    bb = torch.rand(1, T, T, generator=g).to(dev)
    torch.testing.assert_close(b["k_fu"](s, bb, d, v), ((s * bb) * d) @ v, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(b["k_co"](s, v), (s * 0.5) @ v, rtol=1e-5, atol=1e-5)
    # non-contiguous operands fold identically
    sn = torch.randn(B, T, T, generator=g).to(dev).mT
    dn = torch.rand(T, T, generator=g).to(dev).t()
    vn = torch.randn(B, DV, T, generator=g).to(dev).mT
    torch.testing.assert_close(b["k_el"](sn, dn, vn), (sn * dn) @ vn, rtol=1e-5, atol=1e-5)
    # T == 0: the empty output; K == 0: zeros; no launch either way
    got = b["k_el"](torch.randn(2, 0, 4, device=dev), torch.rand(0, 4, device=dev), torch.randn(2, 4, 8, device=dev))
    assert got.shape == (2, 0, 8)
    got = b["k_el"](torch.randn(2, 4, 0, device=dev), torch.rand(4, 0, device=dev), torch.randn(2, 0, 8, device=dev))
    assert torch.equal(got, torch.zeros(2, 4, 8, device=dev))
    # bf16 at a size the tensor-core kernel takes
    sb = torch.randn(2, 4, 256, 256, generator=g).to(dev).bfloat16()
    db = torch.rand(4, 256, 256, generator=g).to(dev).bfloat16()
    vb = torch.randn(2, 4, 256, 64, generator=g).to(dev).bfloat16()
    wantb = ((sb * db).double() @ vb.double())
    gotb = b["k_el"](sb, db, vb)
    assert gotb.dtype == torch.bfloat16
    assert ((gotb.double() - wantb).abs().max() / wantb.abs().max()).item() <= 4e-3
