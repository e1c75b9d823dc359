"""Pin the oracle: every function of oracle/oracle.py must reproduce what the
real reference produced on the same seeded inputs (tests/golden/*.npz, written
by tests/golden/make_golden.py).  CPU only."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from oracle import oracle

GOLD = Path(__file__).resolve().parent / "golden"


def _load(name):
    return np.load(GOLD / name)


# --------------------------------------------------------------------------- verify
@pytest.mark.parametrize("case", cases.verify_cases(), ids=lambda c: c[0])
def test_verify_pair_matches_reference_exactly(case):
    name, ref, out, rtol, atol = case
    want = _load("verify.npz")[name]
    rep = oracle.verify_equiv(ref, out, rtol=rtol, atol=atol)
    for got, exp in ((rep.max_abs, want[0]), (rep.max_rel, want[1])):
        assert (math.isnan(got) and math.isnan(exp)) or got == exp  # float-identical
    assert rep.passed == bool(want[2])


def test_verify_tuple_semantics():
    g = _load("verify.npz")
    cs = cases.verify_cases()
    rep = oracle.verify_equiv((cs[0][1], cs[3][1]), (cs[0][2], cs[3][2]), rtol=2e-2)
    assert [rep.max_abs, rep.max_rel, float(rep.passed), *rep.per_output] == list(g["tuple"])
    rep = oracle.verify_equiv((cs[0][1], cs[3][1]), (cs[0][2],), rtol=2e-2)
    assert rep.max_abs == math.inf and rep.max_rel == math.inf and not rep.passed


# --------------------------------------------------------------------------- decayed
@pytest.mark.parametrize("name", list(cases.DECAYED_CASES))
def test_decayed_oracle_bitwise_vs_reference(name):
    g = _load("decayed.npz")
    q, k, v, gamma, C, scale = cases.decayed_inputs(name)
    stride = cases.ROW_STRIDE.get(name, 1)
    pair = oracle.decayed_chunked_pairwise(q, k, v, gamma, C, scale)[:, :, ::stride]
    quad = oracle.decayed_quadratic(q, k, v, gamma, scale)[:, :, ::stride]
    # same torch ops in the same order as the reference's modules: bit-equal
    assert np.array_equal(pair.numpy(), g[f"{name}.chunked"])
    assert np.array_equal(quad.numpy(), g[f"{name}.quadratic"])


@pytest.mark.parametrize("name", list(cases.DECAYED_CASES))
def test_state_carry_agrees_with_reference_forms(name):
    """The recurrence the CUDA kernels implement equals the reference's
    pairwise executor up to reassociation."""
    g = _load("decayed.npz")
    q, k, v, gamma, C, scale = cases.decayed_inputs(name)
    stride = cases.ROW_STRIDE.get(name, 1)
    carry = oracle.decayed_state_carry(q, k, v, gamma, C, scale)[:, :, ::stride]
    ref = torch.from_numpy(g[f"{name}.chunked"])
    tol = 1e-12 if q.dtype == torch.float64 else 2e-6
    assert (carry - ref).abs().max().item() <= tol * max(ref.abs().max().item(), 1.0)


# --------------------------------------------------------------------------- chain
@pytest.mark.parametrize("name", list(cases.CHAIN_CASES))
def test_chain_fold_bitwise_vs_reference(name):
    g = _load("chain.npz")
    ws, x = cases.chain_inputs(name)
    wf = oracle.fold_chain(ws)
    if name == "small":
        assert np.array_equal(wf.numpy(), g["small.w_folded"])
    else:
        assert np.array_equal(wf[::16, ::16].numpy(), g["c1.w_folded_sample"])
    assert np.array_equal(oracle.linear(x, wf).numpy(), g[f"{name}.y_folded"])
    assert np.array_equal(oracle.chain_eager(x, ws).numpy(), g[f"{name}.y_eager"])


# --------------------------------------------------------------------------- scan
@pytest.mark.parametrize("name", list(cases.SCAN_CASES))
def test_scan_oracle_vs_reference_bindings(name):
    g = _load("scan.npz")
    a, x, b, c, h0 = cases.scan_inputs(name)
    y, hT = oracle.diag_scan_serial(a, x, b, c, h0)
    assert np.array_equal(y.numpy(), g[f"{name}.y"])
    assert np.array_equal(hT.numpy(), g[f"{name}.hT"])


@pytest.mark.parametrize("name", list(cases.SCAN_CASES))
def test_scan_tree_and_prefix_forms(name):
    g = _load("scan.npz")
    a, x, b, c, h0 = cases.scan_inputs(name)
    af, xf, bf, cf = a.float(), x.float(), b.float(), c.float()
    if af.dim() == 3:
        af = af.unsqueeze(-1).expand(*af.shape, bf.shape[1])
    A = af.movedim(1, 0).contiguous()
    U = (bf * xf.unsqueeze(-1)).movedim(1, 0).contiguous()
    h_init = torch.zeros_like(A[0]) if h0 is None else h0
    hT_tree = oracle.fused_diag_levels(A.flip(0), U.flip(0), h_init)
    assert np.array_equal(hT_tree.numpy(), g[f"{name}.hT_tree"])
    Pa, Pb = oracle.prefix_scan_diag(A, U)
    y_prefix = ((Pa * h_init + Pb) * cf).sum(-1).movedim(0, 1)
    assert np.array_equal(y_prefix.numpy(), g[f"{name}.y_prefix"])
    # and all three forms agree to fp32 reassociation error
    y, hT = oracle.diag_scan_serial(a, x, b, c, h0)
    assert (y - y_prefix).abs().max() <= 1e-5 * max(1.0, y.abs().max().item())
    assert (hT - hT_tree).abs().max() <= 1e-5 * max(1.0, hT.abs().max().item())


# --------------------------------------------------------------------------- om causal
@pytest.mark.parametrize("name", list(cases.OM_CAUSAL_CASES))
def test_om_causal_oracle_bitwise_vs_reference_bindings(name):
    g = _load("om_causal.npz")
    q, k, v, sizes, scale = cases.om_causal_inputs(name)
    o = oracle.om_causal_chunked(q, k, v, sizes, scale)[..., :: cases.OM_ROW_STRIDE.get(name, 1), :]
    assert np.array_equal(o.numpy(), g[f"{name}.chunked"])
    if f"{name}.sdpa" in g:
        assert np.abs(o.numpy() - g[f"{name}.sdpa"]).max() < 1e-12


def test_om_decode_row_sees_only_key_zero():
    """T_q = 1: the causal mask hides every key but key 0 (reference behaviour)."""
    q, k, v, sizes, scale = cases.om_causal_inputs("decode_row")
    o = oracle.om_causal_chunked(q, k, v, sizes, scale)
    assert torch.allclose(o[..., 0, :], v[..., 0, :], atol=1e-12)


# --------------------------------------------------------------------------- generated-kernel tier
def _from_gold(arr, dtype):
    t = torch.from_numpy(arr)
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


@pytest.mark.parametrize("name", list(cases.GATED_CASES))
def test_om_decayed_element_bitwise_vs_reference(name):
    s, gate, v = cases.gated_inputs(name)
    want = _from_gold(_load("gated.npz")[f"gated.{name}"], s.dtype)
    assert torch.equal(oracle.om_decayed(s, gate, v), want)


@pytest.mark.parametrize("name", list(cases.FOLD_CASES))
def test_seq_fold_bitwise_vs_reference(name):
    a, b, h = cases.fold_inputs(name)
    want = _from_gold(_load("gated.npz")[f"fold.{name}"], h.dtype)
    n = cases.FOLD_CASES[name][0]
    ar = a if a.dim() == h.dim() + 1 else a.expand(n, *a.shape)
    br = b if b.dim() == h.dim() + 1 else b.expand(n, *b.shape)
    assert torch.equal(oracle.seq_fold(ar, br, h), want)


@pytest.mark.parametrize("name", ["per_step_f32", "shared_decay_f32", "per_step_bf16"])
def test_scan_states_bitwise_vs_reference_evaluation_of_the_stacked_map_form(name):
    a, b, h = cases.fold_inputs(name)
    want = _from_gold(_load("states.npz")[f"states.{name}"], h.dtype)
    n = cases.FOLD_CASES[name][0]
    ar = a if a.dim() == h.dim() + 1 else a.expand(n, *a.shape)
    br = b if b.dim() == h.dim() + 1 else b.expand(n, *b.shape)
    assert torch.equal(oracle.scan_states(ar, br, h), want)
