"""Parity of the CUDA path (through the C ABI) against the oracle and against the
reference's stored outputs.  Needs a B200: run with ``-m gpu``.

Tolerances (relative to the largest reference magnitude, the reference's own
verify metric): 1e-5 for fp32, 2e-2 for bf16; the verify reduction is exact.
"""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from oracle import oracle

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
FP32_TOL = 1e-5
BF16_TOL = 2e-2


def rel_to_max(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return ((got - want).abs().max() / (want.abs().max() + 1e-8)).item()


@pytest.fixture(scope="module")
def dev():
    from catopt_b200 import build

    build.build()
    return torch.device("cuda", 0)


# --------------------------------------------------------------------------- (d) verify
@pytest.mark.parametrize("case", cases.verify_cases(), ids=lambda c: c[0])
def test_verify_exact_vs_reference_fixture(dev, case):
    from catopt_b200 import verify

    name, ref, out, rtol, atol = case
    want = np.load(GOLD / "verify.npz")[name]
    rep = verify.verify_equiv(ref.to(dev), out.to(dev), rtol=rtol, atol=atol)
    for got, exp in ((rep.max_abs, want[0]), (rep.max_rel, want[1])):
        assert (math.isnan(got) and math.isnan(exp)) or got == exp, (name, got, exp)
    assert rep.passed == bool(want[2])


def test_verify_tuple_and_mismatch(dev):
    from catopt_b200 import verify

    g = np.load(GOLD / "verify.npz")
    cs = cases.verify_cases()
    r = (cs[0][1].to(dev), cs[3][1].to(dev))
    o = (cs[0][2].to(dev), cs[3][2].to(dev))
    rep = verify.verify_equiv(r, o, rtol=2e-2)
    assert [rep.max_abs, rep.max_rel, float(rep.passed), *rep.per_output] == list(g["tuple"])
    rep = verify.verify_equiv(r, o[:1], rtol=2e-2)
    assert rep.max_abs == math.inf and not rep.passed


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(3, 4, 512, 64), (5, 1, 77, 8), (2, 1, 1, 3)])
def test_verify_batched_vs_oracle(dev, dtype, shape):
    """Segmented reduction (one segment per check) incl. odd, unaligned sizes."""
    from catopt_b200 import verify

    g = torch.Generator().manual_seed(7)
    ref = torch.randn(shape, generator=g).to(dtype)
    out = (ref.float() + 0.01 * torch.randn(shape, generator=g)).to(dtype)
    reps = verify.verify_batched(ref.to(dev), out.to(dev), shape[0], rtol=2e-2)
    for i, rep in enumerate(reps):
        want = oracle.verify_pair(ref[i], out[i], rtol=2e-2)
        assert (rep.max_abs, rep.max_rel, rep.passed) == (want.max_abs, want.max_rel, want.passed)


def test_verify_full_probe_size_properties(dev):
    """Benchmark config 5's tensor size ([4,512,1024] bf16 per probe, 8 probes x 3
    checks here): planted maxima are found exactly; untouched checks report 0."""
    from catopt_b200 import ops

    n_checks, probes = 3, 8
    ref = torch.randn(n_checks, probes, 4, 512, 1024, device=dev).to(torch.bfloat16)
    out = ref.clone()
    out[1, 5, 3, 100, 77] = ref[1, 5, 3, 100, 77] + 8.0
    ref[2, 0, 0, 0, 0] = 1000.0
    out[2, 0, 0, 0, 0] = 1000.0
    res = ops.verify_reduce(ref, out, n_checks).cpu()
    want1 = (ref[1, 5, 3, 100, 77].float() - out[1, 5, 3, 100, 77].float()).to(torch.bfloat16).abs().item()
    assert res[0, 0] == 0 and res[2, 0] == 0 and res[1, 0] == want1
    assert res[2, 1] == 1000.0
    assert res[0, 1] == ref[0].abs().max().item()
    assert res[:, 2:].sum() == 0


# --------------------------------------------------------------------------- (a) chain
@pytest.mark.parametrize("name", list(cases.CHAIN_CASES))
def test_chain_fold_and_linear_vs_reference(dev, name):
    from catopt_b200.executors import B200FoldedLinear

    g = np.load(GOLD / "chain.npz")
    ws, x = cases.chain_inputs(name)
    mod = B200FoldedLinear([w.to(dev) for w in ws])
    assert mod.is_batched and mod.fused_name == f"fused_{2 * len(ws) - 2}"
    wf_ref = oracle.fold_chain(ws)
    assert rel_to_max(mod.weight, wf_ref) <= FP32_TOL
    y = mod(x.to(dev))
    assert rel_to_max(y, torch.from_numpy(g[f"{name}.y_folded"])) <= FP32_TOL
    assert rel_to_max(y, torch.from_numpy(g[f"{name}.y_eager"])) <= FP32_TOL


@pytest.mark.parametrize("rows,n_in,n_out", [(1, 7, 5), (64, 512, 512), (300, 130, 70), (4096, 512, 512)])
def test_linear_shapes_and_bias(dev, rows, n_in, n_out):
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, n_in, generator=g)
    w = torch.randn(n_out, n_in, generator=g) / math.sqrt(n_in)
    b = torch.randn(n_out, generator=g)
    want = torch.nn.functional.linear(x.double(), w.double(), b.double())
    got = ops.linear_f32(x.to(dev), w.to(dev), b.to(dev))
    assert rel_to_max(got, want) <= FP32_TOL
    got = ops.matmul_f32(x.to(dev), w.t().contiguous().to(dev))
    assert rel_to_max(got, want - b.double()) <= FP32_TOL


def test_linear_is_linear_at_published_size(dev):
    """R=65536 rows (the reference's largest published cell): linearity
    f(ax+by) = a f(x) + b f(y) holds to fp32 rounding."""
    from catopt_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(65536, 512, device=dev, generator=g)
    y = torch.randn(65536, 512, device=dev, generator=g)
    w = torch.randn(512, 512, device=dev, generator=g) / math.sqrt(512)
    lhs = ops.linear_f32(2.0 * x - 3.0 * y, w)
    rhs = 2.0 * ops.linear_f32(x, w) - 3.0 * ops.linear_f32(y, w)
    assert rel_to_max(lhs, rhs) <= FP32_TOL


# --------------------------------------------------------------------------- explicit attention masks
@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("B,H,Tq,Tk,d,mshape", [(2, 4, 384, 384, 128, (384, 384)), (1, 3, 200, 333, 64, (1, 3, 200, 333)),
                                               (2, 2, 128, 512, 64, (2, 1, 128, 512)), (1, 2, 130, 70, 32, (130, 1)),
                                               (2, 2, 64, 256, 128, (1, 1, 1, 256)),
                                               (2, 3, 1, 2000, 64, (2, 1, 1, 2000)),       # decode rows: the streaming kernel
                                               (1, 2, 5, 1500, 128, (5, 1500))])
def test_om_bias_fwd_vs_torch_sdpa_in_fp64(dev, dtype, tol, B, H, Tq, Tk, d, mshape):
    """softmax(scale q k^T + bias) v with biases of every broadcast shape (per (t, j), with a head or a
    batch axis, one value per row, one per key), some keys hidden by -inf, against torch's own masked
    attention in fp64 on the same (rounded) inputs."""
    import torch.nn.functional as F

    from catopt_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(Tq + Tk)
    q, k, v = (torch.randn(B, H, T, d, device=dev, generator=g).to(dtype) for T in (Tq, Tk, Tk))
    bias = torch.randn(*mshape, device=dev, generator=g)
    hide = torch.rand(*mshape, device=dev, generator=g) < 0.3
    if mshape[-1] > 1:
        hide[..., 0] = False                                  # every row keeps a key
        bias = bias.masked_fill(hide, float("-inf"))
    got = ops.om_bias_fwd(q, k, v, bias, 0.125)
    ops.check_device_status(dev)
    want = F.scaled_dot_product_attention(q.double(), k.double(), v.double(), attn_mask=bias.double(), scale=0.125)
    assert got.dtype == dtype and rel_to_max(got, want) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("Tq,mshape", [(256, (256, 640)), (3, (1, 2, 3, 640)), (70, (2, 1, 70, 640))])
def test_om_step_with_a_mask_folds_blocks_into_the_masked_attention(dev, dtype, tol, Tq, mshape):
    """Three key blocks folded one ``cb2_om_bias_step`` at a time (tile kernels for many rows; a handful
    of rows takes the tile kernel for the short blocks and the streaming decode kernel for the 320-key
    one), each with its columns of the mask: the readout equals masked attention over the joined keys."""
    import torch.nn.functional as F

    from catopt_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(Tq)
    B, H, d, sizes = 2, 2, 64, (128, 320, 192)
    q = torch.randn(B, H, Tq, d, device=dev, generator=g).to(dtype)
    ks = [torch.randn(B, H, n, d, device=dev, generator=g).to(dtype) for n in sizes]
    vs = [torch.randn(B, H, n, d, device=dev, generator=g).to(dtype) for n in sizes]
    bias = torch.randn(*mshape, device=dev, generator=g)
    hide = torch.rand(*mshape, device=dev, generator=g) < 0.3
    hide[..., 0] = False
    bias = bias.masked_fill(hide, float("-inf"))
    state, col = None, 0
    for kb, vb in zip(ks, vs):
        state = ops.om_step_qk(state, q, kb, vb, 0.125, False, col, bias=bias[..., col:col + kb.shape[2]])
        col += kb.shape[2]
    ops.check_device_status(dev)
    want = F.scaled_dot_product_attention(q.double(), torch.cat(ks, 2).double(), torch.cat(vs, 2).double(),
                                          attn_mask=bias.double(), scale=0.125)
    assert rel_to_max(ops.om_apply_state(state), want) <= tol


def test_om_bias_fwd_bool_mask_hidden_rows_and_the_causal_flag(dev):
    """A bool keep-mask goes in as 0 / -inf (the reference's ``attnbias``); a row with no visible key is
    NaN, as the reference's unclamped a / l; with the causal flag the two masks combine."""
    import torch.nn.functional as F

    from catopt_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(77)
    q, k, v = (torch.randn(1, 2, 256, 64, device=dev, generator=g).bfloat16() for _ in range(3))
    keep = torch.rand(256, 256, device=dev, generator=g) < 0.5
    keep[7] = False
    got = ops.om_bias_fwd(q, k, v, ops.attn_bias(keep), 0.125)
    want = F.scaled_dot_product_attention(q.double(), k.double(), v.double(), attn_mask=keep, scale=0.125)
    assert torch.isnan(got[:, :, 7]).all()        # (torch's own kernels differ among themselves on such rows)
    rows = [t for t in range(256) if t != 7]
    assert rel_to_max(got[:, :, rows], want[:, :, rows]) <= BF16_TOL
    keep[:, 0] = True
    both = keep & torch.ones(256, 256, dtype=torch.bool, device=dev).tril()
    got = ops.om_bias_fwd(q, k, v, ops.attn_bias(keep), 0.125, causal=True)
    want = F.scaled_dot_product_attention(q.double(), k.double(), v.double(), attn_mask=both, scale=0.125)
    assert rel_to_max(got, want) <= BF16_TOL
    ops.check_device_status(dev)


# --------------------------------------------------------------------------- (b) decayed
@pytest.mark.parametrize("name", [n for n in cases.DECAYED_CASES if n != "tiny_f64"])
def test_decayed_fp32_vs_reference_fixture(dev, name):
    from catopt_b200.executors import B200ChunkedDecay

    g = np.load(GOLD / "decayed.npz")
    q, k, v, gamma, C, scale = cases.decayed_inputs(name)
    mod = B200ChunkedDecay(gamma, q.shape[1], C, scale).to(dev)
    out = mod(q.to(dev), k.to(dev), v.to(dev))
    stride = cases.ROW_STRIDE.get(name, 1)
    want = torch.from_numpy(g[f"{name}.chunked"])
    assert rel_to_max(out[:, :, ::stride], want) <= FP32_TOL
    assert rel_to_max(out[:, :, ::stride], torch.from_numpy(g[f"{name}.quadratic"])) <= FP32_TOL


def test_decayed_f64_case_in_fp32(dev):
    """The reference's fp64 test shape, run in fp32 against its fp64 output."""
    from catopt_b200 import ops

    g = np.load(GOLD / "decayed.npz")
    q, k, v, gamma, C, scale = cases.decayed_inputs("tiny_f64")
    out = ops.decayed_chunk_fwd(q.float().to(dev), k.float().to(dev), v.float().to(dev),
                                gamma.float().to(dev), C, scale)
    assert rel_to_max(out, torch.from_numpy(g["tiny_f64.chunked"])) <= FP32_TOL


# fp32 tensors with dk, dv <= 64 and at least 24 (batch, head) units run on the tensor cores in three
# TF32 passes; fewer units stay on the FMA pipes.
def _decayed_fp64(q, k, v, gamma, scale):
    """All-pairs evaluation in fp64 on the device (the reference's quadratic form)."""
    B, H, T, _ = q.shape
    t = torch.arange(T, device=q.device, dtype=torch.float64)
    e = (t[:, None] - t[None, :]).clamp(min=0)
    out = torch.empty(B, H, T, v.shape[-1], dtype=torch.float64, device=q.device)
    for h in range(H):
        g = torch.tensor(float(gamma[h]), dtype=torch.float64, device=q.device)
        dm = torch.tril(torch.pow(g, e))
        out[:, h] = ((q[:, h].double() @ k[:, h].double().transpose(-1, -2)) * dm) @ v[:, h].double() / scale
    return out


@pytest.mark.parametrize("name", ["tiny_f32_scalar", "odd_f32", "c2_f32"])
def test_decayed_fp32_tensor_core_path_vs_reference_fixture(dev, name):
    """The reference's stored outputs, with the case repeated over the batch until the call has
    enough units for the tensor-core kernel: every copy must match the fixture."""
    from catopt_b200 import _lib, ops

    g = np.load(GOLD / "decayed.npz")
    q, k, v, gamma, C, scale = cases.decayed_inputs(name)
    B, H, T, d = q.shape
    reps = -(-24 // (B * H))
    qq, kk, vv = (t.repeat(reps, 1, 1, 1).contiguous().to(dev) for t in (q, k, v))
    gam = (gamma if gamma.dim() else gamma.repeat(H)).float().to(dev)
    assert _lib.load().cb2_decayed_chunk_on_tensor_cores(B * reps, H, T, d, d, C, _lib.CB2_F32) == 1
    out = ops.decayed_chunk_fwd(qq, kk, vv, gam, C, scale)
    ops.check_device_status(dev)
    stride = cases.ROW_STRIDE.get(name, 1)
    want = torch.from_numpy(g[f"{name}.chunked"])
    for rep in range(reps):
        assert rel_to_max(out[rep * B:(rep + 1) * B, :, ::stride], want) <= FP32_TOL


@pytest.mark.parametrize("B,H,T,dk,dv,C,scale", [(1, 24, 128, 64, 64, 128, 1.0), (2, 16, 512, 64, 64, 64, 1.0),
                                                 (1, 24, 384, 32, 32, 128, 1.0), (1, 24, 192, 48, 24, 64, 1.0),
                                                 (1, 24, 200, 64, 64, 8, 8.0), (3, 8, 136, 4, 60, 8, 0.5)])
def test_decayed_fp32_tensor_core_path_vs_fp64(dev, B, H, T, dk, dv, C, scale):
    """Shapes off the tile grid (ragged last chunk, head dims below 64, dk != dv) and a scale."""
    from catopt_b200 import _lib, ops

    gen = torch.Generator(device="cuda").manual_seed(B * 7 + T + dk)
    q = torch.randn(B, H, T, dk, device=dev, generator=gen) / math.sqrt(dk)
    k = torch.randn(B, H, T, dk, device=dev, generator=gen) / math.sqrt(dk)
    v = torch.randn(B, H, T, dv, device=dev, generator=gen)
    gamma = torch.tensor([1 - 2.0 ** (-5 - 3 * h / H) for h in range(H)], dtype=torch.float32, device=dev)
    assert _lib.load().cb2_decayed_chunk_on_tensor_cores(B, H, T, dk, dv, C, _lib.CB2_F32) == 1
    out = ops.decayed_chunk_fwd(q, k, v, gamma, C, scale)
    ops.check_device_status(dev)
    assert rel_to_max(out, _decayed_fp64(q, k, v, gamma, scale)) <= FP32_TOL


@pytest.mark.parametrize("B,H,T,d", [(10, 32, 200, 64), (40, 8, 128, 32), (5, 64, 392, 48)])
def test_decayed_fp32_tensor_core_path_streams_several_units_per_cta(dev, B, H, T, d):
    """More units than SMs: a persistent CTA walks several units as one stream of chunks, so the state
    must restart, the rate must change and a ragged last chunk must be clipped at every unit boundary."""
    from catopt_b200 import ops

    gen = torch.Generator(device="cuda").manual_seed(T + d)
    q, k, v = (torch.randn(B, H, T, d, device=dev, generator=gen) / math.sqrt(d) for _ in range(3))
    gamma = torch.tensor([0.6 + 0.399 * h / (H - 1) for h in range(H)], dtype=torch.float32, device=dev)
    out = ops.decayed_chunk_fwd(q, k, v, gamma, 8, 1.0)
    ops.check_device_status(dev)
    assert rel_to_max(out, _decayed_fp64(q, k, v, gamma, 1.0)) <= FP32_TOL
    # a unit's result does not depend on which units share its CTA (enough units for the same kernel)
    nb = -(-24 // H)
    part = ops.decayed_chunk_fwd(q[B - nb:].contiguous(), k[B - nb:].contiguous(), v[B - nb:].contiguous(), gamma, 8, 1.0)
    assert torch.equal(part, out[B - nb:])


def test_decayed_fp32_tensor_core_path_takes_every_rate(dev):
    """Rates for which rescaled keys would overflow or vanish (0, 0.05, negative, 1): the kernel decays
    scores by g^(r-c) directly, so it needs no second formulation."""
    from catopt_b200 import ops

    gen = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn(1, 24, 512, 64, device=dev, generator=gen) / 8 for _ in range(3))
    gamma = torch.tensor([0.5, 1.0, 0.9, 0.05, 0.0, 0.999, -0.7, 0.74] * 3, dtype=torch.float32, device=dev)
    out = ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0)
    ops.check_device_status(dev)
    want = _decayed_fp64(q, k, v, gamma, 1.0)
    for h in range(24):
        assert rel_to_max(out[:, h], want[:, h]) <= FP32_TOL, (h, float(gamma[h]))


def test_decayed_fp32_tensor_core_path_agrees_with_the_fma_path_and_the_oracle(dev):
    """The same heads through the tensor-core kernel (32 units) and, four at a time, through the FMA
    path; two of them against the oracle's chunked pairwise executor."""
    from catopt_b200 import _lib, ops

    gen = torch.Generator(device="cuda").manual_seed(9)
    q, k, v = (torch.randn(2, 16, 1024, 64, device=dev, generator=gen) / 8 for _ in range(3))
    gamma = torch.tensor([1 - 2.0 ** (-5 - h / 4) for h in range(16)], dtype=torch.float32, device=dev)
    lib = _lib.load()
    assert lib.cb2_decayed_chunk_on_tensor_cores(2, 16, 1024, 64, 64, 64, _lib.CB2_F32) == 1
    assert lib.cb2_decayed_chunk_on_tensor_cores(1, 4, 1024, 64, 64, 64, _lib.CB2_F32) == 0
    out = ops.decayed_chunk_fwd(q, k, v, gamma, 64, 1.0)
    for h0 in range(0, 16, 4):
        part = ops.decayed_chunk_fwd(q[:1, h0:h0 + 4].contiguous(), k[:1, h0:h0 + 4].contiguous(),
                                     v[:1, h0:h0 + 4].contiguous(), gamma[h0:h0 + 4].contiguous(), 64, 1.0)
        assert rel_to_max(out[:1, h0:h0 + 4], part) <= FP32_TOL
    want = oracle.decayed_chunked_pairwise(q[1:, 14:].cpu(), k[1:, 14:].cpu(), v[1:, 14:].cpu(), gamma[14:].cpu(), 64, 1.0)
    assert rel_to_max(out[1:, 14:], want) <= FP32_TOL


def test_decayed_fp32_tensor_core_path_long_sequence_and_full_waves(dev):
    """B16 H32 T2048 d64 (512 units: several waves of CTAs) against fp64 on sampled units, and T = 8192
    (64 chunks of carried state) on 24 units."""
    from catopt_b200 import ops

    gen = torch.Generator(device="cuda").manual_seed(13)
    q, k, v = (torch.randn(16, 32, 2048, 64, device=dev, generator=gen) / 8 for _ in range(3))
    gamma = torch.tensor([1 - 2.0 ** (-5 - 8 * h / 32) for h in range(32)], dtype=torch.float32, device=dev)
    out = ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0)
    ops.check_device_status(dev)
    for b in (0, 7, 15):
        want = _decayed_fp64(q[b:b + 1], k[b:b + 1], v[b:b + 1], gamma, 1.0)
        assert rel_to_max(out[b:b + 1], want) <= FP32_TOL
    q, k, v = (torch.randn(1, 24, 8192, 64, device=dev, generator=gen) / 8 for _ in range(3))
    gamma = torch.tensor([1 - 2.0 ** (-5 - 8 * h / 24) for h in range(24)], dtype=torch.float32, device=dev)
    out = ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0)
    ops.check_device_status(dev)
    for h in (0, 11, 23):
        want = _decayed_fp64(q[:, h:h + 1], k[:, h:h + 1], v[:, h:h + 1], gamma[h:h + 1], 1.0)
        assert rel_to_max(out[:, h:h + 1], want) <= FP32_TOL


@pytest.mark.parametrize("B,H,T,d,C", [(1, 2, 512, 128, 128), (2, 3, 256, 64, 64), (1, 1, 128, 128, 128),
                                       (1, 2, 96, 32, 32), (2, 2, 1024, 64, 64), (1, 3, 384, 16, 32),
                                       (1, 2, 256, 96, 128), (1, 1, 256, 8, 64)])
def test_decayed_bf16_vs_oracle(dev, B, H, T, d, C):
    """bf16 tensors: the oracle runs the reference's pairwise executor in fp32 on
    the bf16-rounded inputs (a pure-bf16 reference run is unusable: gamma_h
    rounds to 1.0)."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(B * 1000 + T)
    q, k, v = (torch.randn(B, H, T, d, generator=g) / math.sqrt(d) for _ in range(3))
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    gamma = torch.tensor([1 - 2.0 ** (-5 - 8 * h / max(H, 1)) for h in range(H)], dtype=torch.float32)
    want = oracle.decayed_chunked_pairwise(q.float(), k.float(), v.float(), gamma, C, 1.0)
    out = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), C, 1.0)
    assert out.dtype == torch.bfloat16
    assert rel_to_max(out, want) <= BF16_TOL


def test_decayed_chunk_size_invariance(dev):
    """Size-independent property: the result does not depend on the chunk size."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(2, 2, 256, 64, generator=g).to(dev) / 8 for _ in range(3))
    gamma = torch.tensor([0.95, 0.99], device=dev)
    outs = [ops.decayed_chunk_fwd(q, k, v, gamma, C, 1.0) for C in (16, 64, 128, 256)]
    for o in outs[1:]:
        assert rel_to_max(o, outs[0]) <= FP32_TOL


def test_decayed_rejects_ragged_T(dev):
    from catopt_b200 import B200Error, ops

    q = torch.zeros(1, 1, 100, 16, device=dev)
    with pytest.raises(B200Error):
        ops.decayed_chunk_fwd(q, q, q, torch.ones(1, device=dev), 64)


# --------------------------------------------------------------------------- (c) scan
@pytest.mark.parametrize("name", list(cases.SCAN_CASES))
def test_scan_vs_reference_fixture(dev, name):
    from catopt_b200.executors import B200DiagScan

    g = np.load(GOLD / "scan.npz")
    a, x, b, c, h0 = cases.scan_inputs(name)
    mod = B200DiagScan(b, c, return_state=True).to(dev)
    y, hT = mod(a.to(dev), x.to(dev), None if h0 is None else h0.to(dev))
    tol = BF16_TOL if x.dtype == torch.bfloat16 else FP32_TOL
    assert y.dtype == x.dtype
    assert rel_to_max(y, torch.from_numpy(g[f"{name}.y"])) <= tol
    assert rel_to_max(y, torch.from_numpy(g[f"{name}.y_prefix"])) <= tol
    assert rel_to_max(hT, torch.from_numpy(g[f"{name}.hT"])) <= FP32_TOL
    assert rel_to_max(hT, torch.from_numpy(g[f"{name}.hT_tree"])) <= FP32_TOL


@pytest.mark.parametrize("B,T,D,N,dtype", [
    (2, 1, 8, 16, torch.bfloat16), (1, 15, 64, 16, torch.bfloat16), (1, 16, 40, 16, torch.bfloat16),
    (2, 17, 32, 16, torch.bfloat16), (1, 130, 96, 16, torch.bfloat16), (1, 65, 8, 32, torch.float32),
    (1, 64, 16, 2, torch.bfloat16), (3, 33, 8, 8, torch.float32),
])
def test_scan_edges_vs_oracle(dev, B, T, D, N, dtype):
    """Ragged tiles (T around the 16-step tile), partial channel blocks, every N."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(T * 100 + D)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, N, generator=g)).to(dtype)
    b = (torch.randn(D, N, generator=g) / 4).to(dtype)
    c = (torch.randn(D, N, generator=g) / 4).to(dtype)
    h0 = torch.randn(B, D, N, generator=g)
    want_y, want_h = oracle.diag_scan_serial(a, x, b, c, h0)
    y, hT = ops.diag_scan_fwd(a.to(dev), x.to(dev), b.to(dev), c.to(dev), h0.to(dev), want_state=True)
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert rel_to_max(y, want_y) <= tol
    assert rel_to_max(hT, want_h) <= FP32_TOL


@pytest.mark.parametrize("B,T,D,N,dtype,with_h0", [
    (2, 100, 64, 16, torch.bfloat16, True), (1, 33, 32, 8, torch.float32, False),
    (1, 32, 96, 16, torch.bfloat16, False), (2, 257, 32, 1, torch.float32, True),
    (1, 2048, 32, 16, torch.bfloat16, True),
])
def test_scan_shared_decay_vs_oracle(dev, B, T, D, N, dtype, with_h0):
    """`a` shared over n ([B,T,D]): the collapsed scalar recurrence equals the
    N-state serial fold of the oracle."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(T + D)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, generator=g)).to(dtype)
    b = (torch.randn(D, N, generator=g) / 4).to(dtype)
    c = (torch.randn(D, N, generator=g) / 4).to(dtype)
    h0 = torch.randn(B, D, N, generator=g) if with_h0 else None
    want_y, want_h = oracle.diag_scan_serial(a, x, b, c, h0)
    y, hT = ops.diag_scan_fwd(a.to(dev), x.to(dev), b.to(dev), c.to(dev),
                              None if h0 is None else h0.to(dev), want_state=True)
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert rel_to_max(y, want_y) <= tol
    assert rel_to_max(hT, want_h) <= FP32_TOL


def test_scan_segment_composition_at_full_width(dev):
    """Size-independent property at config 3's width (D=1024, N=16, bf16):
    scanning [0,T) equals scanning [0,T/2) then [T/2,T) from the carried state —
    bit for bit, since each step's arithmetic is identical."""
    from catopt_b200 import ops

    B, T, D, N = 2, 512, 1024, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(B, T, D, device=dev, generator=g).to(torch.bfloat16)
    a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, N, device=dev, generator=g)).to(torch.bfloat16)
    b = (torch.randn(D, N, device=dev, generator=g) / 4).to(torch.bfloat16)
    c = (torch.randn(D, N, device=dev, generator=g) / 4).to(torch.bfloat16)
    y, hT = ops.diag_scan_fwd(a, x, b, c, None, want_state=True)
    h = T // 2
    y1, h1 = ops.diag_scan_fwd(a[:, :h].contiguous(), x[:, :h].contiguous(), b, c, None, want_state=True)
    y2, h2 = ops.diag_scan_fwd(a[:, h:].contiguous(), x[:, h:].contiguous(), b, c, h1, want_state=True)
    assert torch.equal(torch.cat([y1, y2], 1), y) and torch.equal(h2, hT)
    want_y, _ = oracle.diag_scan_serial(a[:1, :, :64].cpu(), x[:1, :, :64].cpu(), b[:64].cpu(), c[:64].cpu())
    assert rel_to_max(y[:1, :, :64], want_y) <= BF16_TOL


def test_device_status_clean_midway(dev):
    """No kernel in this file ran into a bounded-wait timeout."""
    from catopt_b200 import ops

    ops.check_device_status(dev)


# --------------------------------------------------------------------------- graphs
def test_cuda_graph_replay_matches_eager(dev):
    from catopt_b200.executors import B200ChunkedDecay

    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(1, 2, 128, 32, generator=g).to(dev) for _ in range(3))
    mod = B200ChunkedDecay(0.97, 2, 32).to(dev)
    eager = mod(q, k, v).clone()
    mod.capture_cuda_graph(q, k, v)
    assert mod.is_graph_captured
    assert torch.equal(mod(q, k, v), eager)
    q2 = q * 0.5
    assert torch.equal(mod(q2, k, v), mod._forward_impl(q2, k, v))
    mod.drop_cuda_graph()
    assert not mod.is_graph_captured


def test_cuda_graph_replay_of_segmented_heads_and_other_executors(dev):
    """Graph capture of the launches that do more than one thing per call: the
    tensor-core decayed kernel with heads cut into segments (flag reset + kernel),
    the 3xTF32 GEMM (weight split + GEMM) and the composed scan map (two kernels).
    Replays on new inputs must equal eager runs bit for bit."""
    from catopt_b200 import ops
    from catopt_b200.executors import B200CausalSoftmax, B200ChunkedDecay, B200FoldedLinear

    g = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(3, 64, 1024, 64, generator=g).bfloat16().to(dev) / 4 for _ in range(3))
    gam = (1 - torch.exp2(-5 - 8 * torch.arange(64) / 64)).float()
    mod = B200ChunkedDecay(gam, 64, 128).to(dev)
    mod.capture_cuda_graph(q, k, v)
    for scale in (1.0, 0.5, 0.25):                     # several replays: the segment flags must be reset each time
        qq = q * scale
        assert torch.equal(mod(qq, k, v), mod._forward_impl(qq, k, v))
    lin = B200FoldedLinear([torch.randn(256, 256, generator=g).to(dev) / 16 for _ in range(3)])
    x = torch.randn(512, 256, generator=g).to(dev)
    lin.capture_cuda_graph(x)
    assert torch.equal(lin(x * 2), lin._forward_impl(x * 2))
    att = B200CausalSoftmax().to(dev)
    att.capture_cuda_graph(q[:1, :4], k[:1, :4], v[:1, :4])
    assert torch.equal(att(q[1:2, :4], k[:1, :4], v[:1, :4]), att._forward_impl(q[1:2, :4], k[:1, :4], v[:1, :4]))
    ops.check_device_status(dev)


# --------------------------------------------------------------------------- more edges
@pytest.mark.parametrize("gam", [1.0, 0.5, 0.01, 1e-4])
def test_decayed_bf16_extreme_rates(dev, gam):
    """Rates from no decay to almost total decay on the tensor-core path; the
    oracle is the spelled quadratic form (the reference's chunked form divides by
    gamma^r and overflows for tiny rates)."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(31)
    B, H, T, d = 1, 2, 384, 128
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(math.sqrt(d)).bfloat16() for _ in range(3))
    gamma = torch.tensor([gam, gam], dtype=torch.float32)
    want = oracle.decayed_quadratic(q.float(), k.float(), v.float(), gamma, 1.0)
    out = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 128, 1.0)
    assert torch.isfinite(out.float()).all()
    assert rel_to_max(out, want) <= BF16_TOL


@pytest.mark.parametrize("B,H,T", [(1, 8, 4096), (2, 80, 1024)])
def test_decayed_bf16_mixed_rates_take_both_formulations(dev, B, H, T):
    """Rates on both sides of the kernel's switch (about 0.74: above it keys are scaled by
    g^-c once and the accumulator is renormalised every 1, 2, 8 or 64 chunks depending on the
    rate; below it the chunk-local decaying powers are used), mixed over the heads of ONE
    launch — with few heads (parallel segments from precomputed pieces) and with more heads
    than SMs (segments that wait for one another) — against the spelled quadratic form."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(77 + H)
    d = 128
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(math.sqrt(d)).bfloat16() for _ in range(3))
    base = torch.tensor([0.3, 0.6, 0.735, 0.745, 0.8, 0.9, 0.97, 1.0])
    gamma = base.repeat((H + 7) // 8)[:H].contiguous()
    out = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 128, 2.0).cpu()
    assert torch.isfinite(out.float()).all()
    heads = range(H) if H <= 8 else (0, 3, 4, 6, 7, 72, 75, 78, 79)
    for b in (0, B - 1):
        for h in heads:
            want = oracle.decayed_quadratic(q[b:b + 1, h:h + 1].float(), k[b:b + 1, h:h + 1].float(),
                                            v[b:b + 1, h:h + 1].float(), gamma[h:h + 1], 2.0)
            assert rel_to_max(out[b:b + 1, h:h + 1], want) <= BF16_TOL, (b, h, float(gamma[h]))
    ops.check_device_status(dev)


def test_decayed_bf16_two_ctas_per_head_without_scratch_give_one_pass_bits(dev):
    """Between a quarter and half as many heads as SMs (one rank's share of config 4 cut over 8
    GPUs): two CTAs per head in one launch, the second accumulating the state of the first's
    chunks from K and V alone before producing the rest — no scratch, no flags.  The same heads
    inside a launch with more heads than SMs (where a head's segments hand their state over and
    the bits are those of one CTA per head) must come out bit-identical; rates on both sides of
    the formulation switch; values against the state-carry oracle."""
    from catopt_b200 import _lib, ops

    g = torch.Generator().manual_seed(91)
    B, H, T, d = 5, 32, 2048, 128
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(math.sqrt(d)).bfloat16().to(dev) for _ in range(3))
    gamma = (1 - torch.exp2(-5 - 8 * torch.arange(H) / H)).float()
    gamma[5], gamma[17] = 0.5, 0.745
    gamma = gamma.to(dev)
    lib = _lib.load()
    assert lib.cb2_decayed_chunk_scratch_bytes(2, H, T, d, d, 128, 1) == 0      # 64 heads: nothing to allocate
    whole = ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0)
    part = ops.decayed_chunk_fwd(q[:2].contiguous(), k[:2].contiguous(), v[:2].contiguous(), gamma, 128, 1.0)
    assert torch.equal(part.view(torch.int16), whole[:2].view(torch.int16))
    for b, h in ((0, 0), (1, 5), (0, 17), (1, 31)):
        want = oracle.decayed_state_carry(q[b:b + 1, h:h + 1].float().cpu(), k[b:b + 1, h:h + 1].float().cpu(),
                                          v[b:b + 1, h:h + 1].float().cpu(), gamma[h:h + 1].cpu(), 128, 1.0)
        assert rel_to_max(part[b:b + 1, h:h + 1], want) <= BF16_TOL, (b, h)
    # a ragged length on the same path (the last chunk is partial)
    T2 = 2048 + 77
    q2, k2, v2 = (torch.randn(2, H, T2, d, generator=g).div_(math.sqrt(d)).bfloat16().to(dev) for _ in range(3))
    o2 = ops.decayed_chunk_fwd(q2, k2, v2, gamma, 1, 1.0)
    want = oracle.decayed_quadratic(q2[1:, 30:31].float().cpu(), k2[1:, 30:31].float().cpu(), v2[1:, 30:31].float().cpu(),
                                    gamma[30:31].cpu(), 1.0)
    assert rel_to_max(o2[1:, 30:31], want) <= BF16_TOL
    ops.check_device_status(dev)


def test_decayed_bf16_many_heads_and_scale(dev):
    """More heads than SMs (several waves of CTAs) and a non-unit divisor."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(32)
    B, H, T, d = 4, 80, 256, 128
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(math.sqrt(d)).bfloat16() for _ in range(3))
    gamma = torch.linspace(0.9, 0.999, H)
    out = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 128, 3.0).cpu()
    for b, h in ((0, 0), (1, 17), (3, 79)):
        want = oracle.decayed_state_carry(q[b:b + 1, h:h + 1].float(), k[b:b + 1, h:h + 1].float(),
                                          v[b:b + 1, h:h + 1].float(), gamma[h:h + 1], 128, 3.0)
        assert rel_to_max(out[b:b + 1, h:h + 1], want) <= BF16_TOL


@pytest.mark.parametrize("B,H,T,d,C", [(1, 2, 1000, 128, 125), (2, 3, 200, 64, 8), (1, 1, 77, 32, 77),
                                       (1, 160, 1100, 128, 100)])
def test_decayed_bf16_sequence_lengths_off_the_tile_grid(dev, B, H, T, d, C):
    """bf16 sequences whose length is not a multiple of the kernel's 128-row tile:
    the last tile is zero-filled on load and clipped on store, per head (the last
    case also cuts 160 heads into segments of an odd number of tiles)."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(T + d)
    q, k, v = (torch.randn(B, H, T, d, generator=g).bfloat16() / 4 for _ in range(3))
    gam = (1 - torch.exp2(-4 - 6 * torch.arange(H) / H)).float()
    out = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gam.to(dev), C, 1.5)
    sel = list(range(H)) if H <= 3 else [0, H // 2, H - 1]   # a store past T would land in the next head
    want = oracle.decayed_quadratic(q[:, sel].double(), k[:, sel].double(), v[:, sel].double(), gam[sel].double(), 1.5)
    assert rel_to_max(out[:, sel], want) <= BF16_TOL
    ops.check_device_status(dev)


def test_decayed_config4_full_size_is_invariant_under_head_segmentation(dev):
    """Benchmark config 4 at full size (B=16, H=32, T=8192, d=128, bf16, 4.3 GB): the
    result with heads cut into segments (the shipped path: 1024 CTAs, state handed over
    in scratch) equals the one-CTA-per-head result bit for bit, and the chunk argument
    does not change it either."""
    from catopt_b200 import _lib, ops

    B, H, T, d = 16, 32, 8192, 128
    lib = _lib.load()
    g = torch.Generator(device=dev).manual_seed(4)
    q, k, v = (torch.randn(B * H, T * d, device=dev, generator=g).mul_(1 / math.sqrt(d)).bfloat16().view(B, H, T, d)
               for _ in range(3))
    gam = (1 - torch.exp2(-5 - 8 * torch.arange(H, device=dev) / H)).float()
    assert lib.cb2_decayed_chunk_scratch_bytes(B, H, T, d, d, 128, 1) > 0
    seg = ops.decayed_chunk_fwd(q, k, v, gam, 128, 1.0)
    one = torch.empty_like(seg)
    st = ops.device_status(dev)
    rc = lib.cb2_decayed_chunk_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), one.data_ptr(), gam.data_ptr(),
                                   B, H, T, d, d, 128, 1.0, 1, None, 0, st.data_ptr(), ops.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(seg.view(torch.int16), one.view(torch.int16))
    other = ops.decayed_chunk_fwd(q, k, v, gam, 64, 1.0)
    assert torch.equal(seg.view(torch.int16), other.view(torch.int16))
    assert torch.isfinite(seg[::5, ::7].float()).all()
    ops.check_device_status(dev)
    # 32 of the 512 (batch, head) slices of that full-size result against the reference's
    # pairwise-chunked algorithm, computed in fp32 on the same bf16-rounded inputs: the first
    # and the last batch entry at heads 0, 15 and 31 (slowest, middle and fastest decay),
    # and 26 seeded draws from the rest
    picks = [(b, h) for b in (0, B - 1) for h in (0, 15, 31)]
    rng = np.random.default_rng(44)
    while len(picks) < 32:
        bh = (int(rng.integers(B)), int(rng.integers(H)))
        if bh not in picks:
            picks.append(bh)
    worst = 0.0
    for b, h in picks:
        qs, ks, vs = (t[b:b + 1, h:h + 1].float().cpu() for t in (q, k, v))
        want = oracle.decayed_chunked_pairwise(qs, ks, vs, gam[h:h + 1].cpu(), 128, 1.0)
        r = rel_to_max(seg[b:b + 1, h:h + 1], want)
        worst = max(worst, r)
        assert r <= BF16_TOL, (b, h, r)
    assert 0.0 < worst <= BF16_TOL
    del q, k, v, seg, one, other
    torch.cuda.empty_cache()


def test_scan_config3_full_size_sampled_against_the_serial_oracle(dev):
    """Benchmark config 3 at full size (B=8, T=4096, D=1024, N=16, bf16 in, fp32 state;
    a alone is 1 GiB): one launch, then 64 channels of EVERY batch entry — channel 0,
    the last one, both sides of the first and the last 32-channel block boundary, and
    seeded draws — against the serial fold of the reference's bindings, for every step
    of y and for the final state."""
    from catopt_b200 import ops

    B, T, D, N = 8, 4096, 1024, 16
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(B, T, D, device=dev, generator=g).bfloat16()
    a = torch.empty(B, T, D, N, device=dev, dtype=torch.bfloat16)
    for bi in range(B):             # built per batch entry: the fp32 draw of the whole tensor would be 2 GiB
        a[bi] = torch.sigmoid(4 + 0.5 * torch.randn(T, D, N, device=dev, generator=g)).bfloat16()
    b = (torch.randn(D, N, device=dev, generator=g) / 4).bfloat16()
    c = (torch.randn(D, N, device=dev, generator=g) / 4).bfloat16()
    y, hT = ops.diag_scan_fwd(a, x, b, c, None, want_state=True)
    ops.check_device_status(dev)
    rng = np.random.default_rng(33)
    ch = {0, 31, 32, 991, 992, D - 1}
    while len(ch) < 64:
        ch.add(int(rng.integers(D)))
    ch = torch.tensor(sorted(ch), device=dev)
    a_s, x_s = a.index_select(2, ch).cpu(), x.index_select(2, ch).cpu()
    want_y, want_h = oracle.diag_scan_serial(a_s, x_s, b.index_select(0, ch).cpu(), c.index_select(0, ch).cpu())
    got_y, got_h = y.index_select(2, ch), hT.index_select(1, ch)
    for bi in range(B):
        assert rel_to_max(got_y[bi], want_y[bi]) <= BF16_TOL, bi
        assert rel_to_max(got_h[bi], want_h[bi]) <= FP32_TOL, bi
    # element by element: y is the fp32 readout rounded once to bf16, so every value sits within one
    # bf16 ulp of the oracle's fp32 value (plus the fp32 summation-order noise of the 16-term readout)
    err = (got_y.float().cpu() - want_y).abs()
    assert (err <= want_y.abs() * 2.0 ** -7 + 2e-5 * want_y.abs().max()).all()
    del a, x, y
    torch.cuda.empty_cache()


def test_decayed_bf16_segmented_heads(dev):
    """More heads than SMs: the tensor-core kernel cuts every head into segments
    that different CTAs run, the state crossing through scratch.  Same result as
    one CTA per head (scratch withheld) and as the oracle."""
    from catopt_b200 import _lib, ops

    B, H, T, d = 3, 64, 1024, 128                      # 192 heads, 8 chunks -> 2 segments of 4
    lib = _lib.load()
    assert lib.cb2_decayed_chunk_scratch_bytes(B, H, T, d, d, 128, 1) >= 192 * (128 * 128 * 4 + 4)
    assert lib.cb2_decayed_chunk_scratch_bytes(1, 64, T, d, d, 128, 1) == 0      # one wave: no cut
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, H, T, d, generator=g).bfloat16() / 4 for _ in range(3))
    gam = (1 - torch.exp2(-5 - 8 * torch.arange(H) / H)).float()
    qd, kd, vd, gd = q.to(dev), k.to(dev), v.to(dev), gam.to(dev)
    out = ops.decayed_chunk_fwd(qd, kd, vd, gd, 128, 2.0)
    # the same call with no scratch: one CTA per head
    o1 = torch.empty_like(out)
    st = ops.device_status(qd.device)
    rc = lib.cb2_decayed_chunk_fwd(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o1.data_ptr(), gd.data_ptr(),
                                   B, H, T, d, d, 128, 2.0, 1, None, 0, st.data_ptr(), ops.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert rel_to_max(out, o1.double()) <= 1e-6      # same arithmetic, state round-trips exactly in fp32
    for (b, h) in ((0, 0), (1, 17), (2, 63)):
        want = oracle.decayed_quadratic(q[b:b + 1, h:h + 1].double(), k[b:b + 1, h:h + 1].double(),
                                        v[b:b + 1, h:h + 1].double(), gam[h:h + 1].double(), 2.0)
        assert rel_to_max(out[b:b + 1, h:h + 1], want) <= BF16_TOL
    ops.check_device_status(dev)



def test_decayed_bf16_long_sequence_state_accuracy(dev):
    """T = 8192 (config 4's length, 64 chunks): the fp32 state in tensor memory
    does not drift — compared against the fp64 state-carry recurrence."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(33)
    B, H, T, d = 1, 2, 8192, 128
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(math.sqrt(d)).bfloat16() for _ in range(3))
    gamma = torch.tensor([1 - 2.0 ** -5, 1 - 2.0 ** -12.75], dtype=torch.float32)
    want = oracle.decayed_state_carry(q.double(), k.double(), v.double(), gamma.double(), 128, 1.0)
    out = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 128, 1.0)
    assert rel_to_max(out, want) <= BF16_TOL
    assert rel_to_max(out[:, :, -128:], want[:, :, -128:]) <= BF16_TOL


def test_verify_many_small_segments(dev):
    """3328 segments (13 checks x 256 probes) of a few KiB each."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(34)
    n_seg, n = 3328, 1536
    ref = torch.randn(n_seg, n, generator=g).bfloat16()
    out = (ref.float() + 0.01 * torch.randn(n_seg, n, generator=g)).bfloat16()
    res = ops.verify_reduce(ref.to(dev), out.to(dev), n_seg).cpu()
    want_abs = (ref - out).abs().amax(dim=1).float()
    want_ref = ref.abs().amax(dim=1).float()
    assert torch.equal(res[:, 0], want_abs) and torch.equal(res[:, 1], want_ref)
    assert res[:, 2:].sum() == 0


def test_scan_long_sequence(dev):
    """T = 4096 (config 3's length) on a narrow slice, against the serial oracle."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(35)
    B, T, D, N = 1, 4096, 32, 16
    x = torch.randn(B, T, D, generator=g).bfloat16()
    a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, N, generator=g)).bfloat16()
    b = (torch.randn(D, N, generator=g) / 4).bfloat16()
    c = (torch.randn(D, N, generator=g) / 4).bfloat16()
    want_y, want_h = oracle.diag_scan_serial(a, x, b, c)
    y, hT = ops.diag_scan_fwd(a.to(dev), x.to(dev), b.to(dev), c.to(dev), None, want_state=True)
    assert rel_to_max(y, want_y) <= BF16_TOL
    assert rel_to_max(hT, want_h) <= FP32_TOL


@pytest.mark.parametrize("rows,n_in,n_out", [(256, 512, 512), (1000, 64, 1000), (300, 136, 72), (513, 1024, 128), (513, 2048, 128)])
def test_linear_tensor_core_path(dev, rows, n_in, n_out):
    """Shapes that take the three-pass TF32 kernel (ragged tiles, deep K, bias)."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(rows + n_in)
    x = torch.randn(rows, n_in, generator=g)
    w = torch.randn(n_out, n_in, generator=g) / math.sqrt(n_in)
    b = torch.randn(n_out, generator=g)
    want = torch.nn.functional.linear(x.double(), w.double(), b.double())
    got = ops.linear_f32(x.to(dev), w.to(dev), b.to(dev))
    assert rel_to_max(got, want) <= FP32_TOL


@pytest.mark.parametrize("n,state", [(6, (8,)), (37, (2, 12)), (128, (4, 4, 4)), (5, (3,)), (4096, (64,)),
                                     (1000, (7, 9)), (300, (8, 1024))])
def test_scan_composed_map_vs_reference_tree(dev, n, state):
    """The reduction the catopt scan adapter swaps in: leaves in product order,
    compared with the reference's level-batched `fused_diag_levels` — short and
    long stacks (n cut into segments), vector and scalar state widths."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(n)
    a = torch.sigmoid(3 + torch.randn(n, *state, generator=g))
    b = torch.randn(n, *state, generator=g)
    h = torch.randn(*state, generator=g)
    want = oracle.fused_diag_levels(a.double(), b.double(), h.double())
    got = ops.diag_compose_apply(a.to(dev), b.to(dev), h.to(dev))
    assert got.shape == want.shape and rel_to_max(got, want) <= FP32_TOL
    # bf16 stacks (fp32 accumulation, one rounding at the end) and a gate shared over the batch axis
    ab, bb, hb = a.bfloat16(), b.bfloat16(), h.bfloat16()
    wantb = oracle.fused_diag_levels(ab.double(), bb.double(), hb.double())
    gotb = ops.diag_compose_apply(ab.to(dev), bb.to(dev), hb.to(dev))
    assert gotb.dtype == torch.bfloat16 and rel_to_max(gotb, wantb) <= BF16_TOL
    if len(state) == 2:
        a1 = a[:, :1].contiguous()
        want1 = oracle.fused_diag_levels(a1.double().expand_as(a).contiguous(), b.double(), h.double())
        got1 = ops.diag_compose_apply(a1.to(dev), b.to(dev), h.to(dev))
        assert rel_to_max(got1, want1) <= FP32_TOL
    assert ops.diag_compose_apply(a.double().to(dev), b.double().to(dev), h.double().to(dev)) is None


# --------------------------------------------------------------------------- (b') om causal
@pytest.mark.parametrize("name", list(cases.OM_CAUSAL_CASES))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_om_causal_vs_reference_fixture(dev, name, dtype):
    from catopt_b200.executors import B200CausalSoftmax

    g = np.load(GOLD / "om_causal.npz")
    q, k, v, sizes, scale = cases.om_causal_inputs(name)
    q, k, v = (t.to(dtype) for t in (q, k, v))
    out = B200CausalSoftmax(scale).to(dev)(q.to(dev), k.to(dev), v.to(dev))
    assert out.dtype == dtype
    if dtype == torch.float32:
        st = cases.OM_ROW_STRIDE.get(name, 1)
        assert rel_to_max(out[..., ::st, :], torch.from_numpy(g[f"{name}.chunked"])) <= FP32_TOL
    else:  # oracle on the bf16-rounded inputs
        want = oracle.om_causal_chunked(q.double(), k.double(), v.double(), sizes, scale)
        assert rel_to_max(out, want) <= BF16_TOL


def test_om_causal_long_block_invariance(dev):
    """T = 1000 (ragged against the 64-wide blocks), d = 128: equal to the oracle's
    fold whatever block sizes the oracle uses."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(41)
    q, k, v = (torch.randn(1, 2, 1000, 128, generator=g) for _ in range(3))
    out = ops.om_causal_fwd(q.to(dev), k.to(dev), v.to(dev))
    want = oracle.om_causal_chunked(q.double(), k.double(), v.double(), [300, 700])
    assert rel_to_max(out, want) <= FP32_TOL
    want2 = oracle.om_causal_chunked(q.double(), k.double(), v.double(), [1000])
    assert rel_to_max(out, want2) <= FP32_TOL


@pytest.mark.parametrize("B,H,Tq,Tk,dk,dv", [(1, 2, 1000, 1000, 128, 128), (2, 3, 2048, 2048, 64, 64),
                                            (1, 1, 300, 130, 128, 64), (1, 2, 128, 128, 128, 128),
                                            (1, 1, 1, 257, 32, 32), (1, 2, 384, 384, 96, 48),
                                            (1, 1, 256, 256, 8, 8), (2, 40, 1024, 1024, 128, 128)])
def test_om_causal_bf16_tensor_core_path(dev, B, H, Tq, Tk, dk, dv):
    """bf16 shapes of the tensor-core kernel: ragged lengths, Tq != Tk, many key
    blocks (running max / rescale path), against fp64 on the bf16-rounded inputs."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(Tq + dk)
    q = torch.randn(B, H, Tq, dk, generator=g).bfloat16()
    k = torch.randn(B, H, Tk, dk, generator=g).bfloat16()
    v = torch.randn(B, H, Tk, dv, generator=g).bfloat16()
    out = ops.om_causal_fwd(q.to(dev), k.to(dev), v.to(dev))
    want = oracle.om_causal_chunked(q.double(), k.double(), v.double(), [Tk])
    assert out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
    assert rel_to_max(out, want) <= BF16_TOL


@pytest.mark.parametrize("B,H,Tq,Tk,dk,dv,dtype", [(1, 2, 300, 300, 64, 64, torch.bfloat16),
                                                   (2, 3, 128, 1000, 128, 128, torch.bfloat16),
                                                   (1, 1, 70, 33, 16, 24, torch.float32),
                                                   (1, 2, 1, 257, 32, 32, torch.bfloat16),
                                                   (2, 4, 3, 5000, 64, 64, torch.bfloat16),
                                                   (1, 2, 8, 1500, 32, 48, torch.float32)])
def test_om_unmasked_softmax_attention(dev, B, H, Tq, Tk, dk, dv, dtype):
    """cb2_om_fwd with causal = 0 (the unmasked om carrier): plain softmax attention
    on both kernels, ragged lengths, Tq != Tk, against fp64."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(Tq * 7 + Tk)
    q = torch.randn(B, H, Tq, dk, generator=g).to(dtype)
    k = torch.randn(B, H, Tk, dk, generator=g).to(dtype)
    v = torch.randn(B, H, Tk, dv, generator=g).to(dtype)
    out = ops.om_fwd(q.to(dev), k.to(dev), v.to(dev), 0.3)
    want = torch.softmax((q.double() * 0.3) @ k.double().transpose(-1, -2), -1) @ v.double()
    assert out.dtype == dtype and rel_to_max(out, want) <= (BF16_TOL if dtype == torch.bfloat16 else FP32_TOL)


def test_om_causal_bf16_growing_and_peaked_scores(dev):
    """Score patterns that stress the lazily updated reference point of the
    tensor-core softmax: maxima that creep up block after block (just under and
    just over the update threshold), and very peaked rows."""
    from catopt_b200 import ops

    T, d = 1024, 64
    g = torch.Generator().manual_seed(99)
    base = torch.randn(1, 2, T, d, generator=g)
    for ramp, gain in ((0.004, 1.0), (0.02, 1.0), (0.0, 12.0)):
        # keys grow along the sequence in the direction of the queries -> row maxima keep rising
        dirn = torch.ones(d) / math.sqrt(d)
        k = (base * 0.3 + ramp * torch.arange(T).view(1, 1, T, 1) * dirn).bfloat16()
        q = ((torch.randn(1, 2, T, d, generator=g) * 0.3 + 4.0 * dirn) * gain).bfloat16()
        v = torch.randn(1, 2, T, d, generator=g).bfloat16()
        out = ops.om_causal_fwd(q.to(dev), k.to(dev), v.to(dev))
        want = oracle.om_causal_chunked(q.double(), k.double(), v.double(), [T])
        assert torch.isfinite(out.float()).all()
        assert rel_to_max(out, want) <= BF16_TOL, (ramp, gain)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_om_streaming_steps_match_reference_monoid(dev, dtype):
    """The decode / growing-cache schedule: fold key blocks one call at a time into
    the carrier (m, l, a) and compare every intermediate state and the final
    readout with the oracle's `om_elem` / `om_compose` (the reference's bindings);
    uneven blocks, a causal mask with its key offset, a block that is entirely
    hidden from some rows, and the identity start."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(17)
    B, H, Tq, dk, dv = 2, 3, 70, 32, 24
    sizes = (5, 64, 1, 90)
    q = torch.randn(B, H, Tq, dk, generator=g).to(dtype)
    ks = [torch.randn(B, H, n, dk, generator=g).to(dtype) for n in sizes]
    vs = [torch.randn(B, H, n, dv, generator=g).to(dtype) for n in sizes]
    # fp32 tensors: FMA kernel, fp32 throughout.  bf16: the tensor-core kernel carries the state
    # (P rounded to bf16 for the P.V product, fp32 accumulation and fp32 state)
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    for causal in (False, True):
        state = ops.om_empty_state((B, H, Tq), dv, dev) if causal else None     # both ways of starting
        want, off = None, 0
        for kb, vb in zip(ks, vs):
            state = ops.om_step_qk(state, q.to(dev), kb.to(dev), vb.to(dev), scale=0.3, causal=causal, key_offset=off)
            sc = (q.double() * 0.3) @ kb.double().transpose(-1, -2)
            if causal:
                t = torch.arange(Tq).view(Tq, 1)
                j = torch.arange(kb.shape[2]).view(1, -1) + off
                sc = sc.masked_fill(j > t, float("-inf"))
            e = oracle.om_elem(sc, vb.double())
            want = e if want is None else oracle.om_compose(want, e)
            off += kb.shape[2]
            m, l, a = (x.double().cpu() for x in state)
            fin = torch.isfinite(want[0])
            assert torch.equal(torch.isfinite(m), fin)                    # rows that saw no key yet stay at -inf
            assert (m[fin] - want[0][fin]).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-4)
            # l and a are relative to m: compare the m-independent readout and l e^m
            assert rel_to_max((l * torch.exp(m))[fin], (want[1] * torch.exp(want[0]))[fin]) <= max(tol, 1e-5)
        got = ops.om_apply_state(state)
        ref = want[2] / want[1]
        assert torch.equal(torch.isnan(got.cpu()), torch.isnan(ref))
        ok = ~torch.isnan(ref)
        assert (got.double().cpu()[ok] - ref[ok]).abs().max() / ref[ok].abs().max() <= max(tol, 2e-6)
        # one-shot attention over the joined blocks agrees with the streamed readout
        one = ops.om_causal_fwd(q.to(dev), torch.cat(ks, 2).to(dev), torch.cat(vs, 2).to(dev), 0.3, causal=causal)
        lim = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
        assert rel_to_max(one.double().cpu()[ok], ref[ok]) <= lim


@pytest.mark.parametrize("Tq,Tk,causal", [(1, 2000, False), (3, 1500, True), (64, 4096, False)])
def test_om_step_decode_shapes_split_the_keys(dev, Tq, Tk, causal):
    """Few queries, many keys: the step cuts the keys over extra CTAs and folds their
    partial carriers.  Same carrier as the oracle's one-block `om_elem` composed onto
    an incoming state."""
    from catopt_b200 import _lib, ops

    B, H, dk, dv = 1, 4, 64, 48
    assert _lib.load().cb2_om_step_scratch_bytes(B, H, Tq, Tk, dv) > 0
    g = torch.Generator().manual_seed(Tq + Tk)
    q = torch.randn(B, H, Tq, dk, generator=g)
    k0, v0 = torch.randn(B, H, 37, dk, generator=g), torch.randn(B, H, 37, dv, generator=g)
    k1, v1 = torch.randn(B, H, Tk, dk, generator=g), torch.randn(B, H, Tk, dv, generator=g)
    off = 37
    q_base = off + Tk - Tq if causal else 0          # decode: the queries are the newest positions
    qpos = torch.arange(Tq).view(Tq, 1) + q_base

    def scores(kb, base):
        sc = (q.double() * 0.2) @ kb.double().transpose(-1, -2)
        if causal:
            j = torch.arange(kb.shape[2]).view(1, -1) + base
            sc = sc.masked_fill(j > qpos, float("-inf"))
        return sc

    st = ops.om_step_qk(None, q.to(dev), k0.to(dev), v0.to(dev), 0.2, causal, 0 - q_base)
    st = ops.om_step_qk(st, q.to(dev), k1.to(dev), v1.to(dev), 0.2, causal, off - q_base)
    want = oracle.om_compose(oracle.om_elem(scores(k0, 0), v0.double()), oracle.om_elem(scores(k1, off), v1.double()))
    got = ops.om_apply_state(st).double().cpu()
    ref = want[2] / want[1]
    assert rel_to_max(got, ref) <= FP32_TOL
    assert (st[0].double().cpu() - want[0]).abs().max() <= 1e-5


@pytest.mark.parametrize("dtype,Tq,Tk,dk,dv", [
    (torch.bfloat16, 1, 5001, 128, 128),     # two full 128-byte segments per key row
    (torch.bfloat16, 2, 4100, 72, 100),      # second segment holds one 16-byte piece; dv off the lane grid
    (torch.bfloat16, 4, 3000, 8, 4),         # one piece per key row
    (torch.bfloat16, 8, 2600, 64, 64),
    (torch.float32, 1, 5001, 128, 128),      # four segments
    (torch.float32, 1, 700, 20, 36),         # five pieces
    (torch.float32, 3, 2049, 100, 8),        # four segments, the last with one piece
    (torch.float32, 7, 1000, 32, 128),
])
def test_om_step_decode_key_row_layouts(dev, dtype, Tq, Tk, dk, dv):
    """The decode kernel copies key rows into shared memory in 128-byte segments: row lengths on and off
    that grid, every query-row count, key counts off the 32-key batches, against fp64 attention of the
    newest Tq positions over all Tk keys."""
    from catopt_b200 import _lib, ops

    B, H = 2, 3
    assert _lib.load().cb2_om_step_scratch_bytes(B, H, Tq, Tk, dv) > 0
    gen = torch.Generator(device="cuda").manual_seed(Tk + dk)
    q = torch.randn(B, H, Tq, dk, device=dev, generator=gen).to(dtype)
    k = torch.randn(B, H, Tk, dk, device=dev, generator=gen).to(dtype)
    v = torch.randn(B, H, Tk, dv, device=dev, generator=gen).to(dtype)
    scale = 1 / math.sqrt(dk)
    st = ops.om_step_qk(None, q, k, v, scale, True, -(Tk - Tq))
    ops.check_device_status(dev)
    sc = (q.double() @ k.double().transpose(-1, -2)) * scale
    t = torch.arange(Tq, device=dev).view(Tq, 1)
    j = torch.arange(Tk, device=dev).view(1, Tk)
    sc = sc.masked_fill(j - (Tk - Tq) > t, float("-inf"))
    want = torch.softmax(sc, -1) @ v.double()
    assert rel_to_max(ops.om_apply_state(st), want) <= FP32_TOL
    assert (st[0].double().reshape(B, H, Tq) - sc.amax(-1)).abs().max() <= 1e-5


@pytest.mark.parametrize("dtype,Tq,Tk,dk,dv,causal", [(torch.bfloat16, 1, 5001, 128, 128, False),
                                                       (torch.bfloat16, 4, 3000, 64, 64, True),
                                                       (torch.float32, 2, 2049, 72, 40, True),
                                                       (torch.float32, 8, 1000, 32, 128, False)])
def test_om_step_decode_with_a_mask(dev, dtype, Tq, Tk, dk, dv, causal):
    """The streaming decode kernel with an additive mask over the block's keys (float bias with hidden
    entries, broadcast over heads; whole 32-key batches hidden, so a warp sees batches without a visible
    key), alone and combined with the causal flag, against fp64 attention."""
    from catopt_b200 import ops

    B, H = 2, 3
    gen = torch.Generator(device="cuda").manual_seed(Tk + dv)
    q = torch.randn(B, H, Tq, dk, device=dev, generator=gen).to(dtype)
    k = torch.randn(B, H, Tk, dk, device=dev, generator=gen).to(dtype)
    v = torch.randn(B, H, Tk, dv, device=dev, generator=gen).to(dtype)
    bias = torch.randn(B, 1, Tq, Tk, device=dev, generator=gen)
    bias = bias.masked_fill(torch.rand(B, 1, Tq, Tk, device=dev, generator=gen) < 0.3, float("-inf"))
    bias[..., 64:160] = float("-inf")
    bias[..., 0] = 0.0
    scale = 1 / math.sqrt(dk)
    st = ops.om_step_qk(None, q, k, v, scale, causal, -(Tk - Tq), bias=bias)
    ops.check_device_status(dev)
    sc = (q.double() @ k.double().transpose(-1, -2)) * scale + bias.double()
    if causal:
        t = torch.arange(Tq, device=dev).view(Tq, 1)
        j = torch.arange(Tk, device=dev).view(1, Tk)
        sc = sc.masked_fill(j - (Tk - Tq) > t, float("-inf"))
    want = torch.softmax(sc, -1) @ v.double()
    assert rel_to_max(ops.om_apply_state(st), want) <= FP32_TOL
    assert (st[0].double().reshape(B, H, Tq) - sc.amax(-1)).abs().max() <= 1e-5
    # the same step through the tile kernel (keys in two short blocks) gives the same carrier readout
    half = 200
    k0, v0, k1, v1 = (t.contiguous() for t in (k[:, :, :half], v[:, :, :half], k[:, :, half:], v[:, :, half:]))
    s2 = ops.om_step_qk(None, q, k0, v0, scale, causal, -(Tk - Tq), bias=bias[..., :half])
    s2 = ops.om_step_qk(s2, q, k1, v1, scale, causal, half - (Tk - Tq), bias=bias[..., half:])
    assert rel_to_max(ops.om_apply_state(s2), want) <= FP32_TOL


def test_om_streaming_prefill_chunks_on_the_tensor_cores(dev):
    """bf16 prefill in chunks against a growing cache: every chunk of queries is folded
    against the cached keys and its own keys with the carrier passed along, on the
    tensor-core kernel (state in and out, causal mask with key offset, a chunk whose
    keys all lie in the future of an earlier query tile)."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(23)
    B, H, T, d = 1, 3, 640, 64
    q, k, v = (torch.randn(B, H, T, d, generator=g).bfloat16() for _ in range(3))
    want = oracle.om_causal_chunked(q.double(), k.double(), v.double(), [T], 0.2)
    # all queries at once, keys arriving in three uneven pieces
    st, off = None, 0
    for n in (200, 300, 140):
        st = ops.om_step_qk(st, q.to(dev), k[:, :, off:off + n].to(dev), v[:, :, off:off + n].to(dev), 0.2, True, off)
        off += n
    assert rel_to_max(ops.om_apply_state(st), want) <= BF16_TOL
    # query chunks of 256 rows, each against everything cached so far (key_offset = -first row)
    outs = []
    for q0 in range(0, T, 256):
        q1 = min(T, q0 + 256)
        st = ops.om_step_qk(None, q[:, :, q0:q1].to(dev), k[:, :, :q1].to(dev), v[:, :, :q1].to(dev), 0.2, True, -q0)
        outs.append(ops.om_apply_state(st))
    assert rel_to_max(torch.cat(outs, 2), want) <= BF16_TOL
    ops.check_device_status(dev)


def test_causal_softmax_blocks_entry_point(dev):
    """What the catopt-facing causal module runs after evaluating its operands:
    key/value blocks of uneven sizes joined on the key axis, rank-3 and rank-4
    operands, fp32 and bf16."""
    from catopt_b200.executors import causal_softmax_blocks

    g = torch.Generator().manual_seed(11)
    for lead, sizes, Tq, dt, tol in (((2, 3), (5, 9, 130), 144, torch.float32, FP32_TOL),
                                     ((4,), (128, 128), 256, torch.bfloat16, BF16_TOL),
                                     ((), (3, 4), 1, torch.float32, FP32_TOL)):
        q = torch.randn(*lead, Tq, 32, generator=g).to(dt)
        ks = [torch.randn(*lead, n, 32, generator=g).to(dt) for n in sizes]
        vs = [torch.randn(*lead, n, 16, generator=g).to(dt) for n in sizes]
        out = causal_softmax_blocks(q.to(dev), [t.to(dev) for t in ks], [t.to(dev) for t in vs], 0.25)
        want = oracle.om_causal_chunked(q.double(), torch.cat(ks, -2).double(), torch.cat(vs, -2).double(),
                                        list(sizes), 0.25)
        assert out.shape == want.shape and out.dtype == dt
        assert rel_to_max(out, want) <= tol
    assert causal_softmax_blocks(q.double().to(dev), [t.double().to(dev) for t in ks],
                                 [t.double().to(dev) for t in vs], 0.25) is None
    # the streaming form of the same fold: state after the first block, then the rest
    from catopt_b200 import ops
    from catopt_b200.executors import softmax_blocks_state

    lead, sizes, Tq = (2, 3), (5, 9, 130), 144
    q = torch.randn(*lead, Tq, 32, generator=g)
    ks = [torch.randn(*lead, n, 32, generator=g) for n in sizes]
    vs = [torch.randn(*lead, n, 16, generator=g) for n in sizes]
    st = softmax_blocks_state(q.to(dev), [ks[0].to(dev)], [vs[0].to(dev)], 0.25)
    st = softmax_blocks_state(q.to(dev), [t.to(dev) for t in ks[1:]], [t.to(dev) for t in vs[1:]], 0.25,
                              state=st, key_offset=sizes[0])
    assert st[0].shape == (*lead, Tq, 1) and st[2].shape == (*lead, Tq, 16)
    want = oracle.om_causal_chunked(q.double(), torch.cat(ks, -2).double(), torch.cat(vs, -2).double(),
                                    list(sizes), 0.25)
    assert rel_to_max(ops.om_apply_state(st), want) <= FP32_TOL


def test_decayed_whole_sequence_entry_point(dev):
    """What the catopt-facing decayed module runs for a ragged partition: no chunk
    from the plan (the kernel picks one), rank-3 operands with a scalar rate,
    rank-4 with per-head rates."""
    from catopt_b200.executors import decayed_whole_sequence

    g = torch.Generator().manual_seed(12)
    q, k, v = (torch.randn(2, 320, 16, generator=g) / 2 for _ in range(3))       # [B, T, d]: T = 320 -> chunk 80
    out = decayed_whole_sequence(q.to(dev), k.to(dev), v.to(dev), torch.tensor(0.9), None, 4.0)
    want = oracle.decayed_quadratic(q.double()[None], k.double()[None], v.double()[None],
                                    torch.tensor(0.9, dtype=torch.float64), 4.0)[0]
    assert out.shape == (2, 320, 16) and rel_to_max(out, want) <= FP32_TOL
    q, k, v = (torch.randn(2, 3, 256, 64, generator=g).bfloat16() for _ in range(3))
    gam = torch.tensor([0.9, 0.97, 0.995])
    out = decayed_whole_sequence(q.to(dev), k.to(dev), v.to(dev), gam.to(dev), None, 8.0)
    want = oracle.decayed_quadratic(q.double(), k.double(), v.double(), gam.double(), 8.0)
    assert rel_to_max(out, want) <= BF16_TOL
    assert decayed_whole_sequence(q.double().to(dev), k.double().to(dev), v.double().to(dev), gam, None, 1.0) is None


def test_diag_prefix_maps_vs_reference_prefix_scan(dev):
    """All-prefix maps of a diagonal step sequence (the omd executor's hot step)
    against the oracle's restatement of the reference's blocked prefix scan, which
    the golden fixtures pin to the real ``_prefix_scan``."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(21)
    for T, shape in ((37, (8, 12)), (256, (4, 64)), (5, (16,))):
        A = torch.sigmoid(2 + torch.randn(T, *shape, generator=g))
        Bv = torch.randn(T, *shape, generator=g)
        pa, pb = ops.diag_prefix_maps(A.to(dev), Bv.to(dev))
        wa, wb = oracle.prefix_scan_diag(A.double(), Bv.double())
        assert pa.shape == wa.shape and pb.shape == wb.shape
        assert rel_to_max(pa, wa) <= FP32_TOL and rel_to_max(pb, wb) <= FP32_TOL
    # a shared (broadcast) gate, as LTI scans have
    A = torch.sigmoid(torch.randn(40, 1, 8, generator=g)).expand(40, 3, 8)
    Bv = torch.randn(40, 3, 8, generator=g)
    pa, pb = ops.diag_prefix_maps(A.to(dev), Bv.to(dev))
    wa, wb = oracle.prefix_scan_diag(A.double().contiguous(), Bv.double())
    assert rel_to_max(pa, wa) <= FP32_TOL and rel_to_max(pb, wb) <= FP32_TOL
    assert ops.diag_prefix_maps(A.double().to(dev), Bv.double().to(dev)) is None     # fp64: caller keeps its scan


def test_bounded_device_wait_runs_out_and_surfaces_as_an_error(dev):
    """The timeout route end to end, without faulting or hanging anything: a bounded wait
    against a flag nobody sets gives up after its budget (1 ms), the kernel ends by itself
    with CB2_WAIT_TIMEOUT in the status word, ``check_device_status`` raises ``B200Error``
    (a message catopt's failure taxonomy files under "timeout"), the word is cleared, and
    the next launches on the same stream — a satisfied wait and a real kernel — are clean."""
    import time

    from catopt_b200 import B200Error, _lib, ops

    ops.check_device_status(dev)                      # nothing pending from earlier tests
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    ops.wait_for_flag(flag, budget_us=1000)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0            # gave up after about a millisecond, by itself
    assert int(ops.device_status(dev).item()) == _lib.CB2_WAIT_TIMEOUT
    with pytest.raises(B200Error, match="timed out") as err:
        ops.check_device_status(dev)
    msg = str(err.value).lower()
    assert "timed out" in msg or "timeout" in msg    # what catopt_core.failures.classify reads as TIMEOUT
    assert int(ops.device_status(dev).item()) == 0   # the check consumed the status
    # the same stream is usable: a wait whose flag is set returns at once, then a real kernel
    flag.fill_(1)
    ops.wait_for_flag(flag, budget_us=1000)
    ref = torch.zeros(4096, device=dev)
    res = ops.verify_reduce(ref, ref + 0.5, 1).cpu()
    assert res[0, 0].item() == 0.5 and res[0, 2:].sum() == 0
    ops.check_device_status(dev)
    # argument errors are return codes, not launches
    lib = _lib.load()
    assert lib.cb2_wait_for_flag(None, 10, None, None) != 0
    assert lib.cb2_wait_for_flag(flag.data_ptr(), 0, None, None) != 0
    assert lib.cb2_wait_for_flag(flag.data_ptr(), 3_000_000, None, None) != 0


def test_device_status_clean(dev):
    """No kernel in this file ran into a bounded-wait timeout."""
    from catopt_b200 import ops

    ops.check_device_status(dev)


# --------------------------------------------------------------------------- generated-kernel tier
def _gold_tensor(arr, dtype):
    t = torch.from_numpy(arr)
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


@pytest.mark.parametrize("name", list(cases.GATED_CASES))
def test_gated_contract_vs_reference_fixture(dev, name):
    """(s*g)@v against what the reference's `om_decayed` binding returned."""
    from catopt_b200 import ops

    s, gate, v = cases.gated_inputs(name)
    want = _gold_tensor(np.load(GOLD / "gated.npz")[f"gated.{name}"], s.dtype)
    got = ops.gated_contract(s.to(dev), gate.to(dev), v.to(dev))
    ops.check_device_status(dev)
    assert got.shape == want.shape and got.dtype == want.dtype
    tol = BF16_TOL if s.dtype == torch.bfloat16 else FP32_TOL
    assert rel_to_max(got, want) <= tol, name
    # against the same element evaluated in fp64 on the rounded product: much tighter
    p = (s * gate).double()
    exact = p @ v.double()
    assert rel_to_max(got, exact) <= (4e-3 if s.dtype == torch.bfloat16 else 2e-6), name


@pytest.mark.parametrize("B,H,T,K,dv,gate_kind", [(2, 4, 1024, 1024, 128, "head"), (1, 3, 384, 640, 64, "one"),
                                                  (2, 2, 200, 136, 96, "full"), (3, 1, 129, 64, 8, "batch")])
def test_gated_contract_tensor_core_path_vs_oracle(dev, B, H, T, K, dv, gate_kind):
    from catopt_b200 import _lib, ops

    assert _lib.load().cb2_gated_contract_on_tensor_cores(B * H, T, K, dv, _lib.CB2_BF16) == 1
    g = torch.Generator().manual_seed(31)
    s = torch.randn(B, H, T, K, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, K, dv, generator=g).to(torch.bfloat16)
    gshape = {"head": (H, T, K), "one": (T, K), "full": (B, H, T, K), "batch": (B, 1, T, K)}[gate_kind]
    gate = torch.rand(gshape, generator=g).to(torch.bfloat16)
    got = ops.gated_contract(s.to(dev), gate.to(dev), v.to(dev))
    ops.check_device_status(dev)
    want = ((s * gate).double() @ v.double())
    assert got.shape == (B, H, T, dv)
    assert rel_to_max(got, want) <= 4e-3      # only the output rounding separates them
    # neighbouring batches must not leak into one another: each batch alone gives the same bits
    one = ops.gated_contract(s[:1, :1].to(dev), (gate if gate_kind == "one" else
                                                 gate[:1] if gate_kind == "head" else gate[:1, :1]).to(dev),
                             v[:1, :1].to(dev))
    assert torch.equal(one[0, 0], got[0, 0])


def test_gated_contract_is_the_quadratic_decayed_form(dev):
    """With s = q k^T and g = decay(gamma, T) the element is the decayed attention the
    chunked kernel computes (two routes to one function)."""
    from catopt_b200 import ops

    B, H, T, d = 1, 4, 512, 64
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, H, T, d, generator=g) / d ** 0.5 for _ in range(3))
    gamma = torch.tensor([0.9, 0.95, 0.98, 0.995])
    s = q @ k.transpose(-1, -2)
    gate = oracle.decay_matrix(gamma, T)
    got = ops.gated_contract(s.to(dev), gate.to(dev), v.to(dev))
    want = oracle.decayed_quadratic(q.double(), k.double(), v.double(), gamma.double())
    assert rel_to_max(got, want) <= FP32_TOL
    chunked = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 64)
    assert rel_to_max(chunked, got) <= FP32_TOL


@pytest.mark.parametrize("name", list(cases.FOLD_CASES))
def test_seq_fold_vs_reference_fixture(dev, name):
    from catopt_b200 import ops

    a, b, h = cases.fold_inputs(name)
    want = _gold_tensor(np.load(GOLD / "gated.npz")[f"fold.{name}"], h.dtype)
    got = ops.diag_fold_apply(a.to(dev), b.to(dev), h.to(dev))
    tol = BF16_TOL if h.dtype == torch.bfloat16 else FP32_TOL
    assert got.shape == want.shape and got.dtype == want.dtype
    assert rel_to_max(got, want) <= tol, name


def test_seq_fold_equals_product_order_fold_at_width(dev):
    """Time order and product order are two storage orders of one fold: flipping the rows
    and calling the product-order entry point gives the same state (fp32, 1e-6)."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(11)
    n, S = 4096, 8 * 1024
    a = torch.sigmoid(4 + 0.5 * torch.randn(n, S, generator=g)).to(dev)
    b = (0.1 * torch.randn(n, S, generator=g)).to(dev)
    h = torch.randn(S, generator=g).to(dev)
    t_order = ops.diag_fold_apply(a, b, h)
    p_order = ops.diag_compose_apply(a.flip(0).contiguous(), b.flip(0).contiguous(), h)
    assert rel_to_max(t_order, p_order) <= 2e-6
    # a decay row shared by every step is read in place
    shared = ops.diag_fold_apply(a[0], b, h)
    full = ops.diag_fold_apply(a[0].expand(n, S).contiguous(), b, h)
    assert torch.equal(shared, full)


@pytest.mark.parametrize("dtype,T,state", [(torch.float32, 700, (4, 16)), (torch.float32, 9, (7,)),
                                           (torch.bfloat16, 130, (3, 40)), (torch.bfloat16, 33, (5,))])
def test_diag_prefix_maps_one_pass_shapes(dev, dtype, T, state):
    """Vector and scalar layouts, fp32 and bf16, step counts off the unroll grid; the last
    prefix is the whole fold (cb2_diag_fold_apply) and a shared decay row is read in place."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(8)
    A = torch.sigmoid(2 + torch.randn(T, *state, generator=g)).to(dtype)
    Bv = torch.randn(T, *state, generator=g).to(dtype)
    pa, pb = ops.diag_prefix_maps(A.to(dev), Bv.to(dev))
    # exact recurrence in fp64 on the stored values
    wa, wb = torch.empty(T, *state, dtype=torch.float64), torch.empty(T, *state, dtype=torch.float64)
    ca, cb = torch.ones(state, dtype=torch.float64), torch.zeros(state, dtype=torch.float64)
    for t in range(T):
        cb = A[t].double() * cb + Bv[t].double()
        ca = A[t].double() * ca
        wa[t], wb[t] = ca, cb
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert pa.dtype == dtype and pa.shape == wa.shape
    assert rel_to_max(pa, wa) <= tol and rel_to_max(pb, wb) <= tol
    h = torch.randn(state, generator=g).to(dtype)
    last = ops.diag_fold_apply(A.to(dev), Bv.to(dev), h.to(dev))
    want = wa[-1] * h.double() + wb[-1]
    assert rel_to_max(last, want) <= tol
    sa, sb = ops.diag_prefix_maps(A[:1].expand(T, *state).to(dev).contiguous()[:1].expand(T, *state), Bv.to(dev))
    fa, fb = ops.diag_prefix_maps(A[:1].expand(T, *state).contiguous().to(dev), Bv.to(dev))
    assert torch.equal(sa, fa) and torch.equal(sb, fb)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,state", [(37, (8, 12)), (4096, (2, 64)), (1000, (3, 5)), (64, (4, 8192)), (1, (16,))])
def test_diag_scan_states_vs_oracle(dev, dtype, T, state):
    """Every state of the recurrence in one pass (cb2_diag_scan_states): vector and scalar layouts,
    one pass and segments (a small state with many steps), against the oracle's composition of the
    prefix maps and against the plain recurrence in fp64; the last state is the whole fold."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(9 + T)
    A = torch.sigmoid(2 + torch.randn(T, *state, generator=g)).to(dtype)
    Bv = torch.randn(T, *state, generator=g).to(dtype)
    h = torch.randn(state, generator=g).to(dtype)
    got = ops.diag_scan_states(A.to(dev), Bv.to(dev), h.to(dev))
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert got.dtype == dtype and got.shape == (T, *state)
    hh, rows = h.double(), []
    for t in range(T):
        hh = A[t].double() * hh + Bv[t].double()
        rows.append(hh)
    want = torch.stack(rows)
    assert rel_to_max(got, want) <= tol
    if T <= 64:
        assert rel_to_max(got, oracle.scan_states(A.float(), Bv.float(), h.float())) <= tol
    assert rel_to_max(got[-1], ops.diag_fold_apply(A.to(dev), Bv.to(dev), h.to(dev))) <= tol
    # an operand every step shares is read in place: same bits as the expanded copy
    if T > 1:
        shared = A[:1].to(dev).expand(T, *state)
        assert torch.equal(ops.diag_scan_states(shared, Bv.to(dev), h.to(dev)),
                           ops.diag_scan_states(shared.contiguous(), Bv.to(dev), h.to(dev)))
    assert ops.diag_scan_states(A.double().to(dev), Bv.double().to(dev), h.double().to(dev)) is None


def test_linear_with_a_weight_split_once_equals_the_per_call_split(dev):
    """A module's constant weight is split into its TF32 parts once (cb2_linear_f32_split_weight) and
    every forward runs cb2_linear_f32_presplit: same kernel on the same parts, so the same bits as
    cb2_linear_f32; small row counts keep the FMA path."""
    from catopt_b200 import _lib, ops
    from catopt_b200.executors import B200FoldedLinear

    g = torch.Generator().manual_seed(61)
    w = (torch.randn(384, 512, generator=g) / 16).to(dev)
    b = torch.randn(384, generator=g).to(dev)
    split = ops.linear_split_weight(w)
    assert split is not None and split.shape == (2, 384, 512)
    assert torch.equal(split[0] + split[1], w)                  # hi + lo is the weight exactly
    for rows in (256, 1000, 4096):
        x = torch.randn(rows, 512, generator=g).to(dev)
        assert torch.equal(ops.linear_f32(x, w, b, w_split=split), ops.linear_f32(x, w, b))
        want = oracle.linear(x.double().cpu(), w.double().cpu(), b.double().cpu())
        assert rel_to_max(ops.linear_f32(x, w, b, w_split=split), want) <= FP32_TOL
    x = torch.randn(64, 512, generator=g).to(dev)               # below the tensor-core path: split ignored
    assert torch.equal(ops.linear_f32(x, w, b, w_split=split), ops.linear_f32(x, w, b))
    assert ops.linear_split_weight(torch.randn(10, 6, device=dev)) is None
    ws = [(torch.randn(256, 256, generator=g) / 16).to(dev) for _ in range(3)]
    mod = B200FoldedLinear(ws)
    assert mod.fused_split is not None
    xx = torch.randn(2048, 256, generator=g).to(dev)
    assert rel_to_max(mod(xx), oracle.chain_eager(xx.double().cpu(), [t.double().cpu() for t in ws])) <= FP32_TOL
    lib = _lib.load()
    assert lib.cb2_linear_f32_presplit(xx.data_ptr(), split.data_ptr(), None, xx.data_ptr(), 64, 512, 384, None,
                                       None) != 0              # too few rows: an error code, not a launch
    ops.check_device_status(dev)


def test_host_pipeline_runs_the_lowered_module_slab_by_slab(dev):
    """``DecayedHostPipeline``: pinned host tensors in, the module's forward per slab of batch entries on
    three streams, pinned result out — equal to one call of the same module on the whole batch."""
    from catopt_b200.executors import B200ChunkedDecay
    from catopt_b200.host_api import DecayedHostPipeline

    g = torch.Generator().manual_seed(62)
    B, H, T, d = 6, 4, 512, 64
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(8).bfloat16().pin_memory() for _ in range(3))
    gamma = torch.tensor([0.9, 0.95, 0.97, 0.99])
    mod = B200ChunkedDecay(gamma, H, 128).to(dev)
    out = torch.empty(B, H, T, d, dtype=torch.bfloat16).pin_memory()
    pipe = DecayedHostPipeline(B, H, T, d, d, torch.bfloat16, n_slabs=4, device=dev, module=mod)
    assert [e - b for b, e in pipe.bounds] == [2, 2, 2]
    pipe.run(q, k, v, out)
    torch.cuda.synchronize()
    whole = mod(q.to(dev), k.to(dev), v.to(dev)).cpu()
    assert rel_to_max(out, whole) <= 2.0 ** -7            # same function; segmenting may differ between the calls
    want = oracle.decayed_state_carry(q.float(), k.float(), v.float(), gamma, 128, 1.0)
    assert rel_to_max(out, want) <= BF16_TOL
    pipe.run(k, q, v, out)                                # buffers and events are reusable
    torch.cuda.synchronize()
    assert rel_to_max(out, mod(k.to(dev), q.to(dev), v.to(dev)).cpu()) <= 2.0 ** -7
    built = DecayedHostPipeline(B, H, T, d, d, torch.bfloat16, gamma, 128, 1.0, n_slabs=2, device=dev)
    built.run(q, k, v, out)
    torch.cuda.synchronize()
    assert rel_to_max(out, want) <= BF16_TOL
    ops_err = pytest.raises(Exception)
    with ops_err:
        pipe.run(q.to(dev), k, v, out)                    # device tensors are not what it takes


def test_gated_contract_past_two_billion_scores(dev):
    """2^31 + 2^27 score elements (4.6 GB): batch and row offsets must not wrap.  The last batch,
    computed alone, gives the same bits as inside the large call, and scaling one batch's values
    scales only that batch's output (linearity in v)."""
    from catopt_b200 import ops

    nb, T, K, dv = 17, 8192, 16384, 128
    g = torch.Generator(device=dev).manual_seed(13)
    s = torch.empty(nb, T, K, dtype=torch.bfloat16, device=dev)
    for b in range(nb):
        s[b].copy_(torch.randn(T, K, device=dev, generator=g))
    gate = torch.rand(T, K, device=dev, generator=g).bfloat16()
    v = torch.randn(nb, K, dv, device=dev, generator=g).bfloat16()
    assert s.numel() > 2 ** 31
    out = ops.gated_contract(s, gate, v)
    alone = ops.gated_contract(s[-1:], gate, v[-1:])
    assert torch.equal(out[-1], alone[0])
    v2 = v.clone()
    v2[3] *= 2
    out2 = ops.gated_contract(s, gate, v2)
    assert torch.equal(out2[3], out[3] * 2) and torch.equal(out2[4], out[4]) and torch.equal(out2[0], out[0])
    ref_rows = ((s[-1, -64:] * gate[-64:]).double() @ v[-1].double())
    assert rel_to_max(out[-1, -64:], ref_rows) <= 4e-3
    ops.check_device_status(dev)


@pytest.mark.parametrize("rows,n_in,n_out", [(512, 2048, 256), (300, 4096, 132), (1024, 1056, 512), (256, 8192, 128)])
def test_linear_deep_reductions_on_the_tensor_cores(dev, rows, n_in, n_out):
    """Reductions deeper than one accumulator segment: the result stays within the fp32 budget
    (the segments' sums are added in fp32), with bias, ragged tiles and a ragged last segment."""
    from catopt_b200 import ops

    g = torch.Generator().manual_seed(rows + n_in)
    x = torch.randn(rows, n_in, generator=g)
    w = torch.randn(n_out, n_in, generator=g) / math.sqrt(n_in)
    b = torch.randn(n_out, generator=g)
    want = x.double() @ w.double().t() + b.double()
    got = ops.linear_f32(x.to(dev), w.to(dev), b.to(dev))
    ops.check_device_status(dev)
    assert rel_to_max(got, want) <= FP32_TOL, (rows, n_in, n_out, rel_to_max(got, want))
    # the same inputs, all positive: the worst case for a truncating accumulator
    xp, wp = x.abs(), w.abs()
    wantp = xp.double() @ wp.double().t()
    gotp = ops.linear_f32(xp.to(dev), wp.to(dev))
    assert rel_to_max(gotp, wantp) <= FP32_TOL, (rows, n_in, n_out, rel_to_max(gotp, wantp))


@pytest.mark.parametrize("B,H,T,d,gam", [(1, 4, 4096, 128, (0.97, 0.999, 0.5, 1.0)), (2, 3, 2048, 64, (0.9, 0.99, 0.9999)),
                                          (1, 2, 3000, 128, (0.98, 0.995)), (1, 16, 8192, 128, None), (4, 8, 4096, 64, None)])
def test_decayed_bf16_few_heads_run_their_segments_in_parallel(dev, B, H, T, d, gam):
    """Fewer heads than half the SMs: the sequence is cut into segments that run at once, each from
    a start state computed up front.  Same function as one CTA walking the head (the C ABI without
    scratch), and within the bf16 budget of the fp64 recurrence."""
    from catopt_b200 import _lib, ops

    lib = _lib.load()
    g = torch.Generator().manual_seed(T + H)
    q, k, v = (torch.randn(B, H, T, d, generator=g).div_(math.sqrt(d)).bfloat16() for _ in range(3))
    gamma = torch.tensor(gam, dtype=torch.float32) if gam else bench_gamma(H)
    assert lib.cb2_decayed_chunk_scratch_bytes(B, H, T, d, d, 128 if T % 128 == 0 else T // 8, _lib.CB2_BF16) > 0
    C = 128 if T % 128 == 0 else T // 8
    qd, kd, vd, gd = q.to(dev), k.to(dev), v.to(dev), gamma.to(dev)
    par = ops.decayed_chunk_fwd(qd, kd, vd, gd, C, 2.0)
    ops.check_device_status(dev)
    serial = torch.empty_like(vd)
    rc = lib.cb2_decayed_chunk_fwd(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), serial.data_ptr(), gd.data_ptr(),
                                   B, H, T, d, d, C, 2.0, _lib.CB2_BF16, None, 0,
                                   ops.device_status(dev).data_ptr(), _lib.stream_ptr())
    assert rc == 0
    ops.check_device_status(dev)
    assert rel_to_max(par, serial) <= 8e-3          # two bf16 roundings of one function
    if T <= 4096:
        want = oracle.decayed_state_carry(q.double(), k.double(), v.double(), gamma.double(), C, 2.0)
        assert rel_to_max(par, want) <= BF16_TOL
        assert rel_to_max(par[:, :, -128:], want[:, :, -128:]) <= BF16_TOL


def bench_gamma(H):
    return torch.tensor([1 - 2.0 ** (-5 - 8 * h / H) for h in range(H)], dtype=torch.float32)


@pytest.mark.parametrize("B,T,D,N,dtype,with_h0", [(1, 2048, 64, 16, torch.float32, True), (1, 4096, 256, 8, torch.bfloat16, False),
                                                    (2, 1024, 96, 4, torch.float32, False), (1, 3072, 32, 32, torch.bfloat16, True)])
def test_scan_few_units_runs_segments_side_by_side(dev, B, T, D, N, dtype, with_h0):
    """A scan with few (batch, channel-block) units is cut into segments that start from
    states computed up front; same function as the one-pass kernel and as the serial oracle."""
    from catopt_b200 import _lib, ops
    from catopt_b200.ops import _scan_parallel_segments

    assert _scan_parallel_segments(B, T, D, N) > 1
    g = torch.Generator().manual_seed(T + D)
    a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, N, generator=g)).to(dtype)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    b = (torch.randn(D, N, generator=g) / 4).to(dtype)
    c = (torch.randn(D, N, generator=g) / 4).to(dtype)
    h0 = torch.randn(B, D, N, generator=g) if with_h0 else None
    wy, wh = oracle.diag_scan_serial(a, x, b, c, h0)
    ad, xd, bd, cd = a.to(dev), x.to(dev), b.to(dev), c.to(dev)
    h0d = h0.to(dev) if with_h0 else None
    y, hT = ops.diag_scan_fwd(ad, xd, bd, cd, h0d, want_state=True)
    ops.check_device_status(dev)
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert rel_to_max(y, wy) <= tol and rel_to_max(hT, wh) <= FP32_TOL
    # the one-pass kernel through the C ABI
    y1 = torch.empty_like(xd)
    h1 = torch.empty(B, D, N, device=dev)
    rc = _lib.load().cb2_diag_scan_fwd(ad.data_ptr(), xd.data_ptr(), bd.data_ptr(), cd.data_ptr(),
                                       h0d.data_ptr() if with_h0 else None, y1.data_ptr(), h1.data_ptr(), B, T, D, N, 0,
                                       _lib.dtype_code(dtype), ops.device_status(dev).data_ptr(), _lib.stream_ptr())
    assert rc == 0
    assert rel_to_max(y.float(), y1.float()) <= (8e-3 if dtype == torch.bfloat16 else 2e-6)
    assert rel_to_max(hT, h1) <= 2e-6


def test_cuda_graph_replay_of_the_segment_parallel_paths(dev):
    """The few-heads decayed path (end states, scan, attention) and the few-units scan path (maps,
    starts, scan) are three launches each; captured and replayed on new inputs they must equal
    eager runs bit for bit."""
    from catopt_b200 import ops
    from catopt_b200.executors import B200ChunkedDecay, B200DiagScan

    g = torch.Generator().manual_seed(12)
    q, k, v = (torch.randn(1, 4, 4096, 64, generator=g).bfloat16().to(dev) / 4 for _ in range(3))
    mod = B200ChunkedDecay(torch.tensor([0.9, 0.97, 0.99, 0.999]), 4, 128).to(dev)
    mod.capture_cuda_graph(q, k, v)
    for scale in (1.0, 0.5):
        kk = k * scale
        assert torch.equal(mod(q, kk, v), mod._forward_impl(q, kk, v))
    assert ops._scan_parallel_segments(1, 2048, 128, 16) > 1
    a = torch.sigmoid(4 + 0.5 * torch.randn(1, 2048, 128, 16, generator=g)).bfloat16().to(dev)
    x = torch.randn(1, 2048, 128, generator=g).bfloat16().to(dev)
    b = (torch.randn(128, 16, generator=g) / 4).bfloat16().to(dev)
    c = (torch.randn(128, 16, generator=g) / 4).bfloat16().to(dev)
    scan = B200DiagScan(b, c, return_state=True).to(dev)
    scan.capture_cuda_graph(a, x)
    x2 = x * 0.5
    y_r, h_r = scan(a, x2)
    y_r, h_r = y_r.clone(), h_r.clone()
    y_e, h_e = scan._forward_impl(a, x2)
    assert torch.equal(y_r, y_e) and torch.equal(h_r, h_e)
    ops.check_device_status(dev)


def test_decayed_bf16_few_heads_unequal_head_dims(dev):
    """Parallel segments with dk != dv below the tile width (zero-filled columns in both kernels)."""
    from catopt_b200 import ops

    B, H, T, dk, dv = 1, 3, 2048, 32, 96
    g = torch.Generator().manual_seed(77)
    q = torch.randn(B, H, T, dk, generator=g).div_(math.sqrt(dk)).bfloat16()
    k = torch.randn(B, H, T, dk, generator=g).div_(math.sqrt(dk)).bfloat16()
    v = torch.randn(B, H, T, dv, generator=g).bfloat16()
    gamma = torch.tensor([0.95, 0.99, 0.999])
    want = oracle.decayed_state_carry(q.double(), k.double(), v.double(), gamma.double(), 128, 1.0)
    par = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 128, 1.0)
    one = ops.decayed_chunk_fwd(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), 128, 1.0, one_pass=True)
    ops.check_device_status(dev)
    assert rel_to_max(par, want) <= BF16_TOL and rel_to_max(one, want) <= BF16_TOL
    assert rel_to_max(par, one) <= 8e-3
