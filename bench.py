"""Benchmark of the lowered-executor hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this repo's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on host cores

Headline workload (``config.workload``): benchmark config 4, decayed causal linear
attention B=16 H=32 T=8192 d=128 bf16, per-head gamma, chunk 128 — per GPU; at
N>1 every rank owns its own contiguous range of the flattened batch x head axis
of a global batch of 16*N (weak scaling, no collective on the path).  A "token"
is one (batch, time) position; a step is one pass of the executor over the
rank's shard.  ``value`` is measured with inputs resident in HBM, ``e2e`` through
the lowered module a catopt user holds (``B200Sink().executors`` on the chunked term
when catopt is importable, else its catopt-free twin) with pinned host buffers copied
in and the result copied out inside the timed region.  ``strong_scaling`` is config 4
itself (global batch 16) with rank r owning ``shard_range(512, r, N)`` of the
(batch, head) units; ``roofline.sustained`` the same launch back to back for two
seconds with the clocks sampled.  ``kernels`` carries the same measurement for the other
lowered executors (configs 1, 2, 3, 5, each with a ``cpu_baseline`` of its own: the
reference's algorithm on the host cores over a bounded sample) and for the kernels
without a config of their own.  One JSON line on stdout (rank 0).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

C4 = dict(B=16, H=32, T=8192, d=128, chunk=128)
L2_BYTES = 126 * 2**20
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic
# bytes, from the ncu captures summarised under profiles/ (small cases of the
# same kernels; traffic grows in proportion to the units processed, so the ratio
# carries over to the full launch).
NCU_TRAFFIC_RATIO = {"decayed_tc": 287.4 / 310.4, "diag_scan": 301.1 / 302.0, "verify": 439.9 / 436.2}
TRAFFIC_SOURCE = "scaled from the ncu capture of a small case of the same kernel (profiles/), not measured in this run"


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def c4_gamma(H: int) -> torch.Tensor:
    return torch.tensor([1 - 2.0 ** (-5 - 8 * h / H) for h in range(H)], dtype=torch.float32)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while a region runs
    (NVML every 2 ms; read-only queries)."""

    def __init__(self, index: int) -> None:
        self.index = index
        self.mhz: list[int] = []
        self.max_mhz: int | None = None
        self.reason_bits = 0
        self._stop = threading.Event()
        self._thr: threading.Thread | None = None

    def _run(self) -> None:
        try:
            import pynvml as nv

            nv.nvmlInit()
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[self.index]) if self.index < len(ids) else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            while not self._stop.is_set():
                self.mhz.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                self.reason_bits |= nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self._stop.wait(0.002)
        except Exception:
            pass

    def __enter__(self):
        self._stop.clear()
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        time.sleep(0.05)   # let NVML come up before the timed region starts
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=10)

    def summary(self) -> dict:
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap"}
        mhz = sorted(self.mhz)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_min_mhz": mhz[0] if mhz else None,
                "sm_max_mhz": self.max_mhz,
                "reasons": [n for bit, n in names.items() if self.reason_bits & bit],
                "samples": len(mhz)}


# --------------------------------------------------------------------------- timing
def dist_info():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, local, world


def barrier(world: int) -> None:
    if world > 1:
        torch.distributed.barrier()


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def time_steps(step, steps: int, warmup: int, world: int, flush: torch.Tensor | None = None) -> float:
    """Total device milliseconds of exactly ``steps`` calls, max over ranks.

    Large workloads (inputs > L2) are timed as one region; with ``flush`` given,
    each step is timed by its own event pair and L2 is overwritten in between.
    """
    for _ in range(warmup):
        step()
    barrier(world)
    torch.cuda.synchronize()
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(steps)]
        for a, b in evs:
            flush.add_(1)
            a.record()
            step()
            b.record()
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in evs)
    barrier(world)
    return max_over_ranks(ms, world)


# --------------------------------------------------------------------------- CPU legs
def cpu_reference_step_fn(heads: int = 1):
    """One bounded sample of the headline workload on the host cores: the
    reference's pairwise-chunked executor algorithm (restated in oracle/), fp32
    on bf16-rounded inputs, for ``heads`` of the 512 (batch, head) slices."""
    from oracle import oracle

    T, d, C, H = C4["T"], C4["d"], C4["chunk"], C4["H"]
    g = torch.Generator().manual_seed(1234)
    q, k, v = (torch.randn(1, heads, T, d, generator=g).div_(math.sqrt(d)).bfloat16().float()
               for _ in range(3))
    gamma = c4_gamma(H)[:heads]

    def step():
        with torch.no_grad():
            return oracle.decayed_chunked_pairwise(q, k, v, gamma, C, 1.0)

    tokens = heads * T / H  # token-equivalents: a token is one (b,t) position over all 32 heads
    return step, tokens


def cpu_extras(cores: int) -> dict:
    """The reference's CPU algorithm (oracle port, all host threads) on a bounded sample of the
    other configs, keyed like ``bench_extras``'s entries; a few seconds in total."""
    from oracle import oracle

    g = torch.Generator().manual_seed(99)
    out = {}

    def entry(step, tokens, passes, sample, n_calls=30):
        def call():
            for _ in range(passes):
                step()

        m = meter_cpu(call, 5, n_calls)
        return {"value": tokens * passes / m["median_s"], "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": sample + f"; median of {m['n_calls']} calls after {m['warmup']} warm-ups "
                                   f"(iqr {m['iqr_s'] * 1e3:.3f} ms)"}

    with torch.no_grad():
        # config 1: the folded module's forward, linear(x, W_folded)
        wf = torch.randn(512, 512, generator=g) / math.sqrt(512)
        x = torch.randn(64, 512, generator=g)
        out["config1_folded_chain_fp32"] = entry(lambda: oracle.linear(x, wf), 64, 200,
                                                 "200 forwards of the folded module at full size")
        # config 2 at full size: the pairwise-chunked executor algorithm
        q, k, v = (torch.randn(2, 4, 1024, 64, generator=g) / 8 for _ in range(3))
        g2 = torch.tensor(0.97)
        out["config2_decayed_fp32"] = entry(lambda: oracle.decayed_chunked_pairwise(q, k, v, g2, 64, 1.0),
                                            2 * 1024, 1, "1 pass at full size per call")
        # config 3: a quarter of the steps of one of the 8 batch entries, serial fold of the
        # reference's bindings with readout
        a = torch.sigmoid(4 + 0.5 * torch.randn(1, 1024, 1024, 16, generator=g)).bfloat16()
        xs = torch.randn(1, 1024, 1024, generator=g).bfloat16()
        b3 = (torch.randn(1024, 16, generator=g) / 4).bfloat16()
        c3 = (torch.randn(1024, 16, generator=g) / 4).bfloat16()
        out["config3_diag_scan_bf16"] = entry(lambda: oracle.diag_scan_serial(a, xs, b3, c3), 1024, 1,
                                              "1 pass over 1024 of the 4096 steps of 1 of the 8 batch entries "
                                              "(D=1024, N=16)", n_calls=10)
        # config 5: one check of 4 probes (the reference's four eager passes per pair)
        ref = torch.randn(4, 4 * 512 * 1024, generator=g).bfloat16()
        outp = (ref.float() * 1.003).bfloat16()
        out["config5_verify_bf16"] = entry(
            lambda: [oracle.verify_pair(ref[i], outp[i], rtol=2e-2) for i in range(4)], 4 * 4 * 512, 1,
            "1 check x 4 probes of [4,512,1024] bf16 (of 13 x 256) per call")
    return out


def time_cpu(step, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) * 1e3


def meter_cpu(step, warmup: int = 5, n_calls: int = 30) -> dict:
    """The reference's timing contract (``TorchMeter.time``, catopt_torch/meter.py:77-136):
    ``warmup`` untimed calls, then ``n_calls`` timed ones; median and inter-quartile range
    of the wall seconds of a call."""
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(max(n_calls, 1)):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    n = len(ts)
    return {"median_s": ts[n // 2], "iqr_s": ts[(3 * n) // 4] - ts[n // 4], "n_calls": n, "warmup": warmup}


def run_reference(args) -> None:
    rank, _, world = dist_info()
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    step, tokens = cpu_reference_step_fn(heads=4)
    m = meter_cpu(step, args.warmup, args.steps)
    ms = m["median_s"] * 1e3 * args.steps
    value = tokens / m["median_s"]
    sample = ("4 of 512 (batch,head) slices of config 4 per step (T=8192, d=128, chunk 128), fp32 on "
              "bf16-rounded inputs, pairwise-chunked executor algorithm; tokens = slice share of a "
              f"32-head position; median of {m['n_calls']} timed steps after {m['warmup']} warm-ups "
              f"(iqr {m['iqr_s'] * 1e3:.1f} ms), the reference's own timing contract")
    line = {
        "impl": "reference", "metric": "tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int) -> dict:
    return {"workload": "config4_decayed_attention_B16_H32_T8192_d128_bf16_chunk128_per_gpu",
            "global_batch": C4["B"] * n_gpus, "heads": C4["H"], "seq_len": C4["T"], "d_head": C4["d"],
            "chunk": C4["chunk"], "parallelism": f"batch x head shards over {n_gpus} GPU(s), no collective",
            "l2_policy": "inputs (4.3 GB per GPU) exceed L2; small kernels flush L2 between steps"}


# --------------------------------------------------------------------------- catopt-facing pieces
def catopt_importable() -> str | None:
    """Put catopt on the path when it is around ($CATOPT_SRC checkout, or the offline install
    under baseline/_ref that travels with this tree); returns where it came from."""
    try:
        import catopt_core  # noqa: F401

        return "already importable"
    except ImportError:
        pass
    import glob

    src = os.environ.get("CATOPT_SRC")
    paths = sorted(glob.glob(os.path.join(src, "packages", "*", "src"))) if src else []
    if paths:
        sys.path[:0] = paths
        return "source checkout"
    ref = ROOT / "baseline" / "_ref"
    if (ref / "catopt_core").is_dir():
        sys.path.insert(0, str(ref))
        return "baseline/_ref"
    return None


def lowered_decay_module(slab_batch: int, H: int, T: int, d: int, C: int, gamma: torch.Tensor, dev):
    """The module a catopt user holds for config 4's block: the chunked term routed through
    ``B200Sink().executors`` (the optimizer's own routing, optimize.py:485-495) and lowered by the
    spec it picks.  Without catopt: the catopt-free twin ``executors.B200ChunkedDecay``."""
    where = catopt_importable()
    if where is not None:
        from catopt_orchestrator.optimize import _route_spec

        from catopt_b200 import sink as b200

        ir = b200.uniform_decayed_term(slab_batch, H, T, d, C, per_head=True, scale=1.0)
        spec = _route_spec(ir.root, b200.B200Sink())
        if spec is None or spec.name != "b200_om_decayed_chunked":
            raise SystemExit(f"config 4's term was routed to {getattr(spec, 'name', None)}")
        mod = spec.lower(ir, {"g": gamma.to(dev)})
        if not spec.engaged(mod):
            raise SystemExit("the lowered module did not engage the kernel path")
        return mod, f"sink.B200ChunkedDecayModule via B200Sink().executors[{spec.name}] (catopt from {where})"
    from catopt_b200.executors import B200ChunkedDecay

    return B200ChunkedDecay(gamma, H, C, 1.0).to(dev), "executors.B200ChunkedDecay (catopt not importable here)"


def decoder_pairs(probes: range, dev, n_blocks: int = 12):
    """Config 5's tensor pairs from REAL decoder outputs: for every probe (seeded by its index)
    the bf16 original of the 12-block decoder against its optimized graph — fused q/k/v and
    gate/up projections (the pairings the reference's search finds on this model) and the decayed
    attention of every block through this library's chunked kernel instead of the quadratic form
    — per block on the input the ORIGINAL forward hands that block (the reference's block gate,
    optimize.py:1334-1368, 3555) plus the end-to-end pair.  Returns ref, out as
    ``[13, probes * 4*512*1024]`` bf16 (all probes of a check back to back)."""
    sys.path.insert(0, str(ROOT / "tests"))
    from decoder_model import decoder

    from catopt_b200 import ops

    model = decoder(n_blocks).to(dev).bfloat16()
    H, dh = 16, 64
    gam = torch.full((H,), 0.97, device=dev)
    fused = []
    for blk in model:
        a, m = blk.attn, blk.mlp
        fused.append((torch.cat([a.q.weight, a.k.weight, a.v.weight]).contiguous(),
                      torch.cat([m.gate.weight, m.up.weight]).contiguous()))

    def opt_block(blk, wf, x):
        B, T, dim = x.shape
        h = blk.norm1(x)
        q, k, v = (t.reshape(B, T, H, dh).transpose(1, 2).contiguous() for t in (h @ wf[0].T).split(dim, -1))
        o = ops.decayed_chunk_fwd(q, k, v, gam, 128, math.sqrt(dh))
        x = x + blk.attn.o(o.transpose(1, 2).reshape(B, T, dim))
        gu = blk.norm2(x) @ wf[1].T
        g_, u_ = gu.split(gu.shape[-1] // 2, -1)
        return x + blk.mlp.down(torch.nn.functional.silu(g_) * u_)

    n = 4 * 512 * 1024
    ref = torch.empty(n_blocks + 1, len(probes) * n, dtype=torch.bfloat16, device=dev)
    out = torch.empty_like(ref)
    with torch.no_grad():
        for j, p in enumerate(probes):
            x = torch.randn(4, 512, 1024, generator=torch.Generator().manual_seed(5000 + p)).bfloat16().to(dev)
            xo = x
            for i, blk in enumerate(model):
                y = blk(x)
                ref[i, j * n:(j + 1) * n] = y.reshape(-1)
                out[i, j * n:(j + 1) * n] = opt_block(blk, fused[i], x).reshape(-1)
                xo = opt_block(blk, fused[i], xo)
                x = y
            ref[n_blocks, j * n:(j + 1) * n] = x.reshape(-1)
            out[n_blocks, j * n:(j + 1) * n] = xo.reshape(-1)
    return ref, out


# --------------------------------------------------------------------------- GPU side
def _randn_bf16(shape, gen, scale=1.0, dev="cuda"):
    """Seeded N(0,1)*scale in bf16, generated slab by slab to bound fp32 temporaries."""
    out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
    flat = out.view(shape[0], -1)
    for i in range(shape[0]):
        flat[i].copy_(torch.randn(flat.shape[1], device=dev, generator=gen).mul_(scale))
    return out


def graph_replay_us(module, inputs: tuple, K: int, W: int, world: int, flush: torch.Tensor) -> float:
    """Microseconds per call of ``module`` once captured with its own ``capture_cuda_graph``
    (inputs copied into the static buffers, one graph launch), L2 flushed between calls."""
    module.capture_cuda_graph(*inputs)
    with torch.no_grad():
        ms = time_steps(lambda: module(*inputs), K, W, world, flush)
    module.drop_cuda_graph()
    return ms / K * 1e3


def bench_extras(args, rank: int, world: int, pk: dict, flush: torch.Tensor) -> dict:
    """The other lowered executors (configs 1, 2, 3, 5), same timing contract."""
    from catopt_b200 import ops
    from catopt_b200.executors import B200FoldedLinear
    from catopt_b200.sharding import shard_range

    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    K, W = args.steps, args.warmup
    hbm = pk["hbm_gbs"] * 1e9
    out = {}

    def entry(ms_total, tokens, abytes, launches, note, flops=None, traffic_key=None):
        t = ms_total / K / 1e3
        traffic = int(abytes * NCU_TRAFFIC_RATIO[traffic_key]) if traffic_key else None
        e = {"tokens_per_s": world * tokens / t, "us_per_step": t * 1e6,
             "roofline": {"bound": "hbm", "achieved": abytes / t / 1e9, "peak": pk["hbm_gbs"],
                          "unit": "GB/s", "frac": abytes / t / hbm, "traffic": traffic,
                          "traffic_source": TRAFFIC_SOURCE if traffic else None},
             "gpu_launches_per_step": launches, "note": note}
        if flops:
            e["tflops"] = flops / t / 1e12
        return e

    # config 1: 8 x Linear(512,512) fp32 folded once, then one GEMM on x[64,512]
    ws = [torch.randn(512, 512, device=dev, generator=gen) / math.sqrt(512) for _ in range(8)]
    mod = B200FoldedLinear(ws)
    x = torch.randn(64, 512, device=dev, generator=gen)
    y = torch.empty(64, 512, device=dev)
    ms = time_steps(lambda: ops.linear_f32(x, mod.weight, out=y), K, W, world, flush)
    out["config1_folded_chain_fp32"] = entry(ms, 64, (512 * 512 + 2 * 64 * 512) * 4, 1,
                                             "latency-bound: 64 rows; L2 flushed between steps",
                                             flops=2 * 64 * 512 * 512)
    # the reference delivers small modules as CUDA graphs (executors/base.py:180-220): replay cost per call
    out["config1_folded_chain_fp32"]["graph_replay_us"] = graph_replay_us(mod, (x,), K, W, world, flush)
    # the reference's published shape: R=4096 rows through the folded weight
    x4 = torch.randn(4096, 512, device=dev, generator=gen)
    y4 = torch.empty(4096, 512, device=dev)
    ms = time_steps(lambda: ops.linear_f32(x4, mod.weight, out=y4), K, W, world, flush)
    out["folded_chain_fp32_R4096"] = entry(ms, 4096, (512 * 512 + 2 * 4096 * 512) * 4, 1,
                                           "reference's published cell k8_d512_R4096",
                                           flops=2 * 4096 * 512 * 512)
    del ws, x4, y4

    # config 2: B=2 H=4 T=1024 d=64 fp32, gamma 0.97, chunk 64
    q, k, v = (torch.randn(2, 4, 1024, 64, device=dev, generator=gen) / 8 for _ in range(3))
    g2 = torch.full((4,), 0.97, device=dev)
    o2 = torch.empty_like(v)
    ms = time_steps(lambda: ops.decayed_chunk_fwd(q, k, v, g2, 64, 1.0, out=o2), K, W, world, flush)
    out["config2_decayed_fp32"] = entry(ms, 2 * 1024, 4 * 2 * 4 * 1024 * 64 * 4, 1,
                                        "latency-bound: 8 heads; L2 flushed between steps",
                                        flops=8 * 1024 * (4 * 64 * 64 + 4 * 64 * 64))
    from catopt_b200.executors import B200ChunkedDecay

    out["config2_decayed_fp32"]["graph_replay_us"] = graph_replay_us(B200ChunkedDecay(0.97, 4, 64).to(dev), (q, k, v),
                                                                     K, W, world, flush)
    del q, k, v, o2

    # fp32 decayed attention at many heads (B=16 H=32 T=2048 d=64): three-pass TF32 on the tensor cores.
    # Flops: per 128-row chunk Q.K^T and P.V (2*128*128*64 each), Q.St and K^T.V (2*128*64*64 each),
    # each taken three times.
    Bf, Hf, Tf, df = 16, 32, 2048, 64
    qf, kf, vf = (torch.randn(Bf, Hf, Tf, df, device=dev, generator=gen) / 8 for _ in range(3))
    gf = c4_gamma(Hf).to(dev)
    of = torch.empty_like(vf)
    ms = time_steps(lambda: ops.decayed_chunk_fwd(qf, kf, vf, gf, 128, 1.0, out=of), K, W, world)
    out["decayed_fp32_B16_H32_T2048_d64"] = entry(
        ms, Bf * Tf, 4 * Bf * Hf * Tf * df * 4, 1,
        "fp32 tensors, 3xTF32 tcgen05 (one CTA per unit, 512 units = 3.5 waves); 1.07 GB exceed L2; tflops counts "
        "the three passes",
        flops=3 * Bf * Hf * (Tf // 128) * (2 * 2 * 128 * 128 * df + 2 * 2 * 128 * df * df))
    del qf, kf, vf, of

    # config 3: scan B=8 D=1024 N=16 T=4096 bf16; ranks own channel blocks of the (b,d) axis
    B, T, D, N = 8, 4096, 1024, 16
    x3 = _randn_bf16((B, T, D), gen)
    a3 = torch.empty(B, T, D, N, dtype=torch.bfloat16, device=dev)
    for b in range(B):
        a3[b].copy_(torch.sigmoid(4 + 0.5 * torch.randn(T, D, N, device=dev, generator=gen)))
    b3 = (torch.randn(D, N, device=dev, generator=gen) / 4).bfloat16()
    c3 = (torch.randn(D, N, device=dev, generator=gen) / 4).bfloat16()
    y3 = torch.empty_like(x3)
    ms = time_steps(lambda: ops.diag_scan_fwd(a3, x3, b3, c3, None, out=y3), K, W, world)
    out["config3_diag_scan_bf16"] = entry(ms, B * T, (B * T * D * (N + 2) + 2 * D * N) * 2, 1,
                                          "inputs 1.2 GB exceed L2", flops=5 * B * T * D * N,
                                          traffic_key="diag_scan")
    # config 3 with the decay shared over n (a is [B,T,D]): 201 MB
    a3s = torch.empty(B, T, D, dtype=torch.bfloat16, device=dev)
    for b in range(B):
        a3s[b].copy_(torch.sigmoid(4 + 0.5 * torch.randn(T, D, device=dev, generator=gen)))
    ms = time_steps(lambda: ops.diag_scan_fwd(a3s, x3, b3, c3, None, out=y3), K, W, world)
    out["config3_shared_decay_bf16"] = entry(ms, B * T, (3 * B * T * D + 2 * D * N) * 2, 1,
                                             "a broadcast over n: collapsed scalar recurrence; 201 MB exceed L2",
                                             flops=4 * B * T * D)
    del a3, a3s, x3, y3

    # config 3 as the reference's scan executor sees it (a tree of 4096 leaf maps over the state
    # [8,1024,16], final state only): stacked leaves in product order, fp32, 2 x 2.1 GB
    Tt, St = 4096, 8 * 1024 * 16
    al = torch.empty(Tt, St, device=dev)
    bl = torch.empty(Tt, St, device=dev)
    for t0 in range(0, Tt, 512):
        al[t0:t0 + 512].copy_(torch.sigmoid(4 + 0.5 * torch.randn(512, St, device=dev, generator=gen)))
        bl[t0:t0 + 512].copy_(torch.randn(512, St, device=dev, generator=gen))
    hl = torch.zeros(St, device=dev)
    ms = time_steps(lambda: ops.diag_compose_apply(al, bl, hl), K, W, world)
    out["config3_scan_tree_final_state_fp32"] = entry(
        ms, 8 * Tt, 2 * Tt * St * 4, 2,
        "composed map of 4096 stacked leaf maps (what BatchedScanModule reduces level by level); 4.3 GB exceed L2",
        flops=3 * Tt * St)
    del al, bl, hl

    # all prefix maps of 1024 diagonal steps over config 3's state (what the omd executor's
    # _prefix_scan builds), fp32: a and b read once, both maps written once (4 x 0.54 GB)
    Tp = 1024
    ap = torch.sigmoid(4 + 0.5 * torch.randn(Tp, St, device=dev, generator=gen))
    bp = torch.randn(Tp, St, device=dev, generator=gen)
    ms = time_steps(lambda: ops.diag_prefix_maps(ap, bp), K, W, world)
    out["config3_all_prefix_maps_fp32_T1024"] = entry(
        ms, 8 * Tp, 4 * Tp * St * 4, 1,
        "one pass: 2 reads + 2 writes of [1024, 8*1024*16] fp32 (2.1 GB > L2); includes the allocation of the two outputs",
        flops=3 * Tp * St)
    # every state of the same 1024 steps from an initial state (the stacked-map form of an unrolled
    # scan, spec b200_scan_all): a and b read once, the states written once (3 x 0.54 GB)
    hp = torch.randn(St, device=dev, generator=gen)
    ms = time_steps(lambda: ops.diag_scan_states(ap, bp, hp), K, W, world)
    out["config3_all_states_fp32_T1024"] = entry(
        ms, 8 * Tp, 3 * Tp * St * 4, 1,
        "one pass: 2 reads + 1 write of [1024, 8*1024*16] fp32 (1.6 GB > L2); includes the allocation of the output",
        flops=2 * Tp * St)
    del ap, bp, hp

    # causal online-softmax executor (no config of its own in the benchmark spec), bf16, d=128:
    # a long-sequence case that fills the GPU (268 MB > L2) and a short one (256 CTAs: tail-bound)
    for (Bo, Ho, To) in ((1, 32, 8192), (2, 8, 2048)):
        qo, ko, vo = (_randn_bf16((Bo * Ho, To * 128), gen).view(Bo, Ho, To, 128) for _ in range(3))
        oo = torch.empty_like(vo)
        ms = time_steps(lambda: ops.om_causal_fwd(qo, ko, vo, out=oo), K, W, world,
                        flush if To < 8192 else None)
        e = entry(ms, Bo * To, 4 * Bo * Ho * To * 128 * 2, 1,
                  "tcgen05 online-softmax kernel; causal FLOPs (lower triangle) against the burst bf16 peak; "
                  + ("inputs exceed L2" if To >= 8192 else "L2 flushed between steps"),
                  flops=4 * Bo * Ho * (To * (To + 1) // 2) * 128)
        e["roofline"] = {"bound": "tensor", "achieved": e["tflops"], "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": e["tflops"] / pk["bf16_tflops"], "traffic": None}
        out[f"om_causal_bf16_B{Bo}_H{Ho}_T{To}_d128"] = e
        del qo, ko, vo, oo

    # streaming step of the same monoid in the decode regime: one query row per head against 65536
    # cached keys (bf16, d=128): K and V are read once (1.07 GB)
    qd = _randn_bf16((32, 128), gen).view(1, 32, 1, 128)
    kd, vd = (_randn_bf16((32, 65536 * 128), gen).view(1, 32, 65536, 128) for _ in range(2))
    ms = time_steps(lambda: ops.om_step_qk(None, qd, kd, vd, 0.09, True, -65535), K, W, world)
    out["om_step_decode_bf16_H32_Tk65536_d128"] = entry(
        ms, 32, 2 * 32 * 65536 * 128 * 2, 2,
        "one decode step (Tq = 1) folding 65536 keys into the carrier (m, l, a); K + V read once (1.07 GB > L2)",
        flops=4 * 32 * 65536 * 128)
    del qd, kd, vd

    # decayed attention with few heads (small batch, long sequence): 16 heads x T=8192, d=128 bf16;
    # a head's segments run in parallel from start states computed up front (3 launches)
    qf, kf, vf = (_randn_bf16((16, 8192 * 128), gen, 1 / math.sqrt(128)).view(2, 8, 8192, 128) for _ in range(3))
    gf = c4_gamma(8).to(dev)
    of = torch.empty_like(vf)
    ms = time_steps(lambda: ops.decayed_chunk_fwd(qf, kf, vf, gf, 128, 1.0, out=of), K, W, world, flush)
    out["decayed_bf16_few_heads_B2_H8_T8192_d128"] = entry(
        ms, 2 * 8192, 4 * 16 * 8192 * 128 * 2, 3,
        "16 heads on 148 SMs: 8 parallel segments per head, start states from decayed_seg_state (K and V read "
        "twice); 134 MB, L2 flushed between steps; one CTA per head takes 189 us",
        flops=16 * 8192 * (4 * 128 * 128 + 4 * 128 * 128))
    del qf, kf, vf, of

    # the om_decayed element on materialised scores, (s*g)@v (the site the reference's generated
    # fused-contraction kernel lowers): B=2 H=16 T=K=4096 dv=128 bf16, one gate for all heads
    sg = _randn_bf16((32, 4096 * 4096), gen).view(2, 16, 4096, 4096)
    vg = _randn_bf16((32, 4096 * 128), gen).view(2, 16, 4096, 128)
    gg = torch.rand(4096, 4096, device=dev, generator=gen).bfloat16()
    ms = time_steps(lambda: ops.gated_contract(sg, gg, vg), K, W, world)
    out["gated_contract_bf16_B2_H16_T4096_K4096_dv128"] = entry(
        ms, 2 * 4096, (sg.numel() + gg.numel() + 2 * vg.numel()) * 2, 1,
        "scores 1.07 GB read once, gate (33.5 MB) shared by all heads; P = s*g kept in tensor memory",
        flops=2 * 32 * 4096 * 4096 * 128)
    del sg, vg, gg

    # config 5: verify 13 checks x 256 probes x [4,512,1024] bf16; probes sharded over ranks.
    # The pairs are real decoder outputs: the bf16 original against its optimized graph, per block
    # and end to end, for every probe of this rank (built once, outside the timed region).
    n_probes = args.probes
    p0, p1 = shard_range(n_probes, rank, world)
    probes = p1 - p0
    ref, outp = decoder_pairs(range(p0, p1), dev)
    res = torch.empty(13, 4, device=dev)

    def verify_step():
        ops.verify_reduce(ref, outp, 13, result=res)
        if world > 1:
            torch.distributed.all_reduce(res, op=torch.distributed.ReduceOp.MAX)

    ms = time_steps(verify_step, K, W, world)
    # the gate's numbers, recomputed with plain tensor ops (and their own max all-reduce): the kernel
    # and the collective must reproduce them exactly
    want = torch.zeros(13, 4, device=dev)
    for ci in range(13):                       # row by row: the difference of one check is a 1 GiB temporary
        want[ci, 0] = (ref[ci] - outp[ci]).abs().max().float()
        want[ci, 1] = ref[ci].abs().max().float()
    if world > 1:
        torch.distributed.all_reduce(want, op=torch.distributed.ReduceOp.MAX)
    if not torch.equal(res, want):
        raise SystemExit("config 5: the verify kernel (+ all-reduce) disagrees with the eager maxima")
    max_rel = (res[:, 0] / (res[:, 1] + 1e-8)).tolist()
    e = entry(ms, probes * 4 * 512, 2 * ref.numel() * 2, 2,
              "13 checks per step (12 block pairs + 1 end-to-end pair of real decoder outputs: bf16 original vs "
              "its optimized graph); ends with one max all-reduce when sharded; result checked against eager maxima",
              traffic_key="verify")
    e["tokens_per_s"] = n_probes * 4 * 512 * 13 / (ms / K / 1e3)  # probe tokens x checks, whole job
    e["probes"] = n_probes
    e["max_rel_per_check"] = [round(v, 6) for v in max_rel]
    e["checks_within_rtol_2e-2"] = f"{sum(v < 2e-2 for v in max_rel)} of 13 (the end-to-end pair carries the bf16 rounding of all 12 blocks)"
    out["config5_verify_bf16"] = e
    del ref, outp

    # a wider folded chain (2048 -> 2048, R = 16384): the reduction is cut into four accumulator segments
    xw = torch.randn(16384, 2048, device=dev, generator=gen)
    ww = torch.randn(2048, 2048, device=dev, generator=gen) / math.sqrt(2048)
    yw = torch.empty(16384, 2048, device=dev)
    ms = time_steps(lambda: ops.linear_f32(xw, ww, out=yw), K, W, world)
    e = entry(ms, 16384, (2048 * 2048 + 2 * 16384 * 2048) * 4, 2,
              "3xTF32 tcgen05, four 512-deep accumulator segments added in fp32 (285 MB > L2); timed last, its sustained tensor load lowers the clocks of whatever follows; fp32-equivalent "
              "FLOPs against a third of the bf16 burst peak's TF32 half (three passes)",
              flops=2 * 16384 * 2048 * 2048)
    tf32_equiv_peak = pk["bf16_tflops"] / 2 / 3
    e["roofline"] = {"bound": "tensor", "achieved": e["tflops"], "peak": tf32_equiv_peak, "unit": "TFLOP/s",
                     "frac": e["tflops"] / tf32_equiv_peak, "traffic": None}
    out["folded_chain_fp32_R16384_2048x2048"] = e
    del xw, ww, yw
    ops.check_device_status(dev)
    return out


def run_ours(args) -> None:
    rank, local, world = dist_info()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # Keep stdout for the ONE JSON line: anything libraries print on fd 1 (NCCL's
    # version banner, for one) is sent to stderr; the line is written to the saved
    # descriptor at the end.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    from catopt_b200 import _lib, build, ops
    from catopt_b200.host_api import DecayedHostPipeline

    if not _lib.LIB_PATH.exists() and rank == 0:
        build.build()
    barrier(world)
    pk = peaks()
    B, H, T, d, C = (C4[k] for k in ("B", "H", "T", "d", "chunk"))
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v = (_randn_bf16((B * H, T * d), gen, 1 / math.sqrt(d)).view(B, H, T, d) for _ in range(3))
    gamma = c4_gamma(H).to(dev)
    o = torch.empty_like(v)
    code = _lib.CB2_BF16
    path = "tcgen05" if _lib.load().cb2_decayed_chunk_on_tensor_cores(B, H, T, d, d, C, code) else "ffma"
    launches_per_step = 1 if path == "tcgen05" else 3

    def step():
        ops.decayed_chunk_fwd(q, k, v, gamma, C, 1.0, out=o)

    def region_status(region: str) -> None:
        """A bounded device wait that ran out inside a timed region invalidates it: say which."""
        try:
            ops.check_device_status(dev)
        except Exception as e:  # noqa: BLE001
            raise SystemExit(f"rank {rank}: {e} after {region}") from e

    clk = ClockSampler(local)
    with clk:
        ms = time_steps(step, args.steps, args.warmup, world)
    region_status("the headline region")
    ops.check_device_status(dev)
    tokens = B * T
    t_step = ms / args.steps / 1e3
    abytes = 4 * B * H * T * d * 2
    flops = B * H * T * (4 * C * d + 4 * d * d)

    # strong scaling: config 4 ITSELF (global batch 16, 512 (batch, head) units) cut over the ranks;
    # every rank runs its contiguous share of the units (64 per rank at 8 GPUs), no collective
    from catopt_b200.sharding import shard_units_of_heads

    u0, u1, gs = shard_units_of_heads(gamma, B, rank, world)
    nu = u1 - u0
    qs, ks, vs = (t.view(B * H, T, d)[u0:u1].unsqueeze(0) for t in (q, k, v))     # [1, units, T, d] views
    os_ = torch.empty(1, nu, T, d, dtype=torch.bfloat16, device=dev)
    lib = _lib.load()
    sbytes = lib.cb2_decayed_chunk_scratch_bytes(1, nu, T, d, d, C, code)

    def strong_step():
        ops.decayed_chunk_fwd(qs, ks, vs, gs, C, 1.0, out=os_)

    fl = torch.zeros(2 * L2_BYTES, dtype=torch.uint8, device=dev) if nu * T * d * 8 < 2 * L2_BYTES else None
    ms_strong = time_steps(strong_step, args.steps, args.warmup, world, fl)
    from catopt_b200 import verify

    rep_s = verify.verify_equiv(o.view(B * H, T, d)[u0:u1].contiguous(), os_.view(nu, T, d), rtol=1e-2)
    if not rep_s.passed:          # same units, other segmenting: equal within bf16 rounding
        raise SystemExit(f"strong-scaling shard differs from the same units of the full launch: {rep_s}")
    t_strong = ms_strong / args.steps / 1e3
    strong = {"global_batch": B, "units_total": B * H, "units_per_rank": nu, "ms_per_step": t_strong * 1e3,
              "tokens_per_s": tokens / t_strong, "speedup_over_one_gpu_sized_step": t_step / t_strong,
              "note": "speedup = this run's own 512-unit step time (the headline step, one GPU's worth) over the "
                      "sharded step time, max over ranks",
              "path": {-1: "not on the tensor cores", 0: "one CTA per unit",
                       1: "segments of a unit handing their state over in scratch",
                       2: "parallel segments from start states computed by a pre-pass",
                       3: "two CTAs per unit in one launch, the second accumulating the first's state itself"}[
                  lib.cb2_decayed_chunk_plan(1, nu, T, d, d, C, code)],
              "scratch_bytes": int(sbytes), "vs_full_launch_max_rel": rep_s.max_rel,
              "hbm_floor_ms": 4 * nu * T * d * 2 / (pk["hbm_gbs"] * 1e9) * 1e3}
    del qs, ks, vs, os_, fl

    # sustained: the same launch back to back for two seconds and more, clocks sampled throughout
    # (after the burst measurements above: it leaves the GPU at its power cap)
    n_sus = max(50, int(2.2 / t_step))
    clk_sus = ClockSampler(local)
    with clk_sus:
        ms_sus = time_steps(step, n_sus, 3, world)
    region_status("the sustained loop")
    sus = clk_sus.summary()
    t_sus = ms_sus / n_sus / 1e3
    chunks_per_sm = B * H * (T // 128) / 148.0
    sustained = {"launches": n_sus, "seconds": ms_sus / 1e3, "ms_per_launch": t_sus * 1e3,
                 "achieved": abytes / t_sus / 1e9, "frac": abytes / t_sus / (pk["hbm_gbs"] * 1e9),
                 "sm_mhz_median": sus["sm_mhz"], "sm_mhz_min": sus["sm_min_mhz"], "reasons": sus["reasons"],
                 "cycles_per_128_row_chunk": (t_sus * (sus["sm_mhz"] or 0) * 1e6 / chunks_per_sm) if sus["sm_mhz"] else None,
                 "hbm_floor_cycles_per_chunk": (abytes / (pk["hbm_gbs"] * 1e9) * (sus["sm_mhz"] or 0) * 1e6 / chunks_per_sm)
                 if sus["sm_mhz"] else None}

    # end to end: pinned host buffers in, result out, every step, through the lowered module
    n_slabs = 8
    mod, mod_name = lowered_decay_module(B // n_slabs, H, T, d, C, gamma, dev)
    pipe = DecayedHostPipeline(B, H, T, d, d, torch.bfloat16, n_slabs=n_slabs, device=dev, module=mod)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(B, H, T, d, dtype=torch.bfloat16).pin_memory()
    del q, k, v
    clk_e2e = ClockSampler(local)   # its own sampler: this region is PCIe-bound and barely loads the SMs
    with clk_e2e:
        ms_e2e = time_steps(lambda: pipe.run(hq, hk, hv, ho), args.steps, args.warmup, world)
    region_status("the end-to-end region")
    # same function, other segmenting (a slab has few heads: its segments start from precomputed
    # states): equal within bf16 rounding, checked with the library's own gate
    rep = verify.verify_equiv(o, ho.to(dev), rtol=1e-2)
    if not rep.passed:
        raise SystemExit(f"e2e result differs from the device-resident result: {rep}")
    slab_units = (B // n_slabs) * H
    slab_launches = 1 if slab_units * 2 > 148 else 2
    e2e_launches = (launches_per_step if path != "tcgen05" else slab_launches) * len(pipe.bounds)
    del pipe, hq, hk, hv, ho, o
    torch.cuda.empty_cache()

    flush = torch.zeros(2 * L2_BYTES, dtype=torch.uint8, device=dev)
    extras = bench_extras(args, rank, world, pk, flush) if not args.no_extras else {}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        cstep, ctok = cpu_reference_step_fn(heads=4)
        cm = meter_cpu(cstep, 5, 30)
        cpu = {"value": ctok / cm["median_s"], "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": "4 of 512 (batch,head) slices of config 4 per call, fp32 on bf16-rounded inputs, the "
                         f"reference's pairwise-chunked algorithm; median of {cm['n_calls']} calls after "
                         f"{cm['warmup']} warm-ups (iqr {cm['iqr_s'] * 1e3:.1f} ms)"}
        if extras:
            for name, cb in cpu_extras(cores).items():
                if name in extras:
                    extras[name]["cpu_baseline"] = cb
    if rank != 0:
        return
    line = {
        "metric": "tokens/s", "value": world * tokens / t_step, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(world),
        "roofline": {"bound": "hbm", "achieved": abytes / t_step / 1e9, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": abytes / t_step / (pk["hbm_gbs"] * 1e9),
                     "traffic": int(abytes * NCU_TRAFFIC_RATIO["decayed_tc"]) if path == "tcgen05" else None,
                     "peak_source": pk["source"], "kernel": f"decayed_chunk ({path})",
                     "traffic_source": TRAFFIC_SOURCE if path == "tcgen05" else None,
                     "tensor_tflops": flops / t_step / 1e12,
                     "tensor_frac_of_sustained": flops / t_step / (pk["bf16_tflops_sustained"] * 1e12),
                     "sustained": sustained},
        "e2e": {"value": world * tokens / (ms_e2e / args.steps / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": 3 * B * H * T * d * 2, "d2h_bytes_per_step": B * H * T * d * 2,
                "ms_per_step": ms_e2e / args.steps, "clocks": clk_e2e.summary(), "module": mod_name,
                "slabs": n_slabs, "vs_device_resident_max_rel": rep.max_rel},
        "strong_scaling": strong,
        "gpu_launches": args.steps * launches_per_step,
        "e2e_gpu_launches": args.steps * e2e_launches,
        "clocks": clk.summary(),
        "kernels": extras,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    sys.stdout.flush()
    os.write(json_fd, (json.dumps(line) + "\n").encode())


def run_profile_case(args) -> None:
    """A small, L2-exceeding case of ONE kernel, a few launches, for ncu captures."""
    from catopt_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(7)
    n = max(args.steps, 1)
    if args.profile_case == "decayed":      # 148 heads x T=2048: 310 MB of q,k,v,o
        B, H, T, d = 2, 74, 2048, 128
        q, k, v = (_randn_bf16((B * H, T * d), gen, 1 / math.sqrt(d)).view(B, H, T, d) for _ in range(3))
        gamma = c4_gamma(H).to(dev)
        o = torch.empty_like(v)
        fn = lambda: ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0, out=o)  # noqa: E731
    elif args.profile_case == "scan":       # config 3 at T=1024: 302 MB
        B, T, D, N = 8, 1024, 1024, 16
        x = _randn_bf16((B, T * D), gen).view(B, T, D)
        a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, N, device=dev, generator=gen)).bfloat16()
        b = (torch.randn(D, N, device=dev, generator=gen) / 4).bfloat16()
        c = (torch.randn(D, N, device=dev, generator=gen) / 4).bfloat16()
        y = torch.empty_like(x)
        fn = lambda: ops.diag_scan_fwd(a, x, b, c, None, out=y)  # noqa: E731
    elif args.profile_case == "scan_shared":  # config 3 with the decay shared over n, full size: 201 MB
        B, T, D, N = 8, 4096, 1024, 16
        x = _randn_bf16((B, T * D), gen).view(B, T, D)
        a = torch.sigmoid(4 + 0.5 * torch.randn(B, T, D, device=dev, generator=gen)).bfloat16()
        b = (torch.randn(D, N, device=dev, generator=gen) / 4).bfloat16()
        c = (torch.randn(D, N, device=dev, generator=gen) / 4).bfloat16()
        y = torch.empty_like(x)
        fn = lambda: ops.diag_scan_fwd(a, x, b, c, None, out=y)  # noqa: E731
    elif args.profile_case == "om_causal":    # B=1 H=32 T=8192 d=128 bf16 (268 MB; tensor-bound)
        q, k, v = (_randn_bf16((32, 8192 * 128), gen).view(1, 32, 8192, 128) for _ in range(3))
        o = torch.empty_like(v)
        fn = lambda: ops.om_causal_fwd(q, k, v, out=o)  # noqa: E731
    elif args.profile_case == "compose":      # 1024 stacked leaf maps over config 3's state, fp32: 1.07 GB
        al = torch.sigmoid(4 + 0.5 * torch.randn(1024, 8 * 1024 * 16, device=dev, generator=gen))
        bl = torch.randn(1024, 8 * 1024 * 16, device=dev, generator=gen)
        hl = torch.zeros(8 * 1024 * 16, device=dev)
        fn = lambda: ops.diag_compose_apply(al, bl, hl)  # noqa: E731
    elif args.profile_case == "gated":      # (s*g)@v, B=2 H=16 T=K=2048 dv=128 bf16, one gate: 285 MB
        sg = _randn_bf16((32, 2048 * 2048), gen).view(2, 16, 2048, 2048)
        vg = _randn_bf16((32, 2048 * 128), gen).view(2, 16, 2048, 128)
        gg = torch.rand(2048, 2048, device=dev, generator=gen).bfloat16()
        fn = lambda: ops.gated_contract(sg, gg, vg)  # noqa: E731
    elif args.profile_case == "decayed_few":  # 16 heads x T=8192, d=128 bf16 (134 MB): parallel segments
        q, k, v = (_randn_bf16((16, 8192 * 128), gen, 1 / math.sqrt(128)).view(2, 8, 8192, 128) for _ in range(3))
        gamma = c4_gamma(8).to(dev)
        o = torch.empty_like(v)
        fn = lambda: ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0, out=o)  # noqa: E731
    elif args.profile_case == "decayed_fp32":  # 148 heads x T=2048, d=64 fp32 (310 MB): three-pass TF32 kernel
        q, k, v = (torch.randn(2, 74, 2048, 64, device=dev, generator=gen) / 8 for _ in range(3))
        gamma = c4_gamma(74).to(dev)
        o = torch.empty_like(v)
        fn = lambda: ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0, out=o)  # noqa: E731
    elif args.profile_case == "decayed_strong":  # one rank's share of config 4 cut over 8 GPUs: 64 units (537 MB)
        q, k, v = (_randn_bf16((64, 8192 * 128), gen, 1 / math.sqrt(128)).view(2, 32, 8192, 128) for _ in range(3))
        gamma = c4_gamma(32).to(dev)
        o = torch.empty_like(v)
        fn = lambda: ops.decayed_chunk_fwd(q, k, v, gamma, 128, 1.0, out=o)  # noqa: E731
    elif args.profile_case == "scan_few":     # config 3 with one batch entry (151 MB): 8 segments side by side
        x = _randn_bf16((1, 4096 * 1024), gen).view(1, 4096, 1024)
        a = torch.sigmoid(4 + 0.5 * torch.randn(1, 4096, 1024, 16, device=dev, generator=gen)).bfloat16()
        b = (torch.randn(1024, 16, device=dev, generator=gen) / 4).bfloat16()
        c = (torch.randn(1024, 16, device=dev, generator=gen) / 4).bfloat16()
        y = torch.empty_like(x)
        fn = lambda: ops.diag_scan_fwd(a, x, b, c, None, out=y)  # noqa: E731
    elif args.profile_case == "linear_deep":  # 2048 -> 2048 at R = 16384: four accumulator segments (285 MB)
        x = torch.randn(16384, 2048, device=dev, generator=gen)
        w = torch.randn(2048, 2048, device=dev, generator=gen) / math.sqrt(2048)
        y = torch.empty(16384, 2048, device=dev)
        fn = lambda: ops.linear_f32(x, w, out=y)  # noqa: E731
    elif args.profile_case == "prefix":     # all prefix maps of 256 steps over config 3's state, fp32: 537 MB
        ap_ = torch.sigmoid(4 + 0.5 * torch.randn(256, 8 * 1024 * 16, device=dev, generator=gen))
        bp_ = torch.randn(256, 8 * 1024 * 16, device=dev, generator=gen)
        fn = lambda: ops.diag_prefix_maps(ap_, bp_)  # noqa: E731
    elif args.profile_case == "states":     # every state of 256 steps over config 3's state, fp32: 403 MB
        ap_ = torch.sigmoid(4 + 0.5 * torch.randn(256, 8 * 1024 * 16, device=dev, generator=gen))
        bp_ = torch.randn(256, 8 * 1024 * 16, device=dev, generator=gen)
        hp_ = torch.randn(8 * 1024 * 16, device=dev, generator=gen)
        fn = lambda: ops.diag_scan_states(ap_, bp_, hp_)  # noqa: E731
    elif args.profile_case == "decayed_small":  # config 2 itself (2 MB: a latency case, not a bandwidth one)
        qs, ks, vs = (torch.randn(2, 4, 1024, 64, device=dev, generator=gen) / 8 for _ in range(3))
        gs = torch.full((4,), 0.97, device=dev)
        os_ = torch.empty_like(vs)
        fn = lambda: ops.decayed_chunk_fwd(qs, ks, vs, gs, 64, 8.0, out=os_)  # noqa: E731
    elif args.profile_case == "decode":     # one query row per head against 32768 keys, bf16: K + V = 537 MB
        qd = _randn_bf16((32, 128), gen).view(1, 32, 1, 128)
        kd, vd = (_randn_bf16((32 * 32768, 128), gen).view(1, 32, 32768, 128) for _ in range(2))
        fn = lambda: ops.om_step_qk(None, qd, kd, vd, 0.1, True, -(32768 - 1))  # noqa: E731
    elif args.profile_case == "verify":     # 13 checks x 4 probes of config 5's tensor: 436 MB
        ref = _randn_bf16((13, 4 * 4 * 512 * 1024), gen)
        outp = ref.clone()
        res = torch.empty(13, 4, device=dev)
        fn = lambda: ops.verify_reduce(ref, outp, 13, result=res)  # noqa: E731
    else:                                   # folded chain, R=65536 rows: 269 MB
        x = torch.randn(65536, 512, device=dev, generator=gen)
        w = torch.randn(512, 512, device=dev, generator=gen) / math.sqrt(512)
        y = torch.empty(65536, 512, device=dev)
        fn = lambda: ops.linear_f32(x, w, out=y)  # noqa: E731
    for _ in range(n):
        fn()
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": args.profile_case, "launch_ms": e0.elapsed_time(e1) / n}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile-case", default=None,
                    choices=["decayed", "decayed_fp32", "decayed_strong", "states", "scan", "scan_shared", "verify", "linear", "om_causal", "compose", "gated", "prefix", "decayed_few", "scan_few", "linear_deep", "decode", "decayed_small"],
                    help="run a small case of one kernel only (for ncu captures)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the per-kernel lines")
    ap.add_argument("--probes", type=int, default=256,
                    help="probes of config 5's verify step (256 = the benchmark config; fewer for profiler runs)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
