"""The N>1 host logic on CPU: unit sharding and the single max all-reduce that
ends a sharded verify step, run as world_size-2 gloo ranks."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from catopt_b200.sharding import shard_leading, shard_range, shard_units_of_heads


def test_shard_range_tiles_the_axis():
    for n in (0, 1, 7, 256, 512, 8192):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_shard_leading_by_batch_times_head():
    t = torch.arange(2 * 4 * 3 * 5).reshape(2, 4, 3, 5)
    parts = [shard_leading(t, r, 3, n_leading=2) for r in range(3)]
    assert [p.shape[0] for p in parts] == [3, 3, 2]
    assert torch.equal(torch.cat(parts), t.reshape(8, 3, 5))


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_decayed_attention_sharded_by_unit_equals_the_whole(world):
    """Config 4's partition (contiguous ranges of the batch x head axis, ranks exchange nothing):
    every rank runs its units as a [1, units, T, d] problem with one rate per unit; the shards,
    concatenated in rank order, are the unsharded result (CPU oracle stands in for the kernel:
    this test is about the partition, including shards that cut a batch entry)."""
    from oracle import oracle

    g = torch.Generator().manual_seed(5)
    B, H, T, d = 3, 4, 64, 8
    q, k, v = (torch.randn(B, H, T, d, generator=g, dtype=torch.float64) for _ in range(3))
    gamma = torch.tensor([0.8, 0.9, 0.95, 0.99], dtype=torch.float64)
    whole = oracle.decayed_state_carry(q, k, v, gamma, 16, 1.0)
    parts, covered = [], 0
    for r in range(world):
        u0, u1, rates = shard_units_of_heads(gamma, B, r, world)
        assert u0 == covered and rates.numel() == u1 - u0
        covered = u1
        if u1 == u0:
            continue
        sl = lambda t: t.reshape(B * H, T, d)[u0:u1].unsqueeze(0)  # noqa: E731
        parts.append(oracle.decayed_state_carry(sl(q), sl(k), sl(v), rates, 16, 1.0)[0])
    assert covered == B * H
    assert torch.equal(torch.cat(parts).reshape(B, H, T, d), whole)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from catopt_b200 import verify
        from oracle import oracle

        n_checks, probes = 3, 6
        g = torch.Generator().manual_seed(0)           # every rank builds the same job
        ref = torch.randn(n_checks, probes, 64, generator=g).bfloat16()
        out = (ref.float() * 1.01).bfloat16()
        out[1, 4, 7] = float("nan")                     # lives in rank 1's shard only
        b, e = shard_range(probes, rank, world)
        # per-rank partial result in the kernel's [n_checks, 4] format (oracle stands in
        # for the kernel here: this test is about the collective, not the reduction)
        local = torch.zeros(n_checks, 4)
        for c in range(n_checks):
            d = (ref[c, b:e] - out[c, b:e]).abs().float().flatten()
            r = ref[c, b:e].abs().float().flatten()
            local[c] = torch.tensor([d[~d.isnan()].max().item(), r[~r.isnan()].max().item(),
                                     float(d.isnan().any()), float(r.isnan().any())])
        merged = verify.merge_across_ranks(local.clone())
        reps = verify.reports_from_result(merged, rtol=2e-2)
        want = [oracle.verify_pair(ref[c], out[c], rtol=2e-2) for c in range(n_checks)]
        ok = all((math.isnan(a.max_abs) and math.isnan(w.max_abs)) or
                 (a.max_abs, a.max_rel, a.passed) == (w.max_abs, w.max_rel, w.passed)
                 for a, w in zip(reps, want))
        gathered = [torch.zeros_like(merged) for _ in range(world)]
        dist.all_gather(gathered, merged)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        q.put((rank, ok, same, math.isnan(reps[1].max_abs) and not reps[1].passed))
    finally:
        dist.destroy_process_group()


def test_sharded_verify_merge_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, same, nan_seen in res:
        assert ok and same and nan_seen, (rank, ok, same, nan_seen)
