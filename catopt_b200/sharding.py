"""Partition of the hot path's independent units over the GPUs of one box.

Every executor here works on independent units — (batch, head) pairs for the
decayed recurrence, (batch, channel-block) pairs for the scan, rows for the
folded GEMM, probes for the verify gate — so ranks never exchange data on the
hot path.  The only collective is the max all-reduce that ends a sharded
verify step (``verify.verify_batched``).
"""
from __future__ import annotations


def shard_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous ``[begin, end)`` of ``n_units`` owned by ``rank``.

    The first ``n_units % world`` ranks own one unit more, so sizes differ by at
    most one and the ranges tile ``[0, n_units)`` in rank order.
    """
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    if n_units < 0:
        raise ValueError("n_units must be non-negative")
    base, extra = divmod(n_units, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_leading(t, rank: int, world: int, n_leading: int = 1):
    """This rank's slice of a tensor whose first ``n_leading`` dims are flattened
    into the unit axis (e.g. ``[B,H,T,d]`` with ``n_leading=2`` shards by
    batch x head).  Returns a contiguous ``[units, ...]`` view or copy."""
    units = 1
    for s in t.shape[:n_leading]:
        units *= s
    flat = t.reshape(units, *t.shape[n_leading:])
    b, e = shard_range(units, rank, world)
    return flat[b:e].contiguous()


def shard_units_of_heads(gamma, batch: int, rank: int, world: int):
    """Sharding decayed attention ``[B,H,T,d]`` by (batch, head) unit: ``(begin, end, rates)``
    with ``[begin, end)`` this rank's contiguous range of the ``B*H`` flattened units and
    ``rates`` the decay rate of each of them (unit ``u`` belongs to head ``u % H``), ready to
    be passed as the per-head rates of a ``[1, end-begin, T, d]`` view of the rank's slice —
    the kernels take one rate per row of the head axis, so a shard that starts or ends in the
    middle of a batch entry needs no special case."""
    H = int(gamma.numel())
    begin, end = shard_range(batch * H, rank, world)
    rates = gamma.reshape(-1).repeat(batch)[begin:end].contiguous()
    return begin, end, rates
