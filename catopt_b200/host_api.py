"""Executors over HOST buffers: the copy-in / compute / copy-out pipeline.

The lowered modules normally live on the device next to the model.  When the
operands live in (pinned) host memory, the batch axis is cut into slabs and three
streams overlap the host-to-device copy of slab i+1, the module's forward on slab
i and the device-to-host copy of slab i-1, with two device buffers per operand.
Batch entries are independent, so slabbing changes nothing but the schedule.
"""
from __future__ import annotations

from typing import Any

import torch

from ._lib import B200Error
from .executors import B200ChunkedDecay


class DecayedHostPipeline:
    """``o = module(q, k, v)`` for pinned host tensors ``[B,H,T,d]``, slab by slab.

    ``module`` is the lowered executor a user holds — ``sink.B200ChunkedDecayModule``
    as delivered by catopt's optimizer, or ``executors.B200ChunkedDecay`` — taking
    ``[b,H,T,d]`` CUDA tensors and returning ``[b,H,T,dv]``; without one a
    ``B200ChunkedDecay`` is built from ``gamma`` / ``chunk`` / ``scale``.  Every slab
    is a whole number of batch entries, so one module (one rate per head) serves them
    all.  Device staging (2 slabs x 3 operands), streams and events are created once;
    ``run`` enqueues the whole pipeline and returns after the last copy-out has been
    *enqueued* — synchronise (or record an event on the current stream) before
    reading ``out``.
    """

    def __init__(self, B: int, H: int, T: int, dk: int, dv: int, dtype: torch.dtype,
                 gamma: torch.Tensor | None = None, chunk: int = 128, scale: float = 1.0, n_slabs: int = 8,
                 device: torch.device | None = None, module: Any = None) -> None:
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.shape = (B, H, T, dk, dv)
        n_slabs = max(1, min(n_slabs, B))
        self.slab = (B + n_slabs - 1) // n_slabs            # batch entries per slab
        self.bounds = [(b, min(b + self.slab, B)) for b in range(0, B, self.slab)]
        if module is None:
            if gamma is None:
                raise B200Error("DecayedHostPipeline needs a module or the decay rates")
            module = B200ChunkedDecay(gamma, H, chunk, scale).to(self.device)
        self.module = module
        mk = lambda d: [torch.empty(self.slab, H, T, d, dtype=dtype, device=self.device) for _ in range(2)]  # noqa: E731
        self.dq, self.dk_, self.dv_ = mk(dk), mk(dk), mk(dv)
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_comp = [torch.cuda.Event() for _ in range(2)]
        esz = self.dq[0].element_size()
        self.h2d_bytes = B * H * T * (2 * dk + dv) * esz
        self.d2h_bytes = B * H * T * dv * esz

    def run(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_pinned():
                raise B200Error("DecayedHostPipeline takes pinned host tensors")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        for i, (b, e) in enumerate(self.bounds):
            n, buf = e - b, i % 2
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(self.ev_comp[buf])   # the forward on slab i-2 has read its inputs
                self.dq[buf][:n].copy_(q[b:e], non_blocking=True)
                self.dk_[buf][:n].copy_(k[b:e], non_blocking=True)
                self.dv_[buf][:n].copy_(v[b:e], non_blocking=True)
                self.ev_in[buf].record(self.s_in)
            with torch.cuda.stream(self.s_comp), torch.no_grad():
                self.s_comp.wait_event(self.ev_in[buf])
                res = self.module(self.dq[buf][:n], self.dk_[buf][:n], self.dv_[buf][:n])
                self.ev_comp[buf].record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_comp[buf])
                out[b:e].copy_(res, non_blocking=True)
                res.record_stream(self.s_out)                 # allocated on the compute stream, read here
        for s in (self.s_in, self.s_comp, self.s_out):
            cur.wait_stream(s)
        return out
