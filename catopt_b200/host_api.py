"""Executors over HOST buffers: the copy-in / compute / copy-out pipeline.

The lowered modules normally live on the device next to the model.  When the
operands live in (pinned) host memory, the (batch x head) axis is cut into
slabs and three streams overlap the host-to-device copy of slab i+1, the kernel
on slab i and the device-to-host copy of slab i-1, with two device buffers per
operand.  Units are independent and every slab takes the one-pass form of the kernel,
so slabbing changes no result bit.
"""
from __future__ import annotations

import torch

from . import ops
from ._lib import B200Error


class DecayedHostPipeline:
    """``o = decayed_attention(q, k, v)`` for pinned host tensors ``[B,H,T,d]``.

    Device staging (2 slabs x 4 operands), streams and events are created once;
    ``run`` enqueues the whole pipeline and returns after the last copy-out has
    been *enqueued* — synchronise (or record an event on the current stream)
    before reading ``out``.
    """

    def __init__(self, B: int, H: int, T: int, dk: int, dv: int, dtype: torch.dtype,
                 gamma: torch.Tensor, chunk: int, scale: float = 1.0, n_slabs: int = 8,
                 device: torch.device | None = None) -> None:
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.shape = (B, H, T, dk, dv)
        self.chunk, self.scale = int(chunk), float(scale)
        units = B * H
        n_slabs = max(1, min(n_slabs, units))
        self.slab = (units + n_slabs - 1) // n_slabs
        self.bounds = [(b, min(b + self.slab, units)) for b in range(0, units, self.slab)]
        g = torch.as_tensor(gamma, dtype=torch.float32).reshape(-1)
        if g.numel() == 1:
            g = g.expand(H)
        if g.numel() != H:
            raise B200Error(f"gamma has {g.numel()} rates for {H} heads")
        # one rate per (batch, head) unit, so a slab may start at any unit
        self.gamma_units = g.repeat(B).contiguous().to(self.device)
        mk = lambda d: [torch.empty(self.slab, T, d, dtype=dtype, device=self.device) for _ in range(2)]  # noqa: E731
        self.dq, self.dk_, self.dv_, self.do = mk(dk), mk(dk), mk(dv), mk(dv)
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_comp = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.h2d_bytes = units * T * (2 * dk + dv) * self.dq[0].element_size()
        self.d2h_bytes = units * T * dv * self.dq[0].element_size()

    def run(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        B, H, T, dk, dv = self.shape
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_pinned():
                raise B200Error("DecayedHostPipeline takes pinned host tensors")
        qf, kf, vf, of = (t.reshape(B * H, T, -1) for t in (q, k, v, out))
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        for i, (b, e) in enumerate(self.bounds):
            n, buf = e - b, i % 2
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(self.ev_comp[buf])   # kernel of slab i-2 has read its inputs
                self.dq[buf][:n].copy_(qf[b:e], non_blocking=True)
                self.dk_[buf][:n].copy_(kf[b:e], non_blocking=True)
                self.dv_[buf][:n].copy_(vf[b:e], non_blocking=True)
                self.ev_in[buf].record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(self.ev_in[buf])
                if i >= 2:
                    self.s_comp.wait_event(self.ev_out[buf])  # slab i-2's result has left the buffer
                ops.decayed_chunk_fwd(self.dq[buf][:n].unsqueeze(0), self.dk_[buf][:n].unsqueeze(0),
                                      self.dv_[buf][:n].unsqueeze(0), self.gamma_units[b:e],
                                      self.chunk, self.scale, out=self.do[buf][:n].unsqueeze(0),
                                      one_pass=True)   # bits must not depend on the slab size
                self.ev_comp[buf].record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_comp[buf])
                of[b:e].copy_(self.do[buf][:n], non_blocking=True)
                self.ev_out[buf].record(self.s_out)
        for s in (self.s_in, self.s_comp, self.s_out):
            cur.wait_stream(s)
        return out
