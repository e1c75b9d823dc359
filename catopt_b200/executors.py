"""Lowered executors as ``nn.Module``s over the sm_100a kernels.

Each class keeps the surface the reference's batched modules expose
(``catopt_core.ports.BatchedExecutor``: ``forward``, a plain ``_plan`` dict,
``is_batched``; plus ``capture_cuda_graph`` / ``drop_cuda_graph`` /
``is_graph_captured`` of ``catopt_torch.executors.base.BatchedExecutorBase``,
base.py:146-224) so catopt's runners and autotuner can drive them unchanged.
They need no catopt install: ``sink.py`` adapts them to catopt's executor table
when catopt is importable.

There is no fallback arithmetic here: inputs must be CUDA tensors and every
forward is one C-ABI call.
"""
from __future__ import annotations

from typing import Any

import torch

from . import ops
from ._lib import B200Error


class _GraphMixin:
    """CUDA-graph capture/replay with the reference's calling convention:
    inputs are copied into static buffers and the returned tensor is a static
    output buffer overwritten by the next call (base.py:180-220)."""

    def _init_graph_state(self) -> None:
        self._graph: torch.cuda.CUDAGraph | None = None
        self._graph_inputs: tuple[torch.Tensor, ...] = ()
        self._graph_out: Any = None

    @property
    def is_graph_captured(self) -> bool:
        return self._graph is not None

    def drop_cuda_graph(self) -> None:
        self._init_graph_state()

    def capture_cuda_graph(self, *example_inputs: torch.Tensor, warmup: int = 3):
        if not example_inputs or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in example_inputs):
            raise ValueError("capture_cuda_graph needs CUDA tensor inputs")
        self._graph_inputs = tuple(t.clone() for t in example_inputs)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(warmup, 1)):  # also sizes every scratch buffer
                self._forward_impl(*self._graph_inputs)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph), torch.no_grad():
            self._graph_out = self._forward_impl(*self._graph_inputs)
        self._graph = graph
        return self

    def _replay_if_captured(self, xs: tuple) -> Any:
        g = self._graph
        if g is None or len(xs) != len(self._graph_inputs):
            return None
        if not all(isinstance(t, torch.Tensor) and t.shape == b.shape and t.dtype == b.dtype
                   and t.device == b.device for t, b in zip(xs, self._graph_inputs)):
            return None
        for buf, t in zip(self._graph_inputs, xs):
            buf.copy_(t, non_blocking=True)
        g.replay()
        return self._graph_out

    def forward(self, *xs: Any) -> Any:
        out = self._replay_if_captured(xs)
        return out if out is not None else self._forward_impl(*xs)


class B200FoldedLinear(_GraphMixin, torch.nn.Module):
    """A chain of bias-free Linear maps folded into one weight at construction
    (``IRModule._fold_weight_chains``, torch_bridge.py:2456-2510) and applied
    with a single fp32 GEMM per call (``linear`` binding, 1251-1253).

    ``weights`` are in application order (first layer first), nn.Linear layout
    ``[out, in]``.  The fold runs on the GPU through ``cb2_chain_fold_f32``; the
    result is registered as parameter ``fused_<index>`` the way the reference
    names its folded weights, so ``state_dict()`` keeps working.
    """

    def __init__(self, weights: list[torch.Tensor], bias: torch.Tensor | None = None,
                 fused_index: int | None = None) -> None:
        super().__init__()
        if not weights:
            raise ValueError("B200FoldedLinear needs at least one weight")
        ws = [w.detach().to(torch.float32).contiguous() for w in weights]
        if not all(w.is_cuda for w in ws):
            raise B200Error("B200FoldedLinear folds on the GPU: weights must be CUDA tensors")
        fused = ops.chain_fold_f32(ws)
        # the reference numbers fused params after the k originals and the k-2 intermediates
        idx = 2 * len(ws) - 2 if fused_index is None else fused_index
        self.fused_name = f"fused_{idx}"
        self.register_parameter(self.fused_name, torch.nn.Parameter(fused, requires_grad=False))
        # the folded weight never changes: its TF32 split for the tensor-core path is made once
        split = ops.linear_split_weight(fused)
        self.register_buffer("fused_split", split, persistent=False)
        self.bias = None if bias is None else torch.nn.Parameter(
            bias.detach().to(torch.float32).contiguous(), requires_grad=False)
        self._plan: dict | None = {"kind": "folded_linear", "k": len(ws),
                                   "in": ws[0].shape[1], "out": ws[-1].shape[0]}
        self._init_graph_state()

    @property
    def is_batched(self) -> bool:
        return True

    @property
    def weight(self) -> torch.Tensor:
        return getattr(self, self.fused_name)

    def _forward_impl(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear_f32(x, self.weight, self.bias, w_split=self.fused_split)


class B200ChunkedDecay(_GraphMixin, torch.nn.Module):
    """Decayed causal linear attention on ``q, k, v`` of shape ``[B,H,T,d]``:
    ``o_t = sum_{s<=t} gamma_h^(t-s) (q_t . k_s) v_s / scale``, the value of the
    reference's ``ChunkedDecayModule`` (decayed_lower.py:381-724) on the
    uniform chunk term, computed with a carried fp32 state instead of all-pairs
    cross products.  ``gamma`` is a scalar or one rate per head.
    """

    def __init__(self, gamma: torch.Tensor | float, n_heads: int, chunk: int, scale: float = 1.0) -> None:
        super().__init__()
        g = torch.as_tensor(gamma, dtype=torch.float32).detach().reshape(-1)
        if g.numel() == 1:
            g = g.expand(n_heads)
        if g.numel() != n_heads:
            raise ValueError(f"gamma has {g.numel()} rates for {n_heads} heads")
        self.register_buffer("gamma", g.contiguous().clone())
        self.chunk = int(chunk)
        self.scale = float(scale)
        self._plan: dict | None = {"kind": "decayed_state_carry", "chunk": self.chunk, "scale": self.scale}
        self._init_graph_state()

    @property
    def is_batched(self) -> bool:
        return True

    @property
    def n_blocks(self) -> int:
        return 0 if self._plan is None else int(self._plan.get("n", 0))

    def _forward_impl(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if self._plan is not None:
            self._plan["n"] = q.shape[-2] // self.chunk
        return ops.decayed_chunk_fwd(q, k, v, self.gamma, self.chunk, self.scale)


class B200DiagScan(_GraphMixin, torch.nn.Module):
    """Diagonal linear recurrence with readout,
    ``h_t = a_t*h_{t-1} + b*x_t``, ``y_t = sum_n c*h_t`` — T applications of the
    reference's ``applyd(aff_diag(a_t, b*x_t), h)`` (torch_bridge.py:1895-1900),
    the sequence its ``BatchedScanModule`` reduces level by level
    (scan_lower.py:569-698).  ``forward(a, x, h0=None)`` returns ``y`` (and the
    final state when ``return_state``).
    """

    def __init__(self, b: torch.Tensor, c: torch.Tensor, return_state: bool = False) -> None:
        super().__init__()
        if b.shape != c.shape or b.dim() != 2:
            raise ValueError("b and c must both be [D, N]")
        self.register_buffer("b", b.detach().contiguous().clone())
        self.register_buffer("c", c.detach().contiguous().clone())
        self.return_state = bool(return_state)
        self._plan: dict | None = {"kind": "diag_scan", "D": b.shape[0], "N": b.shape[1]}
        self._init_graph_state()

    @property
    def is_batched(self) -> bool:
        return True

    def _forward_impl(self, a: torch.Tensor, x: torch.Tensor, h0: torch.Tensor | None = None):
        return ops.diag_scan_fwd(a, x, self.b, self.c, h0, want_state=self.return_state)


class B200CausalSoftmax(_GraphMixin, torch.nn.Module):
    """Causal softmax attention evaluated block by block with the online-softmax
    monoid — the value of the reference's ``BatchedOMModule`` / ``StreamingOMModule``
    (catopt_carriers/om_lower.py:729-835, 996-1040) on a causal ``om`` carrier.
    ``forward(q, k, v)`` on ``[B,H,T,d]`` tensors; ``scale=None`` means ``1/sqrt(d)``."""

    def __init__(self, scale: float | None = None, causal: bool = True) -> None:
        super().__init__()
        self.scale = scale
        self.causal = bool(causal)
        self._plan: dict | None = {"kind": "om_causal" if causal else "om", "scale": scale}
        self._init_graph_state()

    @property
    def is_batched(self) -> bool:
        return True

    def _forward_impl(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        return ops.om_causal_fwd(q, k, v, self.scale, causal=self.causal)


# --------------------------------------------------------------------------- tensor-level entry points
# What the catopt-facing modules of ``sink.py`` run once their operand terms are
# evaluated; kept free of catopt imports so the GPU parity tests can call them.
def kernel_chunk(T: int, plan_chunk: int | None = None) -> int | None:
    """Chunk length handed to the decayed kernel: the plan's own when the term was
    uniform, else the largest divisor of T up to 128 (the value does not depend on
    it); ``None`` when T only has tiny divisors (a long prime-ish sequence)."""
    if plan_chunk:
        return plan_chunk
    for c in range(min(128, T), 0, -1):
        if T % c == 0:
            return c if (c >= 16 or T <= 64) else None
    return None


def decayed_whole_sequence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gamma: Any, chunk: int | None,
                           scale: float) -> torch.Tensor | None:
    """Decayed attention of ``[..., H, T, d]`` tensors (any number of leading axes,
    the last one indexing the decay rates) through ``cb2_decayed_chunk_fwd``.
    Returns ``None`` when the kernel has no path (fp64, awkward length)."""
    if not q.is_cuda:
        raise B200Error("decayed executor runs on CUDA tensors only (no CPU fallback)")
    if q.dim() == 2:                       # one head, no batch: q [T, d] with a scalar rate
        out = decayed_whole_sequence(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), gamma, chunk, scale)
        return None if out is None else out.squeeze(0)
    lead = q.shape[:-2]
    c = kernel_chunk(q.shape[-2], chunk)
    if c is None or q.dtype not in (torch.float32, torch.bfloat16):
        return None
    H = lead[-1]
    g = torch.as_tensor(gamma, dtype=torch.float32, device=q.device).reshape(-1)
    g = (g.expand(H) if g.numel() == 1 else g).contiguous()
    q4, k4, v4 = (t.reshape(-1, H, t.shape[-2], t.shape[-1]).contiguous() for t in (q, k, v))
    out = ops.decayed_chunk_fwd(q4, k4, v4, g, c, scale)
    return out.reshape(*lead, out.shape[-2], out.shape[-1])


def causal_softmax_blocks(q: torch.Tensor, k_blocks: list, v_blocks: list, scale: float,
                          causal: bool = True, mask: torch.Tensor | None = None) -> torch.Tensor | None:
    """Softmax attention (causal by default) of ``q [..., Tq, d]`` over key/value
    blocks joined along the key axis, through ``cb2_om_fwd``; ``None`` for fp64.
    ``mask``: an explicit attention mask (bool keep-mask or float bias, broadcastable to
    ``[..., Tq, Tk]``) added to the scaled scores through ``cb2_om_bias_fwd``."""
    if not q.is_cuda:
        raise B200Error("causal softmax executor runs on CUDA tensors only (no CPU fallback)")
    if q.dtype not in (torch.float32, torch.bfloat16):
        return None
    k = k_blocks[0] if len(k_blocks) == 1 else torch.cat(list(k_blocks), dim=-2)
    v = v_blocks[0] if len(v_blocks) == 1 else torch.cat(list(v_blocks), dim=-2)
    lead = q.shape[:-2]
    H = lead[-1] if lead else 1
    q4, k4, v4 = (t.expand(*lead, *t.shape[-2:]).reshape(-1, H, t.shape[-2], t.shape[-1]).contiguous()
                  for t in (q, k, v))
    if mask is None:
        out = ops.om_causal_fwd(q4, k4, v4, scale, causal=causal)
    else:
        out = ops.om_bias_fwd(q4, k4, v4, _mask_as_bias(mask, lead, H), scale, causal=causal)
    return out.reshape(*lead, out.shape[-2], out.shape[-1])


def _mask_as_bias(mask: torch.Tensor, lead: tuple, H: int) -> torch.Tensor:
    """An attention mask (bool keep-mask or float bias, broadcastable to ``[*lead, Tq, Tk]``) as an fp32
    bias whose leading axes are the ``[-1, H]`` pair the kernels index (broadcast axes unmaterialised)."""
    bias = ops.attn_bias(mask)
    if bias.dim() > 2 and any(s != 1 for s in bias.shape[:-2]):
        return bias.expand(*lead, *bias.shape[-2:]).reshape(-1, H, *bias.shape[-2:])
    return bias.reshape(bias.shape[-2:]) if bias.dim() >= 2 else bias


def softmax_blocks_state(q: torch.Tensor, k_blocks: list, v_blocks: list, scale: float, causal: bool = True,
                         state: tuple | None = None, key_offset: int = 0,
                         mask: torch.Tensor | None = None) -> tuple:
    """Streaming fold of key/value blocks into the online-softmax carrier
    ``(m, l, a)`` (fp32), one ``cb2_om_step`` per block — the state a decode loop
    checkpoints (``StreamingOMModule.forward_state``, catopt_carriers/om_lower.py:
    1003-1040).  Read it out with ``ops.om_apply_state``; feed it back as ``state``
    (with ``key_offset`` = keys already folded) when more blocks arrive."""
    if not q.is_cuda:
        raise B200Error("streaming softmax executor runs on CUDA tensors only (no CPU fallback)")
    lead = q.shape[:-2]
    H = lead[-1] if lead else 1

    def r4(t):
        return t.expand(*lead, *t.shape[-2:]).reshape(-1, H, t.shape[-2], t.shape[-1]).contiguous()

    if state is not None:
        state = tuple(r4(t) for t in state)
    bias = None if mask is None else _mask_as_bias(mask, lead, H)
    col = 0                                          # this call's first key among the mask's columns
    for kb, vb in zip(k_blocks, v_blocks):
        n = kb.shape[-2]
        piece = None
        if bias is not None:
            piece = bias if bias.dim() == 0 or bias.shape[-1] == 1 else bias[..., col:col + n]
        state = ops.om_step_qk(state, r4(q), r4(kb), r4(vb), scale, causal, key_offset, bias=piece)
        key_offset += n
        col += n
    return tuple(t.reshape(*lead, *t.shape[-2:]) for t in state)
