"""The synthetic decoder of benchmark config 5 (not a test module): a stack of
blocks, each RMSNorm -> decayed attention (H heads of d_head) -> residual ->
RMSNorm -> SwiGLU MLP -> residual, bias-free, random-init weights ~N(0, 0.02).
Built as an ``nn.Sequential`` so catopt's compositional strategy takes every block
as one unit (its default block selector picks the children of a Sequential).
The decay mask is spelled in-graph (``tril`` of a power of a position difference),
the form catopt's export recognises and lifts to ``om_decayed``; positions are
built in fp32 whatever the activations' dtype (``arange(512)`` is not exact in bf16).
"""
from __future__ import annotations

import torch
from torch import nn


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


class DecayedAttention(nn.Module):
    def __init__(self, dim: int, heads: int, gamma: float = 0.97) -> None:
        super().__init__()
        self.heads, self.d_head, self.gamma = heads, dim // heads, gamma
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim, bias=False) for _ in range(4))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, dim = x.shape
        q, k, v = (p(x).reshape(B, T, self.heads, self.d_head).transpose(1, 2) for p in (self.q, self.k, self.v))
        pos = torch.arange(T, dtype=torch.float32, device=x.device)
        decay = torch.tril(torch.pow(torch.tensor(self.gamma, dtype=torch.float32, device=x.device),
                                     (pos.unsqueeze(1) - pos.unsqueeze(0)).clamp_min(0))).to(x.dtype)
        s = q @ k.transpose(-1, -2) / (self.d_head ** 0.5)
        return self.o(((s * decay) @ v).transpose(1, 2).reshape(B, T, dim))


class SwiGLU(nn.Module):
    def __init__(self, dim: int, hidden: int) -> None:
        super().__init__()
        self.gate, self.up = nn.Linear(dim, hidden, bias=False), nn.Linear(dim, hidden, bias=False)
        self.down = nn.Linear(hidden, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(torch.nn.functional.silu(self.gate(x)) * self.up(x))


class Block(nn.Module):
    def __init__(self, dim: int, heads: int, hidden: int) -> None:
        super().__init__()
        self.norm1, self.attn = RMSNorm(dim), DecayedAttention(dim, heads)
        self.norm2, self.mlp = RMSNorm(dim), SwiGLU(dim, hidden)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


def decoder(n_blocks: int = 12, dim: int = 1024, heads: int = 16, hidden: int = 2816, seed: int = 0) -> nn.Sequential:
    g = torch.Generator().manual_seed(seed)
    model = nn.Sequential(*[Block(dim, heads, hidden) for _ in range(n_blocks)])
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
    return model.eval()
