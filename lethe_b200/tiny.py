"""A small language-model block around the op, for the training-loop evidence the reference keeps
(``results/gdn2_tiny_train_*.json`` of the reference project: B=4, L=256, H=2, d_k=128, d_v=64, 300 Adam
steps at lr 0.01 on a delayed-copy task, loss 3.67 -> below 1e-3, no NaN; arms for the scalar-gate
delta rule, KDA, GLA and SSD).

The block follows the layout of a gated-delta-rule layer: token embedding, a two-tap causal mixing of
neighbouring tokens (the short convolution such layers put in front of q, k, v), linear maps to q, k, v,
the log decay and the erase / write gate, the six-input op, and an output head.  The op is passed in,
so the same module trains through the CUDA library (``lethe_b200.ops.gdn2_op``) or through any callable
with the reference's signature ``op(q, k, v, g, b, w) -> o``.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

ARMS = ("gdn", "kda", "gla", "ssd")


def delayed_copy_batch(B: int, L: int, vocab: int, delay: int = 1, seed: int = 0) -> tuple[Tensor, Tensor]:
    """Tokens ``x [B, L]`` drawn uniformly and targets ``y[t] = x[t - delay]`` (``y[t] = 0`` for t < delay)."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randint(1, vocab, (B, L), generator=gen)
    y = torch.zeros_like(x)
    y[:, delay:] = x[:, :-delay]
    return x, y


class TinyGdnLM(nn.Module):
    """``arm``: "gdn" scalar gate + beta (b = w = beta broadcast), "kda" channel-wise gate + beta,
    "gla" channel-wise gate without the delta term (b = 0, w = 1), "ssd" scalar gate without it."""

    def __init__(self, op, arm: str = "gdn", vocab: int = 40, d_model: int = 64, H: int = 2, K: int = 128, V: int = 64):
        super().__init__()
        if arm not in ARMS:
            raise ValueError(f"arm must be one of {ARMS}")
        self.op, self.arm, self.vocab, self.H, self.K, self.V = op, arm, vocab, H, K, V
        self.emb = nn.Embedding(vocab, d_model)
        self.mix = nn.Linear(2 * d_model, d_model)
        self.q = nn.Linear(d_model, H * K, bias=False)
        self.k = nn.Linear(d_model, H * K, bias=False)
        self.v = nn.Linear(d_model, H * V, bias=False)
        self.g = nn.Linear(d_model, H * (K if arm in ("kda", "gla") else 1))
        self.beta = nn.Linear(d_model, H)
        self.head = nn.Linear(H * V, vocab)

    def forward(self, x: Tensor) -> Tensor:
        B, L = x.shape
        H, K, V = self.H, self.K, self.V
        e = self.emb(x)
        prev = torch.cat([torch.zeros_like(e[:, :1]), e[:, :-1]], dim=1)
        h = torch.tanh(self.mix(torch.cat([e, prev], dim=-1)))
        q = self.q(h).view(B, L, H, K)
        k = self.k(h).view(B, L, H, K)
        v = self.v(h).view(B, L, H, V)
        g = -torch.nn.functional.softplus(self.g(h)).view(B, L, H, -1).expand(B, L, H, K).contiguous()
        if self.arm in ("gdn", "kda"):
            beta = torch.sigmoid(self.beta(h)).view(B, L, H, 1)
            b, w = beta.expand(B, L, H, K).contiguous(), beta.expand(B, L, H, V).contiguous()
        else:
            b, w = torch.zeros(B, L, H, K, device=x.device), torch.ones(B, L, H, V, device=x.device)
        o = self.op(q, k, v, g, b, w)
        return self.head(o.reshape(B, L, H * V).to(h.dtype))
