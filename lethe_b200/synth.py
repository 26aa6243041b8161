"""Seeded synthetic inputs with the value distributions of the benchmark configurations:
q, k ~ N(0,1) L2-normalised over the key dimension; v ~ N(0,1); beta = sigmoid(N(0,1));
g = -softplus(N(0,1) + 3) (a log decay; ``mild=True`` gives the reference bench's -0.1 * U(0,1),
``src/lethe/bench/gdn2_backward_headtohead.py:45-63``); dO ~ N(0,1); h0 ~ 0.1 * N(0,1).
Drawn on the CPU in fp32 in the order q, k, v, beta, g, do, h0."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def make_inputs(B, L, H, K, V, *, gate="scalar", delta=True, with_h0=True, seed=0, mild=False, full=False):
    """Returns a dict of CPU tensors: q, k, v, do (bf16); g, beta, h0 (fp32; None when absent)."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, L, H, K, generator=gen)
    k = torch.randn(B, L, H, K, generator=gen)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(B, L, H, V, generator=gen)
    beta = torch.randn(B, L, H, generator=gen).sigmoid()
    gshape = (B, L, H, K) if gate == "channel" else (B, L, H)
    if mild:
        g = -0.1 * torch.rand(*gshape, generator=gen)
    else:
        g = -F.softplus(torch.randn(*gshape, generator=gen) + 3.0)
    do = torch.randn(B, L, H, V, generator=gen)
    h0 = 0.1 * torch.randn(B, H, K, V, generator=gen)
    out = dict(q=q.bfloat16(), k=k.bfloat16(), v=v.bfloat16(), do=do.bfloat16(),
               g=None if gate == "none" else g, beta=beta if delta else None,
               h0=h0 if with_h0 else None)
    if full:   # independent per-channel erase gate b [B,L,H,K] and write gate w [B,L,H,V] instead of beta
        out["beta"] = None
        out["b"] = torch.randn(B, L, H, K, generator=gen).sigmoid()
        out["w"] = torch.randn(B, L, H, V, generator=gen).sigmoid()
    return out
