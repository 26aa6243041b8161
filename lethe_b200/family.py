"""Family entry points with the reference's names and argument lists
(``src/lethe/kernels/cute/gdn2_family.py:24-164``): GLA, plain linear attention, SSD-class and KDA
backward passes, each returning the same gradient tuple as the reference's wrapper.  All of them are
the one CUDA op ``gdn_chunk`` at different gate settings."""

from __future__ import annotations

from typing import NamedTuple

import torch
from torch import Tensor

from .ops import gdn_chunk


class GlaGrads(NamedTuple):
    grad_q: Tensor
    grad_k: Tensor
    grad_v: Tensor
    grad_g: Tensor


class LaGrads(NamedTuple):
    grad_q: Tensor
    grad_k: Tensor
    grad_v: Tensor


class SsdGrads(NamedTuple):
    grad_q: Tensor
    grad_k: Tensor
    grad_v: Tensor
    grad_g: Tensor


class KdaGrads(NamedTuple):
    grad_q: Tensor
    grad_k: Tensor
    grad_v: Tensor
    grad_g: Tensor
    grad_beta: Tensor


def _run(q, k, v, g, beta, do, scale, use_qk_l2norm):
    leaves = [t.detach().requires_grad_(True) for t in (q, k, v)]
    gl = None if g is None else g.detach().requires_grad_(True)
    bl = None if beta is None else beta.detach().requires_grad_(True)
    with torch.enable_grad():
        o, _ = gdn_chunk(leaves[0], leaves[1], leaves[2], gl, bl, None, scale=scale,
                         use_qk_l2norm=use_qk_l2norm)
        ins = leaves + [t for t in (gl, bl) if t is not None]
        return torch.autograd.grad(o, ins, do.to(o.dtype))


def gla_backward(q, k, v, g, do, *, scale=None, use_qk_l2norm=True) -> GlaGrads:
    """GLA: channel-wise decay, no delta term (reference ``gla_backward``, gdn2_family.py:24)."""
    return GlaGrads(*_run(q, k, v, g, None, do, scale, use_qk_l2norm))


def la_backward(q, k, v, do, *, scale=None, use_qk_l2norm=True) -> LaGrads:
    """Plain causal linear attention (reference ``la_backward``, gdn2_family.py:53)."""
    return LaGrads(*_run(q, k, v, None, None, do, scale, use_qk_l2norm))


def ssd_backward(q, k, v, g, do, *, scale=None, use_qk_l2norm=True) -> SsdGrads:
    """SSD / Mamba-2 class: one decay per token-head, no delta term (gdn2_family.py:82-115)."""
    if g.dim() != 3:
        raise ValueError(f"SSD-class g must be [B, L, H], got {tuple(g.shape)}")
    return SsdGrads(*_run(q, k, v, g, None, do, scale, use_qk_l2norm))


def kda_backward(q, k, v, g, beta, do, *, scale=None, use_qk_l2norm=True) -> KdaGrads:
    """KDA: channel-wise decay and a scalar beta per token-head (gdn2_family.py:118-164)."""
    if beta.dim() != 3:
        raise ValueError(f"KDA beta must be [B, L, H], got {tuple(beta.shape)}")
    return KdaGrads(*_run(q, k, v, g, beta, do, scale, use_qk_l2norm))
