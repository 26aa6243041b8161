"""Kernel plug-ins with the reference's ``K1Fn`` / ``K2Fn`` signatures
(``src/lethe/kernels/cute/gdn2_assemble.py:29-44``), so that its assembly
(``assemble_gdn2_backward_scalar(..., k1_fn=..., k2_fn=...)``, ``gdn2_assemble.py:242-314``) can be
driven by the CUDA kernels of this package unchanged, and so that each kernel can be checked at the
reference's own "micro-gate" granularity (``build_microgate_bundles``, ``gdn2_chunkwise.py:318-388``).

Both callables take and return head-major chunked fp32 tensors ``[B, H, NT, C, ...]`` (C = 64,
d_k = 128) and return fresh tensors, like the reference's.  They stage their arguments into the
per-chunk records the kernels read (PyTorch is used for that restaging only) and run exactly one
kernel of the backward call each: the adjoint state scan for K#1, the WY / triangular-inverse VJP for
K#2 (``k2_fn`` for the scalar gate, ``k2_fn_cw`` for the channel-wise gate with independent erase and
write gates).
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from . import ops

LN2 = math.log(2.0)


# ------------------------------------------------------------------------------------------------
# tile images (the 128-byte-swizzled layout the kernels keep their records in)
# ------------------------------------------------------------------------------------------------
def to_image(x: Tensor) -> Tensor:
    """[..., rows, cols] 16-bit (cols a multiple of 64) -> [..., rows * cols] tile image: atoms of
    64 columns, row r at r * 128 bytes, 16-byte chunk c stored at chunk c ^ (r & 7)."""
    *lead, rows, cols = x.shape
    t = x.reshape(*lead, rows, cols // 64, 8, 8).transpose(-4, -3)            # [..., atom, row, chunk, 8]
    r = torch.arange(rows, device=x.device)
    src = torch.arange(8, device=x.device)[None, :] ^ (r[:, None] & 7)         # chunk stored at position j
    idx = src.view(*([1] * (len(lead) + 1)), rows, 8, 1).expand(*t.shape)
    return torch.gather(t, -2, idx).reshape(*lead, rows * cols)


def from_image(img: Tensor, rows: int, cols: int) -> Tensor:
    """Inverse of ``to_image`` (the swizzle is its own inverse)."""
    *lead, _ = img.shape
    t = img.reshape(*lead, cols // 64, rows, 8, 8)
    r = torch.arange(rows, device=img.device)
    src = torch.arange(8, device=img.device)[None, :] ^ (r[:, None] & 7)
    idx = src.view(*([1] * (len(lead) + 1)), rows, 8, 1).expand(*t.shape)
    return torch.gather(t, -2, idx).transpose(-4, -3).reshape(*lead, rows, cols)


def _record_view(buf: Tensor, off: int, size: int, Z: int, dtype) -> Tensor:
    return buf[off:off + Z * size].view(dtype).view(Z, -1)


def _layout(B, H, L, V, gate):
    """Record offsets of the two workspaces (mirrors ``make_layout`` of the library)."""
    Z = B * H * (L // 64)
    al = lambda x: (x + 1023) // 1024 * 1024  # noqa: E731
    sz = dict(ta=16384, w=16384, u=64 * V * 2, p=32768, r=128 * V * 2, hc=128 * V * 2, vn=64 * V * 2, ad=512)
    off, o = {}, 0
    for n in ("ta", "w", "u", "p", "r", "hc", "vn", "ad"):
        off[n] = o
        o = al(o + (Z + B * H if n == "hc" else Z) * sz[n])
    if gate == ops.GATE_CHANNEL:
        sz["gt"], off["gt"] = 64 * 128 * 4, o
    sz2 = dict(rb=128 * V * 2, dh=128 * V * 2, dv2=64 * V * 2, dw=16384, dkb=64 * 128 * 4,
               dgb=(64 * 128 if gate == ops.GATE_CHANNEL else 64) * 4)
    off2, o = {}, 0
    for n in ("rb", "dh", "dv2", "dw", "dkb", "dgb"):
        off2[n] = o
        o = al(o + Z * sz2[n])
    if gate == ops.GATE_CHANNEL:
        for n, size in (("da", 8192), ("dm", 8192), ("dqp", 64 * 128 * 4)):
            sz2[n], off2[n] = size, o
            o = al(o + Z * size)
    return Z, sz, off, sz2, off2


def _untok(x: Tensor) -> Tensor:
    """[B, H, NT, C, D] -> [B, L, H, D]"""
    B, H, NT, C, D = x.shape
    return x.reshape(B, H, NT * C, D).transpose(1, 2).contiguous()


def _tok(x: Tensor, C: int = 64) -> Tensor:
    """[B, L, H, D] -> [B, H, NT, C, D]"""
    B, L, H, D = x.shape
    return x.transpose(1, 2).reshape(B, H, L // C, C, D)


# ------------------------------------------------------------------------------------------------
def k1_fn(q: Tensor, k: Tensor, w: Tensor, g2: Tensor, g_last: Tensor, do: Tensor, dv_local: Tensor,
          dht: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    """K#1, the reverse state scan (reference ``k1_reverse_state_ref`` / ``_cw_ref``,
    ``gdn2_assemble.py:71-99``, ``:377-404``): returns ``(dh [B,H,NT,K,V], dv2 [B,H,NT,C,V], dh0)``.
    ``g2`` is the in-chunk cumulative decay in log2 units, ``[B,H,NT,C]`` or ``[B,H,NT,C,K]``."""
    B, H, NT, C, K = q.shape
    V = do.shape[-1]
    if C != 64 or K != 128 or V not in (64, 128):
        raise ops.GdnError("lethe_gdn: k1_fn needs C = 64, d_k = 128, d_v in {64, 128}")
    dev, f32 = q.device, torch.float32
    cw = g2.dim() == 5
    g2f = g2.to(f32) if cw else g2.to(f32)[..., None]
    glf = (g_last.to(f32) if cw else g_last.to(f32)[..., None])[..., None, :]          # [B,H,NT,1,K|1]
    kd = k.to(f32) * torch.exp2(glf - g2f)
    qg = q.to(f32) * torch.exp2(g2f)
    # the adjoint scan D' = a D - P^T D + Rb with P = kd^T w, Rb = qg^T do - w^T dv_local
    P = kd.transpose(-1, -2) @ w.to(f32)
    Rb = qg.transpose(-1, -2) @ do.to(f32) - w.to(f32).transpose(-1, -2) @ dv_local.to(f32)
    a = torch.exp2(glf.squeeze(-2)).expand(B, H, NT, K)
    L = NT * C
    gate = ops.GATE_CHANNEL if cw else ops.GATE_SCALAR
    buf = ops.GdnBuffers(B, L, H, K, V, gate, True, dev)
    Z, sz, off, sz2, off2 = _layout(B, H, L, V, gate)
    _record_view(buf.saved, off["p"], sz["p"], Z, torch.float16).copy_(to_image(P.half()).reshape(Z, -1))
    _record_view(buf.saved, off["ad"], sz["ad"], Z, f32).copy_(a.reshape(Z, K))
    # the scan reads Rb as V / 16 column blocks of [128 rows][16 columns]
    rb_img = Rb.half().reshape(Z, K, V // 16, 16).transpose(1, 2).reshape(Z, -1)
    _record_view(buf.scratch, off2["rb"], sz2["rb"], Z, torch.float16).copy_(rb_img)
    dummy16 = torch.zeros(B, L, H, K, dtype=torch.bfloat16, device=dev)
    dummyv = torch.zeros(B, L, H, V, dtype=torch.bfloat16, device=dev)
    gdummy = torch.zeros((B, L, H, K) if cw else (B, L, H), dtype=f32, device=dev)
    bdummy = torch.zeros(B, L, H, dtype=f32, device=dev)
    ops.backward_into(buf, dummy16, dummy16, dummyv, gdummy, bdummy, None, dummyv, dht.to(f32).contiguous(),
                      1.0, kernel_mask=2)
    dh = from_image(_record_view(buf.scratch, off2["dh"], sz2["dh"], Z, torch.float16), K, V)
    dh = dh.to(f32).reshape(B, H, NT, K, V)
    dv2 = kd @ dh + dv_local.to(f32)
    return dh.clone(), dv2, buf.dh0.clone()


def k2_fn(k: Tensor, v: Tensor, beta: Tensor, g2: Tensor, t_mat: Tensor, dw: Tensor, du: Tensor
          ) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """K#2, the WY / triangular-inverse VJP for the scalar gate (reference ``k2_wy_vjp_ref``,
    ``gdn2_assemble.py:102-147``): returns ``(dk2, dv, dbeta, dg)``, ``dg`` after the in-chunk reverse
    cumulative sum, all head-major chunked."""
    B, H, NT, C, K = k.shape
    V = v.shape[-1]
    if C != 64 or K != 128 or V not in (64, 128) or g2.dim() != 4:
        raise ops.GdnError("lethe_gdn: k2_fn needs the scalar gate, C = 64, d_k = 128, d_v in {64, 128}")
    dev, f32 = k.device, torch.float32
    L = NT * C
    buf = ops.GdnBuffers(B, L, H, K, V, ops.GATE_SCALAR, True, dev)
    Z, sz, off, sz2, off2 = _layout(B, H, L, V, ops.GATE_SCALAR)
    ta = torch.zeros(B, H, NT, 128, 64, dtype=torch.float16, device=dev)
    ta[..., :64, :] = t_mat.half()
    _record_view(buf.saved, off["ta"], sz["ta"], Z, torch.float16).copy_(to_image(ta).reshape(Z, -1))
    _record_view(buf.scratch, off2["dv2"], sz2["dv2"], Z, torch.float16).copy_(to_image(du.half()).reshape(Z, -1))
    _record_view(buf.scratch, off2["dw"], sz2["dw"], Z, torch.float16).copy_(to_image(dw.half()).reshape(Z, -1))
    _record_view(buf.scratch, off2["dkb"], sz2["dkb"], Z, f32).zero_()
    _record_view(buf.scratch, off2["dgb"], sz2["dgb"], Z, f32).zero_()
    # per-token natural-log decay from the in-chunk cumulative log2 decay
    g_cum = g2.to(f32) * LN2
    g_tok = torch.diff(g_cum, dim=-1, prepend=torch.zeros_like(g_cum[..., :1]))
    k16 = _untok(k).to(torch.bfloat16)
    v16 = _untok(v).to(torch.bfloat16)
    g_t = _untok(g_tok[..., None])[..., 0].contiguous()
    b_t = _untok(beta.to(f32)[..., None])[..., 0].contiguous()
    dov = torch.zeros(B, L, H, V, dtype=torch.bfloat16, device=dev)
    ops.backward_into(buf, k16, k16, v16, g_t, b_t, None, dov, None, 1.0, kernel_mask=8)
    dk2 = _tok(buf.dk.to(f32))
    dv = _tok(buf.dv.to(f32))
    db = _tok(buf.dbeta[..., None])[..., 0]
    dg = _tok(buf.dg[..., None])[..., 0]
    return dk2.clone(), dv.clone(), db.clone(), dg.clone()


def _gate_tile_image(G: Tensor) -> Tensor:
    """[Z, 64, 128] fp32 cumulative decay in log2 units -> the record image the kernels read (``gidx`` of
    ``csrc/gdn_common.cuh``): a row is 32 pieces of four channels, even pieces first, then the odd ones, and
    within each 128-byte line the pieces are XOR-ed with the low three row bits (the odd half with 4 more)."""
    Z = G.shape[0]
    row = torch.arange(64, device=G.device)[:, None]
    col = torch.arange(128, device=G.device)[None, :]
    p = col >> 2
    piece = ((p >> 1) + ((p & 1) << 4)) ^ ((row & 7) ^ ((p & 1) << 2))
    dst = (row * 128 + (piece << 2) + (col & 3)).reshape(-1)
    img = torch.empty(Z, 64 * 128, dtype=torch.float32, device=G.device)
    img[:, dst] = G.reshape(Z, -1)
    return img


def k2_fn_cw(k: Tensor, v: Tensor, b: Tensor, w: Tensor, g2: Tensor, t_mat: Tensor, dwy: Tensor, du: Tensor
             ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Channel-wise K#2 with independent per-channel erase gate ``b`` and write gate ``w`` (reference
    ``k2_wy_vjp_cw_ref``, ``gdn2_assemble.py:407-473``): returns ``(dk2, dv, db, dw, dg)``, ``dg`` after the
    in-chunk reverse cumulative sum, all head-major chunked.  ``g2 [B,H,NT,C,K]`` is the in-chunk cumulative
    decay in log2 units."""
    B, H, NT, C, K = k.shape
    V = v.shape[-1]
    if C != 64 or K != 128 or V not in (64, 128) or g2.dim() != 5:
        raise ops.GdnError("lethe_gdn: k2_fn_cw needs the channel-wise gate, C = 64, d_k = 128, d_v in {64, 128}")
    dev, f32 = k.device, torch.float32
    L = NT * C
    buf = ops.GdnBuffers(B, L, H, K, V, ops.GATE_CHANNEL, 2, dev)
    Z, sz, off, sz2, off2 = _layout(B, H, L, V, ops.GATE_CHANNEL)
    ta = torch.zeros(B, H, NT, 128, 64, dtype=torch.float16, device=dev)
    ta[..., :64, :] = t_mat.half()
    _record_view(buf.saved, off["ta"], sz["ta"], Z, torch.float16).copy_(to_image(ta).reshape(Z, -1))
    _record_view(buf.saved, off["gt"], sz["gt"], Z, f32).copy_(_gate_tile_image(g2.to(f32).reshape(Z, C, K)))
    _record_view(buf.scratch, off2["dv2"], sz2["dv2"], Z, torch.float16).copy_(to_image(du.half()).reshape(Z, -1))
    _record_view(buf.scratch, off2["dw"], sz2["dw"], Z, torch.float16).copy_(to_image(dwy.half()).reshape(Z, -1))
    _record_view(buf.scratch, off2["dkb"], sz2["dkb"], Z, f32).zero_()
    _record_view(buf.scratch, off2["dgb"], sz2["dgb"], Z, f32).zero_()
    k16 = _untok(k).to(torch.bfloat16)
    v16 = _untok(v).to(torch.bfloat16)
    g_cum = g2.to(f32) * LN2
    g_tok = torch.diff(g_cum, dim=-2, prepend=torch.zeros_like(g_cum[..., :1, :]))
    g_t = _untok(g_tok)
    b_t, w_t = _untok(b.to(f32)), _untok(w.to(f32))
    dov = torch.zeros(B, L, H, V, dtype=torch.bfloat16, device=dev)
    ops.backward_into(buf, k16, k16, v16, g_t, None, None, dov, None, 1.0, kernel_mask=8, b_gate=b_t, w_gate=w_t)
    return (_tok(buf.dk.to(f32)).clone(), _tok(buf.dv.to(f32)).clone(), _tok(buf.db).clone(), _tok(buf.dw).clone(),
            _tok(buf.dg).clone())
