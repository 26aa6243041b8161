"""CPU model of the CUDA kernels' dataflow, including every bf16 rounding point.

TEST INFRASTRUCTURE ONLY (see ``oracle/gdn_oracle.py``).  The CUDA path feeds its tensor-core
products with bf16 operands and accumulates in fp32; intermediate results that become operands of
a later product are rounded to bf16 on the way.  This module replays exactly that order of
operations in PyTorch so that (a) the error budget of the design can be checked on the CPU against
the fp64 oracle before a kernel exists, and (b) a kernel result that differs from the oracle by
more than this model does points at a bug rather than at rounding.  The reference keeps the same
kind of "kernel spec model" tests for its fp16 kernels (``tests/test_gdn2_l2.py:29-52``,
``tests/test_gdn2_k2_fused.py``).

Only the scalar-gate and no-delta paths are modelled here; the channel-wise sub-block scheme is
modelled in ``cw_model``.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .gdn_oracle import Grads, _chunks, _unchunks


def r16(x: Tensor) -> Tensor:
    """Round to bf16 and come back (an MMA operand or a bf16 store)."""
    return x.to(torch.bfloat16).to(torch.float32)


def mm(a: Tensor, b: Tensor) -> Tensor:
    """Tensor-core product: operands already bf16-valued, fp32 accumulate."""
    return a @ b


def scalar_fwd_bwd(q, k, v, g, beta, h0, do, dhT=None, *, scale=None, C=64):
    """q,k,v,do: bf16-valued fp32 tensors; g, beta, h0: fp32.  Returns (o, hT, Grads, ws)."""
    f32 = torch.float32
    q, k, v, do = (t.to(f32) for t in (q, k, v, do))
    B, L, H, K = k.shape
    V = v.shape[-1]
    NT = L // C
    s = K ** -0.5 if scale is None else scale
    delta = beta is not None
    qc, kc, vc, doc = _chunks(q, C), _chunks(k, C), _chunks(v, C), _chunks(do, C)
    if g is None:
        G = torch.zeros(B, H, NT, C, dtype=f32)
    else:
        G = torch.cumsum(g.to(f32).transpose(1, 2).reshape(B, H, NT, C), -1)
    gam = G.exp()
    Gl = G[..., -1]
    diff = G[..., :, None] - G[..., None, :]
    low = torch.tril(torch.ones(C, C, dtype=torch.bool))
    ratio = torch.where(low, diff.clamp(max=0).exp(), torch.zeros((), dtype=f32))
    dec_end = (Gl[..., None] - G).exp()
    a = Gl.exp()
    # ---- prepare
    KK = mm(kc, kc.transpose(-1, -2))
    QK = mm(qc, kc.transpose(-1, -2))
    A16 = r16(s * ratio * QK)
    eye = torch.eye(C, dtype=f32)
    if delta:
        bc = beta.to(f32).transpose(1, 2).reshape(B, H, NT, C)
        Mm = torch.tril(bc[..., None] * ratio * KK, -1)
        T = torch.linalg.solve_triangular(eye + Mm, eye.expand_as(Mm), upper=False,
                                          unitriangular=True)
        T16 = r16(T)
        bv16 = r16(bc[..., None] * vc)
        bgk16 = r16((bc * gam)[..., None] * kc)
        u16 = r16(mm(T16, bv16))
        w16 = r16(mm(T16, bgk16))
    else:
        bc = None
        u16 = vc
        w16 = torch.zeros_like(kc)
    kd16 = r16(kc * dec_end[..., None])
    P16 = r16(mm(kd16.transpose(-1, -2), w16))
    R16 = r16(mm(kd16.transpose(-1, -2), u16))
    # ---- forward scan (fp32 master state, bf16 operand and bf16 snapshots)
    x = torch.zeros(B, H, K, V, dtype=f32) if h0 is None else h0.to(f32).clone()
    hs = []
    for c in range(NT):
        x16 = r16(x)
        hs.append(x16)
        x = a[:, :, c, None, None] * x - mm(P16[:, :, c], x16) + R16[:, :, c]
    hT = x
    h16 = torch.stack(hs, 2)
    # ---- output
    qg16 = r16((s * gam)[..., None] * qc)
    vn16 = r16(u16 - mm(w16, h16))
    o = r16(mm(qg16, h16) + mm(A16, vn16))
    # ---- backward: pre
    dvl = mm(A16.transpose(-1, -2), doc)
    dvl16 = r16(dvl)
    Rb16 = r16(mm(qg16.transpose(-1, -2), doc) - mm(w16.transpose(-1, -2), dvl16))
    D = torch.zeros(B, H, K, V, dtype=f32) if dhT is None else dhT.to(f32).clone()
    dhs = [None] * NT
    for c in reversed(range(NT)):
        D16 = r16(D)
        dhs[c] = D16
        D = a[:, :, c, None, None] * D - mm(P16[:, :, c].transpose(-1, -2), D16) + Rb16[:, :, c]
    dh0 = D
    dh16 = torch.stack(dhs, 2)
    # ---- backward: stage B
    dv2 = mm(kd16, dh16) + dvl
    dv2_16 = r16(dv2)
    dqg = mm(doc, h16.transpose(-1, -2))
    dA = torch.tril(mm(doc, vn16.transpose(-1, -2)))
    dAr16 = r16(s * dA * ratio)          # the q scale is folded into this operand
    dq_in = mm(dAr16, kc)
    dk_in = mm(dAr16.transpose(-1, -2), qc)
    dk_dec = mm(vn16, dh16.transpose(-1, -2))
    dq = dqg * (s * gam)[..., None] + dq_in
    dk = dk_in + dk_dec * dec_end[..., None]
    # scalar-gate dg: row/column sums of dA.A replace the per-channel products
    dAA = dA * (s * ratio * QK)
    dG = (dqg * qg16).sum(-1) + dAA.sum(-1) - dAA.sum(-2) - (dk_dec * kd16).sum(-1)
    dG_last = a * (dh16 * h16).sum((-1, -2)) + (dk_dec * kd16).sum((-1, -2))
    dG[..., -1] = dG[..., -1] + dG_last
    ws = dict(T=T16 if delta else None, A=A16, u=u16, w=w16, P=P16, R=R16, h=h16, v_new=vn16,
              Rb=Rb16, dh=dh16, dv2=dv2, o=o)
    if delta:
        dw = -mm(dv2_16, h16.transpose(-1, -2))
        dw16 = r16(dw)
        Tt = T16.transpose(-1, -2)
        dbv = mm(Tt, dv2_16)
        dbgk = mm(Tt, dw16)
        dT16 = r16(mm(dv2_16, bv16.transpose(-1, -2)) + mm(dw16, bgk16.transpose(-1, -2)))
        X16 = r16(mm(dT16, Tt))
        dM = torch.tril(-mm(Tt, X16), -1)
        dkk = dM * bc[..., None] * ratio
        sym16 = r16(dkk + dkk.transpose(-1, -2))
        dk = dk + mm(sym16, kc) + (bc * gam)[..., None] * dbgk
        dv = bc[..., None] * dbv
        p = (dbgk * kc).sum(-1)
        rr = (dbv * vc).sum(-1)
        dbeta = rr + gam * p + (dM * ratio * KK).sum(-1)
        e = dkk * KK
        dG = dG + e.sum(-1) - e.sum(-2) + bc * p * gam
        dbeta_tok = dbeta.reshape(B, H, L).transpose(1, 2).contiguous()
        ws.update(dw=dw, dM=dM)
    else:
        dv = dv2
        dbeta_tok = None
    dg = torch.flip(torch.cumsum(torch.flip(dG, [-1]), -1), [-1])
    dg_tok = dg.reshape(B, H, L).transpose(1, 2).contiguous()
    gr = Grads(dq=r16(_unchunks(dq)), dk=r16(_unchunks(dk)), dv=r16(_unchunks(dv)),
               dg=dg_tok if g is not None else None, dbeta=dbeta_tok,
               dh0=dh0 if h0 is not None else None)
    return _unchunks(o), hT, gr, ws
