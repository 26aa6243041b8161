"""CPU oracle for the chunked gated-delta-rule (GDN family) forward and backward.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is the
checker used by the test-suite, by the smoke check and by the CPU-baseline leg of the benchmark.

It restates, in plain PyTorch on the CPU, the algorithm of the reference project
(RishiShah99/lethe).  Two independent statements are kept so that each can check the other:

* ``serial_forward`` / ``serial_backward`` -- the token-by-token recurrence with autograd.  This is
  the ground truth (reference: ``src/lethe/kernels/references/gdn_backward.py:13-55`` for the
  recurrence and ``:70-122`` for the autograd backward; the family variants follow
  ``src/lethe/kernels/references/family_oracles.py:35-235``).
* ``chunk_forward`` / ``chunk_backward`` -- the chunkwise (UT / WY transform) form with a hand-derived
  closed-form backward.  It follows the reference's chunkwise forward
  (``src/lethe/kernels/references/gdn2_chunkwise.py:130-163`` scalar gate,
  ``src/lethe/kernels/references/gdn2_chunkwise_cw.py:139-181`` channel-wise gate), its reverse
  state scan "K#1" (``src/lethe/kernels/cute/gdn2_assemble.py:71-99`` and ``:377-404``), its closed
  "Stage B" VJP (``:521-585``) and its WY / triangular-inverse VJP "K#2" (``:102-147`` and
  ``:407-473``).  It also exposes every intermediate the CUDA kernels write to their workspace so
  that the GPU tests can compare stage by stage.

Parity pin: both statements are checked against golden vectors produced by running the reference
itself (``tests/golden/make_golden.py``), see ``tests/test_oracle_golden.py``.

Conventions (all tensors token-major like the reference op):
  q, k : [B, L, H, K]      v : [B, L, H, V]      beta : [B, L, H] or None (no delta term)
  g    : [B, L, H] (scalar log-decay), [B, L, H, K] (channel-wise) or None (no decay)
  h0   : [B, H, K, V] or None.   ``scale`` multiplies q (default K ** -0.5).
With ``beta=None`` the erase term vanishes and the write gate is one (linear attention, GLA, SSD).
With ``beta`` given, erase and write gates are both ``beta`` (gated delta rule, KDA).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import Tensor


# ----------------------------------------------------------------------------------------------
# metric
# ----------------------------------------------------------------------------------------------
def scale_rel(got: Tensor, ref: Tensor) -> float:
    """max|got - ref| / max|ref| -- the reference's per-tensor parity metric
    (``tests/test_gdn2_assemble.py:50-51``; ``results/*.json`` field ``scale_rel``)."""
    ref = ref.double()
    den = float(ref.abs().max())
    num = float((got.detach().double() - ref.detach()).abs().max())
    return num / den if den > 0 else num


# ----------------------------------------------------------------------------------------------
# token-serial truth
# ----------------------------------------------------------------------------------------------
def _gate_cw(g: Tensor | None, like_k: Tensor) -> Tensor | None:
    """Broadcast a scalar gate over the key channels; leave a channel-wise gate alone."""
    if g is None:
        return None
    return g.unsqueeze(-1).expand_as(like_k) if g.dim() == 3 else g


def serial_forward(q, k, v, g, beta, h0=None, *, scale=None):
    """Token-serial recurrence.  Returns ``(o [B,L,H,V], h_T [B,H,K,V])``.

    Per token: S <- S * exp(g_t);  v_new = w_t v_t - (b_t k_t)^T S;  S <- S + k_t v_new^T;
    o_t = (scale q_t)^T S  (reference ``gdn_backward.py:45-53``), with b = w = beta, or b = 0 and
    w = 1 when ``beta`` is None (``family_oracles.py:50-54``, ``:101-104``, ``:151-155``).
    """
    B, L, H, K = k.shape
    V = v.shape[-1]
    s = K ** -0.5 if scale is None else scale
    S = torch.zeros(B, H, K, V, dtype=q.dtype) if h0 is None else h0.to(q.dtype)
    gc = _gate_cw(g, k)
    outs = []
    for t in range(L):
        kt = k[:, t]  # [B,H,K]
        if gc is not None:
            S = S * gc[:, t].exp().unsqueeze(-1)
        if beta is None:
            vn = v[:, t]
        else:
            bt = beta[:, t].unsqueeze(-1)  # [B,H,1]
            vn = bt * (v[:, t] - torch.einsum("bhk,bhkv->bhv", kt, S))
        S = S + kt.unsqueeze(-1) * vn.unsqueeze(-2)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t] * s, S))
    return torch.stack(outs, dim=1), S


@dataclass
class Grads:
    dq: Tensor
    dk: Tensor
    dv: Tensor
    dg: Tensor | None
    dbeta: Tensor | None
    dh0: Tensor | None


def serial_backward(q, k, v, g, beta, h0, do, dhT=None, *, scale=None):
    """Autograd through ``serial_forward`` (reference ``gdn_backward.py:70-122``).

    Returns ``(o, h_T, Grads)``.  ``dhT`` is the adjoint of the final state (zero if None).
    """
    leaves = {}
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta), ("h0", h0)):
        leaves[name] = None if t is None else t.detach().clone().requires_grad_(True)
    o, hT = serial_forward(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                           leaves["h0"], scale=scale)
    names = [n for n, t in leaves.items() if t is not None]
    outs, gouts = [o], [do]
    if dhT is not None:
        outs.append(hT)
        gouts.append(dhT)
    gr = torch.autograd.grad(outs, [leaves[n] for n in names], gouts, allow_unused=True)
    d = dict(zip(names, gr))
    return o.detach(), hT.detach(), Grads(d["q"], d["k"], d["v"], d.get("g"), d.get("beta"),
                                          d.get("h0"))


# ----------------------------------------------------------------------------------------------
# the full op: independent per-channel erase gate b [B,L,H,K] and write gate w [B,L,H,V]
# ----------------------------------------------------------------------------------------------
def serial_forward_full(q, k, v, g, b, w, h0=None, *, scale=None):
    """Token-serial recurrence of the reference's six-input op (``gdn_backward.py:45-53``):
    S <- S * exp(g_t);  v_new = w_t v_t - (b_t k_t)^T S;  S <- S + k_t v_new^T;  o_t = (scale q_t)^T S,
    with ``g, b [B,L,H,K]`` and ``w [B,L,H,V]``.  Returns ``(o, h_T)``."""
    B, L, H, K = k.shape
    V = v.shape[-1]
    s = K ** -0.5 if scale is None else scale
    S = torch.zeros(B, H, K, V, dtype=q.dtype) if h0 is None else h0.to(q.dtype)
    outs = []
    for t in range(L):
        kt = k[:, t]
        S = S * g[:, t].exp().unsqueeze(-1)
        vn = w[:, t] * v[:, t] - torch.einsum("bhk,bhkv->bhv", b[:, t] * kt, S)
        S = S + kt.unsqueeze(-1) * vn.unsqueeze(-2)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t] * s, S))
    return torch.stack(outs, dim=1), S


def serial_backward_full(q, k, v, g, b, w, h0, do, dhT=None, *, scale=None):
    """Autograd through ``serial_forward_full`` (reference ``gdn_backward.py:70-122``).  Returns
    ``(o, h_T, grads)`` with ``grads`` a dict over q, k, v, g, b, w and h0 (when given)."""
    leaves = {}
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("b", b), ("w", w), ("h0", h0)):
        leaves[name] = None if t is None else t.detach().clone().requires_grad_(True)
    o, hT = serial_forward_full(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["b"], leaves["w"],
                                leaves["h0"], scale=scale)
    names = [n for n, t in leaves.items() if t is not None]
    outs, gouts = [o], [do]
    if dhT is not None:
        outs.append(hT)
        gouts.append(dhT)
    gr = torch.autograd.grad(outs, [leaves[n] for n in names], gouts, allow_unused=True)
    return o.detach(), hT.detach(), dict(zip(names, gr))


# ----------------------------------------------------------------------------------------------
# chunkwise form
# ----------------------------------------------------------------------------------------------
def _chunks(x: Tensor, C: int) -> Tensor:
    """[B, L, H, D] -> [B, H, NT, C, D] (reference ``gdn2_chunkwise.py:19-26``)."""
    B, L, H, D = x.shape
    return x.transpose(1, 2).reshape(B, H, L // C, C, D)


def _unchunks(x: Tensor) -> Tensor:
    """[B, H, NT, C, D] -> [B, L, H, D] (reference ``gdn2_chunkwise.py:28-31``)."""
    B, H, NT, C, D = x.shape
    return x.reshape(B, H, NT * C, D).transpose(1, 2).contiguous()


@dataclass
class ChunkState:
    """Everything the chunkwise forward produces; shapes are head-major ``[B,H,NT,...]``."""

    C: int
    scale: float
    scalar_gate: bool
    delta: bool
    qs: Tensor      # scale * q                         [.., C, K]
    k: Tensor       #                                   [.., C, K]
    v: Tensor       #                                   [.., C, V]
    beta: Tensor | None  #                              [.., C]
    G: Tensor       # in-chunk inclusive cumsum of g (natural log), broadcast to [.., C, K]
    ratio: Tensor   # exp(G_i - G_s), zero for s > i    [.., C, C, K]
    T: Tensor       # (I + strict_lower(M))^-1          [.., C, C]
    A: Tensor       # tril((qs k^T) . ratio)            [.., C, C]
    u: Tensor       # T (beta v)                        [.., C, V]
    w: Tensor       # T (beta gamma k)                  [.., C, K]
    kd: Tensor      # k * exp(G_last - G_i)             [.., C, K]
    a: Tensor       # exp(G_last)                       [.., K]
    P: Tensor       # kd^T w                            [.., K, K]
    R: Tensor       # kd^T u                            [.., K, V]
    h: Tensor       # chunk-entry states, NT+1 of them  [B,H,NT+1,K,V]
    v_new: Tensor   # u - w h_c                         [.., C, V]
    o: Tensor       # token-major output                [B,L,H,V]
    extra: dict = field(default_factory=dict)


def chunk_forward(q, k, v, g, beta, h0=None, *, scale=None, C=64) -> ChunkState:
    """Chunkwise forward with the inter-chunk recurrence written as one affine map per chunk.

    Per chunk (reference ``gdn2_chunkwise.py:130-158``, ``gdn2_chunkwise_cw.py:139-175``):
      M = strict_lower(beta_i * sum_d k_i k_s ratio),  T = (I + M)^-1,  u = T(beta v),
      w = T(beta gamma k),  v_new = u - w h,  o = (qs gamma) h + A v_new,
      h' = exp(G_last) h + kd^T v_new.
    Substituting v_new gives  h' = a*h - (kd^T w) h + kd^T u = a*h - P h + R, which is how the
    CUDA scan kernel advances the state (one product per chunk on the serial path).
    """
    B, L, H, K = k.shape
    V = v.shape[-1]
    assert L % C == 0
    NT = L // C
    s = K ** -0.5 if scale is None else scale
    dt = q.dtype
    qs, kc, vc = _chunks(q * s, C), _chunks(k, C), _chunks(v, C)
    scalar_gate = g is None or g.dim() == 3
    if g is None:
        G = torch.zeros(B, H, NT, C, K, dtype=dt)
    else:
        G = torch.cumsum(_chunks(_gate_cw(g, k), C), dim=-2)
    gam = G.exp()
    # exponent masked before exp so the strict upper triangle is exactly zero and never
    # overflows (reference gdn2_chunkwise.py:33-38)
    diff = G.unsqueeze(-2) - G.unsqueeze(-3)                      # [.., i, s, K]
    upper = torch.triu(torch.ones(C, C, dtype=torch.bool), 1)
    ratio = diff.masked_fill(upper[..., None], float("-inf")).exp()
    A = torch.einsum("...id,...sd,...isd->...is", qs, kc, ratio)
    eye = torch.eye(C, dtype=dt)
    if beta is not None:
        bc = beta.transpose(1, 2).reshape(B, H, NT, C)
        Mm = bc[..., None] * torch.einsum("...id,...sd,...isd->...is", kc, kc, ratio)
        Mm = torch.tril(Mm, -1)
        T = torch.linalg.solve_triangular(eye + Mm, eye.expand_as(Mm), upper=False,
                                          unitriangular=True)
        u = T @ (bc[..., None] * vc)
        w = T @ (bc[..., None] * gam * kc)
    else:
        bc = None
        T = eye.expand(B, H, NT, C, C).clone()
        u = vc.clone()
        w = torch.zeros_like(kc)
    Glast = G[..., -1, :]                                          # [.., K]
    kd = kc * (Glast.unsqueeze(-2) - G).exp()
    a = Glast.exp()
    P = kd.transpose(-1, -2) @ w
    R = kd.transpose(-1, -2) @ u
    h = torch.zeros(B, H, NT + 1, K, V, dtype=dt)
    if h0 is not None:
        h[:, :, 0] = h0
    for c in range(NT):
        h[:, :, c + 1] = a[:, :, c, :, None] * h[:, :, c] - P[:, :, c] @ h[:, :, c] + R[:, :, c]
    hc = h[:, :, :-1]
    v_new = u - w @ hc
    o = (qs * gam) @ hc + A @ v_new
    return ChunkState(C=C, scale=s, scalar_gate=scalar_gate, delta=beta is not None, qs=qs, k=kc,
                      v=vc, beta=bc, G=G, ratio=ratio, T=T, A=A, u=u, w=w, kd=kd, a=a, P=P, R=R,
                      h=h, v_new=v_new, o=_unchunks(o))


def chunk_backward(st: ChunkState, do: Tensor, dhT: Tensor | None = None):
    """Closed-form backward of ``chunk_forward``.  Returns ``(Grads, intermediates dict)``.

    Steps (reference citations in the module docstring):
      dv_local = A^T do;  Rb = (qs gamma)^T do - w^T dv_local;
      reverse scan  dh[c] = D;  D <- a*D - P^T D + Rb   (equal to K#1 after substituting dv2);
      dv2 = kd dh + dv_local;  Stage B;  WY / inverse VJP (K#2);  in-chunk reverse cumsum for dg.
    """
    C, K = st.C, st.k.shape[-1]
    B, H, NT = st.k.shape[:3]
    V = st.v.shape[-1]
    dt = st.k.dtype
    doc = _chunks(do, C)
    gam = st.G.exp()
    qg = st.qs * gam
    dv_local = st.A.transpose(-1, -2) @ doc
    Rb = qg.transpose(-1, -2) @ doc - st.w.transpose(-1, -2) @ dv_local
    D = torch.zeros(B, H, K, V, dtype=dt) if dhT is None else dhT.clone()
    dh = torch.zeros(B, H, NT, K, V, dtype=dt)
    for c in reversed(range(NT)):
        dh[:, :, c] = D
        D = st.a[:, :, c, :, None] * D - st.P[:, :, c].transpose(-1, -2) @ D + Rb[:, :, c]
    dh0 = D
    hc = st.h[:, :, :-1]
    dv2 = st.kd @ dh + dv_local
    # ---- Stage B
    dqg = doc @ hc.transpose(-1, -2)
    dA = torch.tril(doc @ st.v_new.transpose(-1, -2))
    dq_in = torch.einsum("...is,...sd,...isd->...id", dA, st.k, st.ratio)
    dk_in = torch.einsum("...is,...id,...isd->...sd", dA, st.qs, st.ratio)
    dk_dec = st.v_new @ dh.transpose(-1, -2)
    dec_end = (st.G[..., -1:, :] - st.G).exp()
    dqs = dqg * gam + dq_in
    dk = dk_in + dk_dec * dec_end
    dde = dk_dec * st.k * dec_end
    dG = dqg * qg + st.qs * dq_in - st.k * dk_in - dde
    dG_last = st.a * (dh * hc).sum(-1) + dde.sum(-2)
    dG[..., -1, :] = dG[..., -1, :] + dG_last
    inter = dict(dv_local=dv_local, Rb=Rb, dh=dh, dv2=dv2, dqg=dqg, dA=dA, dk_dec=dk_dec)
    # ---- WY / triangular-inverse VJP
    if st.delta:
        bc = st.beta[..., None]
        dw = -dv2 @ hc.transpose(-1, -2)
        Tt = st.T.transpose(-1, -2)
        dp = Tt @ dv2
        dq_wy = Tt @ dw
        bv = bc * st.v
        bgk = bc * gam * st.k
        dT = dv2 @ bv.transpose(-1, -2) + dw @ bgk.transpose(-1, -2)
        dM = torch.tril(-(Tt @ dT @ Tt), -1)
        dv = bc * dp
        dbeta = (dp * st.v).sum(-1)
        dbk_m = torch.einsum("...is,...sd,...isd->...id", dM, st.k, st.ratio)
        dk_m = torch.einsum("...is,...id,...isd->...sd", dM, bc * st.k, st.ratio)
        dbk = dq_wy * gam + dbk_m
        dbeta = dbeta + (dbk * st.k).sum(-1)
        dk = dk + dbk * bc + dk_m
        dG = dG + dq_wy * bgk + bc * st.k * dbk_m - st.k * dk_m
        inter.update(dw=dw, dT=dT, dM=dM, dp=dp, dq_wy=dq_wy)
        dbeta_tok = dbeta.reshape(B, H, NT * C).transpose(1, 2).contiguous()
    else:
        dv = dv2
        dbeta_tok = None
    dg_c = torch.flip(torch.cumsum(torch.flip(dG, [-2]), -2), [-2])
    dg = _unchunks(dg_c)
    if st.scalar_gate:
        dg = dg.sum(-1)
    return Grads(dq=_unchunks(dqs) * st.scale, dk=_unchunks(dk), dv=_unchunks(dv), dg=dg,
                 dbeta=dbeta_tok, dh0=dh0), inter


def chunk_fwd_bwd(q, k, v, g, beta, h0, do, dhT=None, *, scale=None, C=64):
    """Convenience: chunkwise forward + closed-form backward.  Returns (o, h_T, Grads)."""
    st = chunk_forward(q, k, v, g, beta, h0, scale=scale, C=C)
    gr, _ = chunk_backward(st, do, dhT)
    if g is None:
        gr.dg = None
    if h0 is None:
        gr.dh0 = None
    return st.o, st.h[:, :, -1], gr


LN2 = math.log(2.0)
