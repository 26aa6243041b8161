"""Generate the golden vectors under tests/golden/ by running the reference project itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference/src

It imports the reference's own fp64 PyTorch oracles (token-serial GDN-2 and the GLA / LA / SSD /
KDA family oracles) and its chunkwise forward, feeds them seeded inputs and stores inputs and
outputs as compressed ``.npz`` files.  The committed files pin ``oracle/gdn_oracle.py``
(``tests/test_oracle_golden.py``) and are compared with the CUDA path on the GPU
(``tests/test_gpu_parity.py``).  The reference cannot travel to the GPU machine; these files can.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def draw(seed, B, L, H, K, V, gate, strong):
    """q,k L2-normalised N(0,1); v N(0,1); beta sigmoid(N); g = -softplus(N+3) (strong) or
    -0.1*U(0,1) (the reference bench draw); do N(0,1); h0 0.1*N."""
    gen = torch.Generator().manual_seed(seed)
    dt = torch.float64
    q = torch.randn(B, L, H, K, generator=gen, dtype=dt)
    k = torch.randn(B, L, H, K, generator=gen, dtype=dt)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(B, L, H, V, generator=gen, dtype=dt)
    beta = torch.randn(B, L, H, generator=gen, dtype=dt).sigmoid()
    gshape = (B, L, H) if gate == "scalar" else (B, L, H, K)
    if strong:
        g = -F.softplus(torch.randn(*gshape, generator=gen, dtype=dt) + 3.0)
    else:
        g = -0.1 * torch.rand(*gshape, generator=gen, dtype=dt)
    do = torch.randn(B, L, H, V, generator=gen, dtype=dt)
    h0 = 0.1 * torch.randn(B, H, K, V, generator=gen, dtype=dt)
    # Inputs are rounded to what the CUDA path is fed (bf16 for q, k, v, do; fp32 for the gates
    # and the state) so that the stored fp64 results are exact answers for exactly these inputs.
    q, k, v, do = (t.to(torch.bfloat16).to(dt) for t in (q, k, v, do))
    g, beta, h0 = (t.to(torch.float32).to(dt) for t in (g, beta, h0))
    return q, k, v, g, beta, do, h0


def main(ref_src: str) -> None:
    sys.path.insert(0, ref_src)
    from lethe.kernels.references import family_oracles as fam
    from lethe.kernels.references.gdn2_chunkwise import chunkwise_forward
    from lethe.kernels.references.gdn2_chunkwise_cw import chunkwise_forward_cw
    from lethe.kernels.references.gdn_backward import (
        reference_gdn2_backward,
        reference_gdn2_forward,
    )

    B, L, H, K, V, C = 1, 128, 2, 32, 16, 64
    scale = K ** -0.5

    def save(name, f32=False, **arrs):
        out = {k_: (v_.detach().numpy() if isinstance(v_, torch.Tensor) else np.asarray(v_))
               for k_, v_ in arrs.items() if v_ is not None}
        if f32:  # kernel-sized cases: results stored in fp32 (compared at 1e-6 / 5e-3)
            out = {k_: (v_.astype(np.float32) if v_.dtype == np.float64 and v_.ndim else v_)
                   for k_, v_ in out.items()}
        for k_ in ("q", "k", "v", "g", "beta", "do", "h0"):  # exactly representable in fp32
            if k_ in out:
                out[k_] = out[k_].astype(np.float32)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print("wrote", name, sorted(out))

    for strong in (True, False):
        tag = "strong" if strong else "mild"
        # ---- gated delta rule, scalar gate, with initial state (token-serial GDN-2 oracle with
        #      g, b, w broadcast over channels)
        q, k, v, g, beta, do, h0 = draw(11 + strong, B, L, H, K, V, "scalar", strong)
        gc = g[..., None].expand(B, L, H, K).contiguous()
        bc = beta[..., None].expand(B, L, H, K).contiguous()
        wc = beta[..., None].expand(B, L, H, V).contiguous()
        o = reference_gdn2_forward(q, k, v, gc, bc, wc, scale=scale, initial_state=h0,
                                   use_qk_l2norm=False)
        gr = reference_gdn2_backward(q, k, v, gc, bc, wc, do, scale=scale, initial_state=h0,
                                     use_qk_l2norm=False)
        cf = chunkwise_forward(q, k, v, g, beta, chunk_len=C, scale=scale, initial_state=h0,
                               use_qk_l2norm=False)
        save(f"gdn_scalar_{tag}", q=q, k=k, v=v, g=g, beta=beta, do=do, h0=h0, o=o,
             dq=gr.grad_q, dk=gr.grad_k, dv=gr.grad_v, dg=gr.grad_g.sum(-1),
             dbeta=gr.grad_b.sum(-1) + gr.grad_w.sum(-1), dh0=gr.grad_initial_state,
             cw_T=cf.T, cw_u=cf.u, cw_w=cf.w, cw_h=cf.h, cw_A=cf.A_qk, cw_vnew=cf.v_new,
             scale=scale, C=C)

        # ---- KDA (channel-wise gate + beta), family oracle, no initial state
        q, k, v, g, beta, do, h0 = draw(21 + strong, B, L, H, K, V, "cw", strong)
        o = fam.reference_kda_forward(q, k, v, g, beta, scale=scale, use_qk_l2norm=False)
        gr = fam.reference_kda_backward(q, k, v, g, beta, do, scale=scale, use_qk_l2norm=False)
        bc = beta[..., None].expand(B, L, H, K).contiguous()
        wc = beta[..., None].expand(B, L, H, V).contiguous()
        cf = chunkwise_forward_cw(q, k, v, g, bc, wc, chunk_len=C, scale=scale,
                                  use_qk_l2norm=False)
        save(f"kda_{tag}", q=q, k=k, v=v, g=g, beta=beta, do=do, o=o, dq=gr.grad_q,
             dk=gr.grad_k, dv=gr.grad_v, dg=gr.grad_g, dbeta=gr.grad_beta,
             cw_T=cf.T, cw_u=cf.u, cw_w=cf.wy, cw_h=cf.h, cw_A=cf.A_qk, cw_vnew=cf.v_new,
             scale=scale, C=C)

        # ---- GLA (channel-wise gate, no delta)
        q, k, v, g, beta, do, h0 = draw(31 + strong, B, L, H, K, V, "cw", strong)
        o = fam.reference_gla_forward(q, k, v, g, scale=scale, use_qk_l2norm=False)
        gr = fam.reference_gla_backward(q, k, v, g, do, scale=scale, use_qk_l2norm=False)
        save(f"gla_{tag}", q=q, k=k, v=v, g=g, do=do, o=o, dq=gr.grad_q, dk=gr.grad_k,
             dv=gr.grad_v, dg=gr.grad_g, scale=scale, C=C)

        # ---- SSD (scalar gate, no delta)
        q, k, v, g, beta, do, h0 = draw(41 + strong, B, L, H, K, V, "scalar", strong)
        o = fam.reference_ssd_forward(q, k, v, g, scale=scale, use_qk_l2norm=False)
        gr = fam.reference_ssd_backward(q, k, v, g, do, scale=scale, use_qk_l2norm=False)
        save(f"ssd_{tag}", q=q, k=k, v=v, g=g, do=do, o=o, dq=gr.grad_q, dk=gr.grad_k,
             dv=gr.grad_v, dg=gr.grad_g, scale=scale, C=C)

    # ---- kernel-sized cases (d_k = 128, d_v = 64, two chunks) for the GPU comparison
    Bg, Lg, Hg, Kg, Vg = 1, 128, 1, 128, 64
    sg = Kg ** -0.5
    q, k, v, g, beta, do, h0 = draw(61, Bg, Lg, Hg, Kg, Vg, "scalar", True)
    gc = g[..., None].expand(Bg, Lg, Hg, Kg).contiguous()
    bc = beta[..., None].expand(Bg, Lg, Hg, Kg).contiguous()
    wc = beta[..., None].expand(Bg, Lg, Hg, Vg).contiguous()
    o = reference_gdn2_forward(q, k, v, gc, bc, wc, scale=sg, initial_state=h0,
                               use_qk_l2norm=False)
    gr = reference_gdn2_backward(q, k, v, gc, bc, wc, do, scale=sg, initial_state=h0,
                                 use_qk_l2norm=False)
    save("gdn_scalar_k128", f32=True, q=q, k=k, v=v, g=g, beta=beta, do=do, h0=h0, o=o,
         dq=gr.grad_q, dk=gr.grad_k, dv=gr.grad_v, dg=gr.grad_g.sum(-1),
         dbeta=gr.grad_b.sum(-1) + gr.grad_w.sum(-1), dh0=gr.grad_initial_state, scale=sg, C=C)
    q, k, v, g, beta, do, h0 = draw(62, Bg, Lg, Hg, Kg, Vg, "cw", True)
    o = fam.reference_kda_forward(q, k, v, g, beta, scale=sg, use_qk_l2norm=False)
    gr = fam.reference_kda_backward(q, k, v, g, beta, do, scale=sg, use_qk_l2norm=False)
    save("kda_k128", f32=True, q=q, k=k, v=v, g=g, beta=beta, do=do, o=o, dq=gr.grad_q,
         dk=gr.grad_k, dv=gr.grad_v, dg=gr.grad_g, dbeta=gr.grad_beta, scale=sg, C=C)

    # ---- the full GDN-2 op: independent per-channel erase gate b [B,L,H,K] and write gate w [B,L,H,V]
    #      (reference_gdn2_forward / _backward as they stand), one small case and one kernel-sized case
    def full_gates(seed, Bx, Lx, Hx, Kx, Vx):
        gen = torch.Generator().manual_seed(seed)
        b = torch.randn(Bx, Lx, Hx, Kx, generator=gen, dtype=torch.float64).sigmoid()
        w = torch.randn(Bx, Lx, Hx, Vx, generator=gen, dtype=torch.float64).sigmoid()
        return b.to(torch.float32).to(torch.float64), w.to(torch.float32).to(torch.float64)

    for name, (Bx, Lx, Hx, Kx, Vx), seed, f32 in (("gdn2_full_small", (B, L, H, K, V), 71, False),
                                                    ("gdn2_full_k128", (Bg, Lg, Hg, Kg, Vg), 72, True)):
        q, k, v, g, beta, do, h0 = draw(seed, Bx, Lx, Hx, Kx, Vx, "cw", True)
        b, w = full_gates(seed + 100, Bx, Lx, Hx, Kx, Vx)
        sx = Kx ** -0.5
        o = reference_gdn2_forward(q, k, v, g, b, w, scale=sx, initial_state=h0, use_qk_l2norm=False)
        gr = reference_gdn2_backward(q, k, v, g, b, w, do, scale=sx, initial_state=h0, use_qk_l2norm=False)
        save(name, f32=f32, q=q, k=k, v=v, g=g, b=b.to(torch.float32), w=w.to(torch.float32), do=do, h0=h0, o=o,
             dq=gr.grad_q, dk=gr.grad_k, dv=gr.grad_v, dg=gr.grad_g, db=gr.grad_b, dw=gr.grad_w,
             dh0=gr.grad_initial_state, scale=sx, C=C)

    # ---- plain linear attention
    q, k, v, g, beta, do, h0 = draw(51, B, L, H, K, V, "scalar", True)
    o = fam.reference_la_forward(q, k, v, scale=scale, use_qk_l2norm=False)
    gr = fam.reference_la_backward(q, k, v, do, scale=scale, use_qk_l2norm=False)
    save("la", q=q, k=k, v=v, do=do, o=o, dq=gr.grad_q, dk=gr.grad_k, dv=gr.grad_v,
         scale=scale, C=C)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference/src")
    main(sys.argv[1])
