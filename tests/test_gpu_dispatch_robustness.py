"""GPU: the dispatch rules and the numerics-robustness pins the reference keeps in its own tests
(``tests/test_gdn2_dispatch.py``, ``tests/test_gdn2_drift_robustness.py`` of the reference project),
restated for this library's six-input surface; and the range behaviour of the fp16 operands."""

import math

import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import chunk_fwd_bwd, scale_rel, serial_backward, serial_backward_full

from .wsview import report

pytestmark = pytest.mark.gpu


def _scalar_gates(seed, dk=128, dv=64, B=2, L=64, H=3):
    gen = torch.Generator().manual_seed(seed)
    g_scalar = -torch.rand(B, L, H, 1, generator=gen)
    beta = torch.rand(B, L, H, 1, generator=gen)
    return (g_scalar.expand(B, L, H, dk).contiguous().cuda(), beta.expand(B, L, H, dk).contiguous().cuda(),
            beta.expand(B, L, H, dv).contiguous().cuda())


def test_exact_broadcast_routes_to_scalar():
    """Reference: tests/test_gdn2_dispatch.py:59-61."""
    g, b, w = _scalar_gates(seed=0)
    assert ops.gate_regime(g, b, w) == (True, True, False)


def test_near_constant_gate_routes_to_channelwise():
    """A gate that is constant over the channels only up to a tolerance is a channel-wise gate: the test
    is bitwise, never ``allclose`` (reference: tests/test_gdn2_dispatch.py:64-71,
    cute/gdn2_backward.py:53-60)."""
    g, b, w = _scalar_gates(seed=1)
    jitter = torch.zeros_like(g)
    jitter[..., 0] = 1e-9
    g_near = g + jitter
    assert torch.allclose(g_near, g_near[..., :1].expand_as(g_near))      # the trap a tolerance falls into
    scalar_gate, one_beta, no_delta = ops.gate_regime(g_near, b, w)
    assert scalar_gate is False and one_beta is True and no_delta is False
    # ... and the op really runs the channel-wise kernels for it: same numbers as gdn_chunk with g [B,L,H,K]
    B, L, H, K = g.shape
    V = w.shape[-1]
    inp = make_inputs(B, L, H, K, V, gate="channel", delta=True, seed=3, with_h0=False)
    q, k, v, do = (inp[n].cuda() for n in ("q", "k", "v", "do"))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g_near, b, w)]
    o = ops.gdn2_op(*leaves, use_qk_l2norm=False)
    dq = torch.autograd.grad(o, leaves[0], do)[0]
    q2 = q.clone().requires_grad_(True)
    o2, _ = ops.gdn_chunk(q2, k, v, g_near, b[..., 0].contiguous(), None)
    dq2 = torch.autograd.grad(o2, q2, do)[0]
    assert torch.equal(o, o2) and torch.equal(dq, dq2)


def test_unequal_b_and_w_route_to_the_full_op():
    g, b, w = _scalar_gates(seed=2)
    w2 = (w * 0.5).contiguous()
    assert ops.gate_regime(g, b, w2)[1] is False
    zeros, ones = torch.zeros_like(b), torch.ones_like(w)
    assert ops.gate_regime(g, zeros, ones) == (True, False, True)


def test_backward_declines_a_second_derivative():
    """The reference's native path returns None when ``do.requires_grad`` and its caller falls back to the
    eager oracle (tests/test_gdn2_dispatch.py:118-127, cute/gdn2_backward.py:92).  There is no eager path
    here, so the same situation must fail loudly instead of returning gradients with no graph."""
    inp = make_inputs(1, 64, 1, 128, 64, gate="scalar", delta=True, seed=5, with_h0=False)
    q, k, v, g, beta, do = (inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "do"))
    q = q.float().requires_grad_(True)
    o, _ = ops.gdn_chunk(q, k, v, g, beta, None)
    dof = do.float().requires_grad_(True)
    (dq,) = torch.autograd.grad(o, q, dof, create_graph=True)
    with pytest.raises(RuntimeError, match="differentiate twice|once_differentiable"):
        dq.sum().backward()                       # a derivative of the backward with respect to do
    o, _ = ops.gdn_chunk(q, k, v, g, beta, None)
    (dq,) = torch.autograd.grad(o, q, do.float(), create_graph=True)
    assert not dq.requires_grad                   # no graph is pretended where none exists
    gK, bK, wV = (g[..., None].expand(1, 64, 1, 128).contiguous(), beta[..., None].expand(1, 64, 1, 128).contiguous(),
                  beta[..., None].expand(1, 64, 1, 64).contiguous())
    with pytest.raises(ops.GdnError, match="not differentiable"):
        ops.gdn2_backward(q.detach(), k, v, gK, bK, wV, do.float().requires_grad_(True))


# ---- numerics robustness: decay regimes past the exponent cliffs -------------------------------------------------
def test_channelwise_gate_drifted_regime_finite_and_matches_fp64():
    """Mean log decay -1.7 per token: a 64-token chunk spans ~157 in log2, past the fp32 exp2 cliff (128)
    (reference: tests/test_gdn2_drift_robustness.py:14-52, there at d = 16)."""
    B, L, H, K, V = 2, 128, 2, 128, 64
    gen = torch.Generator().manual_seed(7)
    inp = make_inputs(B, L, H, K, V, gate="channel", delta=True, seed=7, full=True, with_h0=False)
    g = -1.7 - 0.5 * torch.rand(B, L, H, K, generator=gen)
    span = float((-g.reshape(B, 2, 64, H, K).sum(2)).max()) / math.log(2.0)
    assert span > 128
    names = ("q", "k", "v", "g", "b", "w")
    inp["g"] = g
    inp["b"] = torch.rand(B, L, H, K, generator=gen) * 0.9 + 0.05
    inp["w"] = torch.rand(B, L, H, V, generator=gen) * 0.9 + 0.05
    leaves = [inp[n].cuda().requires_grad_(True) for n in names]
    o, _ = ops.gdn_chunk_full(*leaves)
    grads = torch.autograd.grad(o, leaves, inp["do"].cuda())
    f = {n: inp[n].double() for n in names}
    o_ref, _, gr = serial_backward_full(f["q"], f["k"], f["v"], f["g"], f["b"], f["w"], None, inp["do"].double())
    errs = {"o": scale_rel(o.detach().double().cpu(), o_ref)}
    for n, t in zip(names, grads):
        assert torch.isfinite(t).all(), n
        errs["d" + n] = scale_rel(t.double().cpu(), gr[n])
    report(f"drifted channel-wise regime (chunk log2 span {span:.0f})", errs)
    assert max(errs.values()) <= 5e-3, errs


def test_scalar_gate_finite_past_gamma_underflow():
    """Mean log decay -4 per token: chunk log2 span ~370, gamma underflows fp32 inside every chunk
    (reference: tests/test_gdn2_drift_robustness.py:55-70)."""
    B, L, H, K, V = 1, 128, 2, 128, 64
    inp = make_inputs(B, L, H, K, V, gate="scalar", delta=True, seed=11, with_h0=False)
    gen = torch.Generator().manual_seed(11)
    inp["g"] = -4.0 - torch.rand(B, L, H, generator=gen)
    inp["beta"] = torch.rand(B, L, H, generator=gen) * 0.9 + 0.05
    names = ("q", "k", "v", "g", "beta")
    leaves = [inp[n].cuda().requires_grad_(True) for n in names]
    o, _ = ops.gdn_chunk(*leaves, None)
    grads = torch.autograd.grad(o, leaves, inp["do"].cuda())
    f = {n: inp[n].double() for n in names}
    o_ref, _, gr = serial_backward(f["q"], f["k"], f["v"], f["g"], f["beta"], None, inp["do"].double())
    refs = dict(q=gr.dq, k=gr.dk, v=gr.dv, g=gr.dg, beta=gr.dbeta)
    errs = {"o": scale_rel(o.detach().double().cpu(), o_ref)}
    for n, t in zip(names, grads):
        assert torch.isfinite(t).all(), n
        errs["d" + n] = scale_rel(t.double().cpu(), refs[n])
    report("scalar gate past gamma underflow", errs)
    assert max(errs.values()) <= 5e-3, errs


# ---- range of the fp16 operands ------------------------------------------------------------------------------------
def test_values_beyond_fp16_range_saturate_instead_of_poisoning():
    """v and do enter the tensor cores as fp16.  A magnitude beyond 65504 is clamped to the largest finite
    fp16 value by the conversion (never to infinity), so the result equals the result for the clamped
    input and stays finite; nothing turns into NaN."""
    B, L, H, K, V = 1, 128, 2, 128, 64
    inp = make_inputs(B, L, H, K, V, gate="scalar", delta=True, seed=17)
    big = inp["v"].clone()
    big[0, 5, 0, 3] = 3e5                                        # head 0 only
    big[0, 70, 0, 9] = -3e38
    d = {n: (None if t is None else t.cuda()) for n, t in inp.items()}

    def run(v):
        leaves = [d["q"].clone().requires_grad_(True), d["k"].clone().requires_grad_(True),
                  v.cuda().requires_grad_(True)]
        o, hT = ops.gdn_chunk(leaves[0], leaves[1], leaves[2], d["g"], d["beta"], d["h0"])
        return (o.detach(), hT.detach()) + torch.autograd.grad(o, leaves, d["do"])

    base, got = run(inp["v"]), run(big)
    for t in got:
        assert torch.isfinite(t.float()).all()                   # clamped, never inf, never NaN
    # heads are independent: head 1 is bit for bit what it is without the out-of-range values
    for a, b_ in zip(got, base):
        if a.dim() == 4 and a.shape[1] == L:
            assert torch.equal(a[:, :, 1], b_[:, :, 1])
        else:
            assert torch.equal(a[:, 1], b_[:, 1])


def test_backward_entry_point_rescales_extreme_upstream_gradients():
    """``gdn2_backward`` divides ``do`` by a power of two near its largest magnitude before the kernels and
    multiplies the gradients back: upstream gradients a million times larger or smaller than one (far
    outside what fp16 resolves) give the same relative accuracy as ordinary ones."""
    B, L, H, K, V = 1, 128, 2, 128, 64
    inp = make_inputs(B, L, H, K, V, gate="scalar", delta=True, seed=19, with_h0=False)
    q, k, v, g, beta, do = (inp[n] for n in ("q", "k", "v", "g", "beta", "do"))
    gK = g[..., None].expand(B, L, H, K).contiguous()
    bK, wV = beta[..., None].expand(B, L, H, K).contiguous(), beta[..., None].expand(B, L, H, V).contiguous()
    _, _, gr = chunk_fwd_bwd(q.double(), k.double(), v.double(), g.double(), beta.double(), None, do.double())
    for mag in (1.0, 2.0 ** 20, 2.0 ** -20):        # powers of two: do stays exactly representable in bf16
        got = ops.gdn2_backward(q.cuda(), k.cuda(), v.cuda(), gK.cuda(), bK.cuda(), wV.cuda(),
                                (do.float() * mag).cuda(), use_qk_l2norm=False)
        errs = {"dq": scale_rel(got.grad_q.double().cpu(), gr.dq * mag),
                "dk": scale_rel(got.grad_k.double().cpu(), gr.dk * mag),
                "dv": scale_rel(got.grad_v.double().cpu(), gr.dv * mag),
                "dg": scale_rel(got.grad_g.double().cpu().sum(-1), gr.dg * mag),
                "dbeta": scale_rel((got.grad_b.double().sum(-1) + got.grad_w.double().sum(-1)).cpu(), gr.dbeta * mag)}
        report(f"gdn2_backward, |do| ~ {mag:g}", errs)
        assert max(errs.values()) <= 5e-3, (mag, errs)
