"""GPU: the reference's OWN code on both sides of the drop-in boundary, unchanged.

* its backward assemblies ``assemble_gdn2_backward_scalar`` / ``assemble_gdn2_backward_channelwise``
  (``cute/gdn2_assemble.py:242-314, 601-696``) driven through their ``k1_fn`` / ``k2_fn`` hooks by the
  CUDA kernels (``lethe_b200.plugins``), against the same calls with no plug-in (the reference's torch
  statements of K#1 / K#2);
* its autograd function ``_GDN2Function`` / ``gdn2_op`` (``ops/gdn_layer.py:15-111``) with the backward
  entry point ``gdn2_backward`` replaced by ``lethe_b200.ops.gdn2_backward``, against itself unpatched;
* its family wrappers (``cute/gdn2_family.py``) against ``lethe_b200.family`` on the same inputs.

The reference modules come from ``oracle/_ref`` (see tests/refimport.py).  Whatever the reference
computes by itself ("want") runs on CPU tensors, where it has only its eager PyTorch path: its own
device kernels (CuTe-DSL, compiled at run time) are never reached from these tests."""

import os

import pytest
import torch

os.environ.setdefault("FMR_DISABLE_SBE", "1")     # the reference's optional device kernel for Stage B stays off

from lethe_b200 import family, ops, plugins
from oracle.gdn_oracle import scale_rel

from .refimport import reference
from .wsview import report

pytestmark = pytest.mark.gpu
TOL = 5e-3


def _inputs(B, L, H, K, V, seed, channelwise):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, L, H, K, generator=gen)
    k = torch.randn(B, L, H, K, generator=gen)
    v = torch.randn(B, L, H, V, generator=gen)
    g = -0.1 * torch.rand(B, L, H, K if channelwise else 1, generator=gen)
    beta = torch.rand(B, L, H, generator=gen) * 0.8 + 0.1
    do = torch.randn(B, L, H, V, generator=gen)
    # values the kernels read exactly: bf16-representable q, k, v, do
    rb = lambda t: t.bfloat16().float()  # noqa: E731
    return [rb(q), rb(k), rb(v), g if channelwise else g[..., 0], beta, rb(do)]       # CPU tensors


def cu(ts):
    return [t.cuda() for t in ts]


def test_reference_scalar_assembly_driven_by_the_cuda_plugins():
    reference()
    from lethe.kernels.cute.gdn2_assemble import assemble_gdn2_backward_scalar

    cpu = _inputs(2, 256, 2, 128, 64, seed=5, channelwise=False)
    want = assemble_gdn2_backward_scalar(*cpu)                                      # reference K#1 / K#2, CPU
    got = assemble_gdn2_backward_scalar(*cu(cpu), k1_fn=plugins.k1_fn, k2_fn=plugins.k2_fn)
    errs = {n: scale_rel(getattr(got, n).double().cpu(), getattr(want, n).double().cpu())
            for n in ("dq", "dk", "dv", "dg", "db_erase", "dw_write", "dh0")}
    report("reference scalar assembly + CUDA k1/k2", errs)
    assert max(errs.values()) <= TOL, errs


def test_reference_channelwise_assembly_driven_by_the_cuda_plugins():
    reference()
    from lethe.kernels.cute.gdn2_assemble import assemble_gdn2_backward_channelwise

    q, k, v, g, beta, do = _inputs(1, 256, 2, 128, 64, seed=6, channelwise=True)
    gen = torch.Generator().manual_seed(61)
    b = torch.randn(1, 256, 2, 128, generator=gen).sigmoid()                  # independent per-channel gates
    w = torch.randn(1, 256, 2, 64, generator=gen).sigmoid()
    want = assemble_gdn2_backward_channelwise(q, k, v, g, b, w, do)
    got = assemble_gdn2_backward_channelwise(*cu((q, k, v, g, b, w, do)), k1_fn=plugins.k1_fn,
                                             k2_fn=plugins.k2_fn_cw)
    errs = {n: scale_rel(getattr(got, n).double().cpu(), getattr(want, n).double().cpu())
            for n in ("dq", "dk", "dv", "dg", "db", "dw", "dh0")}
    report("reference channel-wise assembly + CUDA k1/k2cw", errs)
    assert max(errs.values()) <= TOL, errs


@pytest.mark.parametrize("regime", ["scalar", "channelwise", "full"])
def test_reference_autograd_function_with_this_backward(regime, monkeypatch):
    """``gdn2_op`` of the reference, forward untouched (its token loop), backward swapped."""
    reference()
    import lethe.kernels.ops.gdn_layer as ref_layer

    B, L, H, K, V = 1, 128, 2, 128, 64
    q, k, v, g, beta, do = _inputs(B, L, H, K, V, seed=7, channelwise=regime != "scalar")
    if regime == "scalar":
        g = g[..., None].expand(B, L, H, K).contiguous()
    if regime == "full":
        gen = torch.Generator().manual_seed(71)
        b = torch.randn(B, L, H, K, generator=gen).sigmoid()
        w = torch.randn(B, L, H, V, generator=gen).sigmoid()
    else:
        b, w = beta[..., None].expand(B, L, H, K).contiguous(), beta[..., None].expand(B, L, H, V).contiguous()

    def run(dev):
        leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v, g, b, w)]
        o = ref_layer.gdn2_op(*leaves)
        return o.detach(), torch.autograd.grad(o, leaves, do.to(dev))

    o_ref, want = run("cpu")                       # the reference alone: eager forward and backward
    calls = []

    def swapped(*a, **kw):
        calls.append(1)
        return ops.gdn2_backward(*a, **kw)

    monkeypatch.setattr(ref_layer, "gdn2_backward", swapped)
    o_got, got = run("cuda")                       # its forward (token loop in torch), this library's backward
    assert calls, "the reference's autograd function did not reach the swapped backward"
    assert scale_rel(o_got.double().cpu(), o_ref.double()) <= 1e-5
    # A gate that was given as one value broadcast over the channels gets its gradient spread evenly over
    # them here (as in the reference's own scalar assembly, gdn2_assemble.py:343-345), while the reference's
    # eager path differentiates every channel: the two agree in the sum over the channels, which is the
    # gradient of the underlying scalar.
    bcast = {"dg": regime == "scalar", "db": regime != "full", "dw": regime != "full"}
    errs = {}
    for n, a, r in zip(("dq", "dk", "dv", "dg", "db", "dw"), got, want):
        a, r = a.double().cpu(), r.double().cpu()
        errs[n] = scale_rel(a.sum(-1), r.sum(-1)) if bcast.get(n) else scale_rel(a, r)
    report(f"reference _GDN2Function + this backward ({regime})", errs)
    assert max(errs.values()) <= TOL, errs
    assert all(a.dtype == r.dtype and a.shape == r.shape for a, r in zip(got, want))


def test_family_wrappers_against_the_reference_wrappers():
    reference()
    import lethe.kernels.cute.gdn2_family as ref_family

    B, L, H, K, V = 1, 256, 2, 128, 64
    q, k, v, g, beta, do = _inputs(B, L, H, K, V, seed=8, channelwise=True)
    gs = g[..., 0].contiguous()
    Q, Kk, Vv, G, Bt, DO, GS = cu((q, k, v, g, beta, do, gs))
    pairs = {
        "kda": (family.kda_backward(Q, Kk, Vv, G, Bt, DO), ref_family.kda_backward(q, k, v, g, beta, do)),
        "gla": (family.gla_backward(Q, Kk, Vv, G, DO), ref_family.gla_backward(q, k, v, g, do)),
        "ssd": (family.ssd_backward(Q, Kk, Vv, GS, DO), ref_family.ssd_backward(q, k, v, gs, do)),
        "la": (family.la_backward(Q, Kk, Vv, DO), ref_family.la_backward(q, k, v, do)),
    }
    for name, (got, want) in pairs.items():
        assert got._fields == want._fields, name
        errs = {f: scale_rel(getattr(got, f).double().cpu(), getattr(want, f).double().cpu()) for f in want._fields}
        report(f"family {name} vs reference wrapper (L2-normalised q, k)", errs)
        assert max(errs.values()) <= TOL, (name, errs)
