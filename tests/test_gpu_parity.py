"""GPU parity of the public op ``gdn_chunk`` (through the C ABI) with the reference's results:
golden vectors produced by the reference itself, and the fp64 oracle on the benchmark
configurations.  Bar: worst max|got - ref| / max|ref| <= 5e-3 per tensor (bf16 inputs, fp32
accumulation), and two runs bitwise equal."""

import os

import numpy as np
import pytest
import torch

from lethe_b200.ops import gdn_chunk
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import chunk_fwd_bwd, scale_rel

from .wsview import report

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 5e-3


def run_op(inp, scale, dhT=None):
    """inp: dict of CPU tensors.  Returns dict of CPU results from the CUDA op."""
    leaves = {}
    for n in ("q", "k", "v", "g", "beta", "h0"):
        t = inp.get(n)
        leaves[n] = None if t is None else t.cuda().requires_grad_(True)
    o, hT = gdn_chunk(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], leaves["h0"],
                      scale=scale)
    outs, gos = [o], [inp["do"].cuda().to(o.dtype)]
    if dhT is not None:
        outs.append(hT)
        gos.append(dhT.cuda())
    names = [n for n in leaves if leaves[n] is not None]
    grads = torch.autograd.grad(outs, [leaves[n] for n in names], gos)
    torch.cuda.synchronize()
    res = {"o": o.detach().cpu(), "hT": hT.detach().cpu()}
    for n, gval in zip(names, grads):
        res["d" + n] = gval.cpu()
    return res


def compare(label, res, ref):
    errs = {}
    for n, r in ref.items():
        if r is not None and n in res:
            errs[n] = scale_rel(res[n].double(), r)
            assert torch.isfinite(res[n].float()).all(), n
    report(label, errs)
    for n, e in errs.items():
        assert e <= TOL, (label, n, e, errs)
    return errs


@pytest.mark.parametrize("name", ["gdn_scalar_k128", "kda_k128"])
def test_golden(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim}
    inp = dict(q=d["q"].bfloat16(), k=d["k"].bfloat16(), v=d["v"].bfloat16(), do=d["do"].bfloat16(),
               g=d.get("g"), beta=d.get("beta"), h0=d.get("h0"))
    res = run_op(inp, float(z["scale"]))
    ref = {n: d[n].double() for n in ("o", "dq", "dk", "dv", "dg", "dbeta", "dh0") if n in d}
    compare(f"golden {name}", res, ref)


def oracle_case(B, L, H, K, V, gate, delta, mild, seed, with_dhT=False):
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=seed, mild=mild)
    dhT = None
    if with_dhT:
        dhT = 0.1 * torch.randn(B, H, K, V, generator=torch.Generator().manual_seed(seed + 100))
    scale = K ** -0.5
    res = run_op(inp, scale, dhT)
    f64 = {k: (None if t is None else t.double()) for k, t in inp.items()}
    o, hT, gr = chunk_fwd_bwd(f64["q"], f64["k"], f64["v"], f64["g"], f64["beta"], f64["h0"], f64["do"],
                              None if dhT is None else dhT.double(), scale=scale)
    ref = dict(o=o, hT=hT, dq=gr.dq, dk=gr.dk, dv=gr.dv, dg=gr.dg, dbeta=gr.dbeta, dh0=gr.dh0)
    return inp, res, ref


@pytest.mark.parametrize("mild", [False, True])
def test_config1_scalar_gdn(mild):
    """B=2, H=8, L=2048, d_k=128, d_v=64, scalar gate, initial state (the headline configuration)."""
    _, res, ref = oracle_case(2, 2048, 8, 128, 64, "scalar", True, mild, seed=1)
    compare(f"config1 mild={mild}", res, ref)


@pytest.mark.parametrize("mild", [False, True])
def test_config2_channelwise_kda(mild):
    """B=2, H=8, L=2048, d_k=128, d_v=128, channel-wise gate + beta (KDA)."""
    _, res, ref = oracle_case(2, 2048, 8, 128, 128, "channel", True, mild, seed=2)
    compare(f"config2 KDA mild={mild}", res, ref)


@pytest.mark.parametrize("V", [64, 128])
def test_gla(V):
    """Channel-wise gate without the delta term (GLA), with initial state and final-state adjoint."""
    _, res, ref = oracle_case(2, 512, 4, 128, V, "channel", False, True, seed=7, with_dhT=True)
    compare(f"gla V={V}", res, ref)
    _, res, ref = oracle_case(1, 256, 2, 128, V, "channel", False, False, seed=8)
    compare(f"gla strong V={V}", res, ref)


def test_config0_shape_d64():
    """B=1, H=2, L=256, d_k=d_v=64 (the reference's CPU-sized case; key channels zero-padded)."""
    inp = make_inputs(1, 256, 2, 64, 64, gate="scalar", delta=True, seed=0, with_h0=False)
    res = run_op(inp, 64 ** -0.5)
    f64 = {k: (None if t is None else t.double()) for k, t in inp.items()}
    o, hT, gr = chunk_fwd_bwd(f64["q"], f64["k"], f64["v"], f64["g"], f64["beta"], None, f64["do"],
                              scale=64 ** -0.5)
    compare("config0", res, dict(o=o, hT=hT, dq=gr.dq, dk=gr.dk, dv=gr.dv, dg=gr.dg, dbeta=gr.dbeta))


@pytest.mark.parametrize("V", [64, 128])
def test_ssd_and_la(V):
    """No-delta variants through the same kernels: SSD (scalar gate) and plain linear attention."""
    _, res, ref = oracle_case(2, 512, 4, 128, V, "scalar", False, True, seed=3, with_dhT=True)
    compare(f"ssd V={V}", res, ref)
    _, res, ref = oracle_case(2, 512, 4, 128, V, "none", False, True, seed=4)
    compare(f"la V={V}", res, ref)


def test_final_state_adjoint_and_v128():
    _, res, ref = oracle_case(1, 512, 4, 128, 128, "scalar", True, True, seed=6, with_dhT=True)
    compare("gdn V=128 dhT", res, ref)


def test_bitwise_deterministic():
    inp = make_inputs(2, 1024, 4, 128, 64, gate="scalar", delta=True, seed=8)
    a = run_op(inp, 128 ** -0.5)
    b = run_op(inp, 128 ** -0.5)
    for n in a:
        assert torch.equal(a[n], b[n]), n


def test_single_chunk_and_ragged_rejection():
    _, res, ref = oracle_case(1, 64, 1, 128, 64, "scalar", True, False, seed=11)
    compare("single chunk", res, ref)
    # the library itself only takes whole chunks (the Python op pads; see test_gpu_decode_ragged.py)
    from lethe_b200 import ops
    with pytest.raises(ops.GdnError):
        ops.GdnBuffers(1, 96, 1, 128, 64, ops.GATE_SCALAR, True, torch.device("cuda"))


def test_repeated_no_delta_forward_keeps_status_clean():
    """The no-delta output kernel commits two product groups back to back; every thread has to be past
    its wait on the first before the second is committed (else a bounded wait runs out).  Many
    launches, status word checked, results bitwise stable."""
    from lethe_b200 import ops

    B, L, H, K, V = 2, 1024, 8, 128, 128
    inp = make_inputs(B, L, H, K, V, gate="scalar", delta=False, seed=13)
    d = {k: t.cuda() for k, t in inp.items() if t is not None}
    buf = ops.GdnBuffers(B, L, H, K, V, ops.GATE_SCALAR, False, torch.device("cuda"), backward=False)
    ops.forward_into(buf, d["q"], d["k"], d["v"], d["g"], None, d["h0"], K ** -0.5)
    ref = buf.o.clone()
    for _ in range(300):
        ops.forward_into(buf, d["q"], d["k"], d["v"], d["g"], None, d["h0"], K ** -0.5, kernel_mask=4)
    torch.cuda.synchronize()
    ops.check_status(buf.status)
    assert torch.equal(buf.o, ref)
