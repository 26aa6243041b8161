"""GPU: the records the backward kernels pass to one another, and all gradients, against the fp64
chunkwise oracle (closed-form backward) on the same bf16-rounded inputs."""

import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import chunk_backward, chunk_forward, scale_rel

from .wsview import layout, records, report, rrecords, unswizzle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gate", ["scalar", "channel"])
@pytest.mark.parametrize("V", [64, 128])
@pytest.mark.parametrize("delta", [True, False])
@pytest.mark.parametrize("mild", [False, True])
def test_backward_records(V, delta, mild, gate):
    B, L, H = 2, 256, 2
    inp = make_inputs(B, L, H, 128, V, gate=gate, delta=delta, seed=5, mild=mild)
    dev = {k: (None if t is None else t.cuda()) for k, t in inp.items()}
    scale = 128 ** -0.5
    gen = torch.Generator().manual_seed(9)
    dhT = 0.1 * torch.randn(B, H, 128, V, generator=gen)
    o, hT, saved, status = ops.gdn_forward_raw(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"],
                                               dev["h0"], scale)
    dq, dk, dv, dg, dbeta, dh0, scratch = ops.gdn_backward_raw(
        dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], dev["h0"], dev["do"], dhT.cuda(),
        saved, status, scale)
    torch.cuda.synchronize()
    ops.check_status(status)
    f64 = {k: (None if t is None else t.double()) for k, t in inp.items()}
    st = chunk_forward(f64["q"], f64["k"], f64["v"], f64["g"], f64["beta"], f64["h0"], scale=scale)
    gr, it = chunk_backward(st, f64["do"], dhT.double())
    Z, _, _, sz2, off2 = layout(B, H, L, V, gate=2 if gate == "channel" else 1)
    NT = L // 64
    shp = (B, H, NT)
    errs = {}
    # with the delta term Rb is stored in per-scan-CTA column blocks, without it as a plain tile image
    rb_rec = (rrecords(scratch, off2["rb"], sz2["rb"], Z, V) if delta
              else unswizzle(records(scratch, off2["rb"], sz2["rb"], Z), 128, V))
    errs["Rb"] = scale_rel(rb_rec.reshape(*shp, 128, V).double(), it["Rb"])
    errs["dh"] = scale_rel(unswizzle(records(scratch, off2["dh"], sz2["dh"], Z), 128, V).reshape(*shp, 128, V).double(),
                           it["dh"])
    if delta:
        errs["dv2"] = scale_rel(unswizzle(records(scratch, off2["dv2"], sz2["dv2"], Z), 64, V).reshape(*shp, 64, V).double(),
                                it["dv2"])
        errs["dw"] = scale_rel(unswizzle(records(scratch, off2["dw"], sz2["dw"], Z), 64, 128).reshape(*shp, 64, 128).double(),
                               it["dw"])
    for n, got in (("dq", dq), ("dk", dk), ("dv", dv), ("dg", dg), ("dbeta", dbeta), ("dh0", dh0)):
        ref = getattr(gr, n)
        if ref is not None and got is not None:
            errs[n] = scale_rel(got.cpu().double(), ref)
    report(f"bwd gate={gate} V={V} delta={delta} mild={mild}", errs)
    for n, e in errs.items():
        assert e < (5e-3 if n in ("dq", "dk", "dv") else 2e-3), (n, e, errs)
