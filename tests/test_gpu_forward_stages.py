"""GPU: every record the forward kernels leave in the workspace, and o / h_T, against the fp64
chunkwise oracle on the same (bf16-rounded) inputs.  Tolerances are scale-relative: fp16 operand
rounding is 2^-11, the bf16 output rounding 2^-8."""

import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import chunk_forward, scale_rel

from .wsview import layout, records, rrecords, report, unswizzle

pytestmark = pytest.mark.gpu


def run_forward(B, L, H, V, delta=True, gate="scalar", mild=False, seed=0, with_h0=True):
    inp = make_inputs(B, L, H, 128, V, gate=gate, delta=delta, seed=seed, mild=mild, with_h0=with_h0)
    dev = {k: (None if t is None else t.cuda()) for k, t in inp.items()}
    scale = 128 ** -0.5
    o, hT, saved, status = ops.gdn_forward_raw(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"],
                                               dev["h0"], scale)
    torch.cuda.synchronize()
    ops.check_status(status)
    f64 = {k: (None if t is None else t.double()) for k, t in inp.items()}
    st = chunk_forward(f64["q"], f64["k"], f64["v"], f64["g"], f64["beta"], f64["h0"], scale=scale)
    return inp, o.cpu(), hT.cpu(), saved, st


@pytest.mark.parametrize("gate", ["scalar", "channel"])
@pytest.mark.parametrize("V", [64, 128])
@pytest.mark.parametrize("delta", [True, False])
@pytest.mark.parametrize("mild", [False, True])
def test_forward_records(V, delta, mild, gate):
    B, L, H = 2, 256, 2
    inp, o, hT, saved, st = run_forward(B, L, H, V, delta=delta, mild=mild, gate=gate)
    Z, sz, off, _, _ = layout(B, H, L, V)
    NT = L // 64
    shp = (B, H, NT)
    tol = 1.5e-3
    ta = unswizzle(records(saved, off["ta"], sz["ta"], Z), 128, 64).reshape(*shp, 128, 64).double()
    errs = {}
    errs["A"] = scale_rel(ta[..., 64:, :], st.A)
    # the chunk decay exp(G_last) underflows fp32 under the strong gate draw: compare absolutely
    ad = records(saved, off["ad"], sz["ad"], Z, torch.float32).reshape(*shp, 128).double()
    errs["ad"] = float((ad - st.a).abs().max())
    # with the delta term R is stored in per-scan-CTA column blocks, without it as a plain tile image
    r_rec = (rrecords(saved, off["r"], sz["r"], Z, V) if delta
             else unswizzle(records(saved, off["r"], sz["r"], Z), 128, V))
    errs["R"] = scale_rel(r_rec.reshape(*shp, 128, V).double(), st.R)
    errs["h"] = scale_rel(unswizzle(records(saved, off["hc"], sz["hc"], Z + B * H), 128, V)
                          .reshape(B, H, NT + 1, 128, V).double(), st.h)
    errs["vn"] = scale_rel(unswizzle(records(saved, off["vn"], sz["vn"], Z), 64, V).reshape(*shp, 64, V).double(),
                           st.v_new)
    errs["u"] = scale_rel(unswizzle(records(saved, off["u"], sz["u"], Z), 64, V).reshape(*shp, 64, V).double(), st.u)
    if delta:
        errs["T"] = scale_rel(ta[..., :64, :], st.T)
        errs["w"] = scale_rel(unswizzle(records(saved, off["w"], sz["w"], Z), 64, 128).reshape(*shp, 64, 128).double(),
                              st.w)
        # P = kd^T w carries the chunk's whole decay: ~1e-80 under the strong draw, zero in fp16, so
        # it is compared on an absolute floor (entries of h, which P multiplies, are O(1))
        Pg = unswizzle(records(saved, off["p"], sz["p"], Z), 128, 128).reshape(*shp, 128, 128).double()
        errs["P"] = float((Pg - st.P).abs().max()) / max(float(st.P.abs().max()), 1e-3)
    errs["hT"] = scale_rel(hT.double(), st.h[:, :, -1])
    errs["o"] = scale_rel(o.double(), st.o)
    report(f"fwd gate={gate} V={V} delta={delta} mild={mild}", errs)
    for n, e in errs.items():
        assert e < (5e-3 if n == "o" else tol), (n, e, errs)
