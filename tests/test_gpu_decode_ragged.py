"""The two extensions around the chunked path: a single-token decode step that continues from a
prompt's final state, and sequence lengths that are not a multiple of the chunk length.  Both are
checked against the token-serial fp64 oracle (reference ``gdn_backward.py:45-53``)."""
import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import scale_rel, serial_backward, serial_forward

from .wsview import report

pytestmark = pytest.mark.gpu
TOL = 5e-3


@pytest.mark.parametrize("gate,delta,V", [("scalar", True, 64), ("channel", True, 128), ("scalar", False, 128),
                                          ("none", False, 64), ("channel", False, 64)])
def test_decode_continues_a_prompt(gate, delta, V):
    B, Lp, T, H, K = 2, 128, 6, 3, 128
    dev = torch.device("cuda")
    inp = make_inputs(B, Lp + T, H, K, V, gate=gate, delta=delta, seed=11)
    f64 = {n: (None if t is None else t.double()) for n, t in inp.items()}
    o_ref, hT_ref = serial_forward(f64["q"], f64["k"], f64["v"], f64["g"], f64["beta"], f64["h0"])

    d = {n: (None if t is None else t.to(dev)) for n, t in inp.items()}
    cut = lambda t, a, b: None if t is None else t[:, a:b].contiguous()   # noqa: E731
    _, state = ops.gdn_chunk(cut(d["q"], 0, Lp), cut(d["k"], 0, Lp), cut(d["v"], 0, Lp), cut(d["g"], 0, Lp),
                             cut(d["beta"], 0, Lp), d["h0"])
    state = state.contiguous()
    outs = []
    for t in range(Lp, Lp + T):
        tok = lambda x: None if x is None else x[:, t].contiguous()       # noqa: E731
        outs.append(ops.gdn_decode_step(tok(d["q"]), tok(d["k"]), tok(d["v"]), tok(d["g"]), tok(d["beta"]), state))
    o = torch.stack(outs, dim=1).double().cpu()
    errs = {"o": scale_rel(o, o_ref[:, Lp:]), "state": scale_rel(state.double().cpu(), hT_ref)}
    report(f"decode gate={gate} delta={delta} V={V}", errs)
    assert max(errs.values()) <= TOL, errs


def test_decode_rejects_bad_arguments():
    dev = torch.device("cuda")
    st = torch.zeros(1, 1, 128, 64, device=dev)
    q = torch.zeros(1, 1, 128, device=dev, dtype=torch.bfloat16)
    v = torch.zeros(1, 1, 64, device=dev, dtype=torch.bfloat16)
    with pytest.raises(ops.GdnError):
        ops.gdn_decode_step(q, q, v, None, None, st.half())
    with pytest.raises(ops.GdnError):
        ops.gdn_decode_step(q, q, v[..., :32], None, None, st)
    with pytest.raises(ops.GdnError):
        ops.gdn_decode_step(q[..., :64], q[..., :64], v, None, None, torch.zeros(1, 1, 64, 64, device=dev))


@pytest.mark.parametrize("gate,delta,L", [("scalar", True, 200), ("channel", True, 70), ("scalar", False, 33)])
def test_lengths_off_the_chunk_grid(gate, delta, L):
    B, H, K, V = 2, 2, 128, 64
    dev = torch.device("cuda")
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=5)
    f64 = {n: (None if t is None else t.double()) for n, t in inp.items()}
    dhT = 0.1 * torch.randn(B, H, K, V, generator=torch.Generator().manual_seed(3))
    o_ref, hT_ref, gr = serial_backward(f64["q"], f64["k"], f64["v"], f64["g"], f64["beta"], f64["h0"], f64["do"],
                                        dhT.double())
    leaves = {n: (None if inp[n] is None else inp[n].to(dev).requires_grad_(True)) for n in ("q", "k", "v", "g", "beta", "h0")}
    o, hT = ops.gdn_chunk(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], leaves["h0"])
    assert o.shape == (B, L, H, V)
    names = [n for n in leaves if leaves[n] is not None]
    grads = torch.autograd.grad([o, hT], [leaves[n] for n in names], [inp["do"].to(dev), dhT.to(dev)])
    got = dict(zip(names, grads))
    ref = {"q": gr.dq, "k": gr.dk, "v": gr.dv, "g": gr.dg, "beta": gr.dbeta, "h0": gr.dh0}
    errs = {"o": scale_rel(o.detach().double().cpu(), o_ref), "hT": scale_rel(hT.detach().double().cpu(), hT_ref)}
    for n in names:
        assert got[n].shape == leaves[n].shape
        errs["d" + n] = scale_rel(got[n].double().cpu(), ref[n])
    report(f"ragged gate={gate} delta={delta} L={L}", errs)
    assert max(errs.values()) <= TOL, errs
