"""CUDA-graph replay of the forward + backward step must give exactly what plain launches give."""
import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gate,delta,V", [("scalar", True, 64), ("channel", True, 128), ("none", False, 64)])
def test_graph_replay_matches_plain_launches(gate, delta, V):
    B, L, H, K = 1, 256, 2, 128
    dev = torch.device("cuda")
    code = {"none": ops.GATE_NONE, "scalar": ops.GATE_SCALAR, "channel": ops.GATE_CHANNEL}[gate]
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=3)
    d = {n: (None if t is None else t.to(dev)) for n, t in inp.items()}
    ref = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
    ops.forward_into(ref, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], K ** -0.5)
    ops.backward_into(ref, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], d["do"], None, K ** -0.5)
    buf = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
    graph = ops.GdnStepGraph(buf, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], d["do"], None, K ** -0.5)
    for t in (buf.o, buf.dq, buf.dk, buf.dv):
        t.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    ops.check_status(buf.status)
    names = ["o", "hT", "dq", "dk", "dv", "dh0"] + (["dg"] if gate != "none" else []) + (["dbeta"] if delta else [])
    for n in names:
        assert torch.equal(getattr(buf, n), getattr(ref, n)), n
    # new data in the captured tensors: the replay follows it
    d["v"].mul_(0.5)
    ops.forward_into(ref, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], K ** -0.5)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(buf.o, ref.o)


def test_head_ranges_and_groups_give_the_same_bits():
    """Calls restricted to (batch, head) ranges, and the graph that runs the ranges as concurrent chains,
    must reproduce the full call bit for bit (the pairs are independent recurrences)."""
    B, L, H, K, V = 2, 256, 3, 128, 64
    dev = torch.device("cuda")
    inp = make_inputs(B, L, H, K, V, gate="scalar", delta=True, seed=8)
    d = {n: (None if t is None else t.to(dev)) for n, t in inp.items()}
    args = (d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"])
    ref = ops.GdnBuffers(B, L, H, K, V, ops.GATE_SCALAR, True, dev)
    ops.forward_into(ref, *args, K ** -0.5)
    ops.backward_into(ref, *args, d["do"], None, K ** -0.5)
    part = ops.GdnBuffers(B, L, H, K, V, ops.GATE_SCALAR, True, dev)
    for rng in ((4, 2), (0, 1), (1, 3)):                     # out of order, uneven
        ops.forward_into(part, *args, K ** -0.5, bh_range=rng)
        ops.backward_into(part, *args, d["do"], None, K ** -0.5, bh_range=rng)
    grp = ops.GdnBuffers(B, L, H, K, V, ops.GATE_SCALAR, True, dev)
    graph = ops.GdnStepGraph(grp, *args, d["do"], None, K ** -0.5, groups=4)
    graph.replay()
    torch.cuda.synchronize()
    for b in (part, grp):
        ops.check_status(b.status)
        for n in ("o", "hT", "dq", "dk", "dv", "dg", "dbeta", "dh0"):
            assert torch.equal(getattr(b, n), getattr(ref, n)), n
    with pytest.raises(ops.GdnError):
        ops.forward_into(part, *args, K ** -0.5, bh_range=(5, 2))     # beyond B * H = 6

