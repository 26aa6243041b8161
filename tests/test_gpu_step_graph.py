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
