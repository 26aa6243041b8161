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



@pytest.mark.parametrize("gate,delta,V", [("scalar", True, 64), ("channel", True, 128), ("scalar", False, 128),
                                          ("channel", False, 64)])
def test_chunk_ranges_and_the_pipelined_graph_give_the_same_bits(gate, delta, V):
    """Calls restricted to chunk ranges (forward ranges ascending, backward ranges descending: the scans hand
    their fp32 state on through the workspace) and the graph that overlaps the two halves of every sequence
    on two streams must reproduce the one-call result bit for bit, final state and initial-state gradient
    included."""
    B, L, H, K = 2, 1024, 3, 128
    NT = L // 64
    dev = torch.device("cuda")
    code = {"scalar": ops.GATE_SCALAR, "channel": ops.GATE_CHANNEL}[gate]
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=9)
    d = {n: (None if t is None else t.to(dev)) for n, t in inp.items()}
    dhT = 0.1 * torch.randn(B, H, K, V, generator=torch.Generator().manual_seed(10)).to(dev)
    args = (d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"])
    sc = K ** -0.5
    ref = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
    ops.forward_into(ref, *args, sc)
    ops.backward_into(ref, *args, d["do"], dhT, sc)
    names = ["o", "hT", "dq", "dk", "dv", "dg", "dh0"] + (["dbeta"] if delta else [])
    # three uneven ranges, kernel by kernel
    part = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
    for t in (part.o, part.dq, part.dk, part.dv, part.hT, part.dh0):
        t.fill_(float("nan"))
    ranges = [(0, 5), (5, 1), (6, NT - 6)]
    for m in (1, 2, 4):
        for cr in ranges:
            ops.forward_into(part, *args, sc, m, c_range=cr)
    for m in (1, 2, 4, 8) if delta else (1, 2, 4):
        for cr in reversed(ranges):
            ops.backward_into(part, *args, d["do"], dhT, sc, m, c_range=cr)
    pipes = []
    for cut, bcuts in ((0, None), (NT // 2, None), (1, None), (NT - 1, None), (NT // 2, (3, 9)), (5, (2, 7, 11, 14)),
                       (0, (4,))):
        pipe = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
        graph = ops.GdnStepGraph(pipe, *args, d["do"], dhT, sc, pipeline=True, cut=cut, bwd_cuts=bcuts)
        assert graph.pipeline and graph.cut == cut and graph.segments == (2 if cut else 1)
        assert graph.bwd_cuts == (tuple(bcuts) if bcuts else ((cut,) if cut else ()))
        for t in (pipe.o, pipe.dq, pipe.dk, pipe.dv, pipe.hT, pipe.dh0):
            t.fill_(float("nan"))
        graph.replay()
        graph.replay()
        pipes.append(pipe)
    torch.cuda.synchronize()
    for b in [part] + pipes:
        ops.check_status(b.status)
        for n in names:
            assert torch.equal(getattr(b, n), getattr(ref, n)), n
    with pytest.raises(ops.GdnError):
        ops.forward_into(part, *args, sc, c_range=(NT - 1, 2))          # beyond the last chunk


@pytest.mark.parametrize("gate,V,B,L,H", [("scalar", 64, 2, 2048, 8), ("channel", 128, 2, 2048, 8), ("scalar", 128, 4, 4096, 16)])
def test_step_graph_at_benchmark_shapes_equals_the_plain_chain_on_every_replay(gate, V, B, L, H):
    """The overlapped schedule at the shapes the benchmark times (the default cut, full grids, every stream of
    the graph busy): twelve replays, each compared bit for bit with the plain chain - an ordering hole between
    the graph's streams would show as a difference that comes and goes."""
    K = 128
    dev = torch.device("cuda")
    delta = gate != "scalar" or V != 128           # the third case is SSD: scalar gate, no delta term
    code = {"scalar": ops.GATE_SCALAR, "channel": ops.GATE_CHANNEL}[gate]
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=5)
    d = {n: (None if t is None else t.to(dev)) for n, t in inp.items()}
    sc = K ** -0.5
    ref = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
    ops.forward_into(ref, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], sc)
    ops.backward_into(ref, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], d["do"], None, sc)
    buf = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
    graph = ops.GdnStepGraph(buf, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], d["do"], None, sc)
    assert graph.pipeline and graph.cut > 0
    names = ["o", "hT", "dq", "dk", "dv", "dh0", "dg"] + (["dbeta"] if delta else [])
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    for rep in range(12):
        for n in names:
            getattr(buf, n).fill_(float("nan"))
        if rep % 2:
            flush.zero_()                          # cold and warm L2: different relative timing of the streams
        graph.replay()
        torch.cuda.synchronize()
        ops.check_status(buf.status)
        for n in names:
            assert torch.equal(getattr(buf, n), getattr(ref, n)), (rep, n)
