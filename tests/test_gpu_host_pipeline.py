"""Host-buffer pipeline: overlapped copy / compute / copy-back must give exactly what the direct calls give."""
import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gate,delta,V", [("scalar", True, 64), ("channel", True, 128), ("scalar", False, 64)])
def test_pipeline_matches_direct_calls(gate, delta, V):
    from lethe_b200.host import HostPipeline

    B, L, H, K = 1, 256, 2, 128
    dev = torch.device("cuda")
    code = ops.GATE_SCALAR if gate == "scalar" else ops.GATE_CHANNEL
    steps = []
    for seed in range(4):
        inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=seed)
        steps.append({n: t.pin_memory() for n, t in inp.items() if t is not None})
    has_h0 = "h0" in steps[0]
    pipe = HostPipeline(B, L, H, K, V, gate=code, delta=delta, has_h0=has_h0, depth=2)
    names = ["o", "hT", "dq", "dk", "dv", "dg", "dh0"] + (["dbeta"] if delta else [])
    outs = []
    for hin in steps:
        ref = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
        shapes = {n: getattr(ref, n) for n in names}
        hout = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory() for n, t in shapes.items()}
        pipe.submit({n: hin[n] for n in pipe.slots[0].inp}, hout)
        outs.append(hout)
    pipe.drain()
    for hin, hout in zip(steps, outs):
        d = {n: t.to(dev) for n, t in hin.items()}
        ref = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
        ops.forward_into(ref, d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), d.get("h0"), K ** -0.5)
        ops.backward_into(ref, d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), d.get("h0"), d["do"], None,
                          K ** -0.5)
        torch.cuda.synchronize()
        ops.check_status(ref.status)
        for n in names:
            assert torch.equal(hout[n], getattr(ref, n).cpu()), n


@pytest.mark.parametrize("gate,delta,V", [("scalar", True, 64), ("channel", 2, 128)])
def test_packed_host_buffers_move_as_one_copy_and_give_the_same_bits(gate, delta, V):
    """Host buffers made by the pipeline itself are laid out like its device buffers: a step then crosses the
    host link as one copy each way.  Four steps in flight on two pairs of such buffers, mixed with a step on
    ordinary per-tensor buffers, against the direct calls."""
    from lethe_b200 import host as host_mod
    from lethe_b200.host import HostPipeline

    B, L, H, K = 1, 256, 2, 128
    dev = torch.device("cuda")
    code = ops.GATE_SCALAR if gate == "scalar" else ops.GATE_CHANNEL
    pipe = HostPipeline(B, L, H, K, V, gate=code, delta=delta, has_h0=True, depth=2)
    pairs = [pipe.make_host_buffers() for _ in range(2)]
    for hin, hout in pairs:        # recognised as packed: one base each way
        assert host_mod._packed_base(hin, pipe.slots[0].in_spec, pipe.slots[0].in_offs, pipe._host_bases) is not None
        assert host_mod._packed_base(hout, pipe.slots[0].out_spec, pipe.slots[0].out_offs, pipe._host_bases) is not None
    loose = {n: t.clone().pin_memory() for n, t in pairs[0][0].items()}
    assert host_mod._packed_base(loose, pipe.slots[0].in_spec, pipe.slots[0].in_offs, pipe._host_bases) is None

    def fill(hin, seed):
        if delta == 2:
            inp = make_inputs(B, L, H, K, V, gate=gate, delta=True, seed=seed)
            gen = torch.Generator().manual_seed(100 + seed)
            inp["b"] = torch.rand(B, L, H, K, generator=gen)
            inp["w"] = torch.rand(B, L, H, V, generator=gen)
        else:
            inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=seed)
        for n in hin:
            hin[n].copy_(inp[n])
        return {n: hin[n].clone() for n in hin}

    def direct(inp):
        d = {n: t.to(dev) for n, t in inp.items()}
        ref = ops.GdnBuffers(B, L, H, K, V, code, delta, dev)
        gates = dict(b_gate=d.get("b"), w_gate=d.get("w"))
        ops.forward_into(ref, d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), d.get("h0"), K ** -0.5, **gates)
        ops.backward_into(ref, d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), d.get("h0"), d["do"], None,
                          K ** -0.5, **gates)
        torch.cuda.synchronize()
        ops.check_status(ref.status)
        return ref

    done = []
    for rnd in range(2):
        kept = []
        for j, (hin, hout) in enumerate(pairs):
            kept.append(fill(hin, 10 * rnd + j))
            pipe.submit(hin, hout)
        pipe.drain()               # the host buffers are reused by the next round
        for (hin, hout), inp in zip(pairs, kept):
            ref = direct(inp)
            for n in hout:
                assert torch.equal(hout[n], getattr(ref, n).cpu()), (rnd, n)
            done.append(1)
    # a per-tensor step on the same pipeline still works
    inp = fill(loose, 77)
    hout = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory() for n, t in pairs[0][1].items()}
    pipe.submit(loose, hout)
    pipe.drain()
    ref = direct(inp)
    for n in hout:
        assert torch.equal(hout[n], getattr(ref, n).cpu()), n
    assert len(done) == 4


def test_pipeline_rejects_wrong_inputs():
    from lethe_b200.host import HostPipeline

    pipe = HostPipeline(1, 64, 1, 128, 64, gate=ops.GATE_SCALAR, delta=True)
    with pytest.raises(ops.GdnError):
        pipe.submit({"q": torch.empty(1)}, {})
