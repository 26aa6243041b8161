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


def test_pipeline_rejects_wrong_inputs():
    from lethe_b200.host import HostPipeline

    pipe = HostPipeline(1, 64, 1, 128, 64, gate=ops.GATE_SCALAR, delta=True)
    with pytest.raises(ops.GdnError):
        pipe.submit({"q": torch.empty(1)}, {})
