"""CPU: where the step graph cuts the sequences (pure host logic of ``lethe_b200.ops``).

The cut points only move kernels between streams of the captured step - results are bit-identical for any
cut (``tests/test_gpu_step_graph.py``) - so what is pinned here is the rule, on the shapes it was measured on."""
import pytest

from lethe_b200 import ops

B200_SMS = 148


@pytest.mark.parametrize("gate,V,delta,NT,BH,cut,bwd", [
    (ops.GATE_SCALAR, 64, True, 32, 16, 18, (9, 18)),       # configuration 1: two CTAs per SM, 18 chunks per wave
    (ops.GATE_CHANNEL, 128, True, 32, 16, 18, (18,)),       # configuration 2: one CTA per SM, 9 chunks per wave
    (ops.GATE_SCALAR, 64, True, 64, 32, 36, (36,)),         # 2048 chunks: four waves, no second backward cut
    (ops.GATE_SCALAR, 128, True, 32, 16, 18, (18,)),        # d_v = 128: Stage B holds an SM alone
    (ops.GATE_CHANNEL, 128, True, 128, 64, 64, (64,)),      # configuration 4a share: two pairs per wave
    (ops.GATE_SCALAR, 128, False, 64, 64, 32, (32,)),       # SSD of configuration 3
    (ops.GATE_SCALAR, 64, True, 4, 2, 0, ()),               # short sequences are not cut
    (ops.GATE_SCALAR, 64, True, 16, 2, 8, (8,)),            # everything fits one wave: halves
    (ops.GATE_SCALAR, 64, True, 16, 400, 8, (8,)),          # more pairs than CTA slots: halves
])
def test_default_cuts(gate, V, delta, NT, BH, cut, bwd):
    assert ops.default_cut(gate, V, NT, BH, B200_SMS) == cut
    assert ops.default_bwd_cuts(gate, V, delta, NT, BH, B200_SMS, cut) == bwd


def test_cuts_stay_inside_the_sequence():
    for gate in (ops.GATE_NONE, ops.GATE_SCALAR, ops.GATE_CHANNEL):
        for V in (64, 128):
            for NT in (1, 2, 7, 8, 9, 31, 32, 33, 100, 1024):
                for BH in (1, 3, 16, 37, 64, 148, 149, 296, 297, 1000):
                    for sms in (1, 20, 132, 148):
                        cut = ops.default_cut(gate, V, NT, BH, sms)
                        assert cut == 0 or 0 < cut < NT, (gate, V, NT, BH, sms, cut)
                        for delta in (False, True):
                            b = ops.default_bwd_cuts(gate, V, delta, NT, BH, sms, cut)
                            assert all(0 < c < NT for c in b) and list(b) == sorted(set(b)), (gate, V, NT, BH, sms, b)
                            assert (cut in b) if cut else b == ()
