"""GPU parity at the shapes the benchmark configurations name, and bitwise determinism at the headline
shapes.  The CUDA op runs the FULL shape; the fp64 chunkwise oracle then checks a subset of (batch,
head) pairs of it (pairs are independent recurrences, and the oracle's per-chunk ``[C, C, K]`` decay
tensors make the full shape impractical on a CPU).  Bar: worst ``max|got - ref| / max|ref|`` <= 5e-3 per
tensor."""

import pytest
import torch

from lethe_b200.ops import gdn_chunk
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import chunk_fwd_bwd, scale_rel

from .test_gpu_parity import run_op
from .wsview import report

pytestmark = pytest.mark.gpu
TOL = 5e-3


def check_pairs(label, inp, res, pairs, dhT=None):
    """Compare the op's results on the listed (b, h) pairs with the oracle run on exactly those pairs."""
    K = inp["q"].shape[-1]
    worst = {}
    for (b, h) in pairs:
        cut = lambda t: None if t is None else t[b:b + 1, :, h:h + 1].double()        # noqa: E731  [1, L, 1, ...]
        cut_state = lambda t: None if t is None else t[b:b + 1, h:h + 1].double()      # noqa: E731  [1, 1, K, V]
        o, hT, gr = chunk_fwd_bwd(cut(inp["q"]), cut(inp["k"]), cut(inp["v"]), cut(inp["g"]), cut(inp["beta"]),
                                  cut_state(inp["h0"]), cut(inp["do"]), cut_state(dhT), scale=K ** -0.5)
        ref = dict(o=o, hT=hT, dq=gr.dq, dk=gr.dk, dv=gr.dv, dg=gr.dg, dbeta=gr.dbeta, dh0=gr.dh0)
        for n, r in ref.items():
            if r is None or n not in res:
                continue
            got = res[n][b:b + 1, h:h + 1] if n in ("hT", "dh0") else res[n][b:b + 1, :, h:h + 1]
            assert torch.isfinite(got.float()).all(), (label, n)
            worst[n] = max(worst.get(n, 0.0), scale_rel(got.double(), r))
    report(f"{label} pairs={pairs}", worst)
    for n, e in worst.items():
        assert e <= TOL, (label, n, e, worst)


@pytest.mark.parametrize("variant,gate", [("la", "none"), ("ssd", "scalar"), ("gla", "channel")])
def test_config3_family_variants_at_their_own_shape(variant, gate):
    """B=4, H=16, L=4096, d_k=d_v=128 without the delta term: plain linear attention (no decay: the state
    grows over all 64 chunks), SSD (scalar gate) and GLA (channel-wise gate)."""
    B, L, H, K, V = 4, 4096, 16, 128, 128
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=False, seed=3)
    res = run_op(inp, K ** -0.5)
    check_pairs(f"config3 {variant}", inp, res, [(0, 0), (3, 15)] if gate != "channel" else [(0, 0), (3, 9)])


def test_config4a_one_gpu_share_kda():
    """One GPU's share of B=16, H=32, L=8192 (batch x head sharding over 8 GPUs): KDA B=2, H=32, L=8192."""
    B, L, H, K, V = 2, 8192, 32, 128, 128
    inp = make_inputs(B, L, H, K, V, gate="channel", delta=True, seed=4)
    res = run_op(inp, K ** -0.5)
    check_pairs("config4a share", inp, res, [(1, 31)])


def test_config4b_one_rank_slice_kda():
    """One rank's slice of the sequence-parallel configuration (B=1, H=32, L=65536 over 8 ranks): L=8192
    with a state coming in from the previous rank and a state adjoint coming in from the next."""
    B, L, H, K, V = 1, 8192, 32, 128, 128
    inp = make_inputs(B, L, H, K, V, gate="channel", delta=True, seed=5)
    dhT = 0.1 * torch.randn(B, H, K, V, generator=torch.Generator().manual_seed(55))
    res = run_op(inp, K ** -0.5, dhT)
    check_pairs("config4b slice", inp, res, [(0, 17)], dhT=dhT)


@pytest.mark.parametrize("cfg", ["config1", "config2"])
def test_headline_shapes_bitwise_deterministic(cfg):
    """Two complete runs (fresh workspaces each) of the two headline configurations are bit-identical in
    every output and gradient."""
    if cfg == "config1":
        inp = make_inputs(2, 2048, 8, 128, 64, gate="scalar", delta=True, seed=1)
    else:
        inp = make_inputs(2, 2048, 8, 128, 128, gate="channel", delta=True, seed=2)
    a = run_op(inp, 128 ** -0.5)
    b = run_op(inp, 128 ** -0.5)
    assert set(a) == set(b)
    for n in a:
        assert torch.equal(a[n], b[n]), (cfg, n)


@pytest.mark.parametrize("gate,V,B,H", [("scalar", 64, 5, 16), ("channel", 128, 5, 8), ("scalar", 128, 3, 16)])
def test_many_pairs_take_the_wide_scan_and_stay_exact(gate, V, B, H):
    """With more (batch, head) pairs than fit the GPU as 16-column scan CTAs (two per SM), the state scans run
    with 32 columns per CTA (a 64-byte-swizzled state operand).  Parity on the first, a middle and the last
    pair - with an initial state and a final-state gradient, so both ends of both scans are covered - and two
    runs must agree bit for bit."""
    L, K = 256, 128
    assert (V // 16) * B * H > 2 * torch.cuda.get_device_properties(0).multi_processor_count
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=True, seed=21)
    dhT = 0.1 * torch.randn(B, H, K, V, generator=torch.Generator().manual_seed(22))
    res = run_op(inp, K ** -0.5, dhT)
    check_pairs(f"wide scan {gate} V={V}", inp, res, [(0, 0), (B // 2, H // 2), (B - 1, H - 1)], dhT=dhT)
    again = run_op(inp, K ** -0.5, dhT)
    for n in res:
        assert torch.equal(res[n], again[n]), n
