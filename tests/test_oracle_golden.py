"""Pin the CPU oracle (both statements) to golden vectors produced by the reference itself."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle.gdn_oracle import chunk_backward, chunk_forward, scale_rel, serial_backward, serial_backward_full

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ALL = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "*.npz")))
FULL_CASES = [n for n in ALL if n.startswith("gdn2_full")]     # independent per-channel gates b, w
CASES = [n for n in ALL if n not in FULL_CASES]


def load(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    d = {k: torch.from_numpy(z[k]).double() if z[k].ndim else z[k].item() for k in z.files}
    return d


def _args(d):
    return d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), d.get("h0")


def test_golden_files_present():
    assert len(CASES) >= 11, CASES
    assert len(FULL_CASES) >= 2, FULL_CASES


@pytest.mark.parametrize("name", FULL_CASES)
def test_full_gate_oracle_matches_reference(name):
    d = load(name)
    tol = 2e-6 if name.endswith("k128") else 1e-9
    o, _hT, gr = serial_backward_full(d["q"], d["k"], d["v"], d["g"], d["b"], d["w"], d["h0"], d["do"],
                                      scale=d["scale"])
    assert scale_rel(o, d["o"]) < tol
    for n in ("q", "k", "v", "g", "b", "w", "h0"):
        assert scale_rel(gr[n], d["d" + n]) < tol, n


@pytest.mark.parametrize("name", CASES)
def test_serial_oracle_matches_reference(name):
    d = load(name)
    tol = 2e-6 if name.endswith("k128") else 1e-9   # kernel-sized cases are stored in fp32
    o, _hT, gr = serial_backward(*_args(d), d["do"], scale=d["scale"])
    assert scale_rel(o, d["o"]) < tol
    for n in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        if n in d:
            assert scale_rel(getattr(gr, n), d[n]) < tol, n


@pytest.mark.parametrize("name", CASES)
def test_chunk_oracle_matches_reference(name):
    d = load(name)
    tol = 2e-6 if name.endswith("k128") else 1e-8
    st = chunk_forward(*_args(d), scale=d["scale"], C=int(d["C"]))
    gr, _ = chunk_backward(st, d["do"])
    assert scale_rel(st.o, d["o"]) < tol
    for n in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        if n in d:
            assert scale_rel(getattr(gr, n), d[n]) < tol, n
    # the reference's own chunkwise intermediates (UT transform, WY factors, chunk states)
    for n, mine in (("cw_T", st.T), ("cw_u", st.u), ("cw_w", st.w), ("cw_h", st.h),
                    ("cw_A", st.A), ("cw_vnew", st.v_new)):
        if n in d:
            assert scale_rel(mine, d[n]) < tol, n


def test_final_state_adjoint_and_small_chunk():
    """Non-zero final-state adjoint and a chunk length other than 64: chunk form == serial form."""
    torch.manual_seed(3)
    B, L, H, K, V = 2, 48, 2, 16, 8
    dt = torch.float64
    q, k = torch.randn(B, L, H, K, dtype=dt), torch.randn(B, L, H, K, dtype=dt)
    v, do = torch.randn(B, L, H, V, dtype=dt), torch.randn(B, L, H, V, dtype=dt)
    beta = torch.rand(B, L, H, dtype=dt)
    g = -torch.rand(B, L, H, K, dtype=dt)
    h0, dhT = torch.randn(B, H, K, V, dtype=dt), torch.randn(B, H, K, V, dtype=dt)
    o, hT, gr = serial_backward(q, k, v, g, beta, h0, do, dhT)
    st = chunk_forward(q, k, v, g, beta, h0, C=16)
    gr2, _ = chunk_backward(st, do, dhT)
    assert scale_rel(st.o, o) < 1e-10 and scale_rel(st.h[:, :, -1], hT) < 1e-10
    for n in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        assert scale_rel(getattr(gr2, n), getattr(gr, n)) < 1e-9, n
