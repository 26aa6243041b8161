"""GPU self-test of the tcgen05 / TMA toolkit: D = A @ B on one CTA for every operand orientation
and tile-fill method the GDN kernels use, against a plain fp32 product."""

import ctypes

import pytest
import torch

from lethe_b200 import _build

pytestmark = pytest.mark.gpu
_PROBE = None


def probe_lib():
    """The test-only library built from tests/native/probe.cu (declared in tests/native/lethe_probe.h)."""
    global _PROBE
    if _PROBE is None:
        _PROBE = ctypes.CDLL(_build.build_probe())
        vp, ci = ctypes.c_void_p, ctypes.c_int
        _PROBE.lethe_probe_umma.restype = ci
        _PROBE.lethe_probe_umma.argtypes = [vp] * 4 + [ci] * 7 + [vp]
        _PROBE.lethe_probe_starved_wait.restype = ci
        _PROBE.lethe_probe_starved_wait.argtypes = [vp, ctypes.c_longlong, vp, vp]
    return _PROBE


def sw128_image(x: torch.Tensor) -> torch.Tensor:
    """Host-side construction of the swizzled tile image of a [rows, cols] 16-bit matrix
    (cols a multiple of 64): atoms of 64 columns, row r at r*128 B, 16-byte chunk c at c ^ (r & 7)."""
    rows, cols = x.shape
    out = torch.empty(cols // 64, rows, 8, 8, dtype=x.dtype)
    xa = x.reshape(rows, cols // 64, 8, 8).permute(1, 0, 2, 3)        # [atom, row, chunk, 8]
    r = torch.arange(rows) & 7
    for c in range(8):
        dst = (c ^ r)                                                  # [rows]
        out[:, torch.arange(rows), dst] = xa[:, :, c]
    return out.reshape(-1)


def run_probe(a_mn, b_mn, N, kc, fill, a_neg=0, twice=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    Am = torch.randn(128, kc, generator=g).half()           # logical A [M=128, kc]
    Bm = torch.randn(N, kc, generator=g).half()             # logical B [N, kc]
    ref = Am.float() @ Bm.float().t()
    if a_neg:
        ref = -ref
    if twice:
        ref = 2 * ref
    A_store = Am.t().contiguous() if a_mn else Am           # tile as stored: [rows, cols]
    B_store = Bm.t().contiguous() if b_mn else Bm
    if fill == 2:
        A_dev = sw128_image(A_store).cuda()
        B_dev = sw128_image(B_store).cuda()
    else:
        A_dev, B_dev = A_store.cuda(), B_store.cuda()
    D = torch.full((128, N), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = probe_lib().lethe_probe_umma(A_dev.data_ptr(), B_dev.data_ptr(), D.data_ptr(),
                                       status.data_ptr(), a_mn, b_mn, N, kc, fill, a_neg, twice,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device wait timed out, code {int(status.item())}"
    err = (D.cpu() - ref).abs().max().item()
    return err, ref.abs().max().item()


CASES = [
    # (a_mn, b_mn, N, kc, fill, a_neg, twice)
    (0, 0, 64, 64, 0, 0, 0),     # both contract along columns, thread-written tiles
    (0, 0, 64, 128, 0, 0, 0),    # two atoms along the contraction
    (0, 0, 16, 128, 0, 0, 0),    # narrow N (the scan kernel's shape)
    (0, 0, 128, 64, 1, 0, 0),    # tensor-map fill
    (0, 0, 64, 128, 2, 0, 0),    # bulk copy of a pre-swizzled image
    (1, 0, 64, 64, 0, 0, 0),     # A contracted along its rows
    (0, 1, 64, 64, 0, 0, 0),     # B contracted along its rows
    (1, 1, 128, 64, 0, 0, 0),    # both
    (1, 1, 192, 64, 1, 0, 0),    # three atoms of N, tensor-map fill
    (1, 1, 256, 64, 2, 0, 0),
    (1, 0, 128, 128, 0, 0, 0),   # A row-contracted over 128 rows (transposed 128x128 operand)
    (0, 0, 64, 64, 0, 1, 0),     # negated A
    (0, 1, 64, 64, 0, 0, 1),     # accumulate
    (0, 0, 256, 128, 1, 0, 0),   # widest tile
]


@pytest.mark.parametrize("case", CASES)
def test_probe(case):
    err, scale = run_probe(*case)
    assert err < 2e-3 * max(scale, 1.0), (case, err, scale)


def test_bounded_wait_runs_out_and_the_gpu_stays_usable():
    """Failure detection without a fault: a CTA waits, with a limit of 1e5 cycles, on a barrier that
    nothing completes.  The wait must give up and leave its site code (101) in the status word, the
    CTA's next wait must fall through at once, the kernel must return by itself with its tensor memory
    freed - and an ordinary probe launched right after on the same stream must still pass."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    trace = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    limit = 100_000
    rc = probe_lib().lethe_probe_starved_wait(status.data_ptr(), limit, trace.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 101
    abort_flag, kcyc_first, kcyc_second = trace[:3].tolist()
    assert abort_flag == 1
    assert limit // 1024 <= kcyc_first <= 50 * limit // 1024          # gave up after about the limit
    assert kcyc_second <= 8                                            # the later wait did not spin
    from lethe_b200 import ops
    with pytest.raises(ops.GdnError, match="101"):
        ops.check_status(status)
    # the context is intact and the tensor memory was given back: a 256-column product still runs
    for _ in range(3):
        err, scale = run_probe(0, 0, 256, 128, 1)
        assert err < 2e-3 * max(scale, 1.0)
