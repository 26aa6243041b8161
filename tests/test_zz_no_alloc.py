"""GPU test of ``lethe_gdn_forward_static``: the forward entry point for hosts that cannot allocate
device memory (a plug-in inside a runtime whose memory pool it may not use, a server whose memory
budget was fixed at start-up).  Its workspace is an array built into the library instead of a
caller buffer, so this test calls it through the C ABI twice in a row -- a larger problem first,
then a smaller one that lands on the leftovers of the first -- and requires the results to equal
those of the ordinary entry point bit for bit.  It also checks that a problem beyond the built-in
capacity is refused.  The file name keeps it last in collection order."""

import ctypes

import pytest
import torch

from lethe_b200 import native, ops
from lethe_b200.synth import make_inputs

pytestmark = pytest.mark.gpu


def _forward_both(B, L, H, V, seed, device="cuda"):
    dev = torch.device(device)
    inp = make_inputs(B, L, H, 128, V, gate="scalar", delta=True, seed=seed)
    d = {k: (None if t is None else t.to(dev)) for k, t in inp.items()}
    scale = 128 ** -0.5
    o_ref, hT_ref, _saved, status_ref = ops.gdn_forward_raw(d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"],
                                                            scale)
    # outputs for the static entry point are ordinary caller tensors, allocated before the call
    o = torch.full_like(o_ref, float("nan"))
    hT = torch.full_like(hT_ref, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize(dev)
    before = torch.cuda.memory_allocated(dev)
    dims = ops._Dims(B, H, L, 128, V, ops.GATE_SCALAR, 1)
    a = ops._Args(dims=dims, scale=scale, q=d["q"].data_ptr(), k=d["k"].data_ptr(), v=d["v"].data_ptr(),
                  g=d["g"].data_ptr(), beta=d["beta"].data_ptr(), h0=d["h0"].data_ptr(), o=o.data_ptr(),
                  hT=hT.data_ptr(), status=status.data_ptr())
    rc = native.lib().lethe_gdn_forward_static(ctypes.byref(a), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0, native.lib().lethe_gdn_strerror(rc)
    torch.cuda.synchronize(dev)
    assert torch.cuda.memory_allocated(dev) == before    # nothing came from torch's allocator
    ops.check_status(status)
    ops.check_status(status_ref)
    return o, hT, o_ref, hT_ref


def test_static_forward_matches_ordinary_forward_twice():
    cap = native.lib().lethe_gdn_forward_static_capacity()
    assert cap == 16 << 20
    # first call: 128 chunks (about 14 MiB of records); second call: 8 chunks on top of the leftovers
    for (B, L, H, V, seed) in ((1, 1024, 8, 64, 21), (1, 256, 2, 128, 22)):
        o, hT, o_ref, hT_ref = _forward_both(B, L, H, V, seed)
        assert torch.equal(o, o_ref)
        assert torch.equal(hT, hT_ref)


def test_static_forward_refuses_oversize():
    B, L, H, V = 2, 2048, 8, 64                          # 512 chunks: far beyond 16 MiB
    dims = ops._Dims(B, H, L, 128, V, ops.GATE_SCALAR, 1)
    assert native.lib().lethe_gdn_saved_bytes(ctypes.byref(dims)) > native.lib().lethe_gdn_forward_static_capacity()
    x = torch.zeros(16, device="cuda")
    a = ops._Args(dims=dims, scale=1.0, q=x.data_ptr(), k=x.data_ptr(), v=x.data_ptr(), g=x.data_ptr(),
                  beta=x.data_ptr(), o=x.data_ptr(), status=x.data_ptr())
    rc = native.lib().lethe_gdn_forward_static(ctypes.byref(a), None)
    assert rc != 0
    assert b"16 MiB" in native.lib().lethe_gdn_strerror(rc)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_static_forward_uses_the_gpu_that_owns_q_not_the_current_device():
    """Every GPU has its own copy of the built-in workspace.  A caller whose thread has GPU 0 selected
    while its tensors live on GPU 1 (a worker thread of a multi-GPU process) must get GPU 1's copy: the
    results on GPU 1 equal the ordinary entry point bit for bit, twice in a row, and GPU 0 is left alone."""
    assert torch.cuda.current_device() == 0
    for (B, L, H, V, seed) in ((1, 512, 4, 64, 31), (1, 256, 2, 128, 32)):
        o, hT, o_ref, hT_ref = _forward_both(B, L, H, V, seed, device="cuda:1")
        assert o.device.index == 1
        assert torch.equal(o, o_ref)
        assert torch.equal(hT, hT_ref)
    assert torch.cuda.current_device() == 0              # the call put the caller's device back
    # and GPU 0's own copy still serves GPU 0
    o, hT, o_ref, hT_ref = _forward_both(1, 256, 2, 64, 33, device="cuda:0")
    assert torch.equal(o, o_ref) and torch.equal(hT, hT_ref)
