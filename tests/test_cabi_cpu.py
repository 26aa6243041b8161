"""CPU checks of the C-ABI library: it loads, exports every symbol the header declares, sizes its
workspaces as documented and rejects bad arguments before touching a GPU."""

import ctypes
import os
import re

import pytest

from lethe_b200 import _build, native, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return native.lib()


def test_exports_every_declared_symbol(lib):
    hdr = open(os.path.join(ROOT, "include", "lethe_gdn.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(lethe_[a-z0-9_]+)\s*\(", hdr))
    assert {"lethe_gdn_forward", "lethe_gdn_backward", "lethe_gdn_saved_bytes", "lethe_gdn_scratch_bytes",
            "lethe_gdn_strerror", "lethe_gdn_forward_static", "lethe_gdn_decode_step", "lethe_gdn_l2norm_qk",
            "lethe_gdn_l2norm_qk_vjp", "lethe_gdn_forward_static_capacity"} <= names
    assert not any("probe" in n for n in names)      # test hooks are not part of the public interface
    for n in names:
        assert hasattr(lib, n), n
    assert not hasattr(lib, "lethe_probe_umma")


def test_probe_library_exports_its_header():
    """The test-only self-test library is separate from the product library and exports what its own
    header declares."""
    plib = ctypes.CDLL(_build.build_probe())
    hdr = open(os.path.join(ROOT, "tests", "native", "lethe_probe.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(lethe_[a-z0-9_]+)\s*\(", hdr))
    assert names == {"lethe_probe_umma", "lethe_probe_starved_wait"}
    for n in names:
        assert hasattr(plib, n), n
    # argument checks come before any launch
    assert plib.lethe_probe_starved_wait(None, ctypes.c_longlong(100000), None, None) != 0


def test_decode_step_argument_errors(lib):
    a = ops._DecodeArgs(B=1, H=1, K=128, V=64, gate=1, delta=1, scale=1.0)      # all pointers null
    rc = lib.lethe_gdn_decode_step(ctypes.byref(a), None)
    assert rc != 0 and b"null" in lib.lethe_gdn_strerror(rc)
    a = ops._DecodeArgs(B=1, H=1, K=64, V=64, gate=0, delta=0, scale=1.0, q=0x1000, k=0x2000, v=0x3000,
                        state=0x4000, o=0x5000)
    rc = lib.lethe_gdn_decode_step(ctypes.byref(a), None)
    assert rc != 0 and b"sizes" in lib.lethe_gdn_strerror(rc)


def test_l2norm_argument_errors(lib):
    rc = lib.lethe_gdn_l2norm_qk(None, None, None, None, 4, 128, 0, 1e-6, None)
    assert rc != 0 and b"null" in lib.lethe_gdn_strerror(rc)
    rc = lib.lethe_gdn_l2norm_qk(0x1000, 0x2000, 0x3000, 0x4000, 4, 96, 0, 1e-6, None)
    assert rc != 0 and b"sizes" in lib.lethe_gdn_strerror(rc)
    rc = lib.lethe_gdn_l2norm_qk_vjp(0x1000, 0x2000, 0x3000, 0x4008, 0x5000, 0x6000, 4, 128, 0, 1e-6, None)
    assert rc != 0 and b"align" in lib.lethe_gdn_strerror(rc)


def test_workspace_sizes(lib):
    d = ops._Dims(2, 8, 2048, 128, 64, 1, 1)
    saved = lib.lethe_gdn_saved_bytes(ctypes.byref(d))
    scratch = lib.lethe_gdn_scratch_bytes(ctypes.byref(d))
    Z = 2 * 8 * 32
    per_saved = 16384 + 16384 + 8192 + 32768 + 16384 + 16384 + 8192 + 512
    carry = 2 * 8 * 128 * 64 * 4            # fp32 state handed between chunk-range calls of the scan
    assert Z * per_saved + carry <= saved <= Z * per_saved + carry + 16 * 16384 + 9 * 1024
    assert scratch >= Z * (16384 + 16384 + 8192 + 16384 + 32768 + 256)
    for bad in (ops._Dims(2, 8, 2000, 128, 64, 1, 1), ops._Dims(2, 8, 2048, 96, 64, 1, 1),
                ops._Dims(2, 8, 2048, 128, 32, 1, 1), ops._Dims(0, 8, 2048, 128, 64, 1, 1),
                ops._Dims(2, 8, 2048, 128, 64, 5, 1)):
        assert lib.lethe_gdn_saved_bytes(ctypes.byref(bad)) == 0


def test_argument_errors_come_before_any_launch(lib):
    d = ops._Dims(1, 1, 64, 128, 64, 1, 1)
    a = ops._Args(dims=d, scale=1.0)                      # all pointers null
    rc = lib.lethe_gdn_forward(ctypes.byref(a), None)
    assert rc != 0 and b"null" in lib.lethe_gdn_strerror(rc)
    a = ops._Args(dims=ops._Dims(1, 1, 65, 128, 64, 1, 1), scale=1.0)
    rc = lib.lethe_gdn_forward(ctypes.byref(a), None)
    assert rc != 0 and b"sizes" in lib.lethe_gdn_strerror(rc)
    # misaligned tensor pointer (fake host addresses: nothing is dereferenced before the checks)
    a = ops._Args(dims=d, scale=1.0, q=0x1008, k=0x2000, v=0x3000, g=0x4000, beta=0x5000, o=0x6000,
                  saved=0x100000, saved_bytes=1 << 30, status=0x7000)
    rc = lib.lethe_gdn_forward(ctypes.byref(a), None)
    assert rc != 0 and b"aligned" in lib.lethe_gdn_strerror(rc)
    a.q = 0x1000
    a.saved_bytes = 1024                                   # workspace too small
    rc = lib.lethe_gdn_forward(ctypes.byref(a), None)
    assert rc != 0 and b"workspace" in lib.lethe_gdn_strerror(rc)
    assert lib.lethe_gdn_strerror(0) == b"ok"
    assert b"timed out" in lib.lethe_gdn_strerror(412)
    # distinct texts for the three host-side failure classes that used to share one
    texts = {lib.lethe_gdn_strerror(c) for c in (5, 9, 10)}
    assert len(texts) == 3 and all(b"unknown" not in t for t in texts)


def test_static_forward_rejects_host_pointers(lib):
    """The entry point without a caller workspace finds its GPU from q; a q that is not device memory is
    refused before anything is looked up or launched."""
    import numpy as np
    d = ops._Dims(1, 1, 64, 128, 64, 1, 1)
    host = np.zeros(64 * 128, dtype=np.uint16)
    a = ops._Args(dims=d, scale=1.0, q=host.ctypes.data, k=host.ctypes.data, v=host.ctypes.data,
                  g=host.ctypes.data, beta=host.ctypes.data, o=host.ctypes.data, status=host.ctypes.data)
    rc = lib.lethe_gdn_forward_static(ctypes.byref(a), None)
    assert rc != 0 and b"device" in lib.lethe_gdn_strerror(rc)


def test_op_refuses_cpu_tensors():
    import torch

    q = torch.zeros(1, 64, 1, 128)
    with pytest.raises(ops.GdnError):
        ops.gdn_chunk(q, q, torch.zeros(1, 64, 1, 64), None, None)
