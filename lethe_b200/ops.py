"""PyTorch surface of the B200 chunked gated-delta-rule path.

``gdn_chunk`` is the differentiable op.  It keeps the argument meaning of the reference project's op
(``gdn2_op``, ``src/lethe/kernels/ops/gdn_layer.py:99-111``: token-major ``[B, L, H, D]`` tensors,
``scale`` applied to q, optional L2 normalisation of q and k) and adds what the reference only has in
its chunkwise references: an initial state in and the final state out
(``src/lethe/kernels/references/gdn2_chunkwise.py:77,157-158``).

PyTorch supplies device memory, the stream and autograd bookkeeping; every number is computed by the
CUDA library behind ``lethe_b200.native`` (there is no other path: a missing library raises).
"""

from __future__ import annotations

import ctypes
from typing import NamedTuple

import torch
from torch import Tensor
from torch.autograd.function import once_differentiable

from . import native

GATE_NONE, GATE_SCALAR, GATE_CHANNEL = 0, 1, 2


class _Dims(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "H", "L", "K", "V", "gate", "delta")]


class _Args(ctypes.Structure):
    _fields_ = [
        ("dims", _Dims), ("scale", ctypes.c_float),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("g", ctypes.c_void_p), ("beta", ctypes.c_void_p), ("h0", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("hT", ctypes.c_void_p),
        ("d_o", ctypes.c_void_p), ("dhT", ctypes.c_void_p),
        ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("dg", ctypes.c_void_p), ("dbeta", ctypes.c_void_p), ("dh0", ctypes.c_void_p),
        ("saved", ctypes.c_void_p), ("saved_bytes", ctypes.c_size_t),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p), ("kernel_mask", ctypes.c_uint32),
        ("dbeta_write", ctypes.c_void_p),
        ("b_gate", ctypes.c_void_p), ("w_gate", ctypes.c_void_p),
        ("db_gate", ctypes.c_void_p), ("dw_gate", ctypes.c_void_p),
        ("bh_begin", ctypes.c_uint32), ("bh_count", ctypes.c_uint32), ("qk_f16", ctypes.c_uint32),
        ("c_begin", ctypes.c_uint32), ("c_count", ctypes.c_uint32),
    ]


def _workspace(nbytes: int, dev) -> Tensor:
    """Byte buffer whose first element is 1024-byte aligned (the tile images inside need it)."""
    raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
    off = (-raw.data_ptr()) % 1024
    return raw[off:off + nbytes]


def _ptr(t: Tensor | None):
    return None if t is None else t.data_ptr()


class GdnError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        msg = native.lib().lethe_gdn_strerror(rc).decode()
        raise GdnError(f"lethe_gdn: {msg} (code {rc})")


def check_status(status: Tensor) -> None:
    """Raise if a device-side wait of an earlier call gave up (synchronises)."""
    code = int(status.item())
    if code != 0:
        raise GdnError(f"lethe_gdn: device-side wait timed out at site {code}; results are invalid")


def _prep16(t: Tensor) -> Tensor:
    return t.to(torch.bfloat16).contiguous()


def _prep_qk(q: Tensor, k: Tensor) -> tuple[Tensor, Tensor]:
    """q and k as the kernels read them: fp16 when both came as fp16 (the tensor-core operand type, kept
    as it is), bf16 otherwise."""
    if q.dtype == torch.float16 and k.dtype == torch.float16:
        return q.contiguous(), k.contiguous()
    return _prep16(q), _prep16(k)


class _StatusWatch:
    """Deferred, sync-free check of the device status words.  After a call the word is copied to a pinned
    host slot on the call's stream; a later call looks at the slots whose copies have completed and
    raises if a device-side wait of that earlier call gave up.  Nothing ever waits for the GPU here, so
    an error surfaces one or two calls late; ``check_status`` is the immediate (synchronising) form."""

    SLOTS = 64

    def __init__(self):
        self._host = None
        self._events = [None] * self.SLOTS
        self._next = 0

    def poll(self) -> None:
        for i, ev in enumerate(self._events):
            if ev is not None and ev.query():
                self._events[i] = None
                code = int(self._host[i])
                if code != 0:
                    raise GdnError(f"lethe_gdn: a device-side wait of an earlier call timed out at site {code}; "
                                   "the results of that call are invalid")

    def watch(self, status: Tensor) -> None:
        if self._host is None:
            self._host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        i = self._next
        self._next = (i + 1) % self.SLOTS
        if self._events[i] is not None:      # ring full: this slot's copy is old enough to have landed
            self._events[i].synchronize()
            self.poll()
        self._host[i:i + 1].copy_(status, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(status.device))
        self._events[i] = ev


_watch = _StatusWatch()


def _prep32(t: Tensor | None) -> Tensor | None:
    return None if t is None else t.to(torch.float32).contiguous()


class GdnBuffers:
    """Every buffer one forward + backward of a fixed problem size needs, allocated once.  The C
    library allocates nothing: callers that must not allocate per step (a training loop, the
    benchmark) keep one of these and call ``forward_into`` / ``backward_into``."""

    def __init__(self, B, L, H, K, V, gate: int, delta: bool, device, backward: bool = True,
                 saved: Tensor | None = None, status: Tensor | None = None, qk_dtype=torch.bfloat16):
        L_ = native.lib()
        # delta: False / True (one beta per token-head), or 2 for the full op's per-channel gates b, w
        self.dims = _Dims(B, H, L, K, V, gate, int(delta))
        full = int(delta) == 2
        nsaved = L_.lethe_gdn_saved_bytes(ctypes.byref(self.dims))
        if nsaved == 0:
            raise GdnError(f"lethe_gdn: unsupported sizes B={B} H={H} L={L} K={K} V={V} "
                           "(need K = 128, V in {64, 128}, L a multiple of 64)")
        bf, f32 = torch.bfloat16, torch.float32
        self.saved = _workspace(nsaved, device) if saved is None else saved
        self.status = torch.zeros(1, dtype=torch.int32, device=device) if status is None else status
        self.o = torch.empty(B, L, H, V, dtype=bf, device=device)
        self.hT = torch.empty(B, H, K, V, dtype=f32, device=device)
        self.scratch = None
        self.db = self.dw = None
        if backward:
            self.scratch = _workspace(L_.lethe_gdn_scratch_bytes(ctypes.byref(self.dims)), device)
            self.dq = torch.empty(B, L, H, K, dtype=qk_dtype, device=device)     # the type of q, k
            self.dk = torch.empty(B, L, H, K, dtype=qk_dtype, device=device)
            self.dv = torch.empty(B, L, H, V, dtype=bf, device=device)
            gshape = (B, L, H, K) if gate == GATE_CHANNEL else (B, L, H)
            self.dg = torch.empty(gshape, dtype=f32, device=device) if gate != GATE_NONE else None
            self.dbeta = torch.empty(B, L, H, dtype=f32, device=device) if (delta and not full) else None
            self.db = torch.empty(B, L, H, K, dtype=f32, device=device) if full else None
            self.dw = torch.empty(B, L, H, V, dtype=f32, device=device) if full else None
            self.dbeta_write = None      # set to a [B, L, H] fp32 tensor to get the erase / write split
            self.dh0 = torch.empty(B, H, K, V, dtype=f32, device=device)


def forward_into(buf: GdnBuffers, q, k, v, g, beta, h0, scale: float, kernel_mask: int = 0, *,
                 b_gate=None, w_gate=None, bh_range: tuple[int, int] = (0, 0),
                 c_range: tuple[int, int] = (0, 0)) -> None:
    """Enqueue the forward kernels on the current stream; results land in ``buf.o`` / ``buf.hT``.
    ``b_gate [B,L,H,K]`` / ``w_gate [B,L,H,V]`` (fp32) replace ``beta`` for buffers made with ``delta=2``.
    ``bh_range = (begin, count)`` restricts the call to those (batch, head) pairs (count 0: all),
    ``c_range = (begin, count)`` to those 64-token chunks of every sequence (the scans carry their state from
    one range to the next: forward ranges in ascending order)."""
    a = _Args(dims=buf.dims, scale=scale, q=_ptr(q), k=_ptr(k), v=_ptr(v), g=_ptr(g), beta=_ptr(beta),
              h0=_ptr(h0), o=_ptr(buf.o), hT=_ptr(buf.hT), saved=_ptr(buf.saved),
              saved_bytes=buf.saved.numel(), status=_ptr(buf.status), kernel_mask=kernel_mask,
              b_gate=_ptr(b_gate), w_gate=_ptr(w_gate), bh_begin=bh_range[0], bh_count=bh_range[1],
              qk_f16=int(q.dtype == torch.float16), c_begin=c_range[0], c_count=c_range[1])
    _check(native.lib().lethe_gdn_forward(ctypes.byref(a), torch.cuda.current_stream(q.device).cuda_stream))


def backward_into(buf: GdnBuffers, q, k, v, g, beta, h0, do, dhT, scale: float, kernel_mask: int = 0, *,
                  b_gate=None, w_gate=None, bh_range: tuple[int, int] = (0, 0),
                  c_range: tuple[int, int] = (0, 0)) -> None:
    """Enqueue the backward kernels; gradients land in ``buf.dq`` ... ``buf.dh0`` (``buf.db`` / ``buf.dw``
    for the per-channel gates of buffers made with ``delta=2``)."""
    a = _Args(dims=buf.dims, scale=scale, q=_ptr(q), k=_ptr(k), v=_ptr(v), g=_ptr(g), beta=_ptr(beta),
              h0=_ptr(h0), d_o=_ptr(do), dhT=_ptr(dhT), dq=_ptr(buf.dq), dk=_ptr(buf.dk), dv=_ptr(buf.dv),
              dg=_ptr(buf.dg), dbeta=_ptr(buf.dbeta), dh0=_ptr(buf.dh0), saved=_ptr(buf.saved),
              saved_bytes=buf.saved.numel(), scratch=_ptr(buf.scratch), scratch_bytes=buf.scratch.numel(),
              status=_ptr(buf.status), kernel_mask=kernel_mask, dbeta_write=_ptr(buf.dbeta_write),
              b_gate=_ptr(b_gate), w_gate=_ptr(w_gate), db_gate=_ptr(buf.db), dw_gate=_ptr(buf.dw),
              bh_begin=bh_range[0], bh_count=bh_range[1], qk_f16=int(q.dtype == torch.float16),
              c_begin=c_range[0], c_count=c_range[1])
    if buf.dq.dtype != q.dtype:
        raise GdnError("lethe_gdn: dq / dk buffers must have the type of q / k (make GdnBuffers with qk_dtype=)")
    _check(native.lib().lethe_gdn_backward(ctypes.byref(a), torch.cuda.current_stream(q.device).cuda_stream))


def default_cut(gate: int, V: int, NT: int, BH: int, sms: int) -> int:
    """Chunk index at which ``GdnStepGraph`` cuts every sequence: the whole number of CTA waves of the chunk
    kernels nearest to half of the sequence.  A chunk kernel runs one CTA per chunk, two per SM for the scalar
    gate at d_v = 64 and one otherwise; when the early segment fills whole waves, the kernels on the serial
    chain (its prepare, its Stage B and WY) do not end on a nearly empty wave, which is worth 7 % of the step
    at B=2, H=8, L=2048.  ``NT`` chunks per sequence, ``BH`` (batch, head) pairs, ``sms`` SMs."""
    if NT < 8:
        return 0
    per_sm = 2 if (gate != GATE_CHANNEL and V == 64) else 1
    wave = (sms * per_sm) // BH                  # chunks of every (batch, head) pair in one wave
    if wave == 0 or wave >= NT:
        return NT // 2
    cut = max(1, int(NT / 2 / wave + 0.5)) * wave
    if cut >= NT:
        cut -= wave
    return cut if cut > 0 else NT // 2


def default_bwd_cuts(gate: int, V: int, delta: bool, NT: int, BH: int, sms: int, cut: int) -> tuple:
    """Where the backward is cut: at the forward's cut, and - when the whole problem is at most two waves of
    two CTAs per SM - once more at half a wave.  The last Stage B and WY launches of a step have nothing to
    hide behind; with half a wave of chunks their CTAs have an SM each and finish sooner (measured at
    B=2, H=8, L=2048, d_v=64: 0.1185 -> 0.1125 ms; larger problems and the one-CTA-per-SM kernels lose)."""
    if not cut:
        return ()
    two_per_sm = gate != GATE_CHANNEL and V == 64 and delta
    wave = (sms * 2) // BH
    if two_per_sm and wave >= 2 and cut == wave and wave < NT <= 2 * wave:
        return (wave // 2, cut)
    return (cut,)


class GdnStepGraph:
    """Forward + backward of one fixed problem, captured once into a CUDA graph and replayed.

    A training step at fixed shapes calls the library with the same pointers every time; replaying the
    captured kernels removes the launch gaps between them.  Two ways to fill the SMs the serial state scans
    leave idle (a scan occupies V / 16 CTAs per (batch, head) pair, V / 32 for very many pairs), both bitwise
    equal to the plain chain:

    ``pipeline`` (default): only the serial chain of the step - prepare, forward scan, adjoint scan, Stage B
    and WY - stays on one stream; the output kernel and the kernel that builds the adjoint scan's input run
    on other streams of the graph beside the scans (the adjoint scan needs neither the outputs nor the
    forward scan).  ``cut`` (default: about half of the chunks, on a whole number of CTA waves, for
    sequences of at least 8 chunks; 0 = no cut) splits every sequence into an early and a late segment of
    chunks (``c_range`` of the C ABI): the late segment is prepared under the forward scan of the early one,
    and its Stage B and WY kernels run under the adjoint scan of the early one.  The scans hand their fp32
    state from segment to segment through the workspace.  ``bwd_cuts`` (default: the forward's cut, plus one
    at half a wave for problems of at most two waves) cuts the backward at places of its own.  (More
    segments than that, and a stream per segment, measured slower: every extra segment adds a scan prologue
    to the serial chain.)

    ``groups > 1``: the (batch, head) pairs are cut into that many ranges and every range runs its own
    kernel chain on its own stream inside the graph (the pairs are independent recurrences).

    Inputs are read from, and results written to, the tensors given here: copy new data into them between
    replays.  Results land in ``buf`` as with ``forward_into`` / ``backward_into``.
    """

    def __init__(self, buf: GdnBuffers, q, k, v, g, beta, h0, do, dhT, scale: float, *, b_gate=None, w_gate=None,
                 groups: int = 1, pipeline: bool | None = None,
                 cut: int | None = None, bwd_cuts=None):
        self.buf = buf
        self._keep = (q, k, v, g, beta, h0, do, dhT, b_gate, w_gate)
        dev = q.device
        BH = buf.dims.B * buf.dims.H
        NT = buf.dims.L // 64
        groups = max(1, min(int(groups), BH))
        bounds = [BH * i // groups for i in range(groups + 1)]
        ranges = [(bounds[i], bounds[i + 1] - bounds[i]) for i in range(groups)]
        self.groups = groups
        if pipeline is None:
            pipeline = groups == 1
        self.pipeline = bool(pipeline) and groups == 1
        if cut is None:
            cut = self._default_cut(buf, NT, BH, dev)
        self.cut = int(cut) if self.pipeline and 0 < int(cut) < NT else 0
        self.segments = 2 if self.cut else 1
        if bwd_cuts is None or not self.pipeline:
            bwd_cuts = self._default_bwd_cuts(buf, NT, BH, dev, self.cut)
        self.bwd_cuts = tuple(sorted(int(c) for c in bwd_cuts))
        if any(c <= 0 or c >= NT for c in self.bwd_cuts) or len(set(self.bwd_cuts)) != len(self.bwd_cuts):
            raise GdnError(f"lethe_gdn: backward cuts {self.bwd_cuts} must be distinct chunk indices inside (0, {NT})")
        gates = dict(b_gate=b_gate, w_gate=w_gate)

        def chain(rng):
            forward_into(buf, q, k, v, g, beta, h0, scale, bh_range=rng, **gates)
            backward_into(buf, q, k, v, g, beta, h0, do, dhT, scale, bh_range=rng, **gates)

        side = torch.cuda.Stream(device=dev)
        self._streams = [torch.cuda.Stream(device=dev) for _ in range(max(groups - 1, 2))]

        def fwd(mask, cr):
            forward_into(buf, q, k, v, g, beta, h0, scale, mask, c_range=cr, **gates)

        def bwd(mask, cr):
            backward_into(buf, q, k, v, g, beta, h0, do, dhT, scale, mask, c_range=cr, **gates)

        def mark(st):
            e = torch.cuda.Event()
            e.record(st)
            return e

        def pipelined():
            # The serial chain of a step is prepare(first segment) -> forward scan -> adjoint scan -> Stage B and
            # WY of the first segment; `side` carries exactly that.  Everything else hangs off it by events:
            # `other` prepares the later segment and builds the adjoint scan's input while the forward scan
            # runs, computes the outputs behind the scan, and runs Stage B / WY of the later segment under the
            # adjoint scan of the first; `third` computes the output of the last segment while the adjoint scan
            # has already started.  Stream order is chosen so that no kernel launched with the
            # programmatic-dependency attribute follows, on its own stream, the kernel whose result it loads
            # before its wait (Stage B loads v_new early: it never follows an output kernel of its own segment).
            other, third = self._streams[0], self._streams[1]
            segs = [(0, self.cut), (self.cut, NT - self.cut)] if self.segments == 2 else [(0, NT)]
            S = len(segs)
            # the backward may be cut at other places than the forward (its ranges only have to be visited in
            # descending order): boundaries self.bwd_cuts, ascending
            bb = [0] + list(self.bwd_cuts) + [NT]
            bsegs = [(bb[i], bb[i + 1] - bb[i]) for i in range(len(bb) - 1)]
            SB = len(bsegs)
            has_wy = buf.dims.delta != 0
            e_p, e_f, e_o = ([None] * S for _ in range(3))
            e_r, e_a = ([None] * SB for _ in range(2))
            with torch.cuda.stream(side):
                fwd(1, segs[0])
                e_p[0] = mark(side)
            other.wait_event(e_p[0])
            with torch.cuda.stream(other):
                for i in range(1, S):
                    fwd(1, segs[i])                          # prepare of the later segment: under the first scan
                    e_p[i] = mark(other)
                for i in reversed(range(SB)):
                    bwd(1, bsegs[i])                         # input of the adjoint scan: needs prepare and do only
                    e_r[i] = mark(other)
            for i in range(S):                               # forward scan, segment after segment
                if i:
                    side.wait_event(e_p[i])
                with torch.cuda.stream(side):
                    fwd(2, segs[i])
                    e_f[i] = mark(side)
            for i in range(S):                               # outputs behind the scan, off the serial chain
                st = third if i == S - 1 else other
                st.wait_event(e_f[i])
                with torch.cuda.stream(st):
                    fwd(4, segs[i])
                    e_o[i] = mark(st)
            for i in reversed(range(SB)):                    # adjoint scan straight behind the forward scan
                side.wait_event(e_r[i])
                with torch.cuda.stream(side):
                    bwd(2, bsegs[i])
                    e_a[i] = mark(side)
            for n, i in enumerate(reversed(range(1, SB))):   # Stage B / WY of the later segments: under the adjoint scan
                st = other if n % 2 == 0 else third
                st.wait_event(e_a[i])
                for e in e_o:
                    st.wait_event(e)
                with torch.cuda.stream(st):
                    bwd(4, bsegs[i])
                    if has_wy:
                        bwd(8, bsegs[i])
            for e in e_o:
                side.wait_event(e)
            with torch.cuda.stream(side):
                bwd(4, bsegs[0])
                if has_wy:
                    bwd(8, bsegs[0])
            side.wait_event(mark(other))
            side.wait_event(mark(third))

        def step():
            if self.pipeline:
                pipelined()
                return
            if groups == 1:
                chain((0, 0))
                return
            fork = torch.cuda.Event()
            fork.record(side)
            joins = []
            for i, rng in enumerate(ranges):
                st = side if i == 0 else self._streams[i - 1]
                if i:
                    st.wait_event(fork)
                with torch.cuda.stream(st):
                    chain(rng)
                if i:
                    e = torch.cuda.Event()
                    e.record(st)
                    joins.append(e)
            for e in joins:
                side.wait_event(e)

        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            chain((0, 0))               # first call outside the capture: one-time driver look-ups and attributes
            side.synchronize()
            check_status(buf.status)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                step()
        torch.cuda.current_stream(dev).wait_stream(side)

    @staticmethod
    def _default_cut(buf, NT: int, BH: int, dev) -> int:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        return default_cut(buf.dims.gate, buf.dims.V, NT, BH, sms)

    @staticmethod
    def _default_bwd_cuts(buf, NT: int, BH: int, dev, cut: int) -> tuple:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        return default_bwd_cuts(buf.dims.gate, buf.dims.V, buf.dims.delta != 0, NT, BH, sms, cut)

    def replay(self) -> None:
        """Enqueue the captured step on the current stream."""
        self.graph.replay()


def _gate_code(g: Tensor | None) -> int:
    return GATE_NONE if g is None else (GATE_SCALAR if g.dim() == 3 else GATE_CHANNEL)


def gdn_forward_raw(q, k, v, g, beta, h0, scale: float):
    """One forward call of the library.  Inputs must be CUDA tensors: q, k (both bf16 or both fp16) and
    v (bf16) contiguous ``[B, L, H, D]``; g, beta, h0 fp32.  Returns ``(o, hT, saved, status)`` in fresh
    buffers."""
    B, L, H, K = q.shape
    buf = GdnBuffers(B, L, H, K, v.shape[-1], _gate_code(g), beta is not None, q.device, backward=False)
    forward_into(buf, q, k, v, g, beta, h0, scale)
    return buf.o, buf.hT, buf.saved, buf.status


def gdn_backward_raw(q, k, v, g, beta, h0, do, dhT, saved, status, scale: float):
    """One backward call of the library.  Returns ``(dq, dk, dv, dg, dbeta, dh0, scratch)``."""
    B, L, H, K = q.shape
    buf = GdnBuffers(B, L, H, K, v.shape[-1], _gate_code(g), beta is not None, q.device,
                     saved=saved, status=status, qk_dtype=q.dtype)
    backward_into(buf, q, k, v, g, beta, h0, do, dhT, scale)
    return buf.dq, buf.dk, buf.dv, buf.dg, buf.dbeta, buf.dh0, buf.scratch


L2_IN_F32, L2_NORM_F16 = 1, 2


def _l2_working(q: Tensor, k: Tensor) -> tuple[Tensor, Tensor, bool]:
    """q, k as the normalisation kernels read them: both bf16 if both came as bf16, else both fp32."""
    f32 = not (q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16)
    dt = torch.float32 if f32 else torch.bfloat16
    return q.to(dt).contiguous(), k.to(dt).contiguous(), f32


def l2norm_qk_raw(q: Tensor, k: Tensor, eps: float = 1e-6, norm_dtype=torch.float16) -> tuple[Tensor, Tensor]:
    """``x * rsqrt(sum x^2 + eps)`` over the last axis of q and of k in one launch (epsilon placed as in
    the reference, ``gdn_backward.py:9-10``).  The rows are formed in fp32 and rounded once: to fp16 by
    default (the operand type of the GDN kernels, which then read them unchanged; the reference rounds
    at the same point, ``gdn2_bwd_dhu_l3.py:477-479``), or to bf16 with ``norm_dtype=torch.bfloat16``."""
    if not q.is_cuda:
        raise GdnError("lethe_gdn: inputs must live on a CUDA device (there is no CPU path)")
    if q.shape != k.shape:
        raise GdnError("lethe_gdn: q and k must have the same shape")
    if norm_dtype not in (torch.float16, torch.bfloat16):
        raise GdnError("lethe_gdn: normalised rows are fp16 or bf16")
    qc, kc, f32 = _l2_working(q, k)
    qn, kn = torch.empty_like(qc, dtype=norm_dtype), torch.empty_like(kc, dtype=norm_dtype)
    D = q.shape[-1]
    flags = (L2_IN_F32 if f32 else 0) | (L2_NORM_F16 if norm_dtype == torch.float16 else 0)
    _check(native.lib().lethe_gdn_l2norm_qk(qc.data_ptr(), kc.data_ptr(), qn.data_ptr(), kn.data_ptr(),
                                            qc.numel() // D, D, flags, eps,
                                            torch.cuda.current_stream(q.device).cuda_stream))
    return qn, kn


def l2norm_qk_vjp_raw(q: Tensor, k: Tensor, dqn: Tensor, dkn: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Gradients with respect to q and k given those with respect to the normalised rows (fp16 or bf16,
    as the backward kernels wrote them).  Returned in the working type of q, k (bf16 or fp32)."""
    qc, kc, f32 = _l2_working(q, k)
    f16 = dqn.dtype == torch.float16 and dkn.dtype == torch.float16
    if f16:
        dqn, dkn = dqn.contiguous(), dkn.contiguous()
    else:
        dqn, dkn = _prep16(dqn), _prep16(dkn)
    dq, dk = torch.empty_like(qc), torch.empty_like(kc)
    D = q.shape[-1]
    flags = (L2_IN_F32 if f32 else 0) | (L2_NORM_F16 if f16 else 0)
    _check(native.lib().lethe_gdn_l2norm_qk_vjp(qc.data_ptr(), kc.data_ptr(), dqn.data_ptr(), dkn.data_ptr(),
                                                dq.data_ptr(), dk.data_ptr(), qc.numel() // D, D, flags, eps,
                                                torch.cuda.current_stream(q.device).cuda_stream))
    return dq, dk


class _L2NormQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, eps):
        ctx.save_for_backward(q, k)
        ctx.eps = eps
        return l2norm_qk_raw(q, k, eps)

    @staticmethod
    @once_differentiable
    def backward(ctx, dqn, dkn):
        q, k = ctx.saved_tensors
        dqn = torch.zeros_like(q, dtype=torch.float16) if dqn is None else dqn
        dkn = torch.zeros_like(k, dtype=torch.float16) if dkn is None else dkn
        dq, dk = l2norm_qk_vjp_raw(q, k, dqn, dkn, ctx.eps)
        return dq.to(q.dtype), dk.to(k.dtype), None


def l2norm_qk(q: Tensor, k: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Differentiable L2 normalisation of q and k over the channel axis (one kernel each way).  Returns
    fp16 rows, which ``gdn_chunk`` / ``gdn_chunk_full`` take as they are."""
    return _L2NormQK.apply(q, k, eps)


class _GdnChunk(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, h0, scale):
        if not q.is_cuda:
            raise GdnError("lethe_gdn: inputs must live on a CUDA device (there is no CPU path)")
        _watch.poll()
        K = q.shape[-1]
        ctx.in_dtypes = tuple(None if t is None else t.dtype for t in (q, k, v, g, beta, h0))
        ctx.pad_k = 0
        (q16, k16), v16 = _prep_qk(q, k), _prep16(v)
        g32, b32, h32 = _prep32(g), _prep32(beta), _prep32(h0)
        if K == 64:
            # the kernels are built for 128 key channels: pad with zero channels (exact)
            ctx.pad_k = 64
            q16 = torch.nn.functional.pad(q16, (0, 64))
            k16 = torch.nn.functional.pad(k16, (0, 64))
            if g32 is not None and g32.dim() == 4:
                g32 = torch.nn.functional.pad(g32, (0, 64))
            if h32 is not None:
                h32 = torch.nn.functional.pad(h32, (0, 0, 0, 64))
        L = q.shape[1]
        ctx.pad_l = (-L) % 64
        if ctx.pad_l:
            # The kernels work on chunks of 64 tokens.  Tokens appended with k = v = q = 0, g = 0 and
            # beta = 0 leave the state untouched (decay 1, nothing erased, nothing written), so the
            # result on the real tokens and the final state are exact.
            def pad_tokens(t):
                return None if t is None else torch.nn.functional.pad(t, (0, 0) * (t.dim() - 2) + (0, ctx.pad_l))
            q16, k16, v16, g32, b32 = (pad_tokens(t) for t in (q16, k16, v16, g32, b32))
        o, hT, saved, status = gdn_forward_raw(q16, k16, v16, g32, b32, h32, scale)
        _watch.watch(status)
        ctx.save_for_backward(q16, k16, v16, g32, b32, h32, saved, status)
        ctx.scale = scale
        if ctx.pad_k:
            hT = hT[:, :, :K].contiguous()
        if ctx.pad_l:
            o = o[:, :L]
        return o.to(v.dtype), hT

    @staticmethod
    @once_differentiable
    def backward(ctx, do, dhT):
        q16, k16, v16, g32, b32, h32, saved, status = ctx.saved_tensors
        _watch.poll()
        do16 = _prep16(do)
        dhT32 = _prep32(dhT)
        if ctx.pad_l:
            do16 = torch.nn.functional.pad(do16, (0, 0, 0, 0, 0, ctx.pad_l))
        if ctx.pad_k and dhT32 is not None:
            dhT32 = torch.nn.functional.pad(dhT32, (0, 0, 0, ctx.pad_k))
        dq, dk, dv, dg, dbeta, dh0, _ = gdn_backward_raw(q16, k16, v16, g32, b32, h32, do16, dhT32,
                                                        saved, status, ctx.scale)
        _watch.watch(status)
        if ctx.pad_k:
            K = q16.shape[-1] - ctx.pad_k
            dq, dk, dh0 = dq[..., :K], dk[..., :K], dh0[:, :, :K]
            if dg is not None and dg.dim() == 4:
                dg = dg[..., :K]
        if ctx.pad_l:
            L = q16.shape[1] - ctx.pad_l
            dq, dk, dv = dq[:, :L], dk[:, :L], dv[:, :L]
            dg = None if dg is None else dg[:, :L]
            dbeta = None if dbeta is None else dbeta[:, :L]
        dts = ctx.in_dtypes
        outs = [dq.to(dts[0]), dk.to(dts[1]), dv.to(dts[2]),
                None if dg is None else dg.to(dts[3]),
                None if dbeta is None else dbeta.to(dts[4]),
                None if dts[5] is None else dh0.to(dts[5]), None]
        return tuple(outs)


def gdn_chunk(q: Tensor, k: Tensor, v: Tensor, g: Tensor | None, beta: Tensor | None,
              h0: Tensor | None = None, *, scale: float | None = None,
              use_qk_l2norm: bool = False) -> tuple[Tensor, Tensor]:
    """Chunked gated delta rule, differentiable.  Returns ``(o [B,L,H,V], h_T [B,H,K,V] fp32)``.

    ``g``: per-token log decay, ``[B,L,H]`` (scalar gate), ``[B,L,H,K]`` (channel-wise) or None.
    ``beta``: ``[B,L,H]`` (erase and write gate) or None for the variants without the delta term
    (linear attention, GLA, SSD).  Gradients flow to q, k, v, g, beta and h0 (first order only: the
    backward is not itself differentiable, asking for a second derivative raises).  ``L`` need not be a
    multiple of the chunk length and d_k may be 64 or 128: both are met by exact zero padding.  q and k
    are read as bf16, or as fp16 when both are given as fp16; with ``use_qk_l2norm`` they are normalised
    in fp32 and rounded once to fp16.
    """
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if use_qk_l2norm:
        q, k = l2norm_qk(q, k)
    return _GdnChunk.apply(q, k, v, g, beta, h0, float(scale))


class _DecodeArgs(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("K", ctypes.c_int32), ("V", ctypes.c_int32),
                ("gate", ctypes.c_int32), ("delta", ctypes.c_int32), ("scale", ctypes.c_float),
                ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("g", ctypes.c_void_p), ("beta", ctypes.c_void_p), ("state", ctypes.c_void_p),
                ("o", ctypes.c_void_p)]


def gdn_decode_step(q: Tensor, k: Tensor, v: Tensor, g: Tensor | None, beta: Tensor | None, state: Tensor,
                    *, scale: float | None = None) -> Tensor:
    """One token of the recurrence for every (batch, head) pair, for generation: the body of the
    reference's token loop (``src/lethe/kernels/references/gdn_backward.py:45-53``).

    ``q, k [B,H,K]``, ``v [B,H,V]``; ``g [B,H]`` (scalar gate), ``[B,H,K]`` (channel-wise) or None;
    ``beta [B,H]`` or None (no delta term); ``state [B,H,K,V]`` fp32 contiguous, **updated in place**
    (start from the ``h_T`` that ``gdn_chunk`` returned for the prompt).  Returns ``o [B,H,V]`` bf16.
    Not differentiable.  K must be 128, V 64 or 128.
    """
    if not state.is_cuda:
        raise GdnError("lethe_gdn: inputs must live on a CUDA device (there is no CPU path)")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise GdnError("lethe_gdn: the decode state must be a contiguous fp32 tensor (it is updated in place)")
    B, H, K, V = state.shape
    q16, k16, v16 = _prep16(q), _prep16(k), _prep16(v)
    g32, b32 = _prep32(g), _prep32(beta)
    if q16.shape != (B, H, K) or k16.shape != (B, H, K) or v16.shape != (B, H, V):
        raise GdnError("lethe_gdn: decode step expects q, k [B,H,K] and v [B,H,V] matching the state")
    if g32 is not None and g32.shape not in ((B, H), (B, H, K)):
        raise GdnError("lethe_gdn: decode step expects g [B,H] or [B,H,K]")
    if b32 is not None and b32.shape != (B, H):
        raise GdnError("lethe_gdn: decode step expects beta [B,H]")
    o = torch.empty(B, H, V, dtype=torch.bfloat16, device=state.device)
    a = _DecodeArgs(B=B, H=H, K=K, V=V, gate=_gate_code(None if g32 is None else g32.unsqueeze(1)),
                    delta=0 if b32 is None else 1, scale=float(K ** -0.5 if scale is None else scale),
                    q=_ptr(q16), k=_ptr(k16), v=_ptr(v16), g=_ptr(g32), beta=_ptr(b32), state=_ptr(state), o=_ptr(o))
    _check(native.lib().lethe_gdn_decode_step(ctypes.byref(a), torch.cuda.current_stream(state.device).cuda_stream))
    return o


class _GdnFull(torch.autograd.Function):
    """The reference's full recurrence (``src/lethe/kernels/references/gdn_backward.py:45-53``): per-channel
    log decay ``g`` and erase gate ``b`` (``[B,L,H,K]``), per-channel write gate ``w`` (``[B,L,H,V]``)."""

    @staticmethod
    def forward(ctx, q, k, v, g, b, w, h0, scale):
        if not q.is_cuda:
            raise GdnError("lethe_gdn: inputs must live on a CUDA device (there is no CPU path)")
        _watch.poll()
        B, L, H, K = q.shape
        V = v.shape[-1]
        if K != 128 or L % 64:
            raise GdnError("lethe_gdn: the full-gate op needs d_k = 128 and L a multiple of 64")
        ctx.in_dtypes = tuple(None if t is None else t.dtype for t in (q, k, v, g, b, w, h0))
        (q16, k16), v16 = _prep_qk(q, k), _prep16(v)
        g32, b32, w32, h32 = _prep32(g), _prep32(b), _prep32(w), _prep32(h0)
        buf = GdnBuffers(B, L, H, K, V, GATE_CHANNEL, 2, q.device, backward=False)
        forward_into(buf, q16, k16, v16, g32, None, h32, scale, b_gate=b32, w_gate=w32)
        _watch.watch(buf.status)
        ctx.save_for_backward(q16, k16, v16, g32, b32, w32, h32, buf.saved, buf.status)
        ctx.scale = scale
        return buf.o.to(v.dtype), buf.hT

    @staticmethod
    @once_differentiable
    def backward(ctx, do, dhT):
        q16, k16, v16, g32, b32, w32, h32, saved, status = ctx.saved_tensors
        _watch.poll()
        B, L, H, K = q16.shape
        buf = GdnBuffers(B, L, H, K, v16.shape[-1], GATE_CHANNEL, 2, q16.device, saved=saved, status=status,
                         qk_dtype=q16.dtype)
        backward_into(buf, q16, k16, v16, g32, None, h32, _prep16(do), _prep32(dhT), ctx.scale,
                      b_gate=b32, w_gate=w32)
        _watch.watch(status)
        dts = ctx.in_dtypes
        return (buf.dq.to(dts[0]), buf.dk.to(dts[1]), buf.dv.to(dts[2]), buf.dg.to(dts[3]), buf.db.to(dts[4]),
                buf.dw.to(dts[5]), None if dts[6] is None else buf.dh0.to(dts[6]), None)


def gdn_chunk_full(q: Tensor, k: Tensor, v: Tensor, g: Tensor, b: Tensor, w: Tensor, h0: Tensor | None = None, *,
                   scale: float | None = None, use_qk_l2norm: bool = False) -> tuple[Tensor, Tensor]:
    """The reference's full six-input recurrence with an initial state in and the final state out:
    ``g, b [B,L,H,K]`` (log decay and erase gate per key channel), ``w [B,L,H,V]`` (write gate per value
    channel).  Returns ``(o, h_T)``; gradients flow to all seven inputs (first order only)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if use_qk_l2norm:
        q, k = l2norm_qk(q, k)
    return _GdnFull.apply(q, k, v, g, b, w, h0, float(scale))


# ------------------------------------------------------------------------------------------------
# The reference's own six-input surface
# ------------------------------------------------------------------------------------------------
def gate_regime(g: Tensor, b: Tensor, w: Tensor) -> tuple[bool, bool, bool]:
    """``(scalar_gate, one_beta, no_delta)`` of a six-input call, decided as the reference decides
    (``src/lethe/kernels/cute/gdn2_backward.py:53-60``): BITWISE equality along the channel axis, never
    a tolerance - a gate that is merely close to constant is a channel-wise gate.  One device
    reduction and one host read for all five tests.

    scalar_gate: g is one value per token-head broadcast over the key channels;
    one_beta:    b and w are the same one value per token-head broadcast over their channels;
    no_delta:    b = 0 everywhere and w = 1 everywhere (no erase term, unit write gate)."""
    with torch.no_grad():
        flags = torch.stack([
            (g == g[..., :1]).all(),
            (b == b[..., :1]).all() & (w == w[..., :1]).all() & (b[..., 0] == w[..., 0]).all(),
            (b == 0).all() & (w == 1).all(),
        ]).tolist()
    return bool(flags[0]), bool(flags[1]), bool(flags[2])


class _Gdn2Op(torch.autograd.Function):
    """``gdn2_op`` of the reference (``src/lethe/kernels/ops/gdn_layer.py:15-111``) on the CUDA library.

    The reference op takes a per-channel log decay ``g``, erase gate ``b`` (both ``[B,L,H,d_k]``) and
    write gate ``w`` (``[B,L,H,d_v]``).  The kernels cover the regimes its native path covers
    (``src/lethe/kernels/cute/gdn2_backward.py:53-60,102-134`` and ``cute/gdn2_family.py``):
    ``b`` and ``w`` both equal to one beta per token-head broadcast over the channels (gated delta
    rule / KDA), or ``b = 0, w = 1`` (no delta term); ``g`` either constant over the channels
    (scalar gate) or not (channel-wise gate).  Independent per-channel ``b`` / ``w`` do not come
    here: ``gdn2_op`` sends them to ``gdn_chunk_full``.

    Gradients of broadcast inputs are spread evenly over the channels, as the reference's scalar
    assembly does (``gdn2_assemble.py:343-345``); ``grad_b`` carries the erase part and ``grad_w`` the
    write part of the beta gradient (``gdn2_assemble.py:150-181``).
    """

    @staticmethod
    def forward(ctx, q, k, v, g, b, w, scale, use_qk_l2norm, scalar_gate, delta):
        if not q.is_cuda:
            raise GdnError("lethe_gdn: inputs must live on a CUDA device (there is no CPU path)")
        _watch.poll()
        K, V = q.shape[-1], v.shape[-1]
        with torch.no_grad():
            beta = b[..., 0].float().contiguous() if delta else None
            g_in = (g[..., 0] if scalar_gate else g).float().contiguous()
        ctx.meta = (q.dtype, k.dtype, v.dtype, g.dtype, b.dtype, w.dtype, K, V, scalar_gate, delta, use_qk_l2norm)
        q16, k16 = l2norm_qk_raw(q, k) if use_qk_l2norm else _prep_qk(q, k)
        v16 = _prep16(v)
        o, _hT, saved, status = gdn_forward_raw(q16, k16, v16, g_in, beta, None, scale)
        _watch.watch(status)
        ctx.save_for_backward(q, k, q16, k16, v16, g_in, beta, saved, status)
        ctx.scale = scale
        return o.to(v.dtype)

    @staticmethod
    @once_differentiable
    def backward(ctx, do):
        q, k, q16, k16, v16, g_in, beta, saved, status = ctx.saved_tensors
        _watch.poll()
        dq_t, dk_t, dv_t, dg_t, db_t, dw_t, K, V, scalar_gate, delta, l2 = ctx.meta
        B, L, H, _ = q16.shape
        buf = GdnBuffers(B, L, H, K, V, _gate_code(g_in), delta, q16.device, saved=saved, status=status,
                         qk_dtype=q16.dtype)
        if delta:
            buf.dbeta_write = torch.empty(B, L, H, dtype=torch.float32, device=q16.device)
        backward_into(buf, q16, k16, v16, g_in, beta, None, _prep16(do), None, ctx.scale)
        _watch.watch(status)
        dq, dk = buf.dq, buf.dk
        if l2:   # VJP of x / sqrt(|x|^2 + eps) (the reference gets it by autograd, gdn2_assemble.py:300-312)
            dq, dk = l2norm_qk_vjp_raw(q, k, dq, dk)
        grad_g = (buf.dg.unsqueeze(-1).expand(B, L, H, K) / K) if scalar_gate else buf.dg
        if delta:
            grad_b = buf.dbeta.unsqueeze(-1).expand(B, L, H, K) / K
            grad_w = buf.dbeta_write.unsqueeze(-1).expand(B, L, H, V) / V
        else:
            grad_b = torch.zeros(B, L, H, K, device=q16.device)
            grad_w = torch.zeros(B, L, H, V, device=q16.device)
        return (dq.to(dq_t), dk.to(dk_t), buf.dv.to(dv_t), grad_g.to(dg_t).contiguous(),
                grad_b.to(db_t).contiguous(), grad_w.to(dw_t).contiguous(), None, None, None, None)


def gdn2_op(q: Tensor, k: Tensor, v: Tensor, g: Tensor, b: Tensor, w: Tensor, *, scale: float | None = None,
            use_qk_l2norm: bool = True) -> Tensor:
    """Drop-in for the reference's ``gdn2_op`` (same argument list, same defaults, returns ``o``).
    First-order gradients only: the backward pass is not differentiable (the reference falls back to its
    eager path for that case, ``cute/gdn2_backward.py:92``; here a second derivative raises)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if q.shape[-1] != 128:
        raise GdnError("lethe_gdn: gdn2_op needs d_k = 128 (use gdn_chunk for d_k = 64)")
    if not q.is_cuda:
        raise GdnError("lethe_gdn: inputs must live on a CUDA device (there is no CPU path)")
    scalar_gate, one_beta, no_delta = gate_regime(g, b, w)
    if one_beta or no_delta:
        # the regimes the scalar-beta kernels cover (cheaper: one gate value per token-head)
        return _Gdn2Op.apply(q, k, v, g, b, w, float(scale), bool(use_qk_l2norm), scalar_gate, bool(one_beta))
    # independent per-channel erase / write gates: the full recurrence
    o, _ = gdn_chunk_full(q, k, v, g, b, w, None, scale=float(scale), use_qk_l2norm=bool(use_qk_l2norm))
    return o


class Gdn2Grads(NamedTuple):
    """Field for field the reference's result type (``src/lethe/kernels/references/gdn_backward.py:58-67``)."""
    grad_q: Tensor
    grad_k: Tensor
    grad_v: Tensor
    grad_g: Tensor
    grad_b: Tensor
    grad_w: Tensor
    grad_initial_state: Tensor | None


def gdn2_backward(q: Tensor, k: Tensor, v: Tensor, g: Tensor, b: Tensor, w: Tensor, do: Tensor, *,
                  scale: float | None = None, use_qk_l2norm: bool = True, fwd_stash=None,
                  rescale_do: bool = True) -> Gdn2Grads:
    """Drop-in for the reference's backward entry point ``gdn2_backward``
    (``src/lethe/kernels/ops/gdn_backward.py:16-57``: same positional arguments, same keywords, same
    result type), which is what its autograd function calls (``ops/gdn_layer.py:69-96``) and what its
    verifier harness takes as the candidate (``verifier/op_harness.py:714-733``).  The six gradients
    come back in the dtypes of the inputs they belong to.

    The reference function gets the inputs only, so the forward is recomputed here (the reference does
    the same, ``cute/gdn2_assemble.py:261-263``); ``fwd_stash`` is accepted and ignored.

    ``rescale_do``: the backward is linear in ``do``, and ``do`` enters the tensor cores as fp16.  With
    this flag (default) ``do`` is first divided by a power of two near its largest magnitude and the
    gradients are multiplied back, so that upstream gradients far outside the fp16 range (1e6, 1e-6)
    neither saturate nor fall into the subnormals.  Exact (a power of two), all on the device, no
    host synchronisation."""
    if do.requires_grad:
        raise GdnError("lethe_gdn: the backward is not differentiable (do.requires_grad): there is no eager "
                       "fallback to route a second derivative to (the reference declines its native path in "
                       "this case, cute/gdn2_backward.py:92)")
    do = do.detach()
    mult = None
    if rescale_do:
        amax = do.abs().amax().float()
        amax = torch.where(torch.isfinite(amax) & (amax > 0), amax, torch.ones_like(amax))
        mult = torch.exp2(torch.round(torch.log2(amax)))          # power of two: scaling is exact
        do = (do.float() / mult).to(do.dtype if do.dtype != torch.float16 else torch.float32)
    leaves = [t.detach().requires_grad_(True) for t in (q, k, v, g, b, w)]
    with torch.enable_grad():
        o = gdn2_op(*leaves, scale=scale, use_qk_l2norm=use_qk_l2norm)
    grads = torch.autograd.grad(o, leaves, do.to(o.dtype))
    if mult is not None:
        grads = tuple((t.float() * mult).to(t.dtype) for t in grads)
    return Gdn2Grads(*grads, None)
