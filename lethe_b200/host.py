"""Forward + backward for callers whose tensors live in host memory.

A training loop that keeps activations on the device calls ``ops.gdn_chunk``.  A host that feeds the
kernels from pinned host buffers and wants the results back in host buffers pays for two PCIe
transfers per step that dwarf the kernels (52 MB against 0.2 ms of kernels at B=2, H=8, L=2048).
``HostPipeline`` overlaps the three legs of consecutive steps - host-to-device copy, kernels,
device-to-host copy - on three CUDA streams with ``depth`` sets of device buffers, so that a stream of
steps runs at the pace of the slowest leg instead of the sum of the three.

Nothing here allocates per step: device buffers are made once per pipeline, and the C library never
allocates.  All calls are asynchronous; ``drain()`` waits and checks the device status words.  Host buffers
made by ``make_host_buffers()`` have the layout of the device side and move as ONE copy per direction and
step, which the host link rewards: 0.61 ms per step against 0.76 ms with one copy per tensor.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


def _arena(specs: dict, device=None, pinned: bool = False):
    """One allocation for all tensors of `specs` (name -> (shape, dtype)), each a view at a 256-byte
    boundary.  Returns ``(base uint8 tensor, {name: view}, {name: byte offset})``."""
    offs, total = {}, 0
    for n, (shape, dt) in specs.items():
        total = (total + 255) & ~255
        offs[n] = total
        total += int(torch.Size(shape).numel()) * torch.empty((), dtype=dt).element_size()
    if pinned:
        base = torch.empty(total, dtype=torch.uint8, pin_memory=True)
    else:
        base = torch.empty(total, dtype=torch.uint8, device=device)
    views = {}
    for n, (shape, dt) in specs.items():
        nbytes = int(torch.Size(shape).numel()) * torch.empty((), dtype=dt).element_size()
        views[n] = base[offs[n]:offs[n] + nbytes].view(dt).view(shape)
    return base, views, offs


class _Slot:
    """Device side of one step in flight.  All inputs live in one allocation and all outputs in another, so
    that a step whose host buffers have the same layout (``HostPipeline.make_host_buffers``) crosses the host
    link as one copy each way: fifteen separate copies per step reach 0.66-0.76 ms on a link that moves the
    same bytes in 0.54 ms as two."""

    def __init__(self, B, L, H, K, V, gate, delta, has_h0, has_dhT, device):
        bf, f32 = torch.bfloat16, torch.float32
        self.buf = ops.GdnBuffers(B, L, H, K, V, gate, delta, device)
        spec = {"q": ((B, L, H, K), bf), "k": ((B, L, H, K), bf), "v": ((B, L, H, V), bf), "do": ((B, L, H, V), bf)}
        if gate != ops.GATE_NONE:
            spec["g"] = ((B, L, H, K) if gate == ops.GATE_CHANNEL else (B, L, H), f32)
        if int(delta) == 2:
            spec["b"] = ((B, L, H, K), f32)
            spec["w"] = ((B, L, H, V), f32)
        elif delta:
            spec["beta"] = ((B, L, H), f32)
        if has_h0:
            spec["h0"] = ((B, H, K, V), f32)
        if has_dhT:
            spec["dhT"] = ((B, H, K, V), f32)
        self.in_spec = spec
        self.in_arena, self.inp, self.in_offs = _arena(spec, device)
        # the outputs GdnBuffers made are replaced by views of one allocation
        b = self.buf
        names = ["o", "hT", "dq", "dk", "dv", "dh0"] + [n for n in ("dg", "dbeta", "db", "dw") if getattr(b, n) is not None]
        self.out_spec = {n: (tuple(getattr(b, n).shape), getattr(b, n).dtype) for n in names}
        self.out_arena, outs, self.out_offs = _arena(self.out_spec, device)
        for n in names:
            setattr(b, n, outs[n])
        self.loaded = torch.cuda.Event()      # inputs of the slot's current step are on the device
        self.computed = torch.cuda.Event()    # its kernels are done (inputs may be overwritten)
        self.stored = torch.cuda.Event()      # its results have left the device (outputs may be overwritten)
        self.used = False

    def outputs(self) -> dict[str, Tensor]:
        return {n: getattr(self.buf, n) for n in self.out_spec}


def _packed_base(tensors: dict, spec: dict, offs: dict, bases: dict):
    """The pinned base allocation if `tensors` are exactly the views ``make_host_buffers`` handed out for this
    layout (every tensor of the layout present, each at its offset of one and the same base), else None."""
    if set(tensors) != set(spec):
        return None
    base = None
    for n, t in tensors.items():
        st = t.untyped_storage()
        b = bases.get(st.data_ptr())
        if b is None or (base is not None and b is not base):
            return None
        base = b
        if (t.storage_offset() * t.element_size() != offs[n] or tuple(t.shape) != tuple(spec[n][0])
                or t.dtype != spec[n][1] or not t.is_contiguous()):
            return None
    return base


class HostPipeline:
    """``submit(host_in, host_out)`` enqueues one forward + backward step:

    * ``host_in``: pinned host tensors ``q, k [B,L,H,K]``, ``v, do [B,L,H,V]`` (bf16), ``g`` (fp32,
      ``[B,L,H]`` or ``[B,L,H,K]``; absent for no gate), ``beta [B,L,H]`` (fp32; absent drops the delta
      term) or, for a pipeline made with ``delta=2``, the per-channel gates ``b [B,L,H,K]``, ``w [B,L,H,V]``;
      optional ``h0``, ``dhT`` ``[B,H,K,V]`` fp32.  The set of names must be the same for every step.
    * ``host_out``: pinned host tensors that receive ``o, hT, dq, dk, dv, dg, dbeta`` (``db, dw`` with
      ``delta=2``), ``dh0`` (any subset).

    A host buffer handed to ``submit`` must not be touched until ``drain()`` returns.  Steps complete
    in submission order.
    """

    def __init__(self, B: int, L: int, H: int, K: int, V: int, *, gate: int, delta: bool, has_h0: bool = False,
                 has_dhT: bool = False, scale: float | None = None, device=None, depth: int = 2):
        if not torch.cuda.is_available():
            raise ops.GdnError("lethe_gdn: HostPipeline needs a CUDA device (there is no CPU path)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.scale = float(K ** -0.5 if scale is None else scale)
        self.delta, self.gate = delta, gate
        with torch.cuda.device(self.device):
            self.slots = [_Slot(B, L, H, K, V, gate, delta, has_h0, has_dhT, self.device) for _ in range(depth)]
            self.s_in = torch.cuda.Stream()
            self.s_run = torch.cuda.Stream()
            self.s_out = torch.cuda.Stream()
            # the buffers were set up on the current stream: the three streams start after that
            ready = torch.cuda.Event()
            ready.record()
            for st in (self.s_in, self.s_run, self.s_out):
                st.wait_event(ready)
        self.n = 0
        self._host_bases = {}   # storage address -> pinned base tensor handed out by make_host_buffers
        self.pre_run = None     # optional callable enqueued on the compute stream before each step's kernels

    def make_host_buffers(self) -> tuple[dict[str, Tensor], dict[str, Tensor]]:
        """Pinned host tensors for one step's inputs and one step's outputs, laid out like the device side:
        ``submit`` moves buffers made here with ONE copy in each direction instead of one per tensor (the same
        bytes cross the host link in about three quarters of the time).  Fill the inputs, submit, read the
        outputs after ``drain()``; make several pairs to have several steps in flight."""
        s0 = self.slots[0]
        in_base, hin, _ = _arena(s0.in_spec, pinned=True)
        out_base, hout, _ = _arena(s0.out_spec, pinned=True)
        self._host_bases[in_base.untyped_storage().data_ptr()] = in_base
        self._host_bases[out_base.untyped_storage().data_ptr()] = out_base
        return hin, hout

    def submit(self, host_in: dict[str, Tensor], host_out: dict[str, Tensor]) -> int:
        slot = self.slots[self.n % len(self.slots)]
        need = set(slot.inp)
        if set(host_in) != need:
            raise ops.GdnError(f"lethe_gdn: HostPipeline expects inputs {sorted(need)}, got {sorted(host_in)}")
        outs = slot.outputs()
        for n in host_out:
            if n not in outs:
                raise ops.GdnError(f"lethe_gdn: this problem has no output {n!r}")
        i = slot.inp
        in_base = _packed_base(host_in, slot.in_spec, slot.in_offs, self._host_bases)
        out_base = _packed_base(host_out, slot.out_spec, slot.out_offs, self._host_bases)
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.s_in):
                if slot.used:
                    self.s_in.wait_event(slot.computed)
                if in_base is not None:
                    slot.in_arena.copy_(in_base, non_blocking=True)
                else:
                    for n, t in host_in.items():
                        i[n].copy_(t, non_blocking=True)
                slot.loaded.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(slot.loaded)
                if slot.used:
                    self.s_run.wait_event(slot.stored)
                if self.pre_run is not None:
                    self.pre_run()
                ops.forward_into(slot.buf, i["q"], i["k"], i["v"], i.get("g"), i.get("beta"), i.get("h0"), self.scale,
                                 b_gate=i.get("b"), w_gate=i.get("w"))
                ops.backward_into(slot.buf, i["q"], i["k"], i["v"], i.get("g"), i.get("beta"), i.get("h0"), i["do"],
                                  i.get("dhT"), self.scale, b_gate=i.get("b"), w_gate=i.get("w"))
                slot.computed.record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(slot.computed)
                if out_base is not None:
                    out_base.copy_(slot.out_arena, non_blocking=True)
                else:
                    for n, t in host_out.items():
                        t.copy_(outs[n], non_blocking=True)
                slot.stored.record(self.s_out)
        slot.used = True
        self.n += 1
        return self.n - 1

    def join(self, stream=None) -> None:
        """Make ``stream`` (default: the current stream) wait for everything submitted so far."""
        stream = torch.cuda.current_stream(self.device) if stream is None else stream
        for s in self.slots:
            if s.used:
                stream.wait_event(s.stored)

    def drain(self) -> None:
        """Wait for every submitted step and raise if a device-side wait gave up."""
        self.s_out.synchronize()
        self.s_run.synchronize()
        for s in self.slots:
            if s.used:
                ops.check_status(s.buf.status)
