"""Forward + backward for callers whose tensors live in host memory.

A training loop that keeps activations on the device calls ``ops.gdn_chunk``.  A host that feeds the
kernels from pinned host buffers and wants the results back in host buffers pays for two PCIe
transfers per step that dwarf the kernels (52 MB against 0.2 ms of kernels at B=2, H=8, L=2048).
``HostPipeline`` overlaps the three legs of consecutive steps - host-to-device copy, kernels,
device-to-host copy - on three CUDA streams with ``depth`` sets of device buffers, so that a stream of
steps runs at the pace of the slowest leg instead of the sum of the three.

Nothing here allocates per step: device buffers are made once per pipeline, and the C library never
allocates.  All calls are asynchronous; ``drain()`` waits and checks the device status words.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


class _Slot:
    def __init__(self, B, L, H, K, V, gate, delta, has_h0, has_dhT, device):
        bf, f32 = torch.bfloat16, torch.float32
        self.buf = ops.GdnBuffers(B, L, H, K, V, gate, delta, device)
        self.inp = {
            "q": torch.empty(B, L, H, K, dtype=bf, device=device),
            "k": torch.empty(B, L, H, K, dtype=bf, device=device),
            "v": torch.empty(B, L, H, V, dtype=bf, device=device),
            "do": torch.empty(B, L, H, V, dtype=bf, device=device),
        }
        if gate != ops.GATE_NONE:
            gshape = (B, L, H, K) if gate == ops.GATE_CHANNEL else (B, L, H)
            self.inp["g"] = torch.empty(gshape, dtype=f32, device=device)
        if int(delta) == 2:
            self.inp["b"] = torch.empty(B, L, H, K, dtype=f32, device=device)
            self.inp["w"] = torch.empty(B, L, H, V, dtype=f32, device=device)
        elif delta:
            self.inp["beta"] = torch.empty(B, L, H, dtype=f32, device=device)
        if has_h0:
            self.inp["h0"] = torch.empty(B, H, K, V, dtype=f32, device=device)
        if has_dhT:
            self.inp["dhT"] = torch.empty(B, H, K, V, dtype=f32, device=device)
        self.loaded = torch.cuda.Event()      # inputs of the slot's current step are on the device
        self.computed = torch.cuda.Event()    # its kernels are done (inputs may be overwritten)
        self.stored = torch.cuda.Event()      # its results have left the device (outputs may be overwritten)
        self.used = False

    def outputs(self) -> dict[str, Tensor]:
        b = self.buf
        out = {"o": b.o, "hT": b.hT, "dq": b.dq, "dk": b.dk, "dv": b.dv, "dh0": b.dh0}
        if b.dg is not None:
            out["dg"] = b.dg
        if b.dbeta is not None:
            out["dbeta"] = b.dbeta
        if b.db is not None:
            out["db"], out["dw"] = b.db, b.dw
        return out


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
        self.pre_run = None     # optional callable enqueued on the compute stream before each step's kernels

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
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.s_in):
                if slot.used:
                    self.s_in.wait_event(slot.computed)
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
