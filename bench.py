#!/usr/bin/env python
"""Benchmark of the chunked gated-delta-rule training step (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one forward + backward of the op over one batch of seeded synthetic inputs.  Per GPU the
workload is the configuration the metric is quoted on: scalar-gate gated delta rule, B=2, H=8,
L=2048, d_k=128, d_v=64, chunk 64, bf16 inputs, initial state.  With N > 1 every rank runs that
workload on its own (batch x head) shard -- the path shards without communication -- so scaling is
"weak" and `value` is the whole job's tokens (B*L per rank) per second.

Prints ONE JSON line (rank 0).  `value`: inputs resident in HBM, the step as the CUDA-graph replay of
`lethe_b200.ops.GdnStepGraph` (`eager_ms_per_step`: the same kernels launched one by one from the host,
`autograd_op_ms`: through `ops.gdn_chunk` + autograd), CUDA events around every step, L2 flushed between
steps, max over ranks.  `e2e`: the same step through `lethe_b200.host.HostPipeline`, the public call for
tensors in host memory: pinned host buffers, host->device copies of all inputs and device->host copies of
all results inside the timed region, consecutive steps overlapped; `e2e.host_link` is the host link measured
in the same process with every rank copying at once, and `host_link_floor_ms` the time those bytes need on
it.  `roofline`: the dominant kernel,
timed alone with CUDA events, plus the whole step against the algorithmic bytes and FLOPs of the path
(HBM and tensor-core fractions for forward, backward and both).  `cpu_baseline`: the reference project's
own PyTorch CPU chunkwise path (its backward assembly, imported from `oracle/_ref`, the reference compiled
to bytecode) timed on this machine's host cores on a bounded sample; the CPU oracle port stands in only
where `oracle/_ref` is absent.  `--impl reference` times that CPU path only (rank 0; other ranks exit):
W warm-up passes, then K timed passes, every pass really executed.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, L, H, K, V, gate, delta)
    "gdn_scalar_B2_H8_L2048_dk128_dv64": (2, 2048, 8, 128, 64, "scalar", True),
    "gdn_scalar_B2_H8_L2048_dk128_dv128": (2, 2048, 8, 128, 128, "scalar", True),
    "gdn_scalar_B4_H8_L4096_dk128_dv64": (4, 4096, 8, 128, 64, "scalar", True),     # > L2: for ncu DRAM figures
    "kda_B2_H8_L2048_dk128_dv128": (2, 2048, 8, 128, 128, "channel", True),          # configuration 2
    # the reference's full six-input op: independent per-channel erase gate b and write gate w (delta = 2)
    "gdn2full_B2_H8_L2048_dk128_dv128": (2, 2048, 8, 128, 128, "channel", 2),
    "gla_B4_H16_L4096_dk128_dv128": (4, 4096, 16, 128, 128, "channel", False),       # configuration 3
    "kda_B4_H8_L4096_dk128_dv128": (4, 4096, 8, 128, 128, "channel", True),          # > L2: for ncu DRAM figures
    "kda_B2_H32_L8192_dk128_dv128": (2, 8192, 32, 128, 128, "channel", True),        # configuration 4a, one GPU's share
    "kda_B1_H32_L65536_dk128_dv128": (1, 65536, 32, 128, 128, "channel", True),      # configuration 4b (use --sp)
    "ssd_B4_H16_L4096_dk128_dv128": (4, 4096, 16, 128, 128, "scalar", False),
    "la_B4_H16_L4096_dk128_dv128": (4, 4096, 16, 128, 128, "none", False),
}
DEFAULT = "gdn_scalar_B2_H8_L2048_dk128_dv64"
METRIC = "GDN fwd+bwd tokens/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": reasons}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own PyTorch CPU chunkwise path
# ------------------------------------------------------------------------------------------------
CPU_TOKEN_HEADS = {"scalar": 32768, "none": 32768, "channel": 8192}     # bounded sample, by gate kind


def cpu_sample_shape(workload: str):
    """(B_s, H_s) of the bounded CPU sample: whole (batch, head) pairs of the workload, as many as fit the
    token-head budget (the headline configuration fits whole).  Pairs are independent recurrences, so the
    sample's time scales linearly to the full workload."""
    B, L, H, K, V, gate, delta = WORKLOADS[workload]
    pairs = max(1, min(B * H, CPU_TOKEN_HEADS[gate] // L))
    Hs = min(H, pairs)
    Bs = max(1, min(B, pairs // Hs))
    return Bs, Hs


def cpu_reference_pass(workload: str):
    """Returns (run, kind, what): `run()` executes one forward + backward of the workload's bounded
    sample on the host cores through the reference's own code (kind "reference") or, when `oracle/_ref` is
    absent, through the CPU oracle port (kind "port")."""
    from lethe_b200.synth import make_inputs

    B, L, H, K, V, gate, delta = WORKLOADS[workload]
    Bs, Hs = cpu_sample_shape(workload)
    # all the host threads this process may use (a torchrun launch exports OMP_NUM_THREADS=1, which would
    # otherwise pin the CPU arm to one core)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    inp = make_inputs(Bs, L, Hs, K, V, gate=gate, delta=bool(delta), seed=0, full=(delta == 2))
    f = {k: (None if t is None else t.float()) for k, t in inp.items()}
    scale = K ** -0.5
    from oracle import make_ref
    if make_ref.import_reference() is not None:
        from lethe.kernels.cute import gdn2_assemble as A
        from lethe.kernels.cute import gdn2_family as F
        kw = dict(scale=scale, use_qk_l2norm=False)
        if delta == 2:
            fn, what = (lambda: A.assemble_gdn2_backward_channelwise(f["q"], f["k"], f["v"], f["g"], f["b"], f["w"],
                                                                     f["do"], **kw)), "assemble_gdn2_backward_channelwise"
        elif delta and gate == "scalar":
            fn, what = (lambda: A.assemble_gdn2_backward_scalar(f["q"], f["k"], f["v"], f["g"], f["beta"], f["do"],
                                                                **kw)), "assemble_gdn2_backward_scalar"
        elif delta:
            fn, what = (lambda: F.kda_backward(f["q"], f["k"], f["v"], f["g"], f["beta"], f["do"], **kw)), "kda_backward"
        elif gate == "channel":
            fn, what = (lambda: F.gla_backward(f["q"], f["k"], f["v"], f["g"], f["do"], **kw)), "gla_backward"
        elif gate == "scalar":
            fn, what = (lambda: F.ssd_backward(f["q"], f["k"], f["v"], f["g"], f["do"], **kw)), "ssd_backward"
        else:
            fn, what = (lambda: F.la_backward(f["q"], f["k"], f["v"], f["do"], **kw)), "la_backward"
        return fn, "reference", (f"the reference's own {what} (chunkwise forward + backward assembly, fp32, no "
                                 "kernels injected, no initial state: its signature has none)")
    from oracle.gdn_oracle import chunk_fwd_bwd
    beta = f.get("beta")
    return (lambda: chunk_fwd_bwd(f["q"], f["k"], f["v"], f["g"], beta, f["h0"], f["do"], scale=scale),
            "port", "oracle.chunk_fwd_bwd (CPU port of the reference's chunkwise path; oracle/_ref absent)")


def cpu_time_passes(workload: str, steps: int, warmup: int, budget_s: float | None = None):
    """Runs `warmup` + up to `steps` passes (stopping early once `budget_s` of timed work is spent, never
    before two).  Returns the cpu_baseline object and the per-pass seconds."""
    B, L, H, K, V, gate, delta = WORKLOADS[workload]
    Bs, Hs = cpu_sample_shape(workload)
    run, kind, what = cpu_reference_pass(workload)
    for _ in range(max(1, warmup)):
        run()
    ts = []
    while len(ts) < steps and (budget_s is None or len(ts) < 2 or sum(ts) < budget_s):
        t0 = time.perf_counter()
        run()
        ts.append(time.perf_counter() - t0)
    t1 = sum(ts) / len(ts)                      # seconds per pass over Bs x Hs pairs
    frac = (Bs * Hs) / (B * H)
    tokens_per_s = (B * L) * frac / t1          # a token spans all H heads; pairs scale linearly
    cb = {"value": tokens_per_s, "unit": "tokens/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
          "kind": kind, "passes": len(ts), "s_per_pass": t1, "sample_fraction": frac,
          "sample": f"{what} on B={Bs}, H={Hs}, L={L} of {workload} ({100 * frac:.0f} % of its (batch, head) pairs"
                    f"{', scaled linearly to all of them' if frac < 1 else ''}); mean of {len(ts)} passes of "
                    f"{t1:.2f} s after {max(1, warmup)} warm-up"}
    return cb, ts


def cpu_baseline(workload: str, budget_s: float = 12.0):
    return cpu_time_passes(workload, steps=10, warmup=1, budget_s=budget_s)[0]


# ------------------------------------------------------------------------------------------------
# Algorithmic work of the path (what a perfectly fused implementation must move and compute)
# ------------------------------------------------------------------------------------------------
# Whole-configuration figures for forward + backward, (GFLOP, MB), for the benchmark configurations:
# dense 2mnk counting per 64-token chunk, every tensor touched once per pass, fp32 chunk-entry state
# written by the forward and read by the backward.  Other workloads use the same formulas (path_model).
PATH_TABLE = {
    "gdn_scalar_B2_H8_L2048_dk128_dv64": (11.86, 105.3),
    "kda_B2_H8_L2048_dk128_dv128": (18.30, 184.7),
    "gla_B4_H16_L4096_dk128_dv128": (77.31, 1476.0),
    "ssd_B4_H16_L4096_dk128_dv128": (77.31, 1476.0),
    "la_B4_H16_L4096_dk128_dv128": (77.31, 1476.0),
    "kda_B2_H32_L8192_dk128_dv128": (2342.0 / 8, 23648.0 / 8),
    "kda_B1_H32_L65536_dk128_dv128": (1171.0, 11824.0),
}


def path_model(workload: str):
    """Algorithmic FLOPs and bytes of forward and backward for a workload: {"fwd": (flop, bytes), "bwd": ...,
    "source": ...}.  Per chunk (C = 64): with the delta term forward 6C^2K + 4C^2V + 6CKV + C^3/3, backward
    12C^2K + 8C^2V + 12CKV + 4C^3; without it 2C^2K + 2C^2V + 4CKV and 4C^2K + 4C^2V + 8CKV.  Per token-head:
    forward 2(2K+V) + 2V + gate bytes, backward 2(2K+V) + 2V + gate bytes + 2(2K+V) + gate-gradient bytes;
    state 2 * 4KV / C.  Configurations listed in PATH_TABLE use its totals, split forward / backward in the
    formulas' proportion."""
    B, L, H, K, V, gate, delta = WORKLOADS[workload]
    C = 64
    Z, TH = B * H * (L // C), B * H * L
    if delta:
        ff = 6 * C * C * K + 4 * C * C * V + 6 * C * K * V + C ** 3 / 3
        fb = 12 * C * C * K + 8 * C * C * V + 12 * C * K * V + 4 * C ** 3
    else:
        ff = 2 * C * C * K + 2 * C * C * V + 4 * C * K * V
        fb = 4 * C * C * K + 4 * C * C * V + 8 * C * K * V
    gbytes = {"none": 0, "scalar": 4, "channel": 4 * K}[gate] + (4 if delta == 1 else (4 * (K + V) if delta == 2 else 0))
    state = 4 * K * V / C
    bf = 2 * (2 * K + V) + 2 * V + gbytes + state
    bb = 2 * (2 * K + V) + 2 * V + gbytes + 2 * (2 * K + V) + gbytes + state
    fwd, bwd, src = (ff * Z, bf * TH), (fb * Z, bb * TH), "formulas"
    if workload in PATH_TABLE:
        gf, mb = PATH_TABLE[workload]
        sf, sb_ = gf * 1e9 / (fwd[0] + bwd[0]), mb * 1e6 / (fwd[1] + bwd[1])
        fwd, bwd, src = (fwd[0] * sf, fwd[1] * sb_), (bwd[0] * sf, bwd[1] * sb_), "configuration table"
    return {"fwd": fwd, "bwd": bwd, "source": src}


def path_fractions(workload: str, fwd_ms: float, bwd_ms: float, step_ms: float, hbm: float, tf: float):
    """HBM and tensor-core fractions of forward, backward and the whole step on the algorithmic counts."""
    m = path_model(workload)
    out = {"source": m["source"], "tensor_peak_tflops": tf}
    for name, (flop, byt), ms in (("fwd", m["fwd"], fwd_ms), ("bwd", m["bwd"], bwd_ms),
                                  ("step", (m["fwd"][0] + m["bwd"][0], m["fwd"][1] + m["bwd"][1]), step_ms)):
        out[name] = {"MB": byt / 1e6, "GFLOP": flop / 1e9, "ms": ms,
                     "hbm_frac": byt / (ms * 1e-3) / 1e9 / hbm, "tensor_frac": flop / (ms * 1e-3) / 1e12 / tf}
    return out


# ------------------------------------------------------------------------------------------------
# DRAM traffic per chunk (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture / chunks of that
# launch), from the captures summarised under profiles/ (2048- and 4096-chunk workloads, records larger than L2;
# every kernel's traffic grows in proportion to its chunks).  Keyed by (kernel, gate, d_v, delta); the
# channel-wise "stageb" and "wy" are two launches each, summed.  Absent combinations report null.
NCU_DRAM_BYTES_PER_CHUNK = {
    # scalar-gate GDN, B4 H8 L4096 d_v 64 (2048 chunks)
    ("prepare", "scalar", 64, True): (85.0e6 + 127.6e6) / 2048,
    ("scan_fwd", "scalar", 64, True): (102.8e6 + 14.0e6) / 2048,
    ("output", "scalar", 64, True): (151.5e6 + 18.1e6) / 2048,
    ("bwd_pre", "scalar", 64, True): (118.0e6 + 14.1e6) / 2048,
    ("scan_bwd", "scalar", 64, True): (101.7e6 + 14.0e6) / 2048,
    ("stageb", "scalar", 64, True): (185.1e6 + 104.6e6) / 2048,
    ("wy", "scalar", 64, True): (203.0e6 + 35.3e6) / 2048,
    # KDA, B4 H8 L4096 d_v 128 (2048 chunks)
    ("prepare", "channel", 128, True): (168.5e6 + 279.2e6) / 2048,
    ("scan_fwd", "channel", 128, True): (137.4e6 + 38.2e6) / 2048,
    ("output", "channel", 128, True): (201.4e6 + 43.8e6) / 2048,
    ("bwd_pre", "channel", 128, True): (134.2e6 + 36.5e6) / 2048,
    ("scan_bwd", "channel", 128, True): (135.3e6 + 37.6e6) / 2048,
    ("stageb", "channel", 128, True): (369.2e6 + 240.3e6 + 352.4e6 + 129.5e6) / 2048,
    ("wy", "channel", 128, True): (235.5e6 + 87.9e6 + 319.9e6 + 81.0e6) / 2048,
    # GLA, B4 H16 L4096 d_v 128 (4096 chunks)
    ("prepare", "channel", 128, False): (335.6e6 + 418.7e6) / 4096,
    ("scan_fwd", "channel", 128, False): (141.0e6 + 93.5e6) / 4096,
    ("output", "channel", 128, False): (335.6e6 + 105.7e6) / 4096,
    ("bwd_pre", "channel", 128, False): (134.2e6 + 89.7e6) / 4096,
    ("scan_bwd", "channel", 128, False): (136.4e6 + 90.6e6) / 4096,
    ("stageb", "channel", 128, False): (738.3e6 + 460.8e6 + 704.7e6 + 244.6e6) / 4096,
    # SSD, B4 H16 L4096 d_v 128 (4096 chunks)
    ("prepare", "scalar", 128, False): (202.5e6 + 217.3e6) / 4096,
    ("scan_fwd", "scalar", 128, False): (141.0e6 + 92.5e6) / 4096,
    ("output", "scalar", 128, False): (336.6e6 + 106.5e6) / 4096,
    ("bwd_pre", "scalar", 128, False): (135.3e6 + 90.4e6) / 4096,
    ("scan_bwd", "scalar", 128, False): (136.4e6 + 91.0e6) / 4096,
    ("stageb", "scalar", 128, False): (571.6e6 + 179.6e6) / 4096,
    # LA, B4 H16 L4096 d_v 128 (4096 chunks)
    ("prepare", "none", 128, False): (201.4e6 + 216.9e6) / 4096,
    ("scan_fwd", "none", 128, False): (141.0e6 + 93.0e6) / 4096,
    ("output", "none", 128, False): (335.6e6 + 105.9e6) / 4096,
    ("bwd_pre", "none", 128, False): (134.2e6 + 90.8e6) / 4096,
    ("scan_bwd", "none", 128, False): (136.4e6 + 89.7e6) / 4096,
    ("stageb", "none", 128, False): (570.5e6 + 178.0e6) / 4096,
}


def measured_traffic(kernel: str, gate: str, V: int, delta: bool, Z: int):
    per = NCU_DRAM_BYTES_PER_CHUNK.get((kernel, gate, V, delta))
    return None if per is None else int(per * Z)


# ------------------------------------------------------------------------------------------------
def algorithmic_bytes(kernel: str, Z: int, BH: int, V: int, delta: bool, cw: bool = False) -> int:
    """Bytes one launch of `kernel` must move: each input tile and each record read once, each
    result written once (Z chunks, 64 tokens each; K = 128).  With the channel-wise gate "prepare" also
    writes the chunk's 32 KB tile of cumulative gate values and the 16 KB record of the scaled, decayed
    query (which "output" and "bwd_pre" read in place of q), the Stage B and WY kernels read the gate
    tile, and "stageb" and "wy" are two launches each that pass three fp32 64 x 128 records (dq / dk / dg
    parts) between them."""
    qk, vv, img = 64 * 128 * 2, 64 * V * 2, 128 * V * 2
    ta, w, p_, r, f32k = 16384, 16384, 32768, 128 * V * 2, 64 * 128 * 4
    if cw:
        g = f32k
        per = {
            "prepare": g + 2 * qk + vv + g + qk + ta + vv + r + ((w + p_) if delta else 0) + 512,
            "scan_fwd": (p_ if delta else 0) + r + img + 512,
            "output": qk + ta + img + vv + vv + vv + (w if delta else 0),
            "bwd_pre": qk + vv + r + ((w + ta) if delta else 0),
            "scan_bwd": (p_ if delta else 0) + r + img + 512,
            "stageb": (g + 2 * qk + vv + ta + vv + 2 * img + 8192 + 3 * f32k + (vv + w if delta else vv))
                      + (g + 2 * qk + 8192 + 3 * f32k + qk + (2 * f32k if delta else qk + f32k)),
            "wy": (g + qk + vv + ta + vv + w + 8192 + f32k + vv) + (g + qk + 8192 + 3 * f32k + qk + f32k),
        }[kernel]
        return per * Z
    per = {
        "prepare": 2 * qk + vv + ta + vv + r + ((w + p_) if delta else 0) + 512,
        "scan_fwd": (p_ if delta else 0) + r + img + 512,
        "output": qk + ta + img + vv + vv + vv + (w if delta else 0),
        "bwd_pre": qk + vv + r + ((w + ta) if delta else 0),
        "scan_bwd": (p_ if delta else 0) + r + img + 512,
        "stageb": 2 * qk + vv + ta + vv + 2 * img + qk + (vv + w + f32k if delta else qk + vv),
        "wy": qk + vv + ta + vv + w + f32k + qk + vv,
    }[kernel]
    return per * Z


def io_bytes(kernel: str, Z: int, V: int, delta, gate: str) -> int:
    """The part of `algorithmic_bytes` that the path itself requires whatever the kernel decomposition: the
    first read of each user tensor in a pass, the final outputs, and the chunk-entry state (written once by
    the forward scan, read once by Stage B).  The rest of a kernel's bytes are records the kernels hand to
    one another and re-reads of inputs - traffic this design chose, not traffic the path needs."""
    qk, vv, img = 64 * 128 * 2, 64 * V * 2, 128 * V * 2
    gin = {"none": 0, "scalar": 64 * 4, "channel": 64 * 128 * 4}[gate]      # gate values of a chunk
    bin_ = 64 * 4 if delta == 1 else (64 * (128 + V) * 4 if delta == 2 else 0)
    per = {
        "prepare": 2 * qk + vv + gin + bin_,                       # q, k, v, g, beta
        "scan_fwd": img,                                           # state entering every chunk
        "output": vv,                                              # o
        "bwd_pre": qk + vv,                                        # q, do (first touch of the backward)
        "scan_bwd": 0,
        # k, state; dq; without the delta term also dk, dv, dg
        "stageb": qk + img + qk + ((qk + vv + gin) if not delta else 0),
        "wy": vv + qk + vv + gin + bin_,                           # v; dk, dv, dg, dbeta
    }[kernel]
    return per * Z


def pcie_probe(dev, world, mbytes: int = 128, reps: int = 4):
    """Host link of this rank while every rank uses its own at the same time: GB/s of pinned-host -> device
    copies, of device -> pinned-host copies, and of both at once (what the end-to-end pipeline does).  Returns
    the slowest rank's figures and the sum over the ranks - the host's aggregate, which is what bounds the
    end-to-end number when several GPUs of one host copy together."""
    import torch.distributed as dist
    n = mbytes << 20
    hbuf = torch.empty(n, dtype=torch.uint8).pin_memory()
    hbuf2 = torch.empty(n, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(n, dtype=torch.uint8, device=dev)
    dbuf2 = torch.empty(n, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def run(which):
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        s1.wait_event(a)
        s2.wait_event(a)
        for _ in range(reps):
            if which in ("h2d", "both"):
                with torch.cuda.stream(s1):
                    dbuf.copy_(hbuf, non_blocking=True)
            if which in ("d2h", "both"):
                with torch.cuda.stream(s2):
                    hbuf2.copy_(dbuf2, non_blocking=True)
        torch.cuda.current_stream(dev).wait_stream(s1)
        torch.cuda.current_stream(dev).wait_stream(s2)
        b.record()
        torch.cuda.synchronize(dev)
        return reps * n / (a.elapsed_time(b) * 1e-3) / 1e9        # GB/s per direction

    run("both")                                                     # warm
    out = {}
    for which in ("h2d", "d2h", "both"):
        g = torch.tensor([run(which)], device=dev, dtype=torch.float64)
        lo, tot = g.clone(), g.clone()
        if world > 1:
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        out[which] = {"slowest_rank_gbs": float(lo), "all_ranks_gbs": float(tot)}
    out["note"] = (f"{mbytes} MiB pinned copies, all {world} ranks at once; 'both' is GB/s per direction with the two "
                   "directions running together")
    return out


def aux_main(args):
    """Timing of the two kernels on either side of the path that the step does not contain: the L2
    normalisation of q, k with its VJP (one launch each way) and the one-token decode step.  Both are
    HBM-bound element-wise kernels; the line reports achieved GB/s against the measured copy bandwidth."""
    from lethe_b200 import ops
    dev = torch.device("cuda", 0)
    hbm = peaks()[0]
    B, L, H, K, V = 2, 8192, 32, 128, 128            # the q, k of one GPU's share of configuration 4a
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(B, L, H, K, generator=gen).bfloat16().to(dev)
    k = torch.randn(B, L, H, K, generator=gen).bfloat16().to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in evs:
            flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / n

    qn, kn = ops.l2norm_qk_raw(q, k)
    rows = q.numel() // K
    t_f = timed(lambda: ops.l2norm_qk_raw(q, k))
    t_b = timed(lambda: ops.l2norm_qk_vjp_raw(q, k, qn, kn))
    by_f, by_b = 2 * rows * K * (2 + 2), 2 * rows * K * (2 + 2 + 2)          # q and k: read x (+ dy), write y / dx
    Bd, Hd = 64, 32
    state = torch.randn(Bd, Hd, K, V, generator=gen).to(dev)
    q1 = torch.randn(Bd, Hd, K, generator=gen).bfloat16().to(dev)
    v1 = torch.randn(Bd, Hd, V, generator=gen).bfloat16().to(dev)
    g1 = -torch.rand(Bd, Hd, generator=gen).to(dev)
    b1 = torch.rand(Bd, Hd, generator=gen).to(dev)
    t_d = timed(lambda: ops.gdn_decode_step(q1, q1, v1, g1, b1, state))
    by_d = 2 * state.numel() * 4                                                # the state is read and written once
    out = {"impl": "aux", "l2norm_qk": {"ms": t_f, "GB/s": by_f / t_f / 1e6, "frac_of_hbm": by_f / t_f / 1e6 / hbm,
                                        "rows_per_tensor": rows},
           "l2norm_qk_vjp": {"ms": t_b, "GB/s": by_b / t_b / 1e6, "frac_of_hbm": by_b / t_b / 1e6 / hbm},
           "decode_step": {"ms": t_d, "GB/s": by_d / t_d / 1e6, "frac_of_hbm": by_d / t_d / 1e6 / hbm,
                           "B": Bd, "H": Hd, "state_MB": by_d / 2e6},
           "peak_gbs": hbm, "l2": "flushed between launches (256 MiB write)"}
    print(json.dumps(out))


def fla_main(args, B, L, H, K, V, gate, delta, config):
    """Extra comparator row, not the reference arm and not part of this package: the flash-linear-attention
    Triton kernels (a third-party library the reference itself times against) on the same workload, same
    seeded inputs resident on the device, forward + backward, CUDA events, L2 flushed between steps.
    Only the two delta-rule workloads have a counterpart there."""
    import torch
    from lethe_b200.synth import make_inputs
    try:
        from fla.ops.kda import chunk_kda
    except Exception as e:   # noqa: BLE001
        print(json.dumps({"impl": "fla", "unavailable": f"cannot import flash-linear-attention: {e}"}))
        return
    if not delta or gate == "none":
        print(json.dumps({"impl": "fla", "unavailable": "no counterpart for this workload"}))
        return
    if gate == "scalar":
        # chunk_gated_delta_rule of this library version ended in a CUDA error on a B200 of this pool with
        # these inputs; it is not run again (the channel-wise comparator below ran cleanly)
        print(json.dumps({"impl": "fla", "unavailable": "the library's scalar-gate kernels raised a CUDA error "
                                                        "on this hardware; not run"}))
        return
    dev = torch.device("cuda", 0)
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=1, mild=args.mild_gate)
    leaves = {n: inp[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")}
    do = inp["do"].to(dev)
    fn = chunk_kda
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        o, _ = fn(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], scale=K ** -0.5,
                  initial_state=leaves["h0"], output_final_state=True)
        torch.autograd.grad(o, list(leaves.values()), do)

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in evs:
        flush.zero_()
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    import fla
    print(json.dumps({"impl": "fla", "library": f"flash-linear-attention {fla.__version__} (Triton)", "metric": METRIC,
                      "value": B * L / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "config": config,
                      "data": "synthetic", "note": "through autograd (includes its Python launch overhead)"}))


def sp_main(args, rank, world, dev, B, L, H, K, V, gate, delta, config):
    """Sequence-parallel timing: rank r owns tokens [r L/N, (r+1) L/N) of every head; chunk-boundary
    states (forward) and adjoint states (backward) travel rank to rank by NCCL point-to-point."""
    import torch.distributed as dist
    from lethe_b200 import ops
    from lethe_b200.parallel import SequenceParallelGdn
    from lethe_b200.synth import make_inputs

    if world == 1:
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1, device_id=dev)
    Ll = L // world
    inp = make_inputs(B, Ll, H, K, V, gate=gate, delta=delta, seed=1 + rank, with_h0=(rank == 0))
    d = {k: t.to(dev) for k, t in inp.items() if t is not None}
    gate_code = {"none": 0, "scalar": 1, "channel": 2}[gate]
    sp = SequenceParallelGdn(B, Ll, H, K, V, gate_code, delta, dev)
    scale = K ** -0.5

    def step():
        sp.forward(d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), d.get("h0"), scale)
        sp.backward(d["do"], None)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ops.check_status(sp.buf.status)
    if rank == 0:
        config = dict(config, mode="sequence parallel", L_per_gpu=Ll, l2="inputs and records exceed L2")
        hbm, _tfb, tfs, _which = peaks()
        m = path_model(args.workload)
        byt, flop = m["fwd"][1] + m["bwd"][1], m["fwd"][0] + m["bwd"][0]
        print(json.dumps({"metric": METRIC, "value": B * L / (float(ms) * 1e-3), "unit": "tokens/s",
                          "hbm_frac": byt / (float(ms) * 1e-3) / 1e9 / (hbm * world),
                          "tensor_frac": flop / (float(ms) * 1e-3) / 1e12 / (tfs * world),
                          "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                          "ms_per_step": float(ms), "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulate (bf16 in/out)",
                          "data": "synthetic", "config": config,
                          "gpu_launches": args.steps * (9 if gate == "channel" and delta else 7)}))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "fla", "aux"],
                    help="reference: the reference's own CPU path (oracle/_ref) or its CPU port; fla: third-party "
                         "comparator (see fla_main); aux: the L2-normalisation and decode-step kernels")
    ap.add_argument("--groups", type=int, default=1,
                    help="cut the (batch, head) pairs into this many ranges that run as concurrent kernel chains "
                         "inside the step graph (helps when the scans leave SMs idle: a few % on the larger workloads)")
    ap.add_argument("--cut", type=int, default=-1,
                    help="chunk index at which the step graph cuts every sequence into an early and a late segment "
                         "(0: no cut; -1: the library's default, about half of the chunks on a whole number of CTA waves)")
    ap.add_argument("--bwd-cuts", default="",
                    help="comma-separated chunk indices at which the backward of the step graph is cut (default: the "
                         "forward's cut)")
    ap.add_argument("--plain-chain", action="store_true",
                    help="capture the step as one chain of kernels on one stream (no overlap inside the graph)")
    ap.add_argument("--mild-gate", action="store_true",
                    help="draw the gate as -0.1 U(0,1), the draw of the reference's own benchmark, instead of "
                         "-softplus(N(0,1) + 3)")
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sp", action="store_true",
                    help="sequence parallel: the workload's L is split over the ranks (strong scaling)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    B, L, H, K, V, gate, delta = WORKLOADS[args.workload]
    config = {"workload": args.workload, "B_per_gpu": B, "H": H, "L": L, "d_k": K, "d_v": V, "chunk": 64,
              "gate": gate, "delta": delta, "sharding": "batch x head, no collective",
              "l2": "flushed between steps (256 MiB write)"}

    if args.impl == "fla":
        if rank == 0:
            fla_main(args, B, L, H, K, V, gate, delta, config)
        return
    if args.impl == "aux":
        if rank == 0:
            aux_main(args)
        return
    if args.impl == "reference":
        if rank != 0:
            return
        t_run = time.perf_counter()
        cb, ts = cpu_time_passes(args.workload, steps=args.steps, warmup=args.warmup)
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": len(ts), "warmup": max(1, args.warmup),
                "ms_per_step": 1e3 * cb["s_per_pass"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "config": config,
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "wall_s": time.perf_counter() - t_run,
                "note": "every step is one executed pass of the CPU sample described in cpu_baseline.sample; "
                        "ms_per_step is the measured time of such a pass, value scales it to the whole workload "
                        "by cpu_baseline.sample_fraction"}
        print(json.dumps(line))
        return

    import torch.distributed as dist
    from lethe_b200 import ops
    from lethe_b200.synth import make_inputs

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.sp:
        sp_main(args, rank, world, dev, B, L, H, K, V, gate, delta, config)
        return
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=bool(delta), seed=1 + rank, mild=args.mild_gate,
                      full=(delta == 2))
    host = {k: t.pin_memory() for k, t in inp.items() if t is not None}
    d = {k: t.to(dev) for k, t in host.items()}
    g, beta, h0 = d.get("g"), d.get("beta"), d.get("h0")
    scale = K ** -0.5
    gate_code = {"none": 0, "scalar": 1, "channel": 2}[gate]
    buf = ops.GdnBuffers(B, L, H, K, V, gate_code, delta, dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    gates = dict(b_gate=d.get("b"), w_gate=d.get("w"))     # per-channel gates of the full op, else None

    def step(mask_f=0, mask_b=0):
        ops.forward_into(buf, d["q"], d["k"], d["v"], g, beta, h0, scale, mask_f, **gates)
        ops.backward_into(buf, d["q"], d["k"], d["v"], g, beta, h0, d["do"], None, scale, mask_b, **gates)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            flush.zero_()
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        barrier()
        for a, b in evs:
            flush.zero_()
            a.record()
            fn()
            b.record()
        barrier()
        return sum(a.elapsed_time(b) for a, b in evs) / steps     # ms per step

    # the clock sampler runs over the whole measured part of the program (timed steps, per-kernel
    # timing and the end-to-end leg): the timed steps alone last only a few milliseconds
    sampler = ClockSampler(local)
    sampler.start()
    # the timed step is the CUDA-graph replay of forward + backward (ops.GdnStepGraph: the public call for a
    # training step at fixed shapes); the per-kernel and fwd / bwd timings below are plain launches
    graph = ops.GdnStepGraph(buf, d["q"], d["k"], d["v"], g, beta, h0, d["do"], None, scale, groups=args.groups,
                             pipeline=not args.plain_chain, cut=None if args.cut < 0 else args.cut,
                             bwd_cuts=[int(x) for x in args.bwd_cuts.split(",")] if args.bwd_cuts else None, **gates)
    ms = timed(graph.replay, args.steps, max(args.warmup, 3))
    ops.check_status(buf.status)
    eager_ms = timed(step, args.steps, 3)

    # ---- per-kernel timing (each kernel alone, same records in place), for the roofline
    kern = {}
    names_f = [("prepare", 1), ("scan_fwd", 2), ("output", 4)]
    names_b = [("bwd_pre", 1), ("scan_bwd", 2), ("stageb", 4)] + ([("wy", 8)] if delta else [])
    step()
    for name, m in names_f:
        kern[name] = timed(lambda m=m: ops.forward_into(buf, d["q"], d["k"], d["v"], g, beta, h0, scale, m, **gates),
                           max(args.steps, 10), 3)
    for name, m in names_b:
        kern[name] = timed(lambda m=m: ops.backward_into(buf, d["q"], d["k"], d["v"], g, beta, h0, d["do"],
                                                         None, scale, m, **gates), max(args.steps, 10), 3)
    fwd_ms = timed(lambda: ops.forward_into(buf, d["q"], d["k"], d["v"], g, beta, h0, scale, **gates), args.steps, 3)
    bwd_ms = timed(lambda: ops.backward_into(buf, d["q"], d["k"], d["v"], g, beta, h0, d["do"], None, scale,
                                             **gates), args.steps, 3)

    ops.check_status(buf.status)

    # ---- end to end through the public host API: pinned host buffers in, pinned host buffers out, every
    # step's copies inside the timed region.  Consecutive steps overlap their copy-in, kernels and
    # copy-out on three streams (two sets of device buffers, together larger than L2; the L2 flush
    # runs on the compute stream inside the timed region).
    from lethe_b200.host import HostPipeline
    pipe = HostPipeline(B, L, H, K, V, gate=gate_code, delta=delta, has_h0="h0" in host, scale=scale)
    pipe.pre_run = flush.zero_
    # pinned host buffers in the pipeline's own layout (one copy per direction and step), filled once
    host_in, outs_host = pipe.make_host_buffers()
    for n in host_in:
        host_in[n].copy_(host[n])

    def e2e_run(steps):
        for _ in range(steps):
            pipe.submit(host_in, outs_host)
        pipe.join()

    # The host link is shared with whatever else runs on the machine, and a run of a few tens of milliseconds
    # catches its moods: three runs of the K steps, the median is reported (all three are in the line).
    e2e_steps = max(6, args.steps)
    e2e_run(3)
    pipe.drain()
    e2e_runs = []
    for _ in range(3):
        barrier()
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        e2e_run(e2e_steps)
        eb.record()
        barrier()
        pipe.drain()
        e2e_runs.append(ea.elapsed_time(eb) / e2e_steps)
    e2e_ms = sorted(e2e_runs)[1]

    # one step alone through the autograd op (copy in, forward, backward, copy out, nothing overlapped)
    single_host = {}

    def e2e_single():
        leaves = {}
        for n in ("q", "k", "v", "g", "beta", "h0"):
            leaves[n] = host[n].to(dev, non_blocking=True).requires_grad_(True) if n in host else None
        do_d = host["do"].to(dev, non_blocking=True)
        if delta == 2:
            for n in ("b", "w"):
                leaves[n] = host[n].to(dev, non_blocking=True).requires_grad_(True)
            o, hT = ops.gdn_chunk_full(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["b"], leaves["w"],
                                       leaves["h0"], scale=scale)
        else:
            o, hT = ops.gdn_chunk(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], leaves["h0"],
                                  scale=scale)
        names = [n for n in leaves if leaves[n] is not None]
        grads = torch.autograd.grad(o, [leaves[n] for n in names], do_d)
        res = [("o", o.detach()), ("hT", hT.detach())] + [("d" + n, t) for n, t in zip(names, grads)]
        for n, t in res:
            if n not in single_host:
                single_host[n] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            single_host[n].copy_(t, non_blocking=True)

    e2e_single_ms = timed(e2e_single, 3, 3)
    pcie = pcie_probe(dev, world)

    # the call a training loop makes: the autograd op on tensors that already live on the device
    dev_leaves = {n: (d[n].clone().requires_grad_(True) if n in d else None) for n in ("q", "k", "v", "g", "beta", "h0")}
    if delta == 2:
        dev_leaves.update({n: d[n].clone().requires_grad_(True) for n in ("b", "w")})

    def op_step():
        L_ = dev_leaves
        if delta == 2:
            o, _ = ops.gdn_chunk_full(L_["q"], L_["k"], L_["v"], L_["g"], L_["b"], L_["w"], L_["h0"], scale=scale)
        else:
            o, _ = ops.gdn_chunk(L_["q"], L_["k"], L_["v"], L_["g"], L_["beta"], L_["h0"], scale=scale)
        torch.autograd.grad(o, [t for t in L_.values() if t is not None], d["do"])

    op_ms = timed(op_step, max(args.steps, 10), 3)
    clocks = sampler.stop()
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in outs_host.values())

    vals = torch.tensor([ms, e2e_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, e2e_ms, fwd_ms, bwd_ms = (float(x) for x in vals.tolist())
    tokens = B * L * world

    if rank == 0:
        hbm, tf_burst, tf_sustained, which = peaks()
        Z, BH = B * H * (L // 64), B * H
        # the roofline kernel is named, not picked by max() over noisy timings: the forward's prepare kernel is
        # the longest single launch of the delta-rule variants, Stage B of the variants without the delta term
        top = "prepare" if delta else "stageb"
        total_b = algorithmic_bytes(top, Z, BH, V, delta, gate == "channel")
        ab = io_bytes(top, Z, V, delta, gate)
        achieved = ab / (kern[top] * 1e-3) / 1e9
        fr = path_fractions(args.workload, fwd_ms, bwd_ms, ms, hbm, tf_sustained)
        line = {
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulate (bf16 in/out)",
            "data": "synthetic", "config": config,
            "launch": f"CUDA graph replay (lethe_b200.ops.GdnStepGraph, groups={args.groups}, overlap={graph.pipeline}, cut={graph.cut}, bwd_cuts={list(graph.bwd_cuts)})",
            "eager_ms_per_step": eager_ms,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "kernel_ms": kern,
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "lethe_b200.host.HostPipeline with its make_host_buffers() (copy-in, kernels and copy-out of "
                           "consecutive steps overlap; one copy per direction and step)", "steps": e2e_steps,
                    "ms_per_step_runs": e2e_runs,
                    "single_step_ms": e2e_single_ms, "single_step_api": "lethe_b200.ops.gdn_chunk + autograd",
                    # the pipelined step moves h2d + d2h bytes per step over the host link in both directions at
                    # once: its floor is bytes / the measured link rate with every rank copying
                    "host_link": pcie,
                    "host_link_floor_ms": max(h2d, d2h) / (pcie["both"]["slowest_rank_gbs"] * 1e9) * 1e3},
            "autograd_op_ms": op_ms,
            # kernels per replayed step: three per forward segment of the step graph, the backward kernels per
            # backward segment
            "gpu_launches": args.steps * ((3 * graph.segments + ((6 if delta else 4) if gate == "channel" else (4 if delta else 3)) * (len(graph.bwd_cuts) + 1))),
            "clocks": clocks,
            "roofline": {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                         "frac": achieved / hbm, "peak_source": which,
                         "traffic": measured_traffic(top, gate, V, delta, Z),
                         "launch_ms": kern[top], "algorithmic_bytes": ab,
                         "algorithmic_bytes_note": "inputs / outputs / state the path itself requires of this "
                                                   "kernel (bench.py::io_bytes); records it writes for later "
                                                   "kernels are counted separately below",
                         "record_bytes": total_b - ab,
                         "with_records": {"bytes": total_b, "achieved": total_b / (kern[top] * 1e-3) / 1e9,
                                          "frac": total_b / (kern[top] * 1e-3) / 1e9 / hbm},
                         # the whole path on its algorithmic bytes and FLOPs (sustained bf16 peak: the step
                         # is timed inside a long loop)
                         "path": fr,
                         "kernels": {n: {"ms": kern[n], "io_bytes": io_bytes(n, Z, V, delta, gate),
                                         "traffic": measured_traffic(n, gate, V, delta, Z),
                                         "record_bytes": algorithmic_bytes(n, Z, BH, V, delta, gate == "channel")
                                         - io_bytes(n, Z, V, delta, gate)} for n in kern}},
            "hbm_frac": fr["step"]["hbm_frac"], "tensor_frac": fr["step"]["tensor_frac"],
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
