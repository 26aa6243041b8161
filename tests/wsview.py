"""Test helper: decode the per-chunk workspace records the CUDA kernels write (tile images)."""

import ctypes

import numpy as np
import torch

from lethe_b200 import native, ops


def unswizzle(img: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of the SW128 tile image: flat fp16 buffer [..., rows*cols] -> [..., rows, cols]."""
    lead = img.shape[:-1]
    x = img.reshape(*lead, cols // 64, rows, 8, 8)
    r = torch.arange(rows) & 7
    out = torch.empty_like(x)
    for c in range(8):
        out[..., torch.arange(rows), c, :] = x[..., torch.arange(rows), (c ^ r), :]
    return out.permute(*range(len(lead)), len(lead) + 1, len(lead), len(lead) + 2, len(lead) + 3) \
              .reshape(*lead, rows, cols)


def layout(B, H, L, V, gate=1, delta=1):
    """Record offsets, mirroring make_layout() of the library."""
    Z = B * H * (L // 64)
    al = lambda x: (x + 1023) // 1024 * 1024
    sz = dict(ta=16384, w=16384, u=64 * V * 2, p=32768, r=128 * V * 2, hc=128 * V * 2, vn=64 * V * 2,
              ad=128 * 4)
    off, o = {}, 0
    for n in ("ta", "w", "u", "p", "r", "hc", "vn", "ad"):
        off[n] = o
        o = al(o + (Z + B * H if n == "hc" else Z) * sz[n])   # states: NT + 1 records per (b, h)
    sz2 = dict(rb=128 * V * 2, dh=128 * V * 2, dv2=64 * V * 2, dw=16384, dkb=64 * 128 * 4,
               dgb=(64 * 128 if gate == 2 else 64) * 4)
    off2, o = {}, 0
    for n in ("rb", "dh", "dv2", "dw", "dkb", "dgb"):
        off2[n] = o
        o = al(o + Z * sz2[n])
    return Z, sz, off, sz2, off2


def records(buf: torch.Tensor, off: int, size: int, Z: int, dtype=torch.float16) -> torch.Tensor:
    raw = buf[off:off + Z * size].cpu()
    return raw.view(dtype).reshape(Z, -1)


def rrecords(buf: torch.Tensor, off: int, size: int, Z: int, V: int) -> torch.Tensor:
    """The scan-input records R / Rb: stored as V / 16 column blocks of [128 rows][16 columns]; returned as
    [Z, 128, V]."""
    blk = records(buf, off, size, Z).reshape(Z, V // 16, 128, 16)
    return blk.permute(0, 2, 1, 3).reshape(Z, 128, V)


def report(label: str, errs: dict) -> None:
    """Print the per-tensor errors of a parity case and append them to a log next to the run."""
    line = label + " " + " ".join(f"{k}={v:.2e}" for k, v in errs.items())
    print(line)
    import os
    d = os.environ.get("LETHE_TEST_LOG_DIR")
    if d and os.path.isdir(d):
        with open(os.path.join(d, "parity.log"), "a") as f:
            f.write(line + "\n")
