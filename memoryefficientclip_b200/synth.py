"""Seeded synthetic feature batches with the shapes and distributions of the five
benchmark configurations.  Everything is drawn with CPU generators so that a CPU
checker and the GPU see identical values.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _randn(rows: int, d: int, seed: int, row_start: int = 0, total_rows: int | None = None) -> torch.Tensor:
    """Rows [row_start, row_start+rows) of the (total_rows, d) matrix drawn from `seed`.

    Drawn in fixed blocks of 4096 rows, each from its own generator, so that a rank of
    the ring can create just its shard and still agree with the single-process draw.
    """
    block = 4096
    out = torch.empty(rows, d, dtype=torch.float32)
    r = row_start
    end = row_start + rows
    while r < end:
        b = r // block
        g = torch.Generator().manual_seed(seed * 1_000_003 + b)
        blk = torch.randn(block, d, generator=g, dtype=torch.float32)
        lo = r - b * block
        hi = min(block, end - b * block)
        out[r - row_start:r - row_start + (hi - lo)] = blk[lo:hi]
        r += hi - lo
    return out


def clip_pair(b: int, d: int, dtype=torch.bfloat16, normalized: bool = True, row_start: int = 0, rows: int | None = None):
    """image ~ N(0,1) seed 0, text ~ N(0,1) seed 1; optionally row-normalised in fp32, then cast."""
    rows = b if rows is None else rows
    img = _randn(rows, d, 0, row_start)
    txt = _randn(rows, d, 1, row_start)
    if normalized:
        img, txt = F.normalize(img, dim=1), F.normalize(txt, dim=1)
    return img.to(dtype), txt.to(dtype)


def noisy_pair(b: int, d: int, noise: float, dtype=torch.bfloat16, row_start: int = 0, rows: int | None = None):
    """image = normalize(N(0,1)); text = normalize(image + noise * N(0,1)).  Returns (image, text)."""
    rows = b if rows is None else rows
    img = F.normalize(_randn(rows, d, 0, row_start), dim=1)
    txt = F.normalize(img + noise * _randn(rows, d, 1, row_start), dim=1)
    return img.to(dtype), txt.to(dtype)


CONFIGS = {
    # name: (kind, B, D, dtype, temperature, normalized_inputs, generator)
    "clip_b4096_d512_f32": ("clip", 4096, 512, torch.float32, 0.07, False, "raw"),
    "clip_b32768_d1152_bf16": ("clip", 32768, 1152, torch.bfloat16, 0.07, True, "normalized"),
    "lit_b32768_d1152_bf16": ("lit", 32768, 1152, torch.bfloat16, 0.07, False, "noisy1.0"),
    "ring_clip_b131072_d768_bf16": ("clip", 131072, 768, torch.bfloat16, 0.07, True, "normalized"),
    "ring_clip_b262144_d1024_bf16": ("clip", 262144, 1024, torch.bfloat16, 0.03, False, "noisy0.5"),
}


def make(name: str, batch: int | None = None, row_start: int = 0, rows: int | None = None):
    """(first_arg, second_arg) in the order the reference modules take them:
    CLIP: (image, text); LiT: (text, image)."""
    kind, b, d, dtype, _t, _n, gen = CONFIGS[name]
    b = batch or b
    if gen == "raw":
        a, t = clip_pair(b, d, dtype, normalized=False, row_start=row_start, rows=rows)
    elif gen == "normalized":
        a, t = clip_pair(b, d, dtype, normalized=True, row_start=row_start, rows=rows)
    else:
        a, t = noisy_pair(b, d, float(gen[5:]), dtype, row_start=row_start, rows=rows)
    return (t, a) if kind == "lit" else (a, t)
