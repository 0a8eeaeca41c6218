"""Generate golden vectors from the reference's own Triton kernels.

Run once, in a container that has the reference checkout and Triton but no GPU:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

The reference's autograd Functions assert ``X.is_cuda`` (clip_loss.py:166), so
the four ``@triton.jit`` kernels are launched directly on CPU tensors through
Triton's interpreter, followed by the same host-side glue the Functions run
(clip_loss.py:181-211, 235-254; lit_loss.py:177-203, 227-245).  The reference
is exact only for B % 128 == 0 (padding columns are summed in), so every case
uses such a B.  Outputs are written next to this script as ``<case>.npz``.
"""
import math
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
import torch.nn.functional as F

CASES = [
    # name, kind, B, D, temperature, stable, grad_output
    ("clip_b128_d64", "clip", 128, 64, 0.07, False, 1.0),
    ("clip_b256_d64_t1", "clip", 256, 64, 1.0, False, 1.0),
    ("clip_stable_b128_d64_go", "clip", 128, 64, 0.07, True, 0.5),
    ("lit_b128_d96", "lit", 128, 96, 0.07, False, 1.0),
    ("lit_stable_b256_d64", "lit", 256, 64, 0.03, True, 1.0),
]


def inputs(b, d, kind):
    g0 = torch.Generator().manual_seed(0)
    g1 = torch.Generator().manual_seed(1)
    a = torch.randn(b, d, generator=g0)
    n = torch.randn(b, d, generator=g1)
    if kind == "lit":
        img = F.normalize(a, dim=1)
        txt = F.normalize(img + 1.0 * n, dim=1)
        return txt.contiguous(), img.contiguous()      # X = text, Y = image
    return F.normalize(a, dim=1).contiguous(), F.normalize(n, dim=1).contiguous()


def run_case(ref_clip, ref_lit, kind, b, d, temperature, stable, grad_output):
    import triton
    x, y = inputs(b, d, kind)
    inv_temp = 1.4426950408889634 / temperature
    inv_temp_orig = math.sqrt(b / temperature) if stable else 1.0 / temperature
    row = torch.zeros(b)
    col = torch.zeros(b)
    grid = (triton.cdiv(b, 128), triton.cdiv(b, 128))
    if kind == "clip":
        ref_clip.clip_sum_exp_kernel[grid](x, y, row, col, b, inv_temp, BLOCK_SIZE_I=128, BLOCK_SIZE_J=128,
                                           BLOCK_SIZE_D=64, D_MODEL=d)
    else:
        ref_lit.lit_sum_exp_kernel[grid](x, y, row, inv_temp, b, BLOCK_SIZE_I=128, BLOCK_SIZE_J=128,
                                         BLOCK_SIZE_D=64, D_MODEL=d)
    sv = torch.einsum("bi,bi->b", x, y) * inv_temp - inv_temp
    logits = torch.log(torch.exp2(sv) / row)
    if kind == "clip":
        logits = logits + torch.log(torch.exp2(sv) / col)
        loss = -logits.mean() / 2.0
    else:
        loss = -logits.mean()
    dx = y.clone().mul_(-inv_temp_orig / b)
    dy = x.clone().mul_(-inv_temp_orig / b)
    bd = min(64, d)
    grid = (triton.cdiv(b, 64), triton.cdiv(b, 64))
    if kind == "clip":
        ref_clip.clip_grad_kernel[grid](x, y, row, col, dx, dy, inv_temp, inv_temp_orig, b, BLOCK_SIZE_I=64,
                                        BLOCK_SIZE_J=64, BLOCK_SIZE_D=bd, D_MODEL=d)
    else:
        ref_lit.lit_grad_kernel[grid](x, y, row, dx, inv_temp, inv_temp_orig, b, BLOCK_SIZE_I=64,
                                      BLOCK_SIZE_J=64, BLOCK_SIZE_D=bd, D_MODEL=d)
    if grad_output != 1.0:
        dx = dx * grad_output
        dy = dy * grad_output
    out = dict(x=x.numpy(), y=y.numpy(), temperature=np.float64(temperature), stable=np.bool_(stable),
               grad_output=np.float64(grad_output), loss=np.float32(loss.item()), row_sum=row.numpy(),
               dx=dx.numpy())
    if kind == "clip":
        out.update(col_sum=col.numpy(), dy=dy.numpy())
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference/checkout")
    ref_dir = sys.argv[1]
    sys.path.insert(0, ref_dir)
    import clip_loss as ref_clip
    import lit_loss as ref_lit
    here = os.path.dirname(os.path.abspath(__file__))
    for name, kind, b, d, t, stable, go in CASES:
        out = run_case(ref_clip, ref_lit, kind, b, d, t, stable, go)
        np.savez_compressed(os.path.join(here, name + ".npz"), kind=kind, **out)
        print(name, "loss", float(out["loss"]))


if __name__ == "__main__":
    main()
