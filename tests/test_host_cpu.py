"""Host-side helpers that need no GPU: synthetic inputs, operand padding rules, gradient scales."""
import math

import torch

from memoryefficientclip_b200 import ops, synth


def test_shards_of_the_synthetic_batch_agree_with_the_whole_draw():
    """A rank of the ring draws only its rows; they must be the rows of the single-process batch."""
    img, txt = synth.clip_pair(12288, 24, torch.float32, True)
    for start, rows in ((0, 4096), (4096, 8192), (5000, 3000), (12000, 288)):
        i2, t2 = synth.clip_pair(12288, 24, torch.float32, True, row_start=start, rows=rows)
        assert torch.equal(i2, img[start:start + rows]) and torch.equal(t2, txt[start:start + rows])
    img, txt = synth.noisy_pair(8192, 16, 0.5, torch.float32)
    i2, t2 = synth.noisy_pair(8192, 16, 0.5, torch.float32, row_start=4096, rows=4096)
    assert torch.equal(i2, img[4096:]) and torch.equal(t2, txt[4096:])
    cos = torch.nn.functional.cosine_similarity(img, txt, dim=1).mean().item()
    assert 0.3 < cos < 0.6            # image + 0.5 N(0,1) on a unit vector in 16 dimensions: positives stand out


def test_configurations_match_the_benchmark_shapes():
    shapes = {name: (cfg[1], cfg[2]) for name, cfg in synth.CONFIGS.items()}
    assert shapes == {"clip_b4096_d512_f32": (4096, 512), "clip_b32768_d1152_bf16": (32768, 1152),
                      "lit_b32768_d1152_bf16": (32768, 1152), "ring_clip_b131072_d768_bf16": (131072, 768),
                      "ring_clip_b262144_d1024_bf16": (262144, 1024)}
    txt, img = synth.make("lit_b32768_d1152_bf16", batch=256)      # LiT order: (text, image)
    assert txt.shape == img.shape == (256, 1152) and txt.dtype == torch.bfloat16


def test_operand_padding_and_direct_gradient_rules():
    assert [ops.padded(d) for d in (1, 7, 8, 9, 1152, 1157)] == [8, 8, 8, 16, 1152, 1160]
    assert ops.direct_grad_dtype(torch.bfloat16, 1152) and ops.direct_grad_dtype(torch.float32, 64)
    assert not ops.direct_grad_dtype(torch.float16, 64)        # fp16 gradients are converted by the row kernel
    assert not ops.direct_grad_dtype(torch.float32, 100)       # as are feature counts that are not multiples of 8


def test_gradient_scales():
    # reference clip_loss.py:182, 235 (1 / (B T)) and clip_loss.py:299 (sqrt(B / T) / B)
    assert math.isclose(ops.grad_scale(4096, 0.07, False), 1.0 / (4096 * 0.07))
    assert math.isclose(ops.grad_scale(4096, 0.07, True), math.sqrt(4096 / 0.07) / 4096)
