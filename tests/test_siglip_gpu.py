"""The sigmoid (SigLIP) loss extension against the dense oracle (same tolerances as the softmax losses).

The operands of the tile kernels are bf16: a logit a_ii = t * s_ii carries an error of about t * 2e-4, and the
positive pair's coefficient sigmoid(a_ii) - 1 changes by that relative amount, so at t = 20 single rows reach the
1e-2 max-relative bar; the cases stay at the scales the loss is used with (t = 10 at initialisation)."""
import math

import pytest
import torch
import torch.nn.functional as F

from oracle import dense

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("b,d,dtype,normalized,t0,b0", [
    (256, 64, torch.float32, False, 10.0, -10.0),
    (520, 128, torch.bfloat16, True, 10.0, -10.0),
    (200, 72, torch.float32, False, 4.0, -2.0),      # ragged tiles, many pairs near the sigmoid's middle
    (1024, 512, torch.bfloat16, False, 10.0, -10.0),
    (640, 256, torch.bfloat16, True, 16.0, -8.0),
])
def test_siglip_matches_dense(b, d, dtype, normalized, t0, b0):
    from memoryefficientclip_b200 import MemoryEfficientSigLIPLoss
    g = torch.Generator().manual_seed(17)
    img = torch.randn(b, d, generator=g)
    txt = img + 0.7 * torch.randn(b, d, generator=g)
    if normalized:
        img, txt = F.normalize(img, dim=1), F.normalize(txt, dim=1)
    img, txt = img.to(dtype), txt.to(dtype)
    mod = MemoryEfficientSigLIPLoss(t0, b0, normalized_inputs=normalized).cuda()
    xg, yg = img.cuda().requires_grad_(True), txt.cuda().requires_grad_(True)
    loss = mod(xg, yg)
    loss.backward(torch.tensor(0.5, device="cuda"))
    torch.cuda.synchronize()
    rl, rx, ry, rt, rb = dense.siglip_dense(img, txt, t0, b0, normalized, grad_output=0.5)
    dense.assert_parity(loss.item(), rl, (xg.grad.float().cpu(), yg.grad.float().cpu()), (rx, ry), f"siglip b={b}")
    # the module's parameter is log(t): d/d log t = t * d/dt
    got_t = mod.log_logit_scale.grad.item() / t0
    got_b = mod.logit_bias.grad.item()
    assert abs(got_t - rt) <= 1e-2 * max(abs(rt), 1e-6), (got_t, rt)
    assert abs(got_b - rb) <= 1e-2 * max(abs(rb), 1e-6), (got_b, rb)


def test_siglip_fixed_scale_and_frozen_text():
    from memoryefficientclip_b200 import MemoryEfficientSigLIPLoss
    g = torch.Generator().manual_seed(18)
    img = F.normalize(torch.randn(384, 96, generator=g), dim=1)
    txt = F.normalize(img + 0.5 * torch.randn(384, 96, generator=g), dim=1)
    mod = MemoryEfficientSigLIPLoss(10.0, -10.0, normalized_inputs=True, learnable=False).cuda()
    xg = img.cuda().requires_grad_(True)
    loss = mod(xg, txt.cuda())
    loss.backward()
    rl, rx, _ry, _rt, _rb = dense.siglip_dense(img, txt, 10.0, -10.0, True)
    dense.assert_parity(loss.item(), rl, (xg.grad.cpu(),), (rx,), "siglip frozen text")
    assert len(list(mod.parameters())) == 0
