"""The benchmark configurations at their full single-GPU sizes (B=32768, D=1152, bf16).

A dense CPU reference would need a 4 GiB matrix per copy, so parity is checked through
(a) the row-blocked streaming oracle: exact loss, exact gradient rows for a sample of rows,
(b) size-independent identities of the loss: it depends on X, Y only through X Y^T, so
    <X, dX> == <Y, dY> and X^T dX + Y^T dY is a symmetric D x D matrix.
"""
import pytest
import torch

from oracle import dense

pytestmark = pytest.mark.gpu

ROWS = [0, 1, 127, 128, 4095, 8191, 8192, 16383, 20000, 32767]


def test_clip_b32768_d1152_bf16():
    from memoryefficientclip_b200 import MemoryEfficientCLIPLoss, synth
    name = "clip_b32768_d1152_bf16"
    _kind, b, d, _dt, t, normed, _g = synth.CONFIGS[name]
    img, txt = synth.make(name)
    x = img.cuda().requires_grad_(True)
    y = txt.cuda().requires_grad_(True)
    loss = MemoryEfficientCLIPLoss(t, normed)(x, y)
    loss.backward()
    torch.cuda.synchronize()
    ref = dense.clip_streaming(img.float(), txt.float(), t, ROWS)
    assert dense.loss_rel_err(loss.item(), ref["loss"]) <= dense.LOSS_RTOL
    gx, gy = x.grad.float(), y.grad.float()
    for got, want in ((gx[ROWS].cpu(), ref["dx_rows"]), (gy[ROWS].cpu(), ref["dy_rows"])):
        max_rel, cos = dense.grad_errors(got, want)
        assert max_rel <= dense.GRAD_MAX_REL and cos >= dense.GRAD_COS_MIN, (max_rel, cos)
    # identities over the whole tensors (fp32 on the GPU, operands exactly as the kernels saw them)
    xf, yf = x.detach().float(), y.detach().float()
    a = (xf * gx).sum().item()
    c = (yf * gy).sum().item()
    assert abs(a - c) <= 2e-2 * max(abs(a), abs(c)), (a, c)     # bf16-rounded gradients
    m = xf.t() @ gx + yf.t() @ gy
    asym = (m - m.t()).norm().item() / m.norm().item()
    assert asym < 2e-2, asym


def test_lit_b32768_d1152_bf16():
    from memoryefficientclip_b200 import MemoryEfficientLiTLoss, synth
    name = "lit_b32768_d1152_bf16"
    _kind, b, d, _dt, t, normed, _g = synth.CONFIGS[name]
    txt, img = synth.make(name)
    x = txt.cuda().requires_grad_(True)
    loss = MemoryEfficientLiTLoss(t, normed)(x, img.cuda())
    loss.backward()
    torch.cuda.synchronize()
    # normalized_inputs=False: the oracle normalises the same bf16 values in fp32
    xn = torch.nn.functional.normalize(txt.float(), dim=1)
    yn = torch.nn.functional.normalize(img.float(), dim=1)
    ref = dense.clip_streaming(xn, yn, t, ROWS, lit=True)
    assert dense.loss_rel_err(loss.item(), ref["loss"]) <= dense.LOSS_RTOL
    # chain the normalise Jacobian onto the oracle's rows (d loss / d x = J^T d loss / d x_hat)
    inv = 1.0 / txt.float().norm(dim=1).clamp_min(1e-12)
    want = dense.normalize_jacobian_np(xn[ROWS].double().numpy(), inv[ROWS].double().numpy(), ref["dx_rows"].numpy())
    max_rel, cos = dense.grad_errors(x.grad.float()[ROWS].cpu(), want)
    assert max_rel <= dense.GRAD_MAX_REL and cos >= dense.GRAD_COS_MIN, (max_rel, cos)
