"""fp32 inputs with tf32 operands for the passes that form S = X Y^T (tcgen05 kind::tf32), the arithmetic of the
reference's tl.dot on fp32 inputs (clip_loss.py:53, :113): against the dense fp64 oracle on the same fp32 values,
and against the default bf16-operand route, whose operand rounding is four times coarser."""
import pytest
import torch
import torch.nn.functional as F

from oracle import dense

pytestmark = pytest.mark.gpu


def _inputs(b, d, seed, normalized):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, d, generator=g)
    y = x + 0.8 * torch.randn(b, d, generator=g)
    if normalized:
        x, y = F.normalize(x, dim=1), F.normalize(y, dim=1)
    return x, y


def _module_step(cls_name, x, y, t, normalized, tf32, monkeypatch):
    import memoryefficientclip_b200 as m
    from memoryefficientclip_b200 import ops
    monkeypatch.setattr(ops, "TF32_OPERANDS", tf32)
    xg = x.cuda().requires_grad_(True)
    yg = y.cuda().requires_grad_(True)
    loss = getattr(m, cls_name)(t, normalized)(xg, yg)
    loss.backward()
    torch.cuda.synchronize()
    ops.check_status()
    return loss.item(), xg.grad.cpu(), None if yg.grad is None else yg.grad.cpu()


@pytest.mark.parametrize("b,d,normalized", [(1024, 512, True), (900, 200, False), (2304, 1152, False), (256, 64, True)])
def test_clip_tf32_operands_match_the_oracle_and_beat_bf16_operands(b, d, normalized, monkeypatch):
    x, y = _inputs(b, d, 3, normalized)
    t = 0.07
    rl, rx, ry = dense.clip_dense(x, y, t, normalized)
    l32, dx32, dy32 = _module_step("MemoryEfficientCLIPLoss", x, y, t, normalized, True, monkeypatch)
    l16, dx16, dy16 = _module_step("MemoryEfficientCLIPLoss", x, y, t, normalized, False, monkeypatch)
    dense.assert_parity(l32, rl, (dx32, dy32), (rx, ry), f"tf32 operands b={b} d={d}")
    # the loss depends on S only: finer operands give a closer loss (the gradients still go through a bf16 panel)
    e32, e16 = dense.loss_rel_err(l32, rl), dense.loss_rel_err(l16, rl)
    assert e32 <= max(e16, 2e-6), (e32, e16)


def test_tf32_sums_are_closer_to_fp64_than_bf16_sums():
    """Row sums of E at T = 0.03 (sharp softmax): the error of s/T is what the operand precision buys."""
    from memoryefficientclip_b200 import _lib, ops
    b, d, t = 2048, 768, 0.03
    x, y = _inputs(b, d, 9, True)
    xg, yg = x.cuda(), y.cuda()
    x16, _ = ops.normalize_fwd(xg, False)
    y16, _ = ops.normalize_fwd(yg, False)
    x32, y32 = ops.operand_f32(xg), ops.operand_f32(yg)
    _l16, r16, _c16, _d16 = ops.loss_forward(_lib.CLIP, x16, y16, t)
    _l32, r32, _c32, d32 = ops.loss_forward(_lib.CLIP, x16, y16, t, f32_operands=(x32, y32))
    torch.cuda.synchronize()
    s = x.double() @ y.double().t()
    ref = torch.exp((s - 1.0) / t).sum(1)
    err16 = ((r16.cpu().double() - ref).abs() / ref).max().item()
    err32 = ((r32.cpu().double() - ref).abs() / ref).max().item()
    assert err32 < 0.5 * err16, (err32, err16)
    assert err32 < 5e-3
    torch.testing.assert_close(d32.cpu().double(), s.diagonal(), rtol=0, atol=2e-3)


def test_lit_tf32_operands(monkeypatch):
    x, y = _inputs(1280, 320, 5, False)
    rl, rx = dense.lit_dense(x, y, 0.07, False)[:2]
    l32, dx32, dy32 = _module_step("MemoryEfficientLiTLoss", x, y, 0.07, False, True, monkeypatch)
    assert dy32 is None
    dense.assert_parity(l32, rl, (dx32,), (rx,), "LiT tf32 operands")


def test_tf32_entry_points_reject_bad_operands():
    from memoryefficientclip_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(256, 72, device="cuda")                     # pitch 72: a multiple of 4 and of 8
    r = torch.zeros(256, device="cuda")
    c = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = lambda xp, ld: (0, xp, x.data_ptr(), 256, 256, 72, ld, 72, 0.07, 0, 0, r.data_ptr(), r.data_ptr(),
                           r.data_ptr(), c.data_ptr(), None, None)
    assert lib.meclip_sum_exp_tf32(*args(x.data_ptr() + 4, 72)) == _lib.EINVAL      # not 16-byte aligned
    assert lib.meclip_sum_exp_tf32(*args(None, 72)) == _lib.EINVAL
    assert lib.meclip_sum_exp_tf32(*args(x.data_ptr(), 70)) == _lib.EINVAL          # pitch below d


def test_operand_f32_is_the_oracles_tf32_rounding_bit_for_bit():
    from memoryefficientclip_b200 import ops
    g = torch.Generator().manual_seed(21)
    x = torch.randn(300, 200, generator=g) * torch.exp(4 * torch.randn(300, 1, generator=g))
    xg = x.cuda()
    plain = ops.operand_f32(xg).cpu()
    assert plain.shape == (300, 200) and torch.equal(plain, dense.round_tf32(x))
    _x16, inv = ops.normalize_fwd(xg, True)
    scaled = ops.operand_f32(xg, inv).cpu()
    assert torch.equal(scaled, dense.round_tf32(x * inv.cpu()[:, None]))
    odd = torch.randn(64, 13, generator=g)                     # pad columns are zero
    out = ops.operand_f32(odd.cuda()).cpu()
    assert out.shape == (64, 16) and torch.equal(out[:, :13], dense.round_tf32(odd)) and not out[:, 13:].any()


def test_tf32_sums_equal_fp64_sums_of_the_rounded_operands():
    """With operands already in tf32 the products are exact and only the tensor cores' fp32 accumulation (which
    truncates: a few 1e-6 on s over 640 terms, i.e. 1e-4 on E at T = 0.03) separates the result from fp64
    arithmetic on the SAME rounded values: far inside what operand rounding itself costs (1e-3 on s for tf32)."""
    from memoryefficientclip_b200 import _lib, ops
    b, d, t = 1536, 640, 0.03
    x, y = _inputs(b, d, 17, True)
    xg, yg = x.cuda(), y.cuda()
    x32, y32 = ops.operand_f32(xg), ops.operand_f32(yg)
    x16, _ = ops.normalize_fwd(xg, False)
    y16, _ = ops.normalize_fwd(yg, False)
    _l, r, c, diag = ops.loss_forward(_lib.CLIP, x16, y16, t, f32_operands=(x32, y32))
    torch.cuda.synchronize()
    xr, yr = dense.round_tf32(x).double(), dense.round_tf32(y).double()
    s = xr @ yr.t()
    e = torch.exp((s - 1.0) / t)
    torch.testing.assert_close(diag.cpu().double(), s.diagonal(), rtol=0, atol=1e-5)
    torch.testing.assert_close(r.cpu().double(), e.sum(1), rtol=1e-3, atol=0)
    torch.testing.assert_close(c.cpu().double(), e.sum(0), rtol=1e-3, atol=0)
