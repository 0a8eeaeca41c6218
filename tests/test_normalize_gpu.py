"""Row kernels (normalise forward / Jacobian) against the oracle's numpy statement."""
import numpy as np
import pytest
import torch

from oracle import dense

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,d,dtype", [(7, 8, torch.float32), (513, 1152, torch.bfloat16), (64, 264, torch.float32)])
def test_normalize_fwd_bwd(rows, d, dtype):
    from memoryefficientclip_b200 import ops
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(rows, d, generator=g) * 3).to(dtype)
    gr = torch.randn(rows, d, generator=g)
    xh, inv = ops.normalize_fwd(x.cuda(), True)
    ref_h, ref_inv = dense.normalize_np(x.double().numpy())
    np.testing.assert_allclose(inv.cpu().numpy(), ref_inv, rtol=1e-5)
    np.testing.assert_allclose(xh.float().cpu().numpy(), ref_h, atol=4e-3 * np.abs(ref_h).max(), rtol=8e-3)
    dx = ops.normalize_bwd(gr.cuda(), xh, inv, torch.float32)
    ref_dx = dense.normalize_jacobian_np(xh.double().cpu().numpy(), inv.double().cpu().numpy(), gr.double().numpy())
    np.testing.assert_allclose(dx.cpu().numpy(), ref_dx, rtol=1e-4, atol=1e-5 * np.abs(ref_dx).max())


def test_zero_row_uses_eps():
    from memoryefficientclip_b200 import ops
    x = torch.zeros(4, 16)
    xh, inv = ops.normalize_fwd(x.cuda(), True)
    assert torch.all(xh == 0) and torch.all(inv == 1e12)


def test_convert_only():
    from memoryefficientclip_b200 import ops
    x = torch.randn(33, 40)
    xh, inv = ops.normalize_fwd(x.cuda(), False)
    assert inv is None
    assert torch.equal(xh.cpu(), x.bfloat16())


@pytest.mark.parametrize("rows,d,dtype", [(37, 1, torch.float32), (130, 13, torch.float16), (65, 100, torch.bfloat16),
                                          (40, 515, torch.float32), (129, 768, torch.float16)])
def test_any_feature_count_and_half(rows, d, dtype):
    """Feature counts that are not multiples of 8 and fp16: the operand is zero padded to 16-byte rows."""
    from memoryefficientclip_b200 import ops
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(rows, d, generator=g) * 2).to(dtype)
    gr = torch.randn(rows, ops.padded(d), generator=g)
    gr[:, d:] = 0
    xh, inv = ops.normalize_fwd(x.cuda(), True)
    assert xh.shape == (rows, ops.padded(d)) and xh.dtype == torch.bfloat16
    assert torch.all(xh[:, d:] == 0)
    ref_h, ref_inv = dense.normalize_np(x.double().numpy())
    np.testing.assert_allclose(inv.cpu().numpy(), ref_inv, rtol=1e-5)
    np.testing.assert_allclose(xh[:, :d].float().cpu().numpy(), ref_h, atol=4e-3 * np.abs(ref_h).max(), rtol=8e-3)
    dx = ops.normalize_bwd(gr.cuda(), xh, inv, dtype, d)
    assert dx.shape == (rows, d) and dx.dtype == dtype
    ref_dx = dense.normalize_jacobian_np(xh[:, :d].double().cpu().numpy(), inv.double().cpu().numpy(),
                                         gr[:, :d].double().numpy())
    tol = 1e-4 if dtype == torch.float32 else 8e-3
    np.testing.assert_allclose(dx.float().cpu().numpy(), ref_dx, rtol=tol, atol=tol * np.abs(ref_dx).max())


def test_unaligned_views_need_no_copy():
    """A column slice of a wider matrix: 4-byte aligned rows with an odd pitch are read element-wise."""
    from memoryefficientclip_b200 import ops
    g = torch.Generator().manual_seed(6)
    wide = torch.randn(50, 75, generator=g).cuda()
    x = wide[:, 3:67]                                    # d = 64, pitch 75, starts 12 bytes in
    assert x.data_ptr() % 16 != 0 and x.stride(0) % 8 != 0
    xh, inv = ops.normalize_fwd(x, True)
    xh2, inv2 = ops.normalize_fwd(x.contiguous(), True)
    # the element-wise and the 16-byte paths sum the squares in different orders: one bf16 ulp at most
    np.testing.assert_allclose(xh.float().cpu().numpy(), xh2.float().cpu().numpy(), rtol=8e-3, atol=1e-6)
    np.testing.assert_allclose(inv.cpu().numpy(), inv2.cpu().numpy(), rtol=1e-5)


def test_gradient_conversion_only():
    from memoryefficientclip_b200 import ops
    g = torch.randn(21, 16)
    g[:, 13:] = 0
    out = ops.normalize_bwd(g.cuda(), None, None, torch.float16, 13)
    assert torch.equal(out.cpu(), g[:, :13].half())
