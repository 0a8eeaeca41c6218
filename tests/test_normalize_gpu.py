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
