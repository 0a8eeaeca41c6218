"""The CPU oracle against the reference's golden vectors and against itself."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import dense

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def test_golden_files_present():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_closed_form_matches_reference_kernels(path):
    """Closed form (fp64) vs. the reference's Triton kernels (fp32, interpreter)."""
    g = np.load(path)
    kind = str(g["kind"])
    t, stable, go = float(g["temperature"]), bool(g["stable"]), float(g["grad_output"])
    if kind == "clip":
        o = dense.clip_closed_form(g["x"], g["y"], t, stable, go)
    else:
        o = dense.lit_closed_form(g["x"], g["y"], t, stable, go)
    assert dense.loss_rel_err(o["loss"], g["loss"]) < 1e-6
    np.testing.assert_allclose(o["row_sum"], g["row_sum"], rtol=5e-5)
    mr, cs = dense.grad_errors(o["dx"], g["dx"])
    assert mr < 5e-5 and cs > 1 - 1e-8
    if kind == "clip":
        np.testing.assert_allclose(o["col_sum"], g["col_sum"], rtol=5e-5)
        mr, cs = dense.grad_errors(o["dy"], g["dy"])
        assert mr < 5e-5 and cs > 1 - 1e-8


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_dense_autograd_matches_reference_kernels(path):
    """Dense cross-entropy + autograd (the parity reference) vs. the golden vectors."""
    g = np.load(path)
    kind = str(g["kind"])
    t, stable, go = float(g["temperature"]), bool(g["stable"]), float(g["grad_output"])
    x, y = torch.from_numpy(g["x"]), torch.from_numpy(g["y"])
    if kind == "clip":
        loss, gx, gy = dense.clip_dense(x, y, t, True, stable, go)
        mr, cs = dense.grad_errors(gy, g["dy"])
        assert mr < 5e-5 and cs > 1 - 1e-8
    else:
        loss, gx = dense.lit_dense(x, y, t, True, stable, go)
    assert dense.loss_rel_err(loss, g["loss"]) < 1e-6
    mr, cs = dense.grad_errors(gx, g["dx"])
    assert mr < 5e-5 and cs > 1 - 1e-8


@pytest.mark.parametrize("b,d", [(192, 48), (200, 64), (64, 16)])
def test_closed_form_equals_dense_any_batch(b, d):
    """B not a multiple of 128: the closed form has no padding pollution."""
    gen = torch.Generator().manual_seed(3)
    x = torch.nn.functional.normalize(torch.randn(b, d, generator=gen, dtype=torch.float64), dim=1)
    y = torch.nn.functional.normalize(torch.randn(b, d, generator=gen, dtype=torch.float64), dim=1)
    loss, gx, gy = dense.clip_dense(x, y, 0.07, True)
    o = dense.clip_closed_form(x.numpy(), y.numpy(), 0.07)
    assert dense.loss_rel_err(o["loss"], loss) < 1e-12
    assert dense.grad_errors(o["dx"], gx)[0] < 1e-10
    assert dense.grad_errors(o["dy"], gy)[0] < 1e-10
    loss, gx = dense.lit_dense(x, y, 0.07, True)
    o = dense.lit_closed_form(x.numpy(), y.numpy(), 0.07)
    assert dense.loss_rel_err(o["loss"], loss) < 1e-12
    assert dense.grad_errors(o["dx"], gx)[0] < 1e-10


def test_normalize_and_jacobian_match_autograd():
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(33, 40, generator=gen, dtype=torch.float64, requires_grad=True)
    g = torch.randn(33, 40, generator=gen, dtype=torch.float64)
    xh = torch.nn.functional.normalize(x, dim=1)
    (dx,) = torch.autograd.grad(xh, x, g)
    xh_np, inv = dense.normalize_np(x.detach().numpy())
    np.testing.assert_allclose(xh_np, xh.detach().numpy(), rtol=1e-13)
    np.testing.assert_allclose(dense.normalize_jacobian_np(xh_np, inv, g.numpy()), dx.numpy(), rtol=1e-10, atol=1e-14)


def test_unnormalised_inputs_chain_rule():
    """normalized_inputs=False: dense autograd == closed form + normalise Jacobian."""
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(96, 32, generator=gen, dtype=torch.float64)
    y = torch.randn(96, 32, generator=gen, dtype=torch.float64)
    loss, gx, gy = dense.clip_dense(x, y, 0.07, False, stable=True, grad_output=2.0)
    xh, ix = dense.normalize_np(x.numpy())
    yh, iy = dense.normalize_np(y.numpy())
    o = dense.clip_closed_form(xh, yh, 0.07, stable=True, grad_output=2.0)
    assert dense.loss_rel_err(o["loss"], loss) < 1e-12
    assert dense.grad_errors(dense.normalize_jacobian_np(xh, ix, o["dx"]), gx)[0] < 1e-10
    assert dense.grad_errors(dense.normalize_jacobian_np(yh, iy, o["dy"]), gy)[0] < 1e-10


def test_streaming_matches_dense():
    gen = torch.Generator().manual_seed(9)
    x = torch.nn.functional.normalize(torch.randn(640, 64, generator=gen), dim=1)
    y = torch.nn.functional.normalize(torch.randn(640, 64, generator=gen), dim=1)
    rows = [0, 5, 639]
    s = dense.clip_streaming(x, y, 0.07, rows, block=256)
    loss, gx, gy = dense.clip_dense(x, y, 0.07, True)
    assert dense.loss_rel_err(s["loss"], loss) < 1e-6
    assert dense.grad_errors(s["dx_rows"], gx[rows])[0] < 1e-5
    assert dense.grad_errors(s["dy_rows"], gy[rows])[0] < 1e-5
    s = dense.clip_streaming(x, y, 0.07, rows, block=256, lit=True)
    loss, gx = dense.lit_dense(x, y, 0.07, True)
    assert dense.loss_rel_err(s["loss"], loss) < 1e-6
    assert dense.grad_errors(s["dx_rows"], gx[rows])[0] < 1e-5


def test_round_tf32_is_nearest_with_ten_mantissa_bits():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 20, 20000))).astype(np.float32)
    r = dense.round_tf32(x)
    assert r.dtype == np.float32 and np.all((r.view(np.uint32) & 0x1FFF) == 0)          # low 13 bits clear
    assert np.array_equal(dense.round_tf32(r), r)                                       # idempotent
    rel = np.abs(r.astype(np.float64) - x.astype(np.float64)) / np.abs(x.astype(np.float64))
    assert rel.max() <= 2.0 ** -11 * (1 + 1e-6)                                         # at most half a unit
    # known values: 1 + 2^-11 is a tie and goes away from zero; just below it rounds down
    one = np.array([1.0 + 2.0 ** -11, 1.0 + 2.0 ** -11 - 2.0 ** -23, -(1.0 + 2.0 ** -11)], dtype=np.float32)
    assert np.array_equal(dense.round_tf32(one), np.array([1.0 + 2.0 ** -10, 1.0, -(1.0 + 2.0 ** -10)], dtype=np.float32))
    t = torch.from_numpy(x)
    assert torch.equal(dense.round_tf32(t), torch.from_numpy(r))
