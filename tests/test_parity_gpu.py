"""CUDA path vs. the CPU oracle on the same seeded inputs (through the public modules,
i.e. through the C ABI).  Tolerances: loss 1e-3 relative; gradients 1e-2 max-relative
and cosine >= 0.9999 (oracle.dense.LOSS_RTOL / GRAD_MAX_REL / GRAD_COS_MIN).
"""
import glob
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import dense

pytestmark = pytest.mark.gpu

@pytest.fixture(autouse=True, params=["step_path", "general_path"])
def both_module_routes(request, monkeypatch):
    """Small CLIP batches take the whole-step entry points (two library calls per step); every case of this
    file also runs with that route switched off, through the block-level entry points."""
    from memoryefficientclip_b200 import _function
    if request.param == "general_path":
        monkeypatch.setattr(_function, "_STEP_PATH_ROWS", 0)
    yield request.param


GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _mods():
    import memoryefficientclip_b200 as m
    return m


def _inputs(b, d, seed=0, normalized=True, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, d, generator=g)
    y = torch.randn(b, d, generator=g)
    if normalized:
        x, y = F.normalize(x, dim=1), F.normalize(y, dim=1)
    return x.to(dtype), y.to(dtype)


def _run_clip(x, y, t, normalized_inputs, stable=False, grad_output=None):
    m = _mods()
    mod = (m.StableMemoryEfficientCLIPLoss if stable else m.MemoryEfficientCLIPLoss)(t, normalized_inputs)
    xg = x.cuda().requires_grad_(True)
    yg = y.cuda().requires_grad_(True)
    loss = mod(xg, yg)
    if grad_output is None:
        loss.backward()
    else:
        loss.backward(torch.tensor(grad_output, device="cuda"))
    torch.cuda.synchronize()
    assert loss.dtype == torch.float32 and loss.dim() == 0
    assert xg.grad.dtype == x.dtype and yg.grad.dtype == y.dtype
    return loss.item(), xg.grad.float().cpu(), yg.grad.float().cpu()


def _run_lit(txt, img, t, normalized_inputs, stable=False):
    m = _mods()
    mod = (m.StableMemoryEfficientLiTLoss if stable else m.MemoryEfficientLiTLoss)(t, normalized_inputs)
    xg = txt.cuda().requires_grad_(True)
    yg = img.cuda().requires_grad_(True)
    loss = mod(xg, yg)
    loss.backward()
    torch.cuda.synchronize()
    assert yg.grad is None            # image tower frozen (reference lit_loss.py:247)
    return loss.item(), xg.grad.float().cpu()


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_against_reference_golden_vectors(path):
    """fp32 inputs of the golden cases; outputs of the reference's own kernels."""
    g = np.load(path)
    kind = str(g["kind"])
    t, stable, go = float(g["temperature"]), bool(g["stable"]), float(g["grad_output"])
    x, y = torch.from_numpy(g["x"]), torch.from_numpy(g["y"])
    if kind == "clip":
        loss, dx, dy = _run_clip(x, y, t, True, stable, None if go == 1.0 else go)
        dense.assert_parity(loss, g["loss"], (dx, dy), (g["dx"], g["dy"]), path)
    else:
        loss, dx = _run_lit(x, y, t, True, stable)
        dense.assert_parity(loss, g["loss"], (dx,), (g["dx"],), path)


@pytest.mark.parametrize("b,d,dtype", [(128, 64, torch.float32), (256, 64, torch.bfloat16), (192, 96, torch.bfloat16),
                                       (200, 48, torch.float32), (1024, 512, torch.bfloat16),
                                       (520, 1152, torch.bfloat16), (8, 16, torch.float32)])
def test_clip_normalized_inputs(b, d, dtype):
    x, y = _inputs(b, d, 0, True, dtype)
    loss, dx, dy = _run_clip(x, y, 0.07, True)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), f"clip b={b} d={d} {dtype}")


@pytest.mark.parametrize("b,d,dtype,t", [(256, 64, torch.float32, 0.07), (384, 128, torch.bfloat16, 0.03),
                                         (200, 72, torch.float32, 1.0)])
def test_clip_unnormalized_inputs_fused_normalize(b, d, dtype, t):
    x, y = _inputs(b, d, 1, False, dtype)
    loss, dx, dy = _run_clip(x, y, t, False)
    rl, rx, ry = dense.clip_dense(x, y, t, False)
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), f"clip raw b={b} d={d} {dtype}")


def test_clip_stable_and_grad_output():
    x, y = _inputs(256, 128, 2, True, torch.float32)
    loss, dx, dy = _run_clip(x, y, 0.07, True, stable=True, grad_output=0.25)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True, stable=True, grad_output=0.25)
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), "stable clip")


@pytest.mark.parametrize("b,d,dtype,norm", [(128, 64, torch.float32, True), (320, 96, torch.bfloat16, False),
                                            (1024, 256, torch.bfloat16, False)])
def test_lit(b, d, dtype, norm):
    g = torch.Generator().manual_seed(4)
    img = F.normalize(torch.randn(b, d, generator=g), dim=1)
    txt = F.normalize(img + torch.randn(b, d, generator=g), dim=1)
    img, txt = img.to(dtype), txt.to(dtype)
    loss, dx = _run_lit(txt, img, 0.07, norm)
    rl, rx = dense.lit_dense(txt, img, 0.07, norm)
    dense.assert_parity(loss, rl, (dx,), (rx,), f"lit b={b} d={d}")
    loss, dx = _run_lit(txt, img, 0.07, norm, stable=True)
    rl, rx = dense.lit_dense(txt, img, 0.07, norm, stable=True)
    dense.assert_parity(loss, rl, (dx,), (rx,), f"stable lit b={b} d={d}")


def test_normed_function_apply_signature():
    """XxxNormed.apply(x, y, temperature) as in the reference (clip_loss.py:271, lit_loss.py:261)."""
    m = _mods()
    x, y = _inputs(128, 64, 5, True)
    xg, yg = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    loss = m.MemoryEfficientCLIPLossNormed.apply(xg, yg, 0.07)
    loss.backward()
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(loss.item(), rl, (xg.grad.cpu(), yg.grad.cpu()), (rx, ry), "normed apply")
    xg.grad = None
    loss = m.MemoryEfficientLiTLossNormed.apply(xg, yg, 0.07)
    loss.backward()
    rl, rx = dense.lit_dense(x, y, 0.07, True)
    dense.assert_parity(loss.item(), rl, (xg.grad.cpu(),), (rx,), "lit normed apply")


def test_backward_is_deterministic():
    """Same saved sums -> bit-identical gradients: the backward has no atomics."""
    from memoryefficientclip_b200 import _lib, ops
    x, y = _inputs(512, 256, 6, True, torch.bfloat16)
    xg, yg = x.cuda(), y.cuda()
    go = torch.ones(1, device="cuda")
    _loss, r, c, _diag = ops.loss_forward(_lib.CLIP, xg, yg, 0.07)
    scale = ops.grad_scale(512, 0.07, False)
    a = ops.loss_backward(_lib.CLIP, xg, yg, 0.07, r, c, go, scale, torch.float32, torch.float32)
    b = ops.loss_backward(_lib.CLIP, xg, yg, 0.07, r, c, go, scale, torch.float32, torch.float32)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_medium_batch_multi_panel_properties():
    """B=4096, D=512 fp32 un-normalised inputs (the CPU-runnable benchmark configuration)."""
    from memoryefficientclip_b200 import synth
    img, txt = synth.make("clip_b4096_d512_f32")
    loss, dx, dy = _run_clip(img, txt, 0.07, False)
    rl, rx, ry = dense.clip_dense(img, txt, 0.07, False, dtype=torch.float32)
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), "clip_b4096_d512_f32")


@pytest.mark.parametrize("kind,stable,b,d,t", [("clip", False, 384, 64, 0.07), ("clip", True, 256, 128, 0.2),
                                              ("lit", False, 320, 96, 0.05)])
def test_learnable_temperature_gradient(kind, stable, b, d, t):
    """Extension: a tensor temperature receives d loss / dT (the reference returns None)."""
    m = _mods()
    x, y = _inputs(b, d, 8, False, torch.float32)
    temp = torch.nn.Parameter(torch.tensor(t, device="cuda"))
    cls = {("clip", False): m.MemoryEfficientCLIPLoss, ("clip", True): m.StableMemoryEfficientCLIPLoss,
           ("lit", False): m.MemoryEfficientLiTLoss}[(kind, stable)]
    xg = x.cuda().requires_grad_(True)
    loss = cls(temp, False)(xg, y.cuda())
    loss.backward(torch.tensor(2.0, device="cuda"))
    want = 2.0 * dense.temperature_grad_dense(x, y, t, kind, False)
    got = temp.grad.item()
    assert abs(got - want) <= 1e-2 * abs(want), (got, want)
    # a float temperature still gets no gradient and the feature gradients are unchanged
    xg2 = x.cuda().requires_grad_(True)
    cls(t, False)(xg2, y.cuda()).backward(torch.tensor(2.0, device="cuda"))
    # forward sums use atomics: last-bit differences; LiT with a constant temperature takes the one-pass route,
    # whose panel holds E instead of E / r (another bf16 rounding of the same quantity)
    assert dense.grad_errors(xg.grad, xg2.grad)[0] < (5e-3 if kind == "lit" else 1e-4)


@pytest.mark.parametrize("frozen", ["image", "text"])
def test_clip_with_one_frozen_tower_skips_its_gradient(frozen, both_module_routes):
    """Only the input that requires a gradient gets one (and only its contraction is launched)."""
    from memoryefficientclip_b200 import _lib
    m = _mods()
    x, y = _inputs(384, 128, 9, False, torch.bfloat16)
    xg = x.cuda().requires_grad_(frozen != "image")
    yg = y.cuda().requires_grad_(frozen != "text")
    before = _lib.load().meclip_launch_count()
    loss = m.MemoryEfficientCLIPLoss(0.07, False)(xg, yg)
    loss.backward()
    torch.cuda.synchronize()
    launches = _lib.load().meclip_launch_count() - before
    rl, rx, ry = dense.clip_dense(x, y, 0.07, False)
    if frozen == "image":
        assert xg.grad is None
        dense.assert_parity(loss.item(), rl, (yg.grad.float().cpu(),), (ry,), "frozen image")
    else:
        assert yg.grad is None
        dense.assert_parity(loss.item(), rl, (xg.grad.float().cpu(),), (rx,), "frozen text")
    if both_module_routes == "general_path":
        # normalise x2, sums, finalize | transpose, coefficient panel, one contraction, one Jacobian
        assert launches == 8, launches
    else:
        # both inputs normalised by one launch, sums, finalize | coefficient panel, one contraction, one Jacobian
        assert launches == 6, launches


def test_noisy_positive_pairs_low_temperature():
    """The distribution of the B=262144 ring configuration at a size the dense oracle handles:
    text = normalize(image + 0.5 noise), T = 0.03, bf16, normalise inside."""
    from memoryefficientclip_b200 import synth
    img, txt = synth.noisy_pair(2048, 1024, 0.5)
    loss, dx, dy = _run_clip(img, txt, 0.03, False)
    rl, rx, ry = dense.clip_dense(img, txt, 0.03, False)
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), "noisy pairs T=0.03")


@pytest.mark.parametrize("b,d,dtype,normalized", [(200, 13, torch.float32, True), (256, 100, torch.bfloat16, False),
                                                  (130, 515, torch.float32, False), (256, 64, torch.float16, True),
                                                  (192, 84, torch.float16, False), (64, 1, torch.float32, False)])
def test_any_feature_count_and_fp16_inputs(b, d, dtype, normalized):
    """The reference takes any D (it masks the last feature block, clip_loss.py:33-38) and any float dtype
    Triton loads; here operands are zero padded to 16-byte rows and fp16 is converted by the row kernels."""
    x, y = _inputs(b, d, 9, normalized, dtype)
    loss, dx, dy = _run_clip(x, y, 0.07, normalized)
    assert dx.shape == (b, d) and dy.shape == (b, d)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, normalized)
    if d == 1:       # every similarity is +-1: only check the loss and that the gradients are finite
        assert dense.loss_rel_err(loss, rl) <= dense.LOSS_RTOL
        assert torch.isfinite(dx).all() and torch.isfinite(dy).all()
        return
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), f"clip b={b} d={d} {dtype}")


def test_lit_odd_feature_count_fp16():
    txt, img = _inputs(160, 50, 10, False, torch.float16)
    loss, dx = _run_lit(txt, img, 0.07, False)
    rl, rx = dense.lit_dense(txt, img, 0.07, False)
    dense.assert_parity(loss, rl, (dx,), (rx,), "lit fp16 d=50")


@pytest.mark.parametrize("b,d", [(1, 8), (2, 16), (3, 5), (127, 24), (129, 40), (257, 8)])
def test_tiny_and_ragged_batches(b, d):
    """One row, fewer rows than a warp, one more or one less than a tile: every B >= 1 is exact here (the
    reference sums its padding columns in unless B is a multiple of 128, clip_loss.py:40-56)."""
    # normalised inputs already rounded to bf16: with so few rows and features nothing averages the operand
    # rounding out, so the kernels and the oracle are given the same representable values
    x, y = _inputs(b, d, 12, True, torch.bfloat16)
    x, y = x.float(), y.float()
    loss, dx, dy = _run_clip(x, y, 0.07, True)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    if b == 1:          # a single pair: the loss is exactly 0 and so are the gradients
        assert abs(loss) <= 1e-5 and float(dx.abs().max()) <= 1e-5 and float(dy.abs().max()) <= 1e-5
        return
    dense.assert_parity(loss, rl, (dx, dy), (rx, ry), f"clip b={b} d={d}")
    tl, tx = _run_lit(x, y, 0.07, True)
    ll, lx = dense.lit_dense(x, y, 0.07, True)
    dense.assert_parity(tl, ll, (tx,), (lx,), f"lit b={b} d={d}")


def test_empty_and_mismatched_inputs_are_rejected():
    m = _mods()
    mod = m.MemoryEfficientCLIPLoss(0.07, False)
    with pytest.raises(AssertionError):
        mod(torch.empty(0, 16, device="cuda"), torch.empty(0, 16, device="cuda"))
    with pytest.raises(AssertionError):
        mod(torch.randn(8, 16, device="cuda"), torch.randn(8, 24, device="cuda"))      # reference clip_loss.py:167
    with pytest.raises(AssertionError):
        mod(torch.randn(8, 16), torch.randn(8, 16))                                        # reference clip_loss.py:166


@pytest.mark.parametrize("b,d,dtype,normalized,stable", [(512, 256, torch.bfloat16, True, False), (384, 100, torch.float32, False, True),
                                                         (1024, 1152, torch.bfloat16, False, False), (200, 64, torch.float16, False, False)])
def test_lit_one_pass_and_two_pass_routes_agree_with_the_oracle(b, d, dtype, normalized, stable, monkeypatch):
    """LiT takes the one-pass route (forward contracts E with [Y | 1], backward is a row kernel) when the text
    input needs a gradient and the temperature is a constant; the two-pass route is what the reference does."""
    from memoryefficientclip_b200 import _function
    g = torch.Generator().manual_seed(21)
    img = F.normalize(torch.randn(b, d, generator=g), dim=1)
    txt = img + 0.8 * torch.randn(b, d, generator=g)
    if normalized:
        txt = F.normalize(txt, dim=1)
    txt, img = txt.to(dtype), img.to(dtype)
    rl, rx = dense.lit_dense(txt, img, 0.07, normalized, stable)
    for fused in (True, False):
        monkeypatch.setattr(_function, "_LIT_FUSED", fused)
        loss, dx = _run_lit(txt, img, 0.07, normalized, stable)
        dense.assert_parity(loss, rl, (dx,), (rx,), f"lit fused={fused} b={b} d={d}")
    # no gradient wanted: the plain forward, same loss
    m = _mods()
    with torch.no_grad():
        l2 = m.MemoryEfficientLiTLoss(0.07, normalized)(txt.cuda(), img.cuda()).item()
    assert dense.loss_rel_err(l2, rl) <= dense.LOSS_RTOL


@pytest.mark.parametrize("b,d,dtype,normalized", [(1000, 96, torch.float32, False), (2304, 256, torch.bfloat16, True),
                                                  (200, 40, torch.float32, True)])
def test_deterministic_forward_makes_the_whole_step_bit_identical(b, d, dtype, normalized, monkeypatch):
    """With the deterministic sums (no atomics in the forward) loss, sums and both gradients of two runs are
    bit-identical, and they are still the dense formulation's; the block-level sums agree with the atomic ones."""
    from memoryefficientclip_b200 import _lib, ops
    m = _mods()
    monkeypatch.setattr(ops, "DETERMINISTIC", True)
    x, y = _inputs(b, d, 31, normalized, dtype)
    runs = []
    for _ in range(2):
        xg, yg = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
        loss = m.MemoryEfficientCLIPLoss(0.07, normalized)(xg, yg)
        loss.backward()
        runs.append((loss.detach().clone(), xg.grad.clone(), yg.grad.clone()))
    torch.cuda.synchronize()
    for a, c in zip(*runs):
        assert torch.equal(a, c)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, normalized)
    dense.assert_parity(runs[0][0].item(), rl, (runs[0][1].float().cpu(), runs[0][2].float().cpu()), (rx, ry), "deterministic")
    # the sums themselves: deterministic against atomic, same kernels otherwise
    xh = ops.normalize_fwd(x.cuda(), not normalized)[0]
    yh = ops.normalize_fwd(y.cuda(), not normalized)[0]
    _l0, r0, c0, d0 = ops.loss_forward(_lib.CLIP, xh, yh, 0.07, deterministic=False)
    _l1, r1, c1, d1 = ops.loss_forward(_lib.CLIP, xh, yh, 0.07, deterministic=True)
    _l2, r2, c2, _d2 = ops.loss_forward(_lib.CLIP, xh, yh, 0.07, deterministic=True)
    assert torch.equal(r1, r2) and torch.equal(c1, c2)
    assert torch.allclose(r0, r1, rtol=1e-5) and torch.allclose(c0, c1, rtol=1e-5) and torch.equal(d0, d1)
