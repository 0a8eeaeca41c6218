"""The backward's blocking (several coefficient panels, several row blocks, ragged last ones,
fp32 partial accumulation, double-buffered panels on side streams) on problems small enough for
the dense oracle, by shrinking the block sizes through the library's test hook."""
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
    yield



@pytest.fixture
def small_blocks():
    from memoryefficientclip_b200 import _lib
    lib = _lib.load()

    def set_blocks(row_block, panel_cols):
        _lib.check(lib.meclip_debug_set_blocking(row_block, row_block * panel_cols * 2))

    yield set_blocks
    lib.meclip_debug_set_blocking(0, 0)


@pytest.mark.parametrize("b,d,row_block,panel_cols,dtype", [
    (1000, 64, 256, 256, torch.float32),     # 4 row blocks x 4 panels, both ragged
    (1536, 128, 512, 512, torch.bfloat16),   # 3 x 3, exact
    (700, 200, 384, 256, torch.bfloat16),    # 2 x 3, ragged, d not a multiple of 64
    (900, 72, 1024, 256, torch.float32),     # 1 row block, 4 panels: dX accumulates, dY does not
    (900, 72, 128, 4096, torch.float32),     # 8 row blocks, 1 panel: dY accumulates, dX does not
])
def test_clip_blocked_backward(small_blocks, b, d, row_block, panel_cols, dtype):
    import memoryefficientclip_b200 as m
    small_blocks(row_block, panel_cols)
    g = torch.Generator().manual_seed(13)
    x = F.normalize(torch.randn(b, d, generator=g), dim=1).to(dtype)
    y = F.normalize(torch.randn(b, d, generator=g), dim=1).to(dtype)
    xg, yg = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    loss = m.MemoryEfficientCLIPLoss(0.07, True)(xg, yg)
    loss.backward(torch.tensor(0.5, device="cuda"))
    torch.cuda.synchronize()
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True, grad_output=0.5)
    dense.assert_parity(loss.item(), rl, (xg.grad.float().cpu(), yg.grad.float().cpu()), (rx, ry), f"blocked b={b}")


def test_lit_blocked_backward_and_determinism(small_blocks):
    import memoryefficientclip_b200 as m
    small_blocks(256, 256)
    g = torch.Generator().manual_seed(14)
    img = F.normalize(torch.randn(840, 96, generator=g), dim=1)
    txt = F.normalize(img + torch.randn(840, 96, generator=g), dim=1)
    grads = []
    for _ in range(2):
        xg = txt.cuda().requires_grad_(True)
        loss = m.MemoryEfficientLiTLoss(0.07, False)(xg, img.cuda())
        loss.backward()
        grads.append(xg.grad.clone())
    torch.cuda.synchronize()
    rl, rx = dense.lit_dense(txt, img, 0.07, False)
    dense.assert_parity(loss.item(), rl, (grads[0].cpu(),), (rx,), "blocked lit")
    # The forward sums use atomics: their last bits can differ between runs, which can flip the bf16
    # rounding of single coefficients; the blocked backward itself adds in a fixed order.
    mr, cs = dense.grad_errors(grads[0], grads[1])
    assert mr < 1e-3


def test_status_word_stays_clear():
    from memoryefficientclip_b200 import _lib, ops
    x = F.normalize(torch.randn(512, 64), dim=1).bfloat16().cuda()
    status = ops.new_status(x.device)
    loss, r, c, _ = ops.loss_forward(_lib.CLIP, x, x, 0.07, status=status)
    ops.loss_backward(_lib.CLIP, x, x, 0.07, r, c, None, 1.0, torch.float32, torch.float32, status=status)
    ops.read_status(status)          # raises MeclipError(ETIMEOUT) if any bounded wait had expired
    assert status.item() == 0
