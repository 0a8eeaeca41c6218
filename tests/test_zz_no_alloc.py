"""meclip_grad_static: the backward for callers that cannot hand over a workspace (a plugin
interface with fixed inputs/outputs, or a process whose device memory is fully owned by
another allocator).  It must give what meclip_grad gives, call after call, although every
call reuses the same built-in scratch array and finds the previous call's data in it.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else; it also passes when run alone in a fresh process.
"""
import gc

import pytest
import torch
import torch.nn.functional as F

from oracle import dense

pytestmark = pytest.mark.gpu


def _case(b, d, kind, seed, strict_free=False, bit_identical=True):
    from memoryefficientclip_b200 import _lib, ops
    g = torch.Generator().manual_seed(seed)
    x = F.normalize(torch.randn(b, d, generator=g), dim=1).bfloat16().cuda()
    y = F.normalize(torch.randn(b, d, generator=g), dim=1).bfloat16().cuda()
    k = _lib.CLIP if kind == "clip" else _lib.LIT
    _loss, r, c, _diag = ops.loss_forward(k, x, y, 0.07)
    go = torch.full((1,), 0.5, device="cuda")
    scale = ops.grad_scale(b, 0.07, False)

    def outputs():
        dx = torch.full((b, d), float("nan"), device="cuda")
        dy = torch.full((b, d), float("nan"), device="cuda") if kind == "clip" else None
        return dx, dy

    status = ops.new_status(x.device)
    dx_ws, dy_ws = outputs()
    ops.grad_block(k, x, y, 0.07, r, c, go, scale, dx_ws, _lib.STORE_F32, dy_ws, _lib.STORE_F32, status=status)
    dx_st, dy_st = outputs()
    # the call itself must not take device memory from anyone: neither from the driver (free bytes of the
    # device unchanged) nor from torch's allocator (bytes handed out unchanged)
    gc.collect()            # garbage of earlier tests must not be freed (or its blocks reused) in between
    torch.cuda.synchronize()
    free0, _total = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    ops.grad_block_static(k, x, y, 0.07, r, c, go, scale, dx_st, _lib.STORE_F32, dy_st, _lib.STORE_F32, status=status)
    torch.cuda.synchronize()
    if strict_free:     # a kernel's first launch lets the driver load its code lazily, which may take device
        assert torch.cuda.mem_get_info()[0] == free0        # memory: checked on a repeat of an earlier case
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    ops.read_status(status)
    # the answer is also right by the CPU oracle, not only equal to the workspace entry point's
    xf, yf = x.float().cpu(), y.float().cpu()
    if kind == "clip":
        _rl, rx, ry = dense.clip_dense(xf, yf, 0.07, True, grad_output=0.5)
        refs = (rx, ry)
    else:
        _rl, rx = dense.lit_dense(xf, yf, 0.07, True, grad_output=0.5)
        refs = (rx, None)
    for got, ref in zip((dx_st, dy_st), refs):
        if ref is None:
            continue
        max_rel, cos = dense.grad_errors(got.cpu(), ref)
        assert max_rel <= dense.GRAD_MAX_REL and cos >= dense.GRAD_COS_MIN, (max_rel, cos)
    for got, ref in ((dx_st, dx_ws), (dy_st, dy_ws)):
        if ref is None:
            continue
        assert torch.isfinite(got).all()
        max_rel, cos = dense.grad_errors(got, ref)
        assert max_rel <= dense.GRAD_MAX_REL and cos >= dense.GRAD_COS_MIN, (max_rel, cos)
        if bit_identical:
            assert torch.equal(got, ref)  # same kernels, same order of additions: bit-identical in practice


def test_static_scratch_matches_workspace_twice_in_a_row():
    # second call: different shape and kind, so it runs over the first call's left-overs
    _case(1024, 256, "clip", 21)
    _case(384, 72, "lit", 22)
    _case(1024, 256, "clip", 21, strict_free=True)


def test_static_scratch_ignores_the_blocking_test_hook():
    """meclip_debug_set_blocking changes how meclip_grad cuts its work into panels; the entry point without
    a workspace plans from its built-in constants, so an override left active by another test neither
    makes it overrun its fixed scratch nor makes it refuse a block inside its limit."""
    from memoryefficientclip_b200 import _lib
    lib = _lib.load()
    _lib.check(lib.meclip_debug_set_blocking(256, 256 * 256 * 2))
    try:
        _case(1024, 256, "clip", 23, bit_identical=False)   # meclip_grad adds its panels in another order here
    finally:
        lib.meclip_debug_set_blocking(0, 0)


def test_static_scratch_rejects_oversize_blocks():
    from memoryefficientclip_b200 import _lib, ops
    x = torch.zeros(4104, 8, dtype=torch.bfloat16, device="cuda")
    r = torch.ones(4104, device="cuda")
    dx = torch.zeros(4104, 8, device="cuda")
    with pytest.raises(_lib.MeclipError) as e:
        ops.grad_block_static(_lib.LIT, x, x, 0.07, r, None, None, 1.0, dx, _lib.STORE_F32, None, 0)
    assert e.value.code == _lib.ENOSPC and "4096" in str(e.value)
