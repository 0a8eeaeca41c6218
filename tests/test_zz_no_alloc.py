"""meclip_grad_static: the backward for callers that cannot hand over a workspace (a plugin
interface with fixed inputs/outputs, or a process whose device memory is fully owned by
another allocator).  It must give what meclip_grad gives, call after call, although every
call reuses the same built-in scratch array and finds the previous call's data in it.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else; it also passes when run alone in a fresh process.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import dense

pytestmark = pytest.mark.gpu


def _case(b, d, kind, seed):
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
    ops.grad_block_static(k, x, y, 0.07, r, c, go, scale, dx_st, _lib.STORE_F32, dy_st, _lib.STORE_F32, status=status)
    ops.read_status(status)
    for got, ref in ((dx_st, dx_ws), (dy_st, dy_ws)):
        if ref is None:
            continue
        assert torch.isfinite(got).all()
        max_rel, cos = dense.grad_errors(got, ref)
        assert max_rel <= dense.GRAD_MAX_REL and cos >= dense.GRAD_COS_MIN, (max_rel, cos)
        assert torch.equal(got, ref)      # same kernels, same order: bit-identical in practice


def test_static_scratch_matches_workspace_twice_in_a_row():
    # second call: different shape and kind, so it runs over the first call's left-overs
    _case(1024, 256, "clip", 21)
    _case(384, 72, "lit", 22)
    _case(1024, 256, "clip", 21)


def test_static_scratch_rejects_oversize_blocks():
    from memoryefficientclip_b200 import _lib, ops
    x = torch.zeros(4104, 8, dtype=torch.bfloat16, device="cuda")
    r = torch.ones(4104, device="cuda")
    dx = torch.zeros(4104, 8, device="cuda")
    with pytest.raises(_lib.MeclipError) as e:
        ops.grad_block_static(_lib.LIT, x, x, 0.07, r, None, None, 1.0, dx, _lib.STORE_F32, None, 0)
    assert e.value.code == _lib.ENOSPC and "4096" in str(e.value)
