"""Ring-distributed CLIP / LiT loss for one NVLink box: one process per GPU.

Rank r keeps its B/N image rows (first argument) for the whole step.  The N text
shards (second argument) rotate around the ring: at step s rank r works on shard
(r + s) mod N while it already sends that shard to rank r-1 and receives the next
one from rank r+1 (NCCL send/recv on the process group's stream, waited on only
after the tile kernels of the step have been queued, so the transfer runs under the
MMAs).  A shard always lands in local HBM before a kernel reads it.

forward   row sums finish locally; per-shard column partial sums [N, b] are
          reduce-scattered so that each rank ends with the column sums of its own
          shard; the loss is the all-reduced sum of the local terms.
backward  column sums are all-gathered (B floats); d(first) accumulates locally in
          fp32 over the N steps; the d(second) partial a rank computes for a visiting
          shard is sent straight to the shard's owner while the next step computes
          (a reduce-scatter spread over the steps: only the last partial's transfer is
          exposed, and no [N, b, D] table exists); the owner adds what it receives.

The reference has no distributed code; the result is defined as the single-process
loss on the concatenated global batch (rank-major row order).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib, ops


def shard_at(rank: int, step: int, world: int) -> int:
    """Index of the text shard rank `rank` holds at ring step `step`."""
    return (rank + step) % world


def ring_neighbours(rank: int, world: int):
    """(destination of this rank's sends, source of its receives)."""
    return (rank - 1) % world, (rank + 1) % world


class CudaBlockOps:
    """Block primitives on the sm_100a kernels (the only product implementation)."""

    def prepare(self, x, normalize):
        if normalize:
            return ops.normalize_fwd(x, True)
        return ops.as_operand(x), None

    def sum_exp(self, kind, x_hat, y_hat, t, row_sum, col_sum, diag, row_off, col_off):
        ops.sum_exp(kind, x_hat, y_hat, t, row_sum, col_sum, diag, row_off, col_off)

    def local_loss_sum(self, kind, row_sum, col_sum, diag, t, scale):
        out = torch.empty((), dtype=torch.float32, device=row_sum.device)
        ops.loss_finalize(kind, row_sum, col_sum, diag, t, scale, out)
        return out

    def grad(self, kind, x_hat, y_hat, t, row_sum, col_sum, go, scale, dx_acc, dy_out, row_off, col_off, workspace):
        ops.grad_block(kind, x_hat, y_hat, t, row_sum, col_sum, go, scale, dx_acc, _lib.ACCUM_F32, dy_out,
                       _lib.STORE_F32, row_off, col_off, workspace)

    def workspace(self, rows, cols, d, device):
        return ops.grad_workspace(rows, cols, d, device)

    def accumulate(self, dst, src):
        ops.accumulate_f32(dst, src)

    def reduce_scatter(self, out, table, group):
        dist.reduce_scatter_tensor(out.view(-1), table.view(-1), op=dist.ReduceOp.SUM, group=group)

    def all_gather(self, table, part, group):
        dist.all_gather_into_tensor(table.view(-1), part.contiguous().view(-1), group=group)

    def finish_grad(self, g_f32, x_hat, inv_norm, out_dtype, d):
        if inv_norm is None and out_dtype == torch.float32 and d == g_f32.shape[1]:
            return g_f32
        return ops.normalize_bwd(g_f32, x_hat, inv_norm, out_dtype, d)


def _rotate(cur: torch.Tensor, nxt: torch.Tensor, group, rank: int, world: int):
    """Start sending `cur` to rank-1 and receiving `nxt` from rank+1; returns the requests."""
    dst, src = ring_neighbours(rank, world)
    dst_g = dist.get_global_rank(group, dst) if group is not None else dst
    src_g = dist.get_global_rank(group, src) if group is not None else src
    p2p = [dist.P2POp(dist.isend, cur, dst_g, group), dist.P2POp(dist.irecv, nxt, src_g, group)]
    return dist.batch_isend_irecv(p2p)


def ring_forward(block, kind, x_hat, y_hat, temperature, group, rank, world):
    """Returns (loss, row_sum [b], col_sum_own [b] or None, diag [b])."""
    b, d = x_hat.shape
    dev = x_hat.device
    clip = kind == _lib.CLIP
    row_sum = torch.zeros(b, dtype=torch.float32, device=dev)
    diag = torch.zeros(b, dtype=torch.float32, device=dev)
    col_part = torch.zeros(world, b, dtype=torch.float32, device=dev) if clip else None
    bufs = [y_hat, torch.empty_like(y_hat)] if world > 1 else [y_hat]
    if world > 2:
        bufs.append(torch.empty_like(y_hat))      # never receive into the caller's own shard
    cur = 0
    for step in range(world):
        shard = shard_at(rank, step, world)
        reqs = []
        if step + 1 < world:
            nxt = 1 + (step % 2) if world > 2 else 1
            reqs = _rotate(bufs[cur], bufs[nxt], group, rank, world)
        block.sum_exp(kind, x_hat, bufs[cur], temperature, row_sum, col_part[shard] if clip else None, diag,
                      rank * b, shard * b)
        for r in reqs:
            r.wait()
        if step + 1 < world:
            cur = nxt
    col_sum = None
    if clip:
        if world > 1:
            col_sum = torch.empty(b, dtype=torch.float32, device=dev)
            block.reduce_scatter(col_sum, col_part, group)
        else:
            col_sum = col_part[0]
    loss = block.local_loss_sum(kind, row_sum, col_sum, diag, temperature, 1.0 / (b * world))
    if world > 1:
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
    return loss, row_sum, col_sum, diag


def _exchange_partial(send_buf, recv_buf, group, rank, world, step):
    """The partial computed at ring step `step` belongs to shard (rank+step): send it to that rank
    and receive, from rank (rank-step), the partial it computed for this rank's own shard."""
    dst = (rank + step) % world
    src = (rank - step) % world
    dst_g = dist.get_global_rank(group, dst) if group is not None else dst
    src_g = dist.get_global_rank(group, src) if group is not None else src
    p2p = [dist.P2POp(dist.isend, send_buf, dst_g, group), dist.P2POp(dist.irecv, recv_buf, src_g, group)]
    return dist.batch_isend_irecv(p2p)


def ring_backward(block, kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, group, rank, world):
    """Returns (dx fp32 [b, D], dy_own fp32 [b, D] or None) w.r.t. the normalised operands."""
    b, d = x_hat.shape
    dev = x_hat.device
    clip = kind == _lib.CLIP
    col_all = None
    if clip:
        if world > 1:
            col_all = torch.empty(world, b, dtype=torch.float32, device=dev)
            block.all_gather(col_all, col_sum, group)
        else:
            col_all = col_sum.view(1, b)
    dx = torch.zeros(b, d, dtype=torch.float32, device=dev)
    dy = torch.empty(b, d, dtype=torch.float32, device=dev) if clip else None          # own shard: step 0 stores it
    part = [torch.empty(b, d, dtype=torch.float32, device=dev) for _ in range(2)] if clip and world > 1 else []
    inbox = [torch.empty(b, d, dtype=torch.float32, device=dev) for _ in range(2)] if clip and world > 1 else []
    workspace = block.workspace(b, b, d, dev)
    bufs = [y_hat, torch.empty_like(y_hat)] if world > 1 else [y_hat]
    if world > 2:
        bufs.append(torch.empty_like(y_hat))
    cur = 0
    pending = None          # (requests, inbox buffer) of the previous step's partial exchange
    for step in range(world):
        shard = shard_at(rank, step, world)
        reqs = []
        if step + 1 < world:
            nxt = 1 + (step % 2) if world > 2 else 1
            reqs = _rotate(bufs[cur], bufs[nxt], group, rank, world)
        out = None
        if clip:
            out = dy if step == 0 else part[step % 2]
        block.grad(kind, x_hat, bufs[cur], temperature, row_sum, col_all[shard] if clip else None, grad_out,
                   grad_scale, dx, out, rank * b, shard * b, workspace)
        if pending is not None:          # the exchange started one step ago ran under this step's kernels
            for r in pending[0]:
                r.wait()
            block.accumulate(dy, pending[1])
            pending = None
        if clip and step > 0:
            pending = (_exchange_partial(part[step % 2], inbox[step % 2], group, rank, world, step), inbox[step % 2])
        for r in reqs:
            r.wait()
        if step + 1 < world:
            cur = nxt
    if pending is not None:
        for r in pending[0]:
            r.wait()
        block.accumulate(dy, pending[1])
    return dx, dy


class RingContrastiveLossFn(torch.autograd.Function):
    """apply(x_local, y_local, temperature, kind, stable, normalize, group, block_ops) -> global loss."""

    @staticmethod
    def forward(ctx, x, y, temperature, kind, stable, normalize, group, block):
        assert x.shape == y.shape and x.dim() == 2
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        block = block or CudaBlockOps()
        x_hat, inv_x = block.prepare(x, normalize)
        y_hat, inv_y = block.prepare(y, normalize)
        loss, row_sum, col_sum, _diag = ring_forward(block, kind, x_hat, y_hat, temperature, group, rank, world)
        saved = [x_hat, y_hat, row_sum]
        if col_sum is not None:
            saved.append(col_sum)
        if normalize:
            saved += [inv_x, inv_y]
        ctx.save_for_backward(*saved)
        ctx.ring = (float(temperature), kind, bool(stable), bool(normalize), x.dtype, y.dtype, x.shape[1], group, rank,
                    world, block)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        temperature, kind, stable, normalize, x_dtype, y_dtype, d, group, rank, world, block = ctx.ring
        saved = list(ctx.saved_tensors)
        x_hat, y_hat, row_sum = saved[:3]
        rest = saved[3:]
        col_sum = rest.pop(0) if kind == _lib.CLIP else None
        inv_x, inv_y = rest if normalize else (None, None)
        b = x_hat.shape[0]
        go = grad_output.detach().to(device=x_hat.device, dtype=torch.float32).reshape(1).contiguous()
        scale = ops.grad_scale(b * world, temperature, stable)
        dx, dy = ring_backward(block, kind, x_hat, y_hat, temperature, row_sum, col_sum, go, scale, group, rank, world)
        dx = block.finish_grad(dx, x_hat, inv_x, x_dtype, d)
        if dy is not None:
            dy = block.finish_grad(dy, y_hat, inv_y, y_dtype, d)
        return dx, dy, None, None, None, None, None, None


class _RingLoss(nn.Module):
    _kind = _lib.CLIP
    _stable = False

    def __init__(self, temperature=0.07, normalized_inputs=False, process_group=None, block_ops=None):
        super().__init__()
        self.temperature = temperature
        self.normalized_inputs = normalized_inputs
        self.process_group = process_group
        self.block_ops = block_ops

    def forward(self, first_local, second_local):
        return RingContrastiveLossFn.apply(first_local, second_local, self.temperature, self._kind, self._stable,
                                           not self.normalized_inputs, self.process_group, self.block_ops)


class RingMemoryEfficientCLIPLoss(_RingLoss):
    """forward(image_features_local, text_features_local): CLIP loss of the global batch."""
    _kind = _lib.CLIP


class RingStableMemoryEfficientCLIPLoss(_RingLoss):
    _kind = _lib.CLIP
    _stable = True


class RingMemoryEfficientLiTLoss(_RingLoss):
    """forward(text_features_local, image_features_local): text rows stay, image shards rotate."""
    _kind = _lib.LIT


class RingStableMemoryEfficientLiTLoss(_RingLoss):
    _kind = _lib.LIT
    _stable = True
