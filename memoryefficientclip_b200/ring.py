"""Ring-distributed CLIP / LiT loss for one NVLink box: one process per GPU.

Rank r keeps its B/N image rows (first argument) for the whole step.  At ring step s it works
on text shard (r + s) mod N, which is in local HBM before any kernel reads it.  How a shard
gets there is the transport's business:
  peer (default on GPUs)  every rank publishes its shard in a buffer the other ranks have mapped
          (CUDA IPC) and fetches the shard of step s+1 from its owner with a copy-engine copy while
          the kernels of step s run (_peer.PeerShards): no SM is taken from the tile kernels;
  send/recv  the shards travel rank to rank (NCCL on GPUs without peer mapping, gloo in the CPU
          tests): rank r sends the shard it works on to r-1 and receives the next one from r+1.

forward   row sums finish locally; per-shard column partial sums [N, b] are
          reduce-scattered so that each rank ends with the column sums of its own
          shard; the loss is the all-reduced sum of the local terms.
backward  column sums are all-gathered (B floats); d(first) accumulates locally in
          fp32 over the N steps; the d(second) partial a rank computes for a visiting
          shard goes straight to the shard's owner while the next step computes
          (copy-engine writes into the owner's inbox, or send/recv), and the owner adds the
          N-1 partials in the order of the ring steps: a reduce-scatter spread over the steps,
          no [N, b, D] table.

The reference has no distributed code; the result is defined as the single-process
loss on the concatenated global batch (rank-major row order).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib, ops


# Phase marks for a per-phase breakdown of one step (benchmarks): while TRACE is a list, the functions below
# append (label, CUDA event) pairs recorded on the current stream; the time between two consecutive marks is
# what the compute stream spent on the phase the LATER mark names.  None (the default) records nothing.
TRACE = None


def _mark(label: str) -> None:
    if TRACE is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        TRACE.append((label, ev))


def _nvtx_push(name: str, t) -> None:
    """NVTX range around one ring step (visible in a profiler's timeline; a no-op on CPU tensors)."""
    if t.is_cuda:
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop(t) -> None:
    if t.is_cuda:
        torch.cuda.nvtx.range_pop()


def trace_durations(trace):
    """{label: milliseconds} summed over the marks of a finished (synchronised) trace."""
    out = {}
    for (_, a), (label, b) in zip(trace[:-1], trace[1:]):
        out[label] = out.get(label, 0.0) + a.elapsed_time(b)
    return out


# how the shards of the second argument reach the ranks: "peer" (copy-engine fetches from the owner's published
# buffer) or "nccl" (send/recv from rank to rank)
_TRANSPORT = __import__("os").environ.get("MECLIP_RING_TRANSPORT", "peer").lower()


def shard_at(rank: int, step: int, world: int) -> int:
    """Index of the text shard rank `rank` holds at ring step `step`."""
    return (rank + step) % world


def ring_neighbours(rank: int, world: int):
    """(destination of this rank's sends, source of its receives)."""
    return (rank - 1) % world, (rank + 1) % world


class CudaBlockOps:
    """Block primitives on the sm_100a kernels (the only product implementation).  Every launch gets the
    device's shared status word, so a bounded wait that ran out surfaces at the next forward."""

    # tensor temperatures / logit scales are read by the kernels on the device (no host synchronisation)
    device_scalars = True

    @staticmethod
    def _st(t):
        return ops.status_word(t.device)

    def begin_step(self, device):
        ops.poll_status(device)

    def end_step(self, device):
        ops.post_status(device)

    def rotation(self, y_own, group, rank, world, token=None):
        """Shard transport: peer-memory fetches by the copy engines (the default on GPUs; see _peer.py) or,
        with MECLIP_RING_TRANSPORT=nccl, send/recv from rank to rank (returns None: the caller's default)."""
        if _TRANSPORT != "peer" or not y_own.is_cuda:
            return None
        from . import _peer
        ex = token[0] if token is not None else _peer.get(group, rank, world, y_own.shape[0], y_own.shape[1],
                                                          y_own.dtype, y_own.device)
        if ex is None:
            return None
        if token is None:
            token = (ex, ex.publish(y_own))       # forward: publish this rank's shard for everyone
            return _PeerRotation(ex, token[1], y_own, rank, world, announce=True), token
        ex.check_live(token[1])                   # backward: the shards of its own forward
        return _PeerRotation(ex, token[1], y_own, rank, world), token

    def partial_inbox(self, rows, cols, device, group, rank, world):
        """Copy-engine transport of the partial text gradients (None: send/recv)."""
        if _TRANSPORT != "peer" or device.type != "cuda":
            return None
        from . import _peer
        return _peer.get_inbox(group, rank, world, rows, cols, device)

    def prepare(self, x, normalize):
        if normalize:
            return ops.normalize_fwd(x, True)
        return ops.as_operand(x), None

    def sum_exp(self, kind, x_hat, y_hat, t, row_sum, col_sum, diag, row_off, col_off):
        ops.sum_exp(kind, x_hat, y_hat, t, row_sum, col_sum, diag, row_off, col_off, status=self._st(x_hat))

    def local_loss_sum(self, kind, row_sum, col_sum, diag, t, scale):
        out = torch.empty((), dtype=torch.float32, device=row_sum.device)
        ops.loss_finalize(kind, row_sum, col_sum, diag, t, scale, out)
        return out

    def grad(self, kind, x_hat, y_hat, t, row_sum, col_sum, go, scale, dx_acc, dy_out, row_off, col_off, workspace,
             sum_g_s=None, scale_rule=0):
        ops.grad_block(kind, x_hat, y_hat, t, row_sum, col_sum, go, scale, dx_acc, _lib.ACCUM_F32, dy_out,
                       _lib.STORE_F32, row_off, col_off, workspace, status=self._st(x_hat), sum_g_s=sum_g_s,
                       scale_rule=scale_rule)

    def new_sum(self, device):
        return torch.zeros(2, dtype=torch.float32, device=device)

    # one-pass LiT (the forward contracts E with [Y | 1]; no ring backward at all)
    lit_one_pass = True

    def prepare_ext(self, y, normalize):
        y_ext, _inv = ops.normalize_fwd(y, normalize, extra_cols=8)
        d_pad = y_ext.shape[1] - 8
        ops.lit_extend(y_ext, d_pad)
        return y_ext, d_pad

    def new_u(self, rows, d_pad, device):
        return torch.zeros(rows, d_pad + 8, dtype=torch.float32, device=device)

    def lit_fused_block(self, x_hat, y_ext, d_pad, t, u, row_off, col_off, workspace):
        ops.lit_fused_block(x_hat, y_ext, d_pad, t, u, _lib.ACCUM_F32, row_off, col_off, workspace,
                            status=self._st(x_hat))

    def lit_fused_stats(self, x_hat, y_ext, u, d_pad):
        return ops.lit_fused_stats(x_hat, y_ext, u, d_pad)

    def lit_fused_bwd(self, u, y_ext, row_sum, go, scale, d_out, out_dtype, temperature=None, scale_rule=0):
        return ops.lit_fused_backward(u, y_ext, row_sum, go, scale, d_out, out_dtype, temperature, scale_rule)

    def siglip_sum(self, x_hat, y_hat, logit_scale, logit_bias, row_sum, diag, row_off, col_off):
        ops.siglip_sum(x_hat, y_hat, logit_scale, logit_bias, row_sum, diag, row_off, col_off, status=self._st(x_hat))

    def siglip_local_loss(self, row_sum, diag, logit_scale, logit_bias, scale):
        out = torch.empty((), dtype=torch.float32, device=row_sum.device)
        ops.siglip_loss_finalize(row_sum, diag, logit_scale, logit_bias, scale, out)
        return out

    def siglip_grad(self, x_hat, y_hat, logit_scale, logit_bias, go, scale, dx_acc, dy_out, row_off, col_off, workspace,
                    sums):
        ops.siglip_grad_block(x_hat, y_hat, logit_scale, logit_bias, go, scale, dx_acc, _lib.ACCUM_F32, dy_out,
                              _lib.STORE_F32, row_off, col_off, workspace, sums, status=self._st(x_hat))

    def workspace(self, rows, cols, d, device):
        return ops.grad_workspace(rows, cols, d, device)

    def accumulate(self, dst, src):
        ops.accumulate_f32(dst, src)

    def accumulate_many(self, dst, srcs):
        ops.accumulate_many_f32(dst, srcs)

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


class _SendRecvRotation:
    """The shards travel rank to rank: at step s a rank sends the shard it works on to rank-1 and receives
    the next one from rank+1 (NCCL on GPUs, gloo in the CPU tests)."""

    def __init__(self, y_own, group, rank, world):
        self.group, self.rank, self.world = group, rank, world
        self.bufs = [y_own, torch.empty_like(y_own)] if world > 1 else [y_own]
        if world > 2:
            self.bufs.append(torch.empty_like(y_own))      # never receive into the caller's own shard
        self.cur = 0
        self.nxt = 0
        self.reqs = []

    def begin(self, step):
        """Called before the step's kernels are queued; returns the shard they work on."""
        if step + 1 < self.world:
            self.nxt = 1 + (step % 2) if self.world > 2 else 1
            self.reqs = _rotate(self.bufs[self.cur], self.bufs[self.nxt], self.group, self.rank, self.world)
        return self.bufs[self.cur]

    def end(self, step):
        """Called after the step's kernels were queued: wait for the transfer that ran under them."""
        for r in self.reqs:
            r.wait()
        self.reqs = []
        if step + 1 < self.world:
            self.cur = self.nxt

    def finish(self):
        pass


class _PeerRotation:
    """Every rank fetches the shard of step s+1 from its owner's published buffer with the copy engines
    while the kernels of step s run (_peer.PeerShards)."""

    def __init__(self, exchange, gen, y_own, rank, world, announce=False):
        self.ex, self.gen, self.rank, self.world = exchange, gen, rank, world
        self.y_own = y_own
        self.announce = announce          # forward: the shards were just published, the ranks have to be told
        self.recv = [torch.empty_like(y_own) for _ in range(min(2, world - 1))]
        self.kernels_done = {}
        self.fetched = {}

    def _prefetch(self, step):
        """Queue the fetch of the shard of `step`; the buffer it lands in was last read by the kernels of step - 2."""
        if step < self.world:
            owner = shard_at(self.rank, step, self.world)
            self.fetched[step] = self.ex.fetch(self.gen, owner, self.recv[step % len(self.recv)],
                                               after=self.kernels_done.get(step - 2))

    def begin(self, step):
        if not (step == 0 and self.announce):
            self._prefetch(step + 1)
        if step == 0:
            return self.y_own
        torch.cuda.current_stream().wait_event(self.fetched.pop(step))
        return self.recv[step % len(self.recv)]

    def end(self, step):
        ev = torch.cuda.Event()
        ev.record()
        self.kernels_done[step] = ev
        if step == 0 and self.announce:       # the own shard's kernels are queued: now the collective, then the fetch
            self.ex.announce()
            self._prefetch(1)

    def finish(self):
        """End of a backward that has no other collective behind its fetches: a one-word all-reduce on the copy
        stream, which the compute stream waits for, so that this rank's next publish (which overwrites a slot)
        cannot overtake another rank that is still fetching from it."""
        torch.cuda.current_stream().wait_event(self.ex.fetches_done_everywhere())


def _rotation(block, y_own, group, rank, world, token=None):
    """(rotation, token): the block implementation may bring its own shard transport; the token is what a
    backward needs to find the same shards again."""
    if world > 1 and hasattr(block, "rotation"):
        made = block.rotation(y_own, group, rank, world, token)
        if made is not None:
            return made
    return _SendRecvRotation(y_own, group, rank, world), None


def ring_forward(block, kind, x_hat, y_hat, temperature, group, rank, world):
    """Returns (loss, row_sum [b], col_sum_own [b] or None, diag [b], transport token for the backward)."""
    b, d = x_hat.shape
    dev = x_hat.device
    clip = kind == _lib.CLIP
    row_sum = torch.zeros(b, dtype=torch.float32, device=dev)
    diag = torch.zeros(b, dtype=torch.float32, device=dev)
    col_part = torch.zeros(world, b, dtype=torch.float32, device=dev) if clip else None
    rot, token = _rotation(block, y_hat, group, rank, world)
    _mark("fwd_setup")
    for step in range(world):
        shard = shard_at(rank, step, world)
        _nvtx_push(f"ring_fwd_step{step}", x_hat)
        y_cur = rot.begin(step)
        _mark("fwd_exposed_shard_wait")
        block.sum_exp(kind, x_hat, y_cur, temperature, row_sum, col_part[shard] if clip else None, diag,
                      rank * b, shard * b)
        _mark("fwd_kernels")
        rot.end(step)
        _nvtx_pop(x_hat)
        _mark("fwd_exposed_shard_wait")
    col_sum = None
    if clip:
        if world > 1:
            col_sum = torch.empty(b, dtype=torch.float32, device=dev)
            block.reduce_scatter(col_sum, col_part, group)
        else:
            col_sum = col_part[0]
    _mark("fwd_reduce_scatter_col_sums")
    loss = block.local_loss_sum(kind, row_sum, col_sum, diag, temperature, 1.0 / (b * world))
    if world > 1:
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
    _mark("fwd_loss_all_reduce")
    return loss, row_sum, col_sum, diag, token


def _exchange_partial(send_buf, recv_buf, group, rank, world, step):
    """The partial computed at ring step `step` belongs to shard (rank+step): send it to that rank
    and receive, from rank (rank-step), the partial it computed for this rank's own shard."""
    dst = (rank + step) % world
    src = (rank - step) % world
    dst_g = dist.get_global_rank(group, dst) if group is not None else dst
    src_g = dist.get_global_rank(group, src) if group is not None else src
    p2p = [dist.P2POp(dist.isend, send_buf, dst_g, group), dist.P2POp(dist.irecv, recv_buf, src_g, group)]
    return dist.batch_isend_irecv(p2p)


def _ring_backward_loop(block, x_hat, y_hat, group, rank, world, want_dy, grad_call, token=None):
    """The backward choreography shared by the softmax and the sigmoid losses.  grad_call(y_shard, shard,
    dx_acc, dy_out, workspace) runs the block kernels: dx_acc accumulates in fp32, dy_out is stored.
    The partial gradient a rank computes for a visiting shard goes straight to the shard's owner while the next
    step computes: with copy-engine writes into the owner's inbox (block.partial_inbox, see _peer.PeerInbox)
    or, without peer memory, with send/recv; the owner adds the partials in the order of the ring steps."""
    b, d = x_hat.shape
    dev = x_hat.device
    dx = torch.zeros(b, d, dtype=torch.float32, device=dev)
    dy = torch.empty(b, d, dtype=torch.float32, device=dev) if want_dy else None       # own shard: step 0 stores it
    exchange = want_dy and world > 1
    inbox_peer = block.partial_inbox(b, d, dev, group, rank, world) if exchange and hasattr(block, "partial_inbox") else None
    part = [torch.empty(b, d, dtype=torch.float32, device=dev) for _ in range(2)] if exchange else []
    inbox = [torch.empty(b, d, dtype=torch.float32, device=dev) for _ in range(2)] if exchange and inbox_peer is None else []
    workspace = block.workspace(b, b, d, dev)
    rot, _ = _rotation(block, y_hat, group, rank, world, token)
    pending = None          # send/recv: (requests, inbox buffer) of the previous step's partial exchange
    pushed = {}             # peer inbox: step -> event after which part[step % 2] may be written again
    _mark("bwd_setup")
    for step in range(world):
        shard = shard_at(rank, step, world)
        _nvtx_push(f"ring_bwd_step{step}", x_hat)
        y_cur = rot.begin(step)
        _mark("bwd_exposed_shard_wait")
        out = None
        if want_dy:
            out = dy if step == 0 else part[step % 2]
            if step - 2 in pushed:      # the copy out of this buffer had a whole ring step to finish
                torch.cuda.current_stream().wait_event(pushed.pop(step - 2))
        grad_call(y_cur, shard, dx, out, workspace)
        _mark("bwd_kernels")
        if pending is not None:          # the exchange started one step ago ran under this step's kernels
            for r in pending[0]:
                r.wait()
            _mark("bwd_exposed_partial_wait")
            block.accumulate(dy, pending[1])
            _mark("bwd_accumulate_f32")
            pending = None
        if exchange and step > 0:
            if inbox_peer is not None:
                done = torch.cuda.Event()
                done.record()
                pushed[step] = inbox_peer.push(step, part[step % 2], done)
            else:
                pending = (_exchange_partial(part[step % 2], inbox[step % 2], group, rank, world, step), inbox[step % 2])
        rot.end(step)
        _nvtx_pop(x_hat)
        _mark("bwd_exposed_shard_wait")
    if pending is not None:
        for r in pending[0]:
            r.wait()
        _mark("bwd_exposed_last_partial_wait")
        block.accumulate(dy, pending[1])
        _mark("bwd_accumulate_f32")
    if inbox_peer is not None:
        torch.cuda.current_stream().wait_event(inbox_peer.arrived())     # every rank's pushes have landed
        _mark("bwd_exposed_last_partial_wait")
        if hasattr(block, "accumulate_many") and dy.numel() % 4 == 0:
            block.accumulate_many(dy, inbox_peer.local)      # one pass, the partial of ring step 1 first
        else:
            for step in range(1, world):
                block.accumulate(dy, inbox_peer.local[step - 1])
        _mark("bwd_accumulate_f32")
    elif world > 1:
        rot.finish()
    return dx, dy


def ring_backward(block, kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, group, rank, world,
                  sum_g_s=None, scale_rule=0, token=None):
    """Returns (dx fp32 [b, D], dy_own fp32 [b, D] or None) w.r.t. the normalised operands.
    sum_g_s: optional zeroed pair; element 0 receives sum_ij G_ij S_ij over this rank's rows and ALL columns."""
    b = x_hat.shape[0]
    clip = kind == _lib.CLIP
    col_all = None
    if clip:
        if world > 1:
            col_all = torch.empty(world, b, dtype=torch.float32, device=x_hat.device)
            _mark("fwd_to_bwd_gap")
            block.all_gather(col_all, col_sum, group)
            _mark("bwd_all_gather_col_sums")
        else:
            col_all = col_sum.view(1, b)
    extra = {} if sum_g_s is None else {"sum_g_s": sum_g_s}
    if scale_rule:
        extra["scale_rule"] = scale_rule

    def grad_call(y_shard, shard, dx_acc, dy_out, workspace):
        block.grad(kind, x_hat, y_shard, temperature, row_sum, col_all[shard] if clip else None, grad_out, grad_scale,
                   dx_acc, dy_out, rank * b, shard * b, workspace, **extra)

    return _ring_backward_loop(block, x_hat, y_hat, group, rank, world, clip, grad_call, token)


def ring_lit_fused_forward(block, x_hat, y_ext, d_pad, temperature, group, rank, world):
    """One-pass LiT over the ring: at every step the visiting shard's block adds E_block [Y_shard | 1] to u, so
    after the N steps u = [E Y | r | 0...] for the local rows and the backward needs no ring at all.
    Returns (loss, u, row_sum)."""
    b = x_hat.shape[0]
    u = block.new_u(b, d_pad, x_hat.device)
    workspace = block.workspace(b, b, d_pad + 8, x_hat.device)
    rot, _ = _rotation(block, y_ext, group, rank, world)
    for step in range(world):
        shard = shard_at(rank, step, world)
        y_cur = rot.begin(step)
        block.lit_fused_block(x_hat, y_cur, d_pad, temperature, u, rank * b, shard * b, workspace)
        rot.end(step)
    row_sum, diag = block.lit_fused_stats(x_hat, y_ext, u, d_pad)        # the positives are the own shard's rows
    loss = block.local_loss_sum(_lib.LIT, row_sum, None, diag, temperature, 1.0 / (b * world))
    if world > 1:
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
    return loss, u, row_sum


def ring_siglip_forward(block, x_hat, y_hat, logit_scale, logit_bias, group, rank, world):
    """Sigmoid loss of the global batch: every block is independent (no row or column sums to finish)."""
    b = x_hat.shape[0]
    dev = x_hat.device
    row_sum = torch.zeros(b, dtype=torch.float32, device=dev)
    diag = torch.zeros(b, dtype=torch.float32, device=dev)
    rot, token = _rotation(block, y_hat, group, rank, world)
    for step in range(world):
        shard = shard_at(rank, step, world)
        y_cur = rot.begin(step)
        block.siglip_sum(x_hat, y_cur, logit_scale, logit_bias, row_sum, diag, rank * b, shard * b)
        rot.end(step)
    loss = block.siglip_local_loss(row_sum, diag, logit_scale, logit_bias, 1.0 / (b * world))
    if world > 1:
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
    return loss, token


def ring_siglip_backward(block, x_hat, y_hat, logit_scale, logit_bias, grad_out, grad_scale, group, rank, world,
                         sums=None, token=None):
    """Returns (dx, dy_own) fp32; sums (optional zeroed pair) receives {sum G S, sum G} over this rank's rows."""
    b = x_hat.shape[0]
    if world > 1 and hasattr(block, "partial_inbox"):
        # The peer inbox is reused by every backward; this loss has no collective at the start of its backward,
        # so a one-word all-reduce takes that place: a rank joins it only after it has consumed the partials of
        # its previous backward, and this backward's pushes are queued behind kernels that wait for it.
        gate = torch.zeros(1, dtype=torch.float32, device=x_hat.device)
        dist.all_reduce(gate, group=group)
        grad_out = grad_out + 0.0 * gate

    def grad_call(y_shard, shard, dx_acc, dy_out, workspace):
        block.siglip_grad(x_hat, y_shard, logit_scale, logit_bias, grad_out, grad_scale, dx_acc, dy_out, rank * b,
                          shard * b, workspace, sums)

    return _ring_backward_loop(block, x_hat, y_hat, group, rank, world, True, grad_call, token)


class RingContrastiveLossFn(torch.autograd.Function):
    """apply(x_local, y_local, temperature, kind, stable, normalize, group, block_ops, temperature_grad)
    -> global loss.

    A tensor temperature that requires grad receives a gradient (the reference has none, clip_loss.py:256):
    temperature_grad "local" gives each rank the part of dL/dT that comes from its own rows, so the parts
    of all ranks ADD UP to the global dL/dT - the same convention as the feature gradients, which are
    d(global loss)/d(local features); "global" all-reduces, every rank gets the whole dL/dT."""

    @staticmethod
    def forward(ctx, x, y, temperature, kind, stable, normalize, group, block, temperature_grad="local"):
        assert x.shape == y.shape and x.dim() == 2
        assert temperature_grad in ("local", "global")
        t_is_tensor = isinstance(temperature, torch.Tensor)
        ctx.ring_t = (temperature, temperature_grad) if t_is_tensor and temperature.requires_grad else None
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        block = block or CudaBlockOps()
        if t_is_tensor and getattr(block, "device_scalars", False):
            temperature = temperature.detach()       # stays on the device: the kernels read it there
        else:
            temperature = float(temperature.detach().item()) if t_is_tensor else float(temperature)
            assert temperature > 0.0, "temperature must be positive"
        if hasattr(block, "begin_step"):
            block.begin_step(x.device)
        from . import _function
        ctx.ring_fused = (kind == _lib.LIT and _function._LIT_FUSED and ctx.needs_input_grad[0] and ctx.ring_t is None
                          and getattr(block, "lit_one_pass", False))
        if ctx.ring_fused:
            x_hat, inv_x = block.prepare(x, normalize)
            y_ext, d_pad = block.prepare_ext(y, normalize)
            loss, u, row_sum = ring_lit_fused_forward(block, x_hat, y_ext, d_pad, temperature, group, rank, world)
            ctx.save_for_backward(*([u, y_ext, row_sum] + ([x_hat, inv_x] if normalize else [])))
            ctx.ring = (temperature, kind, bool(stable), bool(normalize), x.dtype, y.dtype, x.shape[1], group, rank,
                        world, block)
            return loss
        _mark("fwd_begin")
        x_hat, inv_x = block.prepare(x, normalize)
        y_hat, inv_y = block.prepare(y, normalize)
        _mark("fwd_normalize")
        loss, row_sum, col_sum, _diag, ctx.ring_token = ring_forward(block, kind, x_hat, y_hat, temperature, group,
                                                                     rank, world)
        saved = [x_hat, y_hat, row_sum]
        if col_sum is not None:
            saved.append(col_sum)
        if normalize:
            saved += [inv_x, inv_y]
        ctx.save_for_backward(*saved)
        ctx.ring = (temperature, kind, bool(stable), bool(normalize), x.dtype, y.dtype, x.shape[1], group, rank,
                    world, block)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        temperature, kind, stable, normalize, x_dtype, y_dtype, d, group, rank, world, block = ctx.ring
        saved = list(ctx.saved_tensors)
        if getattr(ctx, "ring_fused", False):
            u, y_ext, row_sum = saved[:3]
            go = grad_output.detach().to(device=u.device, dtype=torch.float32).reshape(1).contiguous()
            scale, rule = ops.grad_scale_args(u.shape[0] * world, temperature, stable)
            t_kw = {"temperature": temperature, "scale_rule": rule} if rule else {}
            if normalize:
                x_hat, inv_x = saved[3:]
                g32 = block.lit_fused_bwd(u, y_ext, row_sum, go, scale, x_hat.shape[1], torch.float32, **t_kw)
                dx = block.finish_grad(g32, x_hat, inv_x, x_dtype, d)
            else:
                dx = block.lit_fused_bwd(u, y_ext, row_sum, go, scale, d, x_dtype, **t_kw)
            if hasattr(block, "end_step"):
                block.end_step(u.device)
            return dx, None, None, None, None, None, None, None, None
        x_hat, y_hat, row_sum = saved[:3]
        rest = saved[3:]
        col_sum = rest.pop(0) if kind == _lib.CLIP else None
        inv_x, inv_y = rest if normalize else (None, None)
        b = x_hat.shape[0]
        go = grad_output.detach().to(device=x_hat.device, dtype=torch.float32).reshape(1).contiguous()
        scale, rule = ops.grad_scale_args(b * world, temperature, stable)
        t_info = getattr(ctx, "ring_t", None)
        sum_g_s = block.new_sum(x_hat.device) if t_info is not None else None
        dx, dy = ring_backward(block, kind, x_hat, y_hat, temperature, row_sum, col_sum, go, scale, group, rank, world,
                               sum_g_s=sum_g_s, scale_rule=rule, token=getattr(ctx, "ring_token", None))
        dx = block.finish_grad(dx, x_hat, inv_x, x_dtype, d)
        if dy is not None:
            dy = block.finish_grad(dy, y_hat, inv_y, y_dtype, d)
        _mark("bwd_normalize_jacobian")
        dt = None
        if t_info is not None:
            t_param, mode = t_info
            if mode == "global" and world > 1:
                dist.all_reduce(sum_g_s, op=dist.ReduceOp.SUM, group=group)
            # sum_ij G_ij S_ij = g B dL/d(1/T) with g = grad_out * scale and B the global batch.  With a
            # device-resident temperature `scale` was formed for T = 1 and completed by the kernels, so the
            # same power of T is applied here in tensor arithmetic (no host read).
            if rule:
                t32 = temperature.to(torch.float32).reshape(())
                scale_t = scale / (torch.sqrt(t32) if stable else t32)
                dt = (-sum_g_s[0] / (scale_t * (b * world) * t32 * t32)).reshape(t_param.shape)
            else:
                dt = (sum_g_s[0] * (-1.0 / (scale * b * world * temperature * temperature))).reshape(t_param.shape)
            dt = dt.to(t_param.dtype)
        if hasattr(block, "end_step"):
            block.end_step(x_hat.device)
        return dx, dy, dt, None, None, None, None, None, None


class _RingLoss(nn.Module):
    _kind = _lib.CLIP
    _stable = False

    def __init__(self, temperature=0.07, normalized_inputs=False, process_group=None, block_ops=None,
                 temperature_grad="local"):
        super().__init__()
        self.temperature = temperature          # a float, or a 0-dim tensor / nn.Parameter to learn it
        self.normalized_inputs = normalized_inputs
        self.process_group = process_group
        self.block_ops = block_ops
        self.temperature_grad = temperature_grad

    def forward(self, first_local, second_local):
        return RingContrastiveLossFn.apply(first_local, second_local, self.temperature, self._kind, self._stable,
                                           not self.normalized_inputs, self.process_group, self.block_ops,
                                           self.temperature_grad)


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


class RingSigLIPLossFn(torch.autograd.Function):
    """apply(x_local, y_local, logit_scale, logit_bias, normalize, group, block_ops, param_grad) -> global
    sigmoid loss (1/B) sum_ij softplus(-z_ij (t <x_i, y_j> + b)) over the concatenated batch.

    Gradients: d(global loss)/d(local features); for a tensor scale / bias, param_grad "local" returns the part
    that comes from this rank's rows (the parts of all ranks add up to the global gradient), "global" all-reduces."""

    @staticmethod
    def forward(ctx, x, y, logit_scale, logit_bias, normalize, group, block, param_grad="local"):
        assert x.shape == y.shape and x.dim() == 2
        assert param_grad in ("local", "global")
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        block = block or CudaBlockOps()
        x_hat, inv_x = block.prepare(x, normalize)
        y_hat, inv_y = block.prepare(y, normalize)
        if getattr(block, "device_scalars", False):
            t = logit_scale.detach() if isinstance(logit_scale, torch.Tensor) else float(logit_scale)
            bias = logit_bias.detach() if isinstance(logit_bias, torch.Tensor) else float(logit_bias)
        else:
            t = float(logit_scale.detach().item()) if isinstance(logit_scale, torch.Tensor) else float(logit_scale)
            bias = float(logit_bias.detach().item()) if isinstance(logit_bias, torch.Tensor) else float(logit_bias)
        if hasattr(block, "begin_step"):
            block.begin_step(x.device)
        loss, ctx.ring_token = ring_siglip_forward(block, x_hat, y_hat, t, bias, group, rank, world)
        ctx.save_for_backward(*([x_hat, y_hat] + ([inv_x, inv_y] if normalize else [])))
        ctx.ring = (t, bias, bool(normalize), x.dtype, y.dtype, x.shape[1], group, rank, world, block, param_grad,
                    (logit_scale.shape, logit_scale.dtype) if isinstance(logit_scale, torch.Tensor) else None,
                    (logit_bias.shape, logit_bias.dtype) if isinstance(logit_bias, torch.Tensor) else None)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        t, bias, normalize, x_dtype, y_dtype, d, group, rank, world, block, param_grad, t_tensor, b_tensor = ctx.ring
        saved = list(ctx.saved_tensors)
        x_hat, y_hat = saved[:2]
        inv_x, inv_y = saved[2:] if normalize else (None, None)
        need = ctx.needs_input_grad
        b = x_hat.shape[0]
        go = grad_output.detach().to(device=x_hat.device, dtype=torch.float32).reshape(1).contiguous()
        want_tb = bool(need[2] or need[3])
        sums = block.new_sum(x_hat.device) if want_tb else None
        # grad_scale = t / B; with a device-resident t the kernel multiplies 1/B by t itself
        gscale = 1.0 / (b * world) if ops.is_dev(t) else t / (b * world)
        dx, dy = ring_siglip_backward(block, x_hat, y_hat, t, bias, go, gscale, group, rank, world, sums,
                                      token=getattr(ctx, "ring_token", None))
        dx = block.finish_grad(dx, x_hat, inv_x, x_dtype, d)
        dy = block.finish_grad(dy, y_hat, inv_y, y_dtype, d)
        dt = db = None
        if want_tb:
            if param_grad == "global" and world > 1:
                dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
            # G = g (sigmoid(a) - I) with g = grad_out * t / B: grad_out * dL/dt = sum(G S) / t, dL/db = sum(G) / t
            if need[2] and t_tensor is not None:
                dt = (sums[0] / t).reshape(t_tensor[0]).to(t_tensor[1])
            if need[3] and b_tensor is not None:
                db = (sums[1] / t).reshape(b_tensor[0]).to(b_tensor[1])
        if hasattr(block, "end_step"):
            block.end_step(x_hat.device)
        return dx, dy, dt, db, None, None, None, None


class RingMemoryEfficientSigLIPLoss(nn.Module):
    """forward(image_features_local, text_features_local): sigmoid loss of the global batch, with
    log_logit_scale and logit_bias as parameters (t = exp(log_logit_scale)) unless learnable=False."""

    def __init__(self, init_logit_scale=10.0, init_logit_bias=-10.0, normalized_inputs=False, learnable=True,
                 process_group=None, block_ops=None, param_grad="local"):
        super().__init__()
        import math
        self.normalized_inputs = normalized_inputs
        self.process_group = process_group
        self.block_ops = block_ops
        self.param_grad = param_grad
        ls = torch.tensor(math.log(init_logit_scale), dtype=torch.float32)
        lb = torch.tensor(float(init_logit_bias), dtype=torch.float32)
        if learnable:
            self.log_logit_scale = nn.Parameter(ls)
            self.logit_bias = nn.Parameter(lb)
        else:
            self.register_buffer("log_logit_scale", ls)
            self.register_buffer("logit_bias", lb)

    def forward(self, first_local, second_local):
        return RingSigLIPLossFn.apply(first_local, second_local, self.log_logit_scale.exp(), self.logit_bias,
                                      not self.normalized_inputs, self.process_group, self.block_ops, self.param_grad)
