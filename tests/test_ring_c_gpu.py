"""meclip_ring_sum_exp / meclip_ring_grad: one library call queues a rank's whole ring (tile kernels on the
compute stream, shard fetches and partial-gradient pushes on the copy stream).

On one GPU the ranks are emulated one after the other in one process: every "peer" address is a local
one, the copies are real copy-engine copies, and the host synchronises where a multi-process caller has its
barrier.  Checked against the dense oracle on the concatenated batch and against the single-GPU kernels."""
import pytest
import torch

from oracle import dense

pytestmark = pytest.mark.gpu


def _operands(batch, d, seed):
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(seed)
    x = F.normalize(torch.randn(batch, d, generator=g), dim=1).bfloat16()
    y = F.normalize(x.float() + 0.7 * F.normalize(torch.randn(batch, d, generator=g), dim=1), dim=1).bfloat16()
    return x, y


def _ring_step(kind, world, b, d, temperature, x_cpu, y_cpu):
    """(loss, dx [B, d] fp32, dy [B, d] fp32 or None, row_sum [B], col_sum [B] or None) through the ring calls."""
    from memoryefficientclip_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    batch = world * b
    x, y = x_cpu.to(dev), y_cpu.to(dev)
    xs = [x[p * b:(p + 1) * b] for p in range(world)]
    ys = [y[p * b:(p + 1) * b] for p in range(world)]
    copy = torch.cuda.Stream(device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    calls = [ops.RingCall(p, world, xs[p], [s.data_ptr() for s in ys], ys[p], copy) for p in range(world)]
    clip = kind == _lib.CLIP

    sums = [ops.ring_sum_exp(c, kind, temperature, status=status) for c in calls]
    row_sum = [s[0] for s in sums]
    diag = [s[2] for s in sums]
    col_sum = torch.stack([s[1] for s in sums]).sum(0) if clip else None        # the caller's reduce-scatter
    loss = torch.zeros((), dtype=torch.float32, device=dev)
    for p in range(world):
        ops.loss_finalize(kind, row_sum[p], col_sum[p] if clip else None, diag[p], temperature, 1.0 / batch, loss,
                          accumulate=True)

    go = torch.ones(1, dtype=torch.float32, device=dev)
    scale = ops.grad_scale(batch, temperature, False)
    inbox = [torch.full((max(world - 1, 1), b, d), float("nan"), dtype=torch.float32, device=dev) for _ in range(world)]
    col_all = col_sum.reshape(-1).contiguous() if clip else None
    grads = [ops.ring_grad(calls[p], kind, temperature, row_sum[p], col_all, go, scale,
                           [t.data_ptr() for t in inbox], status=status) for p in range(world)]
    torch.cuda.synchronize()                                                     # the caller's barrier
    dys = None
    if clip:
        dys = [g[1] for g in grads]
        if world > 1:
            for p in range(world):
                ops.accumulate_many_f32(dys[p], inbox[p])
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    dx = torch.cat([g[0] for g in grads])
    return (loss.item(), dx, torch.cat(dys) if clip else None, torch.cat(row_sum),
            col_sum.reshape(-1) if clip else None)


@pytest.mark.parametrize("world,b,d", [(1, 384, 64), (2, 256, 128), (3, 320, 72), (4, 256, 64), (5, 128, 200)])
def test_ring_calls_clip_match_the_dense_oracle(world, b, d):
    from memoryefficientclip_b200 import _lib
    x, y = _operands(world * b, d, 31 + world)
    loss, dx, dy, _r, _c = _ring_step(_lib.CLIP, world, b, d, 0.07, x, y)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(loss, rl, (dx.cpu(), dy.cpu()), (rx, ry), f"ring calls, {world} ranks")


@pytest.mark.parametrize("world,b,d", [(1, 256, 64), (3, 256, 96)])
def test_ring_calls_lit_match_the_dense_oracle(world, b, d):
    from memoryefficientclip_b200 import _lib
    x, y = _operands(world * b, d, 41 + world)
    loss, dx, dy, _r, _c = _ring_step(_lib.LIT, world, b, d, 0.05, x, y)
    assert dy is None
    rl, rx = dense.lit_dense(x, y, 0.05, True)[:2]
    dense.assert_parity(loss, rl, (dx.cpu(),), (rx,), f"ring calls LiT, {world} ranks")


def test_ring_calls_match_the_single_gpu_kernels_at_a_size_with_many_tiles():
    """4 ranks of 2048 rows, D = 256: every step has several tiles per SM pair and the fetches overlap them."""
    from memoryefficientclip_b200 import _lib, ops
    world, b, d, t = 4, 2048, 256, 0.07
    x, y = _operands(world * b, d, 5)
    loss, dx, dy, row_sum, col_sum = _ring_step(_lib.CLIP, world, b, d, t, x, y)
    xg, yg = x.cuda(), y.cuda()
    l1, r1, c1, _d1 = ops.loss_forward(_lib.CLIP, xg, yg, t)
    go = torch.ones(1, dtype=torch.float32, device="cuda")
    dx1, dy1 = ops.loss_backward(_lib.CLIP, xg, yg, t, r1, c1, go, ops.grad_scale(world * b, t, False), torch.float32,
                                 torch.float32)
    torch.cuda.synchronize()
    assert abs(loss - l1.item()) <= 1e-5 * abs(l1.item())
    torch.testing.assert_close(row_sum, r1, rtol=1e-5, atol=0)
    torch.testing.assert_close(col_sum, c1, rtol=1e-5, atol=0)
    for got, ref in ((dx, dx1), (dy, dy1)):
        mr, cs = dense.grad_errors(got.cpu(), ref.cpu())
        assert mr <= 2e-3 and cs >= 0.999999, (mr, cs)


def test_ring_calls_reject_bad_descriptors():
    from memoryefficientclip_b200 import _lib, ops
    x, y = _operands(256, 64, 3)
    xg, yg = x.cuda(), y.cuda()
    copy = torch.cuda.Stream()
    call = ops.RingCall(0, 2, xg[:128], [yg[:128].data_ptr(), 0], yg[:128], copy)      # a peer address is missing
    with pytest.raises(_lib.MeclipError):
        ops.ring_sum_exp(call, _lib.CLIP, 0.07)
    call = ops.RingCall(0, 2, xg[:128], [yg[:128].data_ptr(), yg[128:].data_ptr()], yg[:128], torch.cuda.current_stream())
    with pytest.raises(_lib.MeclipError):                                              # compute == copy stream
        ops.ring_sum_exp(call, _lib.CLIP, 0.07)


def _two_process_worker(rank, world, port, b, d, outdir):
    """Real peers: one process per GPU, shards and inboxes mapped through CUDA IPC, NCCL only for the small
    collectives and the barriers of the caller."""
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from memoryefficientclip_b200 import _lib, _peer, ops
        t, batch = 0.07, world * b
        x, y = _operands(batch, d, 77)
        xl = x[rank * b:(rank + 1) * b].to(dev)
        published = y[rank * b:(rank + 1) * b].to(dev)
        inbox = torch.full((world - 1, b, d), float("nan"), dtype=torch.float32, device=dev)
        shard_addr, ok1 = _peer._map_everywhere(published, None, rank, world, dev)
        inbox_addr, ok2 = _peer._map_everywhere(inbox, None, rank, world, dev)
        assert ok1 and ok2
        copy = torch.cuda.Stream(device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        call = ops.RingCall(rank, world, xl, shard_addr, published, copy)
        torch.cuda.synchronize()
        dist.barrier()                                        # every shard is in place
        row_sum, col_part, diag = ops.ring_sum_exp(call, _lib.CLIP, t, status=status)
        col_sum = torch.empty(b, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(col_sum, col_part.reshape(-1))
        loss = torch.zeros((), dtype=torch.float32, device=dev)
        ops.loss_finalize(_lib.CLIP, row_sum, col_sum, diag, t, 1.0 / batch, loss)
        dist.all_reduce(loss)
        col_all = torch.empty(batch, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(col_all, col_sum)
        go = torch.ones(1, dtype=torch.float32, device=dev)
        dx, dy = ops.ring_grad(call, _lib.CLIP, t, row_sum, col_all, go, ops.grad_scale(batch, t, False), inbox_addr,
                               status=status)
        torch.cuda.synchronize()
        dist.barrier()                                        # every rank's pushes have landed
        ops.accumulate_many_f32(dy, inbox)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        torch.save({"loss": loss.item(), "dx": dx.cpu(), "dy": dy.cpu()}, os.path.join(outdir, f"r{rank}.pt"))
        dist.barrier()                                        # nobody unmaps while a peer could still copy
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ring_calls_between_processes(world):
    import os
    import socket
    import tempfile
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    b, d = 512, 128
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_two_process_worker, args=(world, port, b, d, outdir), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"r{r}.pt")) for r in range(world)]
    x, y = _operands(world * b, d, 77)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(res[0]["loss"], rl, (torch.cat([r["dx"] for r in res]), torch.cat([r["dy"] for r in res])),
                        (rx, ry), f"ring calls, {world} processes")
