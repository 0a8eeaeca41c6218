"""The ring-distributed loss on real GPUs (NCCL), one process per GPU, against the dense
oracle on the concatenated batch.  Skipped on a box with a single GPU."""
import os
import socket
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from oracle import dense

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, kind, b_global, d, dtype_name, normalize, outdir, transport="peer"):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if transport == "peer_unexportable":
        # memory from virtual-memory segments has no IPC handle: the peer transport must notice and every rank must
        # fall back to send/recv together
        transport = "peer"
        torch.cuda.memory._set_allocator_settings("expandable_segments:True")
    os.environ["MECLIP_RING_TRANSPORT"] = transport      # read when the ring module is imported (below)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from memoryefficientclip_b200 import ring
        dtype = getattr(torch, dtype_name)
        g = torch.Generator().manual_seed(0)
        x = torch.randn(b_global, d, generator=g)
        y = torch.randn(b_global, d, generator=g)
        if not normalize:
            x, y = torch.nn.functional.normalize(x, dim=1), torch.nn.functional.normalize(y, dim=1)
        x, y = x.to(dtype), y.to(dtype)
        b = b_global // world
        xl = x[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
        yl = y[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
        cls = ring.RingMemoryEfficientCLIPLoss if kind == "clip" else ring.RingMemoryEfficientLiTLoss
        loss = cls(0.07, not normalize)(xl, yl)
        loss.backward()
        torch.cuda.synchronize()
        torch.save({"loss": loss.item(), "dx": xl.grad.float().cpu(),
                    "dy": None if yl.grad is None else yl.grad.float().cpu()}, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(world, kind, b_global, d, dtype_name, normalize, transport="peer"):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_worker, args=(world, _free_port(), kind, b_global, d, dtype_name, normalize, outdir, transport),
                 nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"r{r}.pt")) for r in range(world)]
    dtype = getattr(torch, dtype_name)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(b_global, d, generator=g)
    y = torch.randn(b_global, d, generator=g)
    if not normalize:
        x, y = torch.nn.functional.normalize(x, dim=1), torch.nn.functional.normalize(y, dim=1)
    x, y = x.to(dtype), y.to(dtype)
    if kind == "clip":
        loss, gx, gy = dense.clip_dense(x, y, 0.07, not normalize)
    else:
        loss, gx = dense.lit_dense(x, y, 0.07, not normalize)
        gy = None
    dx = torch.cat([r["dx"] for r in res])
    for r in res:
        assert dense.loss_rel_err(r["loss"], loss) <= dense.LOSS_RTOL
    if gy is not None:
        dy = torch.cat([r["dy"] for r in res])
        dense.assert_parity(res[0]["loss"], loss, (dx, dy), (gx, gy), f"ring{world} {kind}")
    else:
        assert all(r["dy"] is None for r in res)
        dense.assert_parity(res[0]["loss"], loss, (dx,), (gx,), f"ring{world} {kind}")


@pytest.mark.parametrize("kind,b,d,dtype,normalize", [("clip", 1024, 128, "bfloat16", False),
                                                      ("clip", 768, 64, "float32", True),
                                                      ("lit", 512, 256, "bfloat16", True),
                                                      ("clip", 512, 100, "float16", True),
                                                      ("clip", 640, 52, "float32", False)])
def test_ring_two_gpus(kind, b, d, dtype, normalize):
    _run(2, kind, b, d, dtype, normalize)


def test_ring_two_gpus_send_recv_transport():
    """The fallback transport (NCCL send/recv from rank to rank instead of copy-engine fetches from peer memory)."""
    _run(2, "clip", 1024, 128, "bfloat16", False, transport="nccl")


def test_ring_two_gpus_falls_back_when_memory_cannot_be_exported():
    _run(2, "clip", 768, 64, "float32", True, transport="peer_unexportable")


def _interleaved_worker(rank, world, port, outdir):
    """Two forwards, then their backwards in reverse order: the second forward publishes into the other slot,
    the first backward to run fetches the newer shards, the second one the older ones; the partial-gradient
    inbox is used by two backwards in a row."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from memoryefficientclip_b200 import ring
        b_global, d = 768, 96
        b = b_global // world
        out = {}
        mod = ring.RingMemoryEfficientCLIPLoss(0.07, False)
        batches, losses = [], []
        for seed in (1, 2):
            g = torch.Generator().manual_seed(seed)
            x = torch.randn(b_global, d, generator=g)[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
            y = torch.randn(b_global, d, generator=g)[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
            batches.append((x, y))
            losses.append(mod(x, y))
        losses[1].backward()
        losses[0].backward()
        torch.cuda.synchronize()
        for i, (x, y) in enumerate(batches):
            out[i] = {"loss": losses[i].item(), "dx": x.grad.float().cpu(), "dy": y.grad.float().cpu()}
        torch.save(out, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ring_two_forwards_then_two_backwards():
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_interleaved_worker, args=(world, _free_port(), outdir), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"r{r}.pt")) for r in range(world)]
    for i, seed in enumerate((1, 2)):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(768, 96, generator=g)
        y = torch.randn(768, 96, generator=g)
        loss, gx, gy = dense.clip_dense(x, y, 0.07, False)
        dx = torch.cat([r[i]["dx"] for r in res])
        dy = torch.cat([r[i]["dy"] for r in res])
        dense.assert_parity(res[0][i]["loss"], loss, (dx, dy), (gx, gy), f"interleaved step {i}")


def _large_worker(rank, world, port, outdir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from memoryefficientclip_b200 import ring, synth
        b_global, d = 16384, 768
        b = b_global // world
        img, txt = synth.clip_pair(b_global, d, torch.bfloat16, True, row_start=rank * b, rows=b)
        xl, yl = img.cuda().requires_grad_(True), txt.cuda().requires_grad_(True)
        loss = ring.RingMemoryEfficientCLIPLoss(0.07, True)(xl, yl)
        loss.backward()
        torch.cuda.synchronize()
        torch.save({"loss": loss.item(), "dx": xl.grad.float().cpu(), "dy": yl.grad.float().cpu()},
                   os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ring_two_gpus_large_against_streaming_oracle():
    """Global B = 16384, D = 768 (several tiles, panels and a real overlap of transfers and kernels):
    exact loss and sampled gradient rows from the row-blocked CPU oracle."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    from memoryefficientclip_b200 import synth
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_large_worker, args=(world, _free_port(), outdir), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"r{r}.pt")) for r in range(world)]
    img, txt = synth.clip_pair(16384, 768, torch.bfloat16, True)
    rows = [0, 127, 4096, 8191, 8192, 12000, 16383]
    ref = dense.clip_streaming(img.float(), txt.float(), 0.07, rows)
    dx = torch.cat([r["dx"] for r in res])
    dy = torch.cat([r["dy"] for r in res])
    for r in res:
        assert dense.loss_rel_err(r["loss"], ref["loss"]) <= dense.LOSS_RTOL
    for got, want in ((dx[rows], ref["dx_rows"]), (dy[rows], ref["dy_rows"])):
        max_rel, cos = dense.grad_errors(got, want)
        assert max_rel <= dense.GRAD_MAX_REL and cos >= dense.GRAD_COS_MIN, (max_rel, cos)


def _temperature_worker(rank, world, port, mode, outdir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from memoryefficientclip_b200 import ring
        b_global, d = 768, 96
        g = torch.Generator().manual_seed(4)
        x = torch.randn(b_global, d, generator=g)
        y = torch.randn(b_global, d, generator=g)
        b = b_global // world
        xl = x[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
        yl = y[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
        t = torch.nn.Parameter(torch.tensor(0.1, device="cuda"))
        loss = ring.RingMemoryEfficientCLIPLoss(t, False, temperature_grad=mode)(xl, yl)
        loss.backward()
        torch.cuda.synchronize()
        torch.save({"dt": t.grad.item()}, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["local", "global"])
def test_ring_two_gpus_temperature_gradient(mode):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_temperature_worker, args=(world, _free_port(), mode, outdir), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"r{r}.pt"))["dt"] for r in range(world)]
    g = torch.Generator().manual_seed(4)
    x = torch.randn(768, 96, generator=g)
    y = torch.randn(768, 96, generator=g)
    want = dense.temperature_grad_dense(x, y, 0.1, "clip", False)
    got = [sum(res)] if mode == "local" else res
    for v in got:
        assert abs(v - want) <= 1e-2 * abs(want), (v, want)


def _siglip_inputs(b_global, d):
    g = torch.Generator().manual_seed(17)
    img = torch.randn(b_global, d, generator=g)
    txt = img + 0.7 * torch.randn(b_global, d, generator=g)
    return img.bfloat16(), txt.bfloat16()


def _siglip_worker(rank, world, port, outdir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from memoryefficientclip_b200 import ring
        b_global, d = 1024, 256
        img, txt = _siglip_inputs(b_global, d)
        b = b_global // world
        xl = img[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
        yl = txt[rank * b:(rank + 1) * b].cuda().requires_grad_(True)
        mod = ring.RingMemoryEfficientSigLIPLoss(10.0, -10.0, False, param_grad="global").cuda()
        loss = mod(xl, yl)
        loss.backward()
        torch.cuda.synchronize()
        torch.save({"loss": loss.item(), "dx": xl.grad.float().cpu(), "dy": yl.grad.float().cpu(),
                    "dlogt": mod.log_logit_scale.grad.item(), "db": mod.logit_bias.grad.item()},
                   os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ring_two_gpus_siglip():
    """The sigmoid loss over the ring: every block is independent; text-gradient partials go to their owners."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_siglip_worker, args=(world, _free_port(), outdir), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"r{r}.pt")) for r in range(world)]
    img, txt = _siglip_inputs(1024, 256)
    rl, rx, ry, rt, rb = dense.siglip_dense(img, txt, 10.0, -10.0, False)
    dx = torch.cat([r["dx"] for r in res])
    dy = torch.cat([r["dy"] for r in res])
    for r in res:
        assert dense.loss_rel_err(r["loss"], rl) <= dense.LOSS_RTOL
        assert abs(r["dlogt"] / 10.0 - rt) <= 1e-2 * max(abs(rt), 1e-6), (r["dlogt"] / 10.0, rt)
        assert abs(r["db"] - rb) <= 1e-2 * max(abs(rb), 1e-6), (r["db"], rb)
    dense.assert_parity(res[0]["loss"], rl, (dx, dy), (rx, ry), "ring2 siglip")


def test_ring_four_gpus():
    _run(4, "clip", 2048, 128, "bfloat16", False)


def test_ring_eight_gpus():
    _run(8, "clip", 4096, 64, "bfloat16", True)
