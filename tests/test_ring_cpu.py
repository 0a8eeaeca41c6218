"""Ring choreography on CPU ranks (gloo, world_size 2 and 3): shard rotation, the
reduce-scatter of column sums and of the text-gradient table, the loss all-reduce.
The tile kernels are replaced by a test double built on the oracle's closed form, so
this checks the host-side logic of memoryefficientclip_b200/ring.py only."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dense


class OracleBlockOps:
    """Same interface as ring.CudaBlockOps, fp64 CPU arithmetic."""

    def prepare(self, x, normalize):
        x = x.double()
        if normalize:
            inv = 1.0 / x.norm(dim=1).clamp_min(1e-12)
            return x * inv[:, None], inv
        return x, None

    def sum_exp(self, kind, x_hat, y_hat, t, row_sum, col_sum, diag, row_off, col_off):
        e, r, c = dense.sum_exp(x_hat.numpy(), y_hat.numpy(), t)
        row_sum += torch.from_numpy(r).to(row_sum.dtype)
        if col_sum is not None:
            col_sum += torch.from_numpy(c).to(col_sum.dtype)
        if row_off == col_off:
            diag.copy_((x_hat * y_hat).sum(dim=1).to(diag.dtype))

    def local_loss_sum(self, kind, row_sum, col_sum, diag, t, scale):
        term = torch.log(row_sum.double())
        if col_sum is not None:
            term = 0.5 * (term + torch.log(col_sum.double()))
        return ((term - (diag.double() - 1.0) / t).sum() * scale).float()

    def new_sum(self, device):
        return torch.zeros(2, dtype=torch.float64)

    def grad(self, kind, x_hat, y_hat, t, row_sum, col_sum, go, scale, dx_acc, dy_out, row_off, col_off, workspace,
             sum_g_s=None):
        e, _, _ = dense.sum_exp(x_hat.numpy(), y_hat.numpy(), t)
        e = torch.from_numpy(e)
        g = float(go) * scale
        if col_sum is not None:
            coef = (e / row_sum.double()[:, None] + e / col_sum.double()[None, :]) * (0.5 * g)
        else:
            coef = e / row_sum.double()[:, None] * g
        if row_off == col_off:
            coef -= torch.eye(e.shape[0], dtype=torch.float64) * g
        if sum_g_s is not None:
            sum_g_s[0] += (coef * (x_hat @ y_hat.t())).sum()
        dx_acc += (coef @ y_hat).to(dx_acc.dtype)
        if dy_out is not None:
            dy_out.copy_((coef.t() @ x_hat).to(dy_out.dtype))

    def workspace(self, rows, cols, d, device):
        return None

    # one-pass LiT: u += E_block [Y_shard | 1 | 0...]
    lit_one_pass = True

    def prepare_ext(self, y, normalize):
        y_hat, _ = self.prepare(y, normalize)
        ext = torch.zeros(y_hat.shape[0], 8, dtype=y_hat.dtype)
        ext[:, 0] = 1.0
        return torch.cat([y_hat, ext], dim=1), y_hat.shape[1]

    def new_u(self, rows, d_pad, device):
        return torch.zeros(rows, d_pad + 8, dtype=torch.float64)

    def lit_fused_block(self, x_hat, y_ext, d_pad, t, u, row_off, col_off, workspace):
        e, _, _ = dense.sum_exp(x_hat.numpy(), y_ext[:, :d_pad].contiguous().numpy(), t)
        u += torch.from_numpy(e) @ y_ext

    def lit_fused_stats(self, x_hat, y_ext, u, d_pad):
        return u[:, d_pad].clone(), (x_hat * y_ext[:, :d_pad]).sum(dim=1)

    def lit_fused_bwd(self, u, y_ext, row_sum, go, scale, d_out, out_dtype):
        g = float(go) * scale
        return (g * (u[:, :d_out] / row_sum[:, None] - y_ext[:, :d_out])).to(out_dtype)

    def _siglip_a_z(self, x_hat, y_hat, t, bias, row_off, col_off):
        a = (x_hat @ y_hat.t()) * t + bias
        z = -torch.ones_like(a)
        if row_off == col_off:
            z += 2.0 * torch.eye(a.shape[0], dtype=a.dtype)
        return a, z

    def siglip_sum(self, x_hat, y_hat, t, bias, row_sum, diag, row_off, col_off):
        a, z = self._siglip_a_z(x_hat, y_hat, t, bias, row_off, col_off)
        row_sum += (torch.nn.functional.softplus(-z * a).sum(dim=1) / np.log(2.0)).to(row_sum.dtype)

    def siglip_local_loss(self, row_sum, diag, t, bias, scale):
        return (row_sum.double().sum() * np.log(2.0) * scale).float()

    def siglip_grad(self, x_hat, y_hat, t, bias, go, scale, dx_acc, dy_out, row_off, col_off, workspace, sums):
        a, z = self._siglip_a_z(x_hat, y_hat, t, bias, row_off, col_off)
        coef = (torch.sigmoid(a) - (z + 1.0) / 2.0) * (float(go) * scale)
        if sums is not None:
            sums[0] += (coef * (x_hat @ y_hat.t())).sum()
            sums[1] += coef.sum()
        dx_acc += (coef @ y_hat).to(dx_acc.dtype)
        dy_out.copy_((coef.t() @ x_hat).to(dy_out.dtype))

    def accumulate(self, dst, src):
        dst += src

    def reduce_scatter(self, out, table, group):      # gloo has no reduce_scatter_tensor
        t = table.clone()
        dist.all_reduce(t, group=group)
        out.copy_(t[dist.get_rank(group)])

    def all_gather(self, table, part, group):
        parts = [torch.empty_like(part) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, part.contiguous(), group=group)
        table.copy_(torch.stack(parts))

    def finish_grad(self, g, x_hat, inv_norm, out_dtype, d):
        if inv_norm is not None:
            g = (g.double() - x_hat * (x_hat * g.double()).sum(dim=1, keepdim=True)) * inv_norm[:, None]
        return g.to(out_dtype)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, kind_name, normalize, stable, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from memoryefficientclip_b200 import _lib, ring
        b, d, t = 24, 16, 0.1
        g = torch.Generator().manual_seed(0)
        x = torch.randn(world * b, d, generator=g, dtype=torch.float64)
        y = torch.randn(world * b, d, generator=g, dtype=torch.float64)
        if not normalize:
            x = torch.nn.functional.normalize(x, dim=1)
            y = torch.nn.functional.normalize(y, dim=1)
        xl = x[rank * b:(rank + 1) * b].clone().requires_grad_(True)
        yl = y[rank * b:(rank + 1) * b].clone().requires_grad_(True)
        cls = {("clip", False): ring.RingMemoryEfficientCLIPLoss, ("clip", True): ring.RingStableMemoryEfficientCLIPLoss,
               ("lit", False): ring.RingMemoryEfficientLiTLoss, ("lit", True): ring.RingStableMemoryEfficientLiTLoss}
        mod = cls[(kind_name, stable)](t, not normalize, None, OracleBlockOps())
        loss = mod(xl, yl)
        loss.backward()
        out[rank] = (float(loss.detach()), xl.grad.numpy().copy(), None if yl.grad is None else yl.grad.numpy().copy(),
                     x.numpy(), y.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("kind_name,normalize,stable", [("clip", False, False), ("clip", True, True), ("lit", True, False)])
def test_ring_equals_global_dense(world, kind_name, normalize, stable):
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, kind_name, normalize, stable, out), nprocs=world, join=True)
        res = dict(out)
    b = 24
    x, y = torch.from_numpy(res[0][3]), torch.from_numpy(res[0][4])
    if kind_name == "clip":
        loss, gx, gy = dense.clip_dense(x, y, 0.1, not normalize, stable)
    else:
        loss, gx = dense.lit_dense(x, y, 0.1, not normalize, stable)
        gy = None
    for r in range(world):
        assert abs(res[r][0] - float(loss)) < 1e-5 * abs(float(loss))
        np.testing.assert_allclose(res[r][1], gx[r * b:(r + 1) * b].numpy(), rtol=1e-4, atol=1e-7)
        if gy is not None:
            np.testing.assert_allclose(res[r][2], gy[r * b:(r + 1) * b].numpy(), rtol=1e-4, atol=1e-7)
        else:
            assert res[r][2] is None


def _worker_t(rank, world, port, kind_name, stable, mode, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from memoryefficientclip_b200 import ring
        b, d = 20, 12
        g = torch.Generator().manual_seed(3)
        x = torch.randn(world * b, d, generator=g, dtype=torch.float64)
        y = torch.randn(world * b, d, generator=g, dtype=torch.float64)
        xl = x[rank * b:(rank + 1) * b].clone().requires_grad_(True)
        yl = y[rank * b:(rank + 1) * b].clone().requires_grad_(True)
        t = torch.nn.Parameter(torch.tensor(0.2, dtype=torch.float64))
        cls = {("clip", False): ring.RingMemoryEfficientCLIPLoss, ("clip", True): ring.RingStableMemoryEfficientCLIPLoss,
               ("lit", False): ring.RingMemoryEfficientLiTLoss}[(kind_name, stable)]
        mod = cls(t, False, None, OracleBlockOps(), temperature_grad=mode)
        assert list(mod.parameters()) == [t]
        (mod(xl, yl) * 1.5).backward()
        out[rank] = (float(t.grad), x.numpy(), y.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind_name,stable,mode", [("clip", False, "local"), ("clip", True, "global"), ("lit", False, "local")])
def test_ring_temperature_gradient(kind_name, stable, mode):
    """A tensor temperature gets dL/dT: per-rank parts that add up to it ("local"), or all of it on every rank."""
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker_t, args=(world, port, kind_name, stable, mode, out), nprocs=world, join=True)
        res = dict(out)
    x, y = torch.from_numpy(res[0][1]), torch.from_numpy(res[0][2])
    want = 1.5 * dense.temperature_grad_dense(x, y, 0.2, kind_name, False)   # Stable rescales feature gradients only
    if mode == "local":
        assert abs(sum(res[r][0] for r in range(world)) - want) < 1e-6 * max(1.0, abs(want))   # the ring keeps its sums in fp32
        assert abs(res[0][0] - res[1][0]) > 0            # the parts are different numbers
    else:
        for r in range(world):
            assert abs(res[r][0] - want) < 1e-6 * max(1.0, abs(want))   # the ring keeps its sums in fp32


def _worker_sig(rank, world, port, mode, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from memoryefficientclip_b200 import ring
        b, d = 16, 12
        g = torch.Generator().manual_seed(5)
        x = torch.randn(world * b, d, generator=g, dtype=torch.float64)
        y = torch.randn(world * b, d, generator=g, dtype=torch.float64)
        xl = x[rank * b:(rank + 1) * b].clone().requires_grad_(True)
        yl = y[rank * b:(rank + 1) * b].clone().requires_grad_(True)
        mod = ring.RingMemoryEfficientSigLIPLoss(5.0, -3.0, False, True, None, OracleBlockOps(), mode).double()
        loss = mod(xl, yl)
        loss.backward()
        out[rank] = (float(loss.detach()), xl.grad.numpy().copy(), yl.grad.numpy().copy(),
                     float(mod.log_logit_scale.grad), float(mod.logit_bias.grad), x.numpy(), y.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "local"), (3, "global")])
def test_ring_siglip_equals_global_dense(world, mode):
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker_sig, args=(world, port, mode, out), nprocs=world, join=True)
        res = dict(out)
    b = 16
    x, y = torch.from_numpy(res[0][5]), torch.from_numpy(res[0][6])
    loss, gx, gy, gt, gb = dense.siglip_dense(x, y, 5.0, -3.0, False)
    g_log_t = float(gt) * 5.0                  # the module learns log t
    for r in range(world):
        assert abs(res[r][0] - float(loss)) < 1e-5 * abs(float(loss))
        np.testing.assert_allclose(res[r][1], gx[r * b:(r + 1) * b].numpy(), rtol=1e-4, atol=1e-7)
        np.testing.assert_allclose(res[r][2], gy[r * b:(r + 1) * b].numpy(), rtol=1e-4, atol=1e-7)
    if mode == "local":
        assert abs(sum(res[r][3] for r in range(world)) - g_log_t) < 1e-5 * abs(g_log_t)
        assert abs(sum(res[r][4] for r in range(world)) - float(gb)) < 1e-5 * abs(float(gb))
    else:
        for r in range(world):
            assert abs(res[r][3] - g_log_t) < 1e-5 * abs(g_log_t)
            assert abs(res[r][4] - float(gb)) < 1e-5 * abs(float(gb))


def test_shard_schedule():
    from memoryefficientclip_b200 import ring
    for world in (1, 2, 4, 8):
        for rank in range(world):
            seen = sorted(ring.shard_at(rank, s, world) for s in range(world))
            assert seen == list(range(world))               # every shard visits every rank once
            assert ring.shard_at(rank, 0, world) == rank     # step 0 is the diagonal block
        for s in range(world):
            assert sorted(ring.shard_at(r, s, world) for r in range(world)) == list(range(world))
    assert ring.ring_neighbours(0, 4) == (3, 1)


def _worker_lost_send(rank, world, port, out):
    """Rank 1 never sends its shard (the message is dropped on the host): rank 0's receive must end with an
    error after the process group's time limit instead of blocking forever."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    t0 = time.monotonic()
    try:
        from memoryefficientclip_b200 import ring
        if rank == 1:
            real_rotate = ring._rotate

            def rotate_without_send(cur, nxt, group, rank_, world_):
                # the receive is posted, the send is skipped
                src = ring.ring_neighbours(rank_, world_)[1]
                return [dist.irecv(nxt, src, group)]

            ring._rotate = rotate_without_send
        b, d = 16, 8
        g = torch.Generator().manual_seed(rank)
        xl = torch.nn.functional.normalize(torch.randn(b, d, generator=g, dtype=torch.float64), dim=1).requires_grad_(True)
        yl = torch.nn.functional.normalize(torch.randn(b, d, generator=g, dtype=torch.float64), dim=1).requires_grad_(True)
        mod = ring.RingMemoryEfficientCLIPLoss(0.1, True, None, OracleBlockOps())
        try:
            mod(xl, yl)
            out[rank] = ("finished", time.monotonic() - t0)
        except Exception as e:      # noqa: BLE001 - whatever the backend raises when its wait runs out
            out[rank] = ("error: " + type(e).__name__, time.monotonic() - t0)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:           # noqa: BLE001 - the group is broken by design at this point
            pass


def test_lost_shard_send_surfaces_as_an_error_not_a_hang():
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        ctx = mp.spawn(_worker_lost_send, args=(2, port, out), nprocs=2, join=False)
        deadline = 60.0
        import time
        t0 = time.monotonic()
        while not ctx.join(timeout=1.0):
            if time.monotonic() - t0 > deadline:
                for p in ctx.processes:
                    p.kill()
                pytest.fail("a rank was still blocked after %.0f s" % deadline)
        res = dict(out)
    # rank 0 waited for a shard that was never sent: an error within the group's limit (4 s) plus slack
    assert res[0][0].startswith("error"), res
    assert res[0][1] < 30.0, res
