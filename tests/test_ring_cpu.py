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

    def grad(self, kind, x_hat, y_hat, t, row_sum, col_sum, go, scale, dx_acc, dy_out, row_off, col_off, workspace):
        e, _, _ = dense.sum_exp(x_hat.numpy(), y_hat.numpy(), t)
        e = torch.from_numpy(e)
        g = float(go) * scale
        if col_sum is not None:
            coef = (e / row_sum.double()[:, None] + e / col_sum.double()[None, :]) * (0.5 * g)
        else:
            coef = e / row_sum.double()[:, None] * g
        if row_off == col_off:
            coef -= torch.eye(e.shape[0], dtype=torch.float64) * g
        dx_acc += (coef @ y_hat).to(dx_acc.dtype)
        if dy_out is not None:
            dy_out.copy_((coef.t() @ x_hat).to(dy_out.dtype))

    def workspace(self, rows, cols, d, device):
        return None

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
