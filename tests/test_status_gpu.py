"""Time-out reporting and device-resident scalars of the module path.

A bounded wait that runs out is produced without disturbing any real kernel: the library's wait
probe is one tiny CTA that waits, with the tile kernels' own wait routine and a limit of a
millisecond, on a barrier nobody arrives on; it then sets the status word and ends normally.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import dense

pytestmark = pytest.mark.gpu


def _pair(b, d, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = F.normalize(torch.randn(b, d, generator=g), dim=1).to(dtype)
    y = F.normalize(torch.randn(b, d, generator=g), dim=1).to(dtype)
    return x, y


def test_expired_wait_is_reported_and_context_stays_usable():
    import memoryefficientclip_b200 as m
    from memoryefficientclip_b200 import _lib, ops
    status = ops.new_status(torch.device("cuda", 0))
    ops.read_status(status)                       # clear word: no error
    ops.debug_wait_probe(status, limit_ns=1_000_000)
    with pytest.raises(_lib.MeclipError) as e:
        ops.read_status(status)
    assert e.value.code == _lib.ETIMEOUT
    # the kernel gave up and returned: the context works, and a normal step is still right
    x, y = _pair(384, 64, 3)
    xg, yg = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    loss = m.MemoryEfficientCLIPLoss(0.07, True)(xg, yg)
    loss.backward()
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(loss.item(), rl, (xg.grad.cpu(), yg.grad.cpu()), (rx, ry), "after an expired wait")


def test_module_path_raises_on_the_next_forward():
    import memoryefficientclip_b200 as m
    from memoryefficientclip_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    mod = m.MemoryEfficientCLIPLoss(0.07, True)
    x, y = _pair(256, 64, 4)
    xg, yg = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    mod(xg, yg).backward()                        # a clean step: posts a clear status word
    torch.cuda.synchronize()
    mod(xg, yg).backward()                        # the poll at its start sees the clear word
    # a kernel of "this step" gives up a wait: the probe sets the module path's own status word
    ops.debug_wait_probe(ops.status_word(dev), limit_ns=1_000_000)
    ops.post_status(dev, force=True)
    torch.cuda.synchronize()
    with pytest.raises(_lib.MeclipError) as e:
        mod(xg, yg)
    assert e.value.code == _lib.ETIMEOUT
    # the word was cleared when the error was raised: the next step runs and is right
    xg.grad = yg.grad = None
    loss = mod(xg, yg)
    loss.backward()
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(loss.item(), rl, (xg.grad.cpu(), yg.grad.cpu()), (rx, ry), "after the raised time-out")
    ops.check_status(dev)                         # synchronous form: clean


def test_wait_probe_rejects_long_limits():
    from memoryefficientclip_b200 import _lib, ops
    status = ops.new_status(torch.device("cuda", 0))
    with pytest.raises(_lib.MeclipError) as e:
        ops.debug_wait_probe(status, limit_ns=10_000_000_000)
    assert e.value.code == _lib.EINVAL


@pytest.mark.parametrize("stable", [False, True])
@pytest.mark.parametrize("kind", ["clip", "lit"])
def test_learnable_temperature_without_host_sync(kind, stable):
    """A tensor temperature is read by the kernels on the device: forward + backward issue no
    synchronising call (torch's sync debug mode raises on one), and loss and gradients, the
    temperature's included, match the dense formulation."""
    import memoryefficientclip_b200 as m
    b, d, t0 = 512, 96, 0.05
    x, y = _pair(b, d, 5)
    cls = {("clip", False): m.MemoryEfficientCLIPLoss, ("clip", True): m.StableMemoryEfficientCLIPLoss,
           ("lit", False): m.MemoryEfficientLiTLoss, ("lit", True): m.StableMemoryEfficientLiTLoss}[(kind, stable)]

    def inputs():      # made outside the checked region: a copy from pageable host memory synchronises
        return (x.cuda().requires_grad_(True), y.cuda().requires_grad_(kind == "clip"),
                torch.tensor(t0, device="cuda", requires_grad=True))

    def run(xg, yg, t):
        loss = cls(t, normalized_inputs=False)(xg, yg)
        loss.backward()
        return loss

    run(*inputs())                                 # warm-up: library load, pinned status buffer, side streams
    xg, yg, t = inputs()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        loss = run(xg, yg, t)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    # dense reference with autograd through the temperature
    xr = x.double().requires_grad_(True)
    yr = y.double().requires_grad_(True)
    tr = torch.tensor(t0, dtype=torch.float64, requires_grad=True)
    logits = F.normalize(xr, dim=1) @ F.normalize(yr, dim=1).T / tr
    labels = torch.arange(b)
    ref = F.cross_entropy(logits, labels)
    if kind == "clip":
        ref = 0.5 * (ref + F.cross_entropy(logits.T, labels))
    ref.backward()
    fac = (b * t0) ** 0.5 if stable else 1.0       # the Stable variants scale the FEATURE gradients only
    assert abs(loss.item() - ref.item()) <= 1e-3 * abs(ref.item())
    mr, cs = dense.grad_errors(xg.grad.cpu().double(), xr.grad * fac)
    assert mr <= dense.GRAD_MAX_REL and cs >= dense.GRAD_COS_MIN, (mr, cs)
    if kind == "clip":
        mr, cs = dense.grad_errors(yg.grad.cpu().double(), yr.grad * fac)
        assert mr <= dense.GRAD_MAX_REL and cs >= dense.GRAD_COS_MIN, (mr, cs)
    assert abs(t.grad.item() - tr.grad.item()) <= 1e-2 * abs(tr.grad.item()) + 1e-6, (t.grad.item(), tr.grad.item())


def test_siglip_scale_and_bias_without_host_sync():
    import memoryefficientclip_b200 as m
    b, d = 384, 64
    x, y = _pair(b, d, 6)
    mod = m.MemoryEfficientSigLIPLoss(10.0, -10.0, normalized_inputs=True).cuda()

    def run(xg, yg):
        loss = mod(xg, yg)
        loss.backward()
        return loss

    run(x.cuda().requires_grad_(True), y.cuda().requires_grad_(True))
    mod.zero_grad()
    xg, yg = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        loss = run(xg, yg)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    xr, yr = x.double().requires_grad_(True), y.double().requires_grad_(True)
    ls = torch.tensor(float(mod.log_logit_scale.detach().cpu()), dtype=torch.float64, requires_grad=True)
    lb = torch.tensor(float(mod.logit_bias.detach().cpu()), dtype=torch.float64, requires_grad=True)
    a = ls.exp() * (xr @ yr.T) + lb
    z = 2.0 * torch.eye(b, dtype=torch.float64) - 1.0
    ref = F.softplus(-z * a).sum() / b
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 1e-3 * abs(ref.item())
    for got, want in ((xg.grad, xr.grad), (yg.grad, yr.grad)):
        mr, cs = dense.grad_errors(got.cpu().double(), want)
        assert mr <= dense.GRAD_MAX_REL and cs >= dense.GRAD_COS_MIN, (mr, cs)
    assert abs(mod.log_logit_scale.grad.item() - ls.grad.item()) <= 2e-2 * abs(ls.grad.item()) + 1e-6
    assert abs(mod.logit_bias.grad.item() - lb.grad.item()) <= 2e-2 * abs(lb.grad.item()) + 1e-6
