"""The forward+backward of the public modules inside a CUDA graph.

Small batches are bound by host launch latency (about a dozen launches per step), so the step must be
capturable: no host synchronisation, no allocation outside torch's allocator, side streams forked from and
joined back into the capturing stream inside every call.  Replays on new data must match the oracle.
"""
import pytest
import torch

from oracle import dense

pytestmark = pytest.mark.gpu


def _fresh(b, d, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(b, d, generator=g).to(dtype), torch.randn(b, d, generator=g).to(dtype)


@pytest.mark.parametrize("kind,b,d,normalized_inputs", [("clip", 1024, 256, False), ("clip", 4096, 512, False),
                                                        ("lit", 640, 104, False), ("clip", 512, 64, True)])
def test_whole_step_capture_and_replay(kind, b, d, normalized_inputs):
    import memoryefficientclip_b200 as m
    mod = (m.MemoryEfficientCLIPLoss if kind == "clip" else m.MemoryEfficientLiTLoss)(0.07, normalized_inputs)
    x0, y0 = _fresh(b, d, 0)
    if normalized_inputs:
        x0, y0 = torch.nn.functional.normalize(x0, dim=1), torch.nn.functional.normalize(y0, dim=1)
    x = x0.cuda().requires_grad_(True)
    y = y0.cuda().requires_grad_(kind == "clip")
    # warm-up on a side stream: lazy initialisation (kernel attributes, the library's streams and events)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            x.grad = None
            y.grad = None
            mod(x, y).backward()
    torch.cuda.current_stream().wait_stream(side)
    x.grad = None
    y.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        loss = mod(x, y)
        loss.backward()
    for seed in (1, 2):
        nx, ny = _fresh(b, d, seed)
        if normalized_inputs:
            nx, ny = torch.nn.functional.normalize(nx, dim=1), torch.nn.functional.normalize(ny, dim=1)
        with torch.no_grad():
            x.copy_(nx)
            y.copy_(ny)
        graph.replay()
        torch.cuda.synchronize()
        if kind == "clip":
            rl, rx, ry = dense.clip_dense(nx, ny, 0.07, normalized_inputs)
            dense.assert_parity(loss.item(), rl, (x.grad.cpu(), y.grad.cpu()), (rx, ry), f"graph replay seed {seed}")
        else:
            rl, rx = dense.lit_dense(nx, ny, 0.07, normalized_inputs)
            dense.assert_parity(loss.item(), rl, (x.grad.cpu(),), (rx,), f"graph replay seed {seed}")


def test_replay_is_faster_than_eager_for_a_small_batch():
    """B = 1024, D = 512: the eager step is host-bound; the replay runs at the speed of the kernels."""
    import memoryefficientclip_b200 as m
    mod = m.MemoryEfficientCLIPLoss(0.07, True)
    x0, y0 = _fresh(1024, 512, 3, torch.bfloat16)
    x = torch.nn.functional.normalize(x0.float(), dim=1).bfloat16().cuda().requires_grad_(True)
    y = torch.nn.functional.normalize(y0.float(), dim=1).bfloat16().cuda().requires_grad_(True)

    def step():
        x.grad = None
        y.grad = None
        mod(x, y).backward()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    x.grad = None
    y.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        mod(x, y).backward()

    def timed(f, n=200):
        for _ in range(10):
            f()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    eager_ms = timed(step)
    graph_ms = timed(graph.replay)
    print(f"eager {eager_ms * 1e3:.1f} us/step, graph replay {graph_ms * 1e3:.1f} us/step")
    assert graph_ms < eager_ms


def test_make_graphed_callables_on_the_module():
    """torch.cuda.make_graphed_callables captures the module's forward and backward as two graphs and keeps the
    autograd interface: the drop-in way to run small batches at kernel speed."""
    import memoryefficientclip_b200 as m
    b, d = 2048, 512
    mod = m.MemoryEfficientCLIPLoss(0.07, False)
    sx, sy = _fresh(b, d, 30)
    graphed = torch.cuda.make_graphed_callables(mod, (sx.cuda().requires_grad_(True), sy.cuda().requires_grad_(True)))
    for seed in (31, 32):
        nx, ny = _fresh(b, d, seed)
        x = nx.cuda().requires_grad_(True)
        y = ny.cuda().requires_grad_(True)
        loss = graphed(x, y)
        loss.backward()
        torch.cuda.synchronize()
        rl, rx, ry = dense.clip_dense(nx, ny, 0.07, False)
        dense.assert_parity(loss.item(), rl, (x.grad.cpu(), y.grad.cpu()), (rx, ry), f"graphed callable seed {seed}")
