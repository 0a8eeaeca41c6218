"""The tcgen05 mainloop alone: every operand layout against torch fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(m, n, k, a_mn, b_mn, tile_n=0, accumulate=False, seed=0):
    from memoryefficientclip_b200 import ops
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    b = torch.randn(n, k, generator=g).bfloat16().cuda()
    a_store = a.t().contiguous() if a_mn else a
    b_store = b.t().contiguous() if b_mn else b
    c_in = torch.randn(m, n, generator=g).cuda() if accumulate else None
    status = ops.new_status(a.device)
    c = ops.debug_gemm(a_store, b_store, a_mn, b_mn, m, n, k, tile_n, c_in, status)
    ops.read_status(status)
    ref = a.double() @ b.double().t()
    if accumulate:
        ref = ref + c_in.double()
    err = (c.double() - ref).abs().max().item()
    tol = 1e-3 * max(1.0, k ** 0.5)
    assert err < tol, f"m={m} n={n} k={k} a_mn={a_mn} b_mn={b_mn} tile_n={tile_n}: max err {err} (tol {tol})"


LAYOUTS = [(False, False), (False, True), (True, True), (True, False)]


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_single_tile(a_mn, b_mn):
    _run(128, 256, 64, a_mn, b_mn, 256)


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_multi_k_multi_tile(a_mn, b_mn):
    _run(512, 768, 320, a_mn, b_mn, 256)
    _run(384, 384, 512, a_mn, b_mn, 192)
    _run(256, 128, 192, a_mn, b_mn, 64)


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_ragged_edges(a_mn, b_mn):
    # m, n, k not multiples of the tile: TMA zero-fills, the epilogue masks
    _run(200, 200, 136, a_mn, b_mn, 128)
    _run(72, 1152, 200, a_mn, b_mn, 192)


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_accumulate_input(a_mn, b_mn):
    _run(256, 512, 256, a_mn, b_mn, 256, accumulate=True)


def test_more_tiles_than_sms():
    # 40 x 9 = 360 tiles on 148 persistent CTAs, long K: pipeline wrap-around and TMEM double buffering
    _run(5120, 1152, 2048, False, True, 128)
    _run(2048, 4096, 1152, False, False, 256)


def test_in_kernel_trace_hook():
    """meclip_debug_set_trace: CTA 0 records load / MMA / epilogue timestamps per tile, in order."""
    from memoryefficientclip_b200 import _lib, ops
    lib = _lib.load()
    a = torch.randn(1024, 256).bfloat16().cuda()
    b = torch.randn(512, 256).bfloat16().cuda()
    cap = 300
    buf = torch.zeros(2 + 3 * cap, dtype=torch.int64, device="cuda")
    try:
        _lib.check(lib.meclip_debug_set_trace(buf.data_ptr(), buf.numel()))
        ops.debug_gemm(a, b, False, False, 1024, 512, 256, 256)
        torch.cuda.synchronize()
    finally:
        lib.meclip_debug_set_trace(None, 0)
    rec = [r for r in buf[2:].view(cap, 3).cpu().tolist() if r[0] != 0]
    tags = {r[0] for r in rec}
    assert {1, 2, 10, 11, 12, 20, 21, 22} <= tags, tags
    by_tile = {}
    for tag, tile, t in rec:
        by_tile.setdefault(tile, {})[tag] = t
    for tile, ev in by_tile.items():
        assert ev[1] <= ev[11] <= ev[12] <= ev[21] <= ev[22], (tile, ev)     # loads, data, last MMA, release, end


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("m,n,k,tile_n", [
    (256, 384, 128, 384),       # one wide tile: two MMAs per K step (256 + 128 columns)
    (256, 512, 192, 512),       # 256 + 256 columns
    (512, 1152, 640, 384),      # 3 x 384, several row tiles, wrap-around of the operand ring
    (768, 1160, 512, 512),      # 512, 512 and a narrow last tile (136 -> 160 columns, one MMA)
    (304, 1000, 200, 384),      # ragged rows and a last tile of 232 -> 256 columns
    (1280, 840, 1024, 448),     # 840 = 448 + 392: the last tile is wide too (392 -> 448 columns)
    (2048, 704, 2304, 384),     # last tile 320 wide (two MMAs: 256 + 64)
])
def test_wide_pair_tiles(m, n, k, tile_n, a_mn):
    """Tiles wider than 256 columns on the CTA-pair kernel: the accumulator columns of the two MMAs are
    interleaved halves of the tile (see the epilogue's column map), single-buffered accumulator."""
    _run(m, n, k, a_mn, False, tile_n)
    _run(m, n, k, a_mn, False, tile_n, accumulate=True, seed=3)
