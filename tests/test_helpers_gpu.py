"""Small device helpers of the ring host: one-pass accumulation of several partial gradients, the
device-to-device copy, and the export side of the peer-memory handles."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_src,shape", [(1, (64, 8)), (3, (257, 24)), (7, (1024, 768))])
def test_accumulate_many_adds_in_order(n_src, shape):
    from memoryefficientclip_b200 import ops
    g = torch.Generator().manual_seed(n_src)
    dst0 = torch.randn(*shape, generator=g)
    srcs = torch.randn(n_src, *shape, generator=g)
    dst = dst0.cuda()
    ops.accumulate_many_f32(dst, srcs.cuda())
    want = dst0.clone()
    for s in range(n_src):            # the same order of fp32 additions
        want += srcs[s]
    assert torch.equal(dst.cpu(), want)
    # and it is what n_src single accumulations give
    dst2 = dst0.cuda()
    for s in range(n_src):
        ops.accumulate_f32(dst2, srcs[s].cuda())
    assert torch.equal(dst2, dst)


def test_copy_async_and_handle_export():
    from memoryefficientclip_b200 import _lib
    lib = _lib.load()
    src = torch.arange(1 << 20, dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.meclip_copy_async(dst.data_ptr(), src.data_ptr(), src.numel() * 4, s))
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    # a handle names the ALLOCATION that holds the pointer; two views of one tensor share it and differ in offset
    h0, h1 = ctypes.create_string_buffer(64), ctypes.create_string_buffer(64)
    o0, o1 = ctypes.c_uint64(0), ctypes.c_uint64(0)
    _lib.check(lib.meclip_ipc_export(src.data_ptr(), h0, ctypes.byref(o0)))
    _lib.check(lib.meclip_ipc_export(src[4096:].data_ptr(), h1, ctypes.byref(o1)))
    assert h0.raw == h1.raw and o1.value - o0.value == 4096 * 4
    assert lib.meclip_ipc_export(None, h0, ctypes.byref(o0)) == _lib.EINVAL
