"""CPU-side checks of the boundary: the shared library loads without a GPU, exports every
symbol the header declares, and rejects bad arguments with error codes (no compute)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from memoryefficientclip_b200 import build, _lib
    build.build_library()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "meclip.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(meclip_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from memoryefficientclip_b200 import _lib
    declared = _declared_symbols()
    assert len(declared) >= 12
    assert sorted(_lib.SIGNATURES) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/meclip.h but not exported"


def test_version_and_strings(lib):
    assert lib.meclip_version() >= 100
    assert lib.meclip_status_string(0) == b"ok"
    assert b"workspace" in lib.meclip_status_string(2)


def test_workspace_query_is_pure_host(lib):
    n = lib.meclip_grad_workspace_bytes(32768, 32768, 1152)
    assert 512 * 2**20 <= n <= 2 * 2**30
    assert lib.meclip_grad_workspace_bytes(0, 5, 8) == 0
    small = lib.meclip_grad_workspace_bytes(256, 256, 64)
    assert 256 * 256 * 2 <= small < 2**20


def test_bad_arguments_return_error_codes(lib):
    from memoryefficientclip_b200 import _lib
    # null pointers
    assert lib.meclip_sum_exp(0, None, None, 8, 8, 8, 8, 8, 0.07, 0, 0, None, None, None, None, None, None) == _lib.EINVAL
    assert "null" in _lib.last_error()
    # feature dimension not a multiple of 8
    fake = ctypes.c_void_p(0x1000)
    assert lib.meclip_sum_exp(0, fake, fake, 8, 8, 12, 12, 12, 0.07, 0, 0, fake, fake, fake, None, None, None) == _lib.EINVAL
    # bad kind
    assert lib.meclip_sum_exp(7, fake, fake, 8, 8, 8, 8, 8, 0.07, 0, 0, fake, fake, fake, None, None, None) == _lib.EINVAL
    # non-positive temperature
    assert lib.meclip_sum_exp(0, fake, fake, 8, 8, 8, 8, 8, 0.0, 0, 0, fake, fake, fake, None, None, None) == _lib.EINVAL
    # normalise: the OUTPUT operand must be 16-byte aligned with padded rows (the input may be anything)
    odd = ctypes.c_void_p(0x1004)
    assert lib.meclip_normalize_fwd(fake, 1, 4, 8, 8, 1, odd, 8, fake, None) == _lib.EINVAL
    assert lib.meclip_normalize_fwd(fake, 1, 4, 12, 12, 1, fake, 12, fake, None) == _lib.EINVAL     # ldh < round_up(d, 8)
    assert lib.meclip_normalize_fwd(fake, 9, 4, 8, 8, 1, fake, 8, fake, None) == _lib.EINVAL        # bad dtype
    assert lib.meclip_normalize_bwd(fake, 2, 8, fake, 8, fake, 4, 8, fake, 1, 8, None) == _lib.EINVAL  # g is fp32 or bf16
    # grad: workspace too small is reported before any launch... but only after the device check,
    # so here only the argument validation is exercised
    assert lib.meclip_grad(0, fake, fake, 8, 8, 8, 8, 8, 0.07, 0, 0, fake, None, None, 1.0, fake, 0, 8, None, 0, 8,
                           fake, 0, None, None) == _lib.EINVAL
    # ring calls: the descriptor is checked before anything touches a device
    assert lib.meclip_ring_sum_exp(None, 0, fake, 0.07, fake, fake, fake, fake, None) == _lib.EINVAL
    shards = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    recv = (ctypes.c_void_p * 2)(0x3000, 0x4000)

    def desc(rank=0, nranks=2, d=8, compute=0x10, copy=0x20):
        return _lib.RingDesc(rank, nranks, 8, d, 8, 8, ctypes.cast(shards, ctypes.POINTER(ctypes.c_void_p)), recv,
                             compute, copy)

    for bad in (desc(rank=2), desc(nranks=0), desc(d=12), desc(compute=0x20)):
        assert lib.meclip_ring_sum_exp(ctypes.byref(bad), 0, fake, 0.07, fake, fake, fake, fake, None) == _lib.EINVAL
        assert lib.meclip_ring_grad(ctypes.byref(bad), 0, fake, 0.07, fake, fake, None, 1.0, fake, 8, fake, fake, fake,
                                    None, fake, 0, None) == _lib.EINVAL
    import torch
    if not torch.cuda.is_available():
        # a well-formed descriptor passes the argument checks (every field is read where the C struct has it) and
        # fails only at the first CUDA call; never tried where a GPU could run the fake pointers
        assert lib.meclip_ring_sum_exp(ctypes.byref(desc()), 0, fake, 0.07, fake, fake, fake, fake, None) == _lib.ECUDA
    shards[1] = None                                     # a peer's shard is not mapped
    assert lib.meclip_ring_sum_exp(ctypes.byref(desc()), 0, fake, 0.07, fake, fake, fake, fake, None) == _lib.EINVAL
    shards[1] = 0x2000
    assert lib.meclip_ring_sum_exp(ctypes.byref(desc()), 5, fake, 0.07, fake, fake, fake, fake, None) == _lib.EINVAL
    assert lib.meclip_ring_grad(ctypes.byref(desc()), 0, fake, 0.07, fake, fake, None, 1.0, fake, 8, fake, fake, fake,
                                None, fake, 0, None) == _lib.EINVAL            # CLIP over 2 ranks without an inbox table


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from memoryefficientclip_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="only implementation"):
        _lib.load()


def test_modules_mirror_reference_api():
    import inspect
    import clip_loss
    import lit_loss
    for mod, names in ((clip_loss, ["MemoryEfficientCLIPLoss", "StableMemoryEfficientCLIPLoss"]),
                       (lit_loss, ["MemoryEfficientLiTLoss", "StableMemoryEfficientLiTLoss"])):
        for n in names:
            cls = getattr(mod, n)
            sig = inspect.signature(cls.__init__)
            assert list(sig.parameters)[1:] == ["temperature", "normalized_inputs"]
            assert sig.parameters["temperature"].default == 0.07
            assert sig.parameters["normalized_inputs"].default is False
            m = cls()
            assert len(list(m.parameters())) == 0 and len(m.state_dict()) == 0
    assert list(inspect.signature(clip_loss.MemoryEfficientCLIPLoss.forward).parameters)[1:] == \
        ["image_features", "text_features"]
    assert list(inspect.signature(lit_loss.MemoryEfficientLiTLoss.forward).parameters)[1:] == \
        ["text_features", "image_features"]
    for fn in (clip_loss.MemoryEfficientCLIPLossNormed, clip_loss.StableMemoryEfficientCLIPLossNormed,
               lit_loss.MemoryEfficientLiTLossNormed, lit_loss.StableMemoryEfficientLiTLossNormed):
        assert list(inspect.signature(fn.forward).parameters) == ["ctx", "x_normalized", "y_normalized", "temperature"]


def test_cpu_tensors_are_rejected_like_the_reference():
    import torch
    import clip_loss
    with pytest.raises(AssertionError):
        clip_loss.MemoryEfficientCLIPLoss()(torch.randn(8, 8), torch.randn(8, 8))
