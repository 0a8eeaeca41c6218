"""ctypes binding of libmeclip_sm100.so (the C ABI in include/meclip.h).

There is no fallback: if the shared library is missing this module raises, and
every operation of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# MECLIP_LIBRARY points at another build of the same library (kernel experiments)
LIB_PATH = os.environ.get("MECLIP_LIBRARY") or os.path.join(PKG_DIR, "libmeclip_sm100.so")

OK, EINVAL, ENOSPC, ECUDA, ETIMEOUT, EUNSUPPORTED = range(6)
CLIP, LIT, SIGLIP = 0, 1, 2
BF16, F32, F16 = 0, 1, 2
STORE_BF16, STORE_F32, ACCUM_F32 = 0, 1, 2



class RingDesc(ctypes.Structure):
    """meclip_ring_desc of include/meclip.h."""
    _fields_ = [("rank", c_int), ("nranks", c_int), ("rows", c_int64), ("d", c_int64), ("ldx", c_int64),
                ("ldy", c_int64), ("shards", ctypes.POINTER(c_void_p)), ("recv", c_void_p * 2),
                ("compute_stream", c_void_p), ("copy_stream", c_void_p)]


# name -> (restype, argtypes); mirrors include/meclip.h declaration by declaration
SIGNATURES = {
    "meclip_version": (c_int, []),
    "meclip_status_string": (c_char_p, [c_int]),
    "meclip_last_error": (c_int, [c_char_p, c_size_t]),
    "meclip_read_status": (c_int, [c_void_p, c_void_p]),
    "meclip_bind_device_scalars": (c_int, [c_void_p, c_void_p, c_int]),
    "meclip_ipc_export": (c_int, [c_void_p, c_void_p, c_void_p]),
    "meclip_ipc_open": (c_int, [c_void_p, c_void_p]),
    "meclip_ipc_close": (c_int, [c_void_p]),
    "meclip_copy_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "meclip_ring_sum_exp": (c_int, [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p]),
    "meclip_ring_grad": (c_int, [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                 c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "meclip_debug_wait_probe": (c_int, [ctypes.c_uint64, c_void_p, c_void_p]),
    "meclip_debug_set_blocking": (c_int, [c_int64, c_int64]),
    "meclip_debug_set_trace": (c_int, [c_void_p, c_size_t]),
    "meclip_launch_count": (ctypes.c_longlong, []),
    "meclip_profile_begin": (c_int, []),
    "meclip_profile_end": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "meclip_accumulate_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "meclip_accumulate_many_f32": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "meclip_normalize_fwd": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p,
                                     c_void_p]),
    "meclip_normalize_bwd": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                     c_void_p, c_int, c_int64, c_void_p]),
    "meclip_sum_exp": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                               c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "meclip_sum_exp_det_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "meclip_sum_exp_det": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                   c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
                                   c_void_p]),
    "meclip_loss_finalize": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_float, c_int,
                                     c_void_p, c_void_p]),
    "meclip_grad_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "meclip_grad": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int64,
                            c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int64, c_void_p,
                            c_int, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]),
    "meclip_grad_t": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int64,
                              c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int64, c_void_p,
                              c_int, c_int64, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "meclip_operand_f32": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "meclip_sum_exp_tf32": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                    c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "meclip_grad_tf32": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                 c_int64, c_int64, c_int64, c_float, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                 c_float, c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_size_t,
                                 c_void_p, c_void_p]),
    "meclip_lit_extend": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "meclip_lit_fused_forward": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int64,
                                         c_int64, c_void_p, c_int, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]),
    "meclip_lit_fused_stats": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                       c_void_p, c_void_p]),
    "meclip_lit_fused_backward": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_int64, c_int64,
                                          c_void_p, c_int, c_int64, c_void_p]),
    "meclip_siglip_sum": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_float,
                                  c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "meclip_siglip_loss_finalize": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_float, c_float, c_int, c_void_p,
                                            c_void_p]),
    "meclip_siglip_grad": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_float,
                                   c_int64, c_int64, c_void_p, c_float, c_void_p, c_int, c_int64, c_void_p, c_int,
                                   c_int64, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "meclip_grad_static": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                   c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int64,
                                   c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "meclip_loss_forward": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "meclip_loss_backward": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float,
                                     c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int64, c_void_p,
                                     c_int, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]),
    "meclip_step_saved_bytes": (c_size_t, [c_int64, c_int64]),
    "meclip_step_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "meclip_step_forward": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_float,
                                    c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    "meclip_step_backward": (c_int, [c_int, c_void_p, c_size_t, c_int64, c_int64, c_int, c_float, c_void_p, c_float,
                                     c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]),
    "meclip_debug_gemm": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int64, c_int64, c_int64,
                                  c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
}

_lock = threading.Lock()
_lib = None


class MeclipError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libmeclip_sm100 error {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing. The CUDA extension is the only implementation of this package; build it "
                    "with `python -m memoryefficientclip_b200.build` (needs nvcc with sm_100a support).")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)     # AttributeError if the symbol is not exported
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def last_error() -> str:
    buf = ctypes.create_string_buffer(1024)
    load().meclip_last_error(buf, len(buf))
    return buf.value.decode("utf-8", "replace")


def check(code: int) -> None:
    if code != OK:
        raise MeclipError(code, last_error() or load().meclip_status_string(code).decode())
