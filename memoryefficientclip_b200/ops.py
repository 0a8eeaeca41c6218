"""Torch-tensor front end of the C ABI: every function here launches CUDA kernels from
libmeclip_sm100.so on the current stream of the tensors' device.  Torch is used for
device memory and streams only; no arithmetic of the loss path happens in torch.
"""
from __future__ import annotations

import math
import os

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32, torch.float16: _lib.F16}


# MECLIP_TF32=1 (or ops.TF32_OPERANDS = True): fp32 module inputs keep fp32 operands for the two passes that form
# S = X Y^T, multiplied as tf32 like the reference's tl.dot (clip_loss.py:53); default: bf16 operands
TF32_OPERANDS = os.environ.get("MECLIP_TF32", "0") == "1"


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    """Raw handle of the current stream of t's device (the C getter: no Stream object is built)."""
    return torch._C._cuda_getCurrentRawStream(t.device.index if t.device.index is not None
                                              else torch.cuda.current_device())


class _on_device:
    """`with _on_device(dev):` like torch.cuda.device, but free when dev is already the current device."""
    __slots__ = ("guard",)

    def __init__(self, device):
        idx = device.index
        self.guard = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(idx)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


def _check_matrix(t: torch.Tensor, name: str):
    assert t.is_cuda, f"{name} must be a CUDA tensor"
    assert t.dim() == 2, f"{name} must be 2-D [batch, features]"
    assert t.dtype in _DT, f"{name}: dtype {t.dtype} not supported (float32, bfloat16 or float16)"
    assert t.shape[0] >= 1 and t.shape[1] >= 1, f"{name}: empty input"


def padded(d: int) -> int:
    """Columns of a bf16 operand: the tile loads need 16-byte rows."""
    return (d + 7) // 8 * 8


def new_status(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor) -> None:
    """Synchronise and raise if a kernel recorded an expired wait."""
    with _on_device(status.device):
        _lib.check(_lib.load().meclip_read_status(status.data_ptr(), _stream(status)))


# ---- scalars that may live on the device ----------------------------------------------------------------
GSCALE_FIXED, GSCALE_OVER_T, GSCALE_OVER_SQRT_T, GSCALE_TIMES_T = 0, 1, 2, 3


def _dev_scalar(v, device):
    """fp32 one-element view / copy of a tensor scalar on `device` (no host synchronisation)."""
    v = v.detach()
    if v.dtype != torch.float32 or v.device != device:
        v = v.to(device=device, dtype=torch.float32)
    return v.reshape(1)


def _bind(temperature, device, rule=GSCALE_FIXED, bias=None):
    """Prepares the scalar arguments of the next library call.  A float goes through as it is.  A tensor
    (a learnable temperature / logit scale / bias) stays on the device: its address is bound for the next
    call of this thread (meclip_bind_device_scalars) and the float argument is a placeholder.
    Returns (float for the temperature argument, float for the bias argument, tensors to keep alive)."""
    t_is, b_is = isinstance(temperature, torch.Tensor), isinstance(bias, torch.Tensor)
    if not (t_is or b_is):
        return float(temperature), (0.0 if bias is None else float(bias)), ()
    t_dev = _dev_scalar(temperature, device) if t_is else torch.full((1,), float(temperature), dtype=torch.float32,
                                                                      device=device)
    b_dev = None
    if bias is not None:
        b_dev = _dev_scalar(bias, device) if b_is else torch.full((1,), float(bias), dtype=torch.float32, device=device)
    _lib.check(_lib.load().meclip_bind_device_scalars(t_dev.data_ptr(), _ptr(b_dev), rule))
    return 1.0, 0.0, (t_dev, b_dev)


def is_dev(v) -> bool:
    return isinstance(v, torch.Tensor)


# ---- the status word of the module path -----------------------------------------------------------------
class _DeviceStatus:
    """One status word per device for everything the modules launch, checked without stalling the step:
    after a backward the word is copied to pinned host memory behind an event; the next forward looks at
    the copy if the event has completed and raises MeclipError(ETIMEOUT) when a kernel gave up a bounded
    wait.  MECLIP_CHECK_STATUS=1 checks synchronously after every forward and backward instead."""

    def __init__(self, device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.posted_at = 0.0


_status_by_device = {}
_monotonic = __import__("time").monotonic
_SYNC_CHECK = __import__("os").environ.get("MECLIP_CHECK_STATUS", "0") not in ("", "0")


def _dev_status(device) -> _DeviceStatus:
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _status_by_device.get(key)
    if st is None:
        st = _status_by_device[key] = _DeviceStatus(torch.device("cuda", key))
    return st


def status_word(device) -> torch.Tensor:
    """The device's shared status word (int32[1]); pass it as `status=` to the functions below."""
    return _dev_status(device).word


def _raise_timeout(st: _DeviceStatus):
    st.word.zero_()
    st.host.zero_()
    st.pending = False
    raise _lib.MeclipError(_lib.ETIMEOUT, "a kernel of an earlier step gave up a bounded wait on a barrier; "
                           "its results (loss, gradients) are incomplete")


def poll_status(device) -> None:
    """Non-blocking: raises if the last posted copy of the status word has arrived and is non-zero."""
    st = _dev_status(device)
    if not st.pending or torch.cuda.is_current_stream_capturing():
        return
    if st.event.query():
        st.pending = False
        if int(st.host[0]) != 0:
            _raise_timeout(st)


def post_status(device, force: bool = False) -> None:
    """Queue a copy of the status word to pinned host memory on the current stream (no synchronisation).
    At most one copy per 2 ms unless `force`."""
    st = _dev_status(device)
    if _SYNC_CHECK:
        if not torch.cuda.is_current_stream_capturing():
            check_status(device)
        return
    # A wait gives up after seconds, so a copy every couple of milliseconds loses nothing; steps of small batches
    # (a fifth of a millisecond) do not pay for one each.
    now = _monotonic()
    if (now - st.posted_at < 0.002 and not force) or torch.cuda.is_current_stream_capturing():
        return
    st.posted_at = now
    st.host.copy_(st.word, non_blocking=True)
    if st.word.device.index == torch.cuda.current_device():
        st.event.record()
    else:
        st.event.record(torch.cuda.current_stream(st.word.device))
    st.pending = True


def check_status(device=None) -> None:
    """Synchronous check of the module path's status word: waits for the device's current stream and raises
    MeclipError(ETIMEOUT) if any kernel launched by the modules recorded an expired wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _dev_status(device)
    try:
        read_status(st.word)
    except _lib.MeclipError:
        _raise_timeout(st)
    st.pending = False


def normalize_fwd(x: torch.Tensor, normalize: bool = True, extra_cols: int = 0):
    """Returns (x_hat bf16 [rows, padded(d) + extra_cols], inv_norm fp32 [rows] or None); columns past d are
    zero up to padded(d); extra_cols (a multiple of 8) are left for the caller to fill.

    Any feature count, row pitch and alignment is taken as it is (the kernel reads element-wise when
    16-byte loads are not possible); only a non-unit column stride costs a copy."""
    _check_matrix(x, "x")
    x = x if x.stride(1) == 1 else x.contiguous()
    rows, d = x.shape
    dp = padded(d)
    out = torch.empty(rows, dp + extra_cols, dtype=torch.bfloat16, device=x.device)
    inv = torch.empty(rows, dtype=torch.float32, device=x.device) if normalize else None
    with _on_device(x.device):
        _lib.check(_lib.load().meclip_normalize_fwd(x.data_ptr(), _DT[x.dtype], rows, d, max(x.stride(0), d),
                                                    int(normalize), out.data_ptr(), dp + extra_cols, _ptr(inv),
                                                    _stream(x)))
    return out, inv


def normalize_bwd(g: torch.Tensor, x_hat, inv_norm, out_dtype, d: int | None = None) -> torch.Tensor:
    """Gradient w.r.t. the un-normalised input, [rows, d] in out_dtype, from g (fp32 or bf16, padded(d)
    columns).  inv_norm None: the inputs were already normalised, so this is the conversion of g only."""
    rows = g.shape[0]
    d = g.shape[1] if d is None else d
    assert g.shape[1] == padded(d) and g.stride(1) == 1
    dx = torch.empty(rows, d, dtype=out_dtype, device=g.device)
    with _on_device(g.device):
        _lib.check(_lib.load().meclip_normalize_bwd(g.data_ptr(), _DT[g.dtype], g.stride(0), _ptr(x_hat),
                                                    x_hat.stride(0) if x_hat is not None else 0, _ptr(inv_norm),
                                                    rows, d, dx.data_ptr(), _DT[out_dtype], d, _stream(g)))
    return dx


def accumulate_f32(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst += src (fp32, contiguous, same shape) on the current stream."""
    assert dst.dtype == torch.float32 and src.dtype == torch.float32 and dst.numel() == src.numel()
    with _on_device(dst.device):
        _lib.check(_lib.load().meclip_accumulate_f32(dst.data_ptr(), src.data_ptr(), dst.numel(), _stream(dst)))


def accumulate_many_f32(dst: torch.Tensor, srcs: torch.Tensor) -> None:
    """dst += srcs[0] + srcs[1] + ... in that order; srcs is one contiguous fp32 tensor [n_src, *dst.shape]."""
    assert dst.dtype == torch.float32 and srcs.dtype == torch.float32 and srcs.is_contiguous() and dst.is_contiguous()
    assert srcs.shape[1:] == dst.shape
    with _on_device(dst.device):
        _lib.check(_lib.load().meclip_accumulate_many_f32(dst.data_ptr(), srcs.data_ptr(), srcs.shape[0], dst.numel(),
                                                          dst.numel(), _stream(dst)))


def as_operand(x: torch.Tensor) -> torch.Tensor:
    """bf16, unit-stride rows of padded(d) columns, 16-byte aligned: what the tile kernels read."""
    _check_matrix(x, "operand")
    if (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        return x
    return normalize_fwd(x, normalize=False)[0]


def direct_grad_dtype(dtype, d: int) -> bool:
    """True when the contraction kernels can write the gradient of an input of this dtype and feature
    count themselves; otherwise they write fp32 with padded(d) columns and normalize_bwd converts."""
    return d % 8 == 0 and dtype in (torch.float32, torch.bfloat16)


# MECLIP_DETERMINISTIC=1: forward sums without atomics (meclip_sum_exp_det), so that a whole step is reproducible
# bit for bit; the modules then also stay off the small-batch step path, whose forward uses the atomics.
DETERMINISTIC = __import__("os").environ.get("MECLIP_DETERMINISTIC", "0") not in ("", "0")


def sum_exp(kind, x_hat, y_hat, temperature, row_sum, col_sum, diag_s, row_off=0, col_off=0, status=None,
            deterministic=None):
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    counter = torch.zeros(1, dtype=torch.int32, device=x_hat.device)     # dynamic tile hand-out
    if DETERMINISTIC if deterministic is None else deterministic:
        lib = _lib.load()
        ws = torch.empty(lib.meclip_sum_exp_det_workspace_bytes(rows, cols), dtype=torch.uint8, device=x_hat.device)
        with _on_device(x_hat.device):
            t, _b, _keep = _bind(temperature, x_hat.device)
            _lib.check(lib.meclip_sum_exp_det(kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                              y_hat.stride(0), t, row_off, col_off, row_sum.data_ptr(), _ptr(col_sum),
                                              diag_s.data_ptr(), counter.data_ptr(), ws.data_ptr(), ws.numel(),
                                              _ptr(status), _stream(x_hat)))
        return
    with _on_device(x_hat.device):
        t, _b, _keep = _bind(temperature, x_hat.device)
        _lib.check(_lib.load().meclip_sum_exp(kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                              y_hat.stride(0), t, row_off, col_off, row_sum.data_ptr(),
                                              _ptr(col_sum), diag_s.data_ptr(), counter.data_ptr(), _ptr(status),
                                              _stream(x_hat)))


def loss_finalize(kind, row_sum, col_sum, diag_s, temperature, scale, loss_out, accumulate=False):
    with _on_device(row_sum.device):
        t, _b, _keep = _bind(temperature, row_sum.device)
        _lib.check(_lib.load().meclip_loss_finalize(kind, row_sum.data_ptr(), _ptr(col_sum), diag_s.data_ptr(),
                                                    row_sum.numel(), t, float(scale), int(accumulate),
                                                    loss_out.data_ptr(), _stream(row_sum)))


def operand_f32(x: torch.Tensor, inv_norm=None) -> torch.Tensor:
    """The fp32 operand of the tf32 passes: x * inv_norm (or x itself) with round_up(d, 8) columns, zero padded."""
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    rows, d = x.shape
    dpad = (d + 7) // 8 * 8
    out = torch.empty(rows, dpad, dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        _lib.check(_lib.load().meclip_operand_f32(x.data_ptr(), rows, d, x.stride(0), _ptr(inv_norm), out.data_ptr(),
                                                  dpad, _stream(x)))
    return out


def loss_forward(kind, x_hat, y_hat, temperature, status=None, deterministic=None, f32_operands=None):
    """Returns (loss 0-dim fp32, row_sum, col_sum or None, diag_s).
    f32_operands: optional (x fp32, y fp32) of the same padded shape; S is then formed with tf32 MMAs."""
    b, d = x_hat.shape
    assert y_hat.shape == x_hat.shape
    dev = x_hat.device
    if f32_operands is not None:
        x32, y32 = f32_operands
        assert x32.shape == x_hat.shape and y32.shape == y_hat.shape and x32.dtype == y32.dtype == torch.float32
        row_sum = torch.zeros(b, dtype=torch.float32, device=dev)
        col_sum = torch.zeros(b, dtype=torch.float32, device=dev) if kind == _lib.CLIP else None
        diag_s = torch.zeros(b, dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        with _on_device(dev):
            t, _b, _keep = _bind(temperature, dev)
            _lib.check(_lib.load().meclip_sum_exp_tf32(kind, x32.data_ptr(), y32.data_ptr(), b, b, d, x32.stride(0),
                                                       y32.stride(0), t, 0, 0, row_sum.data_ptr(), _ptr(col_sum),
                                                       diag_s.data_ptr(), counter.data_ptr(), _ptr(status),
                                                       _stream(x_hat)))
        loss_finalize(kind, row_sum, col_sum, diag_s, temperature, 1.0 / b, loss)
        return loss, row_sum, col_sum, diag_s
    if DETERMINISTIC if deterministic is None else deterministic:
        row_sum = torch.zeros(b, dtype=torch.float32, device=dev)
        col_sum = torch.zeros(b, dtype=torch.float32, device=dev) if kind == _lib.CLIP else None
        diag_s = torch.zeros(b, dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        sum_exp(kind, x_hat, y_hat, temperature, row_sum, col_sum, diag_s, 0, 0, status, deterministic=True)
        loss_finalize(kind, row_sum, col_sum, diag_s, temperature, 1.0 / b, loss)
        return loss, row_sum, col_sum, diag_s
    row_sum = torch.empty(b, dtype=torch.float32, device=dev)
    col_sum = torch.empty(b, dtype=torch.float32, device=dev) if kind == _lib.CLIP else None
    diag_s = torch.empty(b, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    counter = torch.empty(1, dtype=torch.int32, device=dev)              # cleared by the call
    with _on_device(dev):
        t, _b, _keep = _bind(temperature, dev)
        _lib.check(_lib.load().meclip_loss_forward(kind, x_hat.data_ptr(), y_hat.data_ptr(), b, d, x_hat.stride(0),
                                                   y_hat.stride(0), t, row_sum.data_ptr(),
                                                   _ptr(col_sum), diag_s.data_ptr(), loss.data_ptr(),
                                                   counter.data_ptr(), _ptr(status), _stream(x_hat)))
    return loss, row_sum, col_sum, diag_s


_MODE = {torch.bfloat16: _lib.STORE_BF16, torch.float32: _lib.STORE_F32}


def grad_workspace(rows, cols, d, device) -> torch.Tensor:
    n = _lib.load().meclip_grad_workspace_bytes(rows, cols, d)
    return torch.empty(n, dtype=torch.uint8, device=device)


def grad_block(kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, dx, dx_mode, dy, dy_mode,
               row_off=0, col_off=0, workspace=None, status=None, sum_g_s=None, scale_rule=GSCALE_FIXED):
    """One rows x cols block of the backward (see meclip_grad in include/meclip.h).
    sum_g_s: optional fp32 pair; its first element gets sum_ij G_ij S_ij of the block ADDED (meclip_grad_t).
    A tensor temperature stays on the device; grad_scale is then the scale for T = 1 and scale_rule says how
    the kernel completes it (see grad_scale_args)."""
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    if workspace is None:
        workspace = grad_workspace(rows, cols, d, x_hat.device)
    with _on_device(x_hat.device):
        t, _b, _keep = _bind(temperature, x_hat.device, scale_rule)
        head = (kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0), y_hat.stride(0), t,
                row_off, col_off, row_sum.data_ptr(), _ptr(col_sum), _ptr(grad_out), float(grad_scale), dx.data_ptr(), dx_mode,
                dx.stride(0), _ptr(dy), dy_mode, dy.stride(0) if dy is not None else 0)
        tail = (workspace.data_ptr(), workspace.numel(), _ptr(status), _stream(x_hat))
        if sum_g_s is None:
            _lib.check(_lib.load().meclip_grad(*head, *tail))
        else:
            _lib.check(_lib.load().meclip_grad_t(*head, sum_g_s.data_ptr(), *tail))


def grad_block_static(kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, dx, dx_mode, dy, dy_mode,
                      row_off=0, col_off=0, status=None):
    """grad_block on the library's built-in 32 MiB scratch (meclip_grad_static): no workspace
    argument and no allocation inside the call, for blocks of at most 4096 x 4096.  Calls share
    the scratch, so keep them on one stream."""
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    with _on_device(x_hat.device):
        _lib.check(_lib.load().meclip_grad_static(kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d,
                                                  x_hat.stride(0), y_hat.stride(0), float(temperature), row_off,
                                                  col_off, row_sum.data_ptr(), _ptr(col_sum), _ptr(grad_out),
                                                  float(grad_scale), dx.data_ptr(), dx_mode, dx.stride(0), _ptr(dy),
                                                  dy_mode, dy.stride(0) if dy is not None else 0, _ptr(status),
                                                  _stream(x_hat)))


def loss_backward(kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, dx_dtype, dy_dtype,
                  status=None, sum_g_s=None, need_dx=True, need_dy=True, scale_rule=GSCALE_FIXED, f32_operands=None):
    """Whole-batch backward on one GPU.  Returns (dx, dy) w.r.t. the normalised operands; an output
    that is not needed (frozen tower, or the second argument of LiT) is None and its contraction is skipped.
    sum_g_s: optional zeroed fp32 scalar that receives sum_ij G_ij S_ij (temperature gradient)."""
    b, d = x_hat.shape
    dev = x_hat.device
    need_dy = need_dy and kind == _lib.CLIP
    if not (need_dx or need_dy):
        return None, None
    dx = torch.empty(b, d, dtype=dx_dtype, device=dev) if need_dx else None
    dy = torch.empty(b, d, dtype=dy_dtype, device=dev) if need_dy else None
    ws = grad_workspace(b, b, d, dev)
    if f32_operands is not None:
        assert sum_g_s is None, "the tf32 route has no temperature gradient"
        x32, y32 = f32_operands
        with _on_device(dev):
            t, _b, _keep = _bind(temperature, dev, scale_rule)
            _lib.check(_lib.load().meclip_grad_tf32(kind, x_hat.data_ptr(), y_hat.data_ptr(), x32.data_ptr(),
                                                    x32.stride(0), y32.data_ptr(), y32.stride(0), b, b, d,
                                                    x_hat.stride(0), y_hat.stride(0), t, 0, 0, row_sum.data_ptr(),
                                                    _ptr(col_sum), _ptr(grad_out), float(grad_scale), _ptr(dx),
                                                    _MODE[dx_dtype], d, _ptr(dy),
                                                    _MODE[dy_dtype] if dy is not None else 0, d, ws.data_ptr(),
                                                    ws.numel(), _ptr(status), _stream(x_hat)))
        return dx, dy
    if sum_g_s is not None:
        with _on_device(dev):
            t, _b, _keep = _bind(temperature, dev, scale_rule)
            _lib.check(_lib.load().meclip_grad_t(kind, x_hat.data_ptr(), y_hat.data_ptr(), b, b, d, x_hat.stride(0),
                                                 y_hat.stride(0), t, 0, 0, row_sum.data_ptr(),
                                                 _ptr(col_sum), _ptr(grad_out), float(grad_scale), _ptr(dx),
                                                 _MODE[dx_dtype], d, _ptr(dy),
                                                 _MODE[dy_dtype] if dy is not None else 0, d, sum_g_s.data_ptr(),
                                                 ws.data_ptr(), ws.numel(), _ptr(status), _stream(x_hat)))
        return dx, dy
    with _on_device(dev):
        t, _b, _keep = _bind(temperature, dev, scale_rule)
        _lib.check(_lib.load().meclip_loss_backward(kind, x_hat.data_ptr(), y_hat.data_ptr(), b, d, x_hat.stride(0),
                                                    y_hat.stride(0), t, row_sum.data_ptr(),
                                                    _ptr(col_sum), _ptr(grad_out), float(grad_scale), _ptr(dx),
                                                    _MODE[dx_dtype], d, _ptr(dy),
                                                    _MODE[dy_dtype] if dy is not None else 0, d, ws.data_ptr(),
                                                    ws.numel(), _ptr(status), _stream(x_hat)))
    return dx, dy


def siglip_sum(x_hat, y_hat, logit_scale, logit_bias, row_sum, diag_s, row_off=0, col_off=0, status=None):
    """One rows x cols block of the sigmoid-loss forward: row_sum[i] += sum_j softplus(-z_ij a_ij) / ln2."""
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    counter = torch.zeros(1, dtype=torch.int32, device=x_hat.device)
    with _on_device(x_hat.device):
        t, b, _keep = _bind(logit_scale, x_hat.device, GSCALE_FIXED, logit_bias)
        _lib.check(_lib.load().meclip_siglip_sum(x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                                 y_hat.stride(0), t, b, row_off, col_off,
                                                 row_sum.data_ptr(), diag_s.data_ptr(), counter.data_ptr(), _ptr(status),
                                                 _stream(x_hat)))


def siglip_loss_finalize(row_sum, diag_s, logit_scale, logit_bias, scale, loss_out, accumulate=False):
    with _on_device(row_sum.device):
        _lib.check(_lib.load().meclip_siglip_loss_finalize(row_sum.data_ptr(), diag_s.data_ptr(), row_sum.numel(),
                                                           0.0, 0.0, float(scale),
                                                           int(accumulate), loss_out.data_ptr(), _stream(row_sum)))


def siglip_forward(x_hat, y_hat, logit_scale, logit_bias, status=None):
    """Sigmoid-loss forward for a whole batch on one GPU; returns the 0-dim fp32 loss."""
    b = x_hat.shape[0]
    dev = x_hat.device
    row_sum = torch.zeros(b, dtype=torch.float32, device=dev)
    diag_s = torch.zeros(b, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    siglip_sum(x_hat, y_hat, logit_scale, logit_bias, row_sum, diag_s, 0, 0, status)
    siglip_loss_finalize(row_sum, diag_s, logit_scale, logit_bias, 1.0 / b, loss)
    return loss


def siglip_grad_block(x_hat, y_hat, logit_scale, logit_bias, grad_out, grad_scale_, dx, dx_mode, dy, dy_mode,
                      row_off=0, col_off=0, workspace=None, sums=None, status=None):
    """One rows x cols block of the sigmoid-loss backward (meclip_siglip_grad)."""
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    if workspace is None:
        workspace = grad_workspace(rows, cols, d, x_hat.device)
    with _on_device(x_hat.device):
        t, b, _keep = _bind(logit_scale, x_hat.device, GSCALE_TIMES_T if is_dev(logit_scale) else GSCALE_FIXED,
                            logit_bias)
        _lib.check(_lib.load().meclip_siglip_grad(x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                                  y_hat.stride(0), t, b, row_off,
                                                  col_off, _ptr(grad_out), float(grad_scale_), _ptr(dx), dx_mode,
                                                  dx.stride(0) if dx is not None else 0, _ptr(dy), dy_mode,
                                                  dy.stride(0) if dy is not None else 0, _ptr(sums),
                                                  workspace.data_ptr(), workspace.numel(), _ptr(status),
                                                  _stream(x_hat)))


def siglip_backward(x_hat, y_hat, logit_scale, logit_bias, grad_out, grad_scale_, dx_dtype, dy_dtype, sums=None,
                    need_dx=True, need_dy=True, status=None):
    """Sigmoid-loss backward for a whole batch; returns (dx, dy) w.r.t. the normalised operands.
    sums: optional two zeroed floats that receive {sum G S, sum G} for the scale / bias gradients."""
    b, d = x_hat.shape
    dev = x_hat.device
    if not (need_dx or need_dy):
        return None, None
    dx = torch.empty(b, d, dtype=dx_dtype, device=dev) if need_dx else None
    dy = torch.empty(b, d, dtype=dy_dtype, device=dev) if need_dy else None
    ws = grad_workspace(b, b, d, dev)
    with _on_device(dev):
        t, bias, _keep = _bind(logit_scale, dev, GSCALE_TIMES_T if is_dev(logit_scale) else GSCALE_FIXED, logit_bias)
        _lib.check(_lib.load().meclip_siglip_grad(x_hat.data_ptr(), y_hat.data_ptr(), b, b, d, x_hat.stride(0),
                                                  y_hat.stride(0), t, bias, 0, 0,
                                                  _ptr(grad_out), float(grad_scale_), _ptr(dx), _MODE[dx_dtype], d,
                                                  _ptr(dy), _MODE[dy_dtype], d, _ptr(sums), ws.data_ptr(), ws.numel(),
                                                  _ptr(status), _stream(x_hat)))
    return dx, dy


def lit_extend(y_ext, d_pad):
    """Writes the ones column (and seven zeros) at column d_pad of y_ext [rows, d_pad + 8]."""
    with _on_device(y_ext.device):
        _lib.check(_lib.load().meclip_lit_extend(y_ext.data_ptr(), y_ext.shape[0], d_pad, y_ext.stride(0), _stream(y_ext)))


def lit_fused_block(x_hat, y_ext, d_pad, temperature, u, u_mode, row_off=0, col_off=0, workspace=None, status=None):
    """One rows x cols block of the one-pass LiT forward: u (=|+=) E [y_ext] (meclip_lit_fused_forward)."""
    rows, cols = x_hat.shape[0], y_ext.shape[0]
    if workspace is None:
        workspace = grad_workspace(rows, cols, d_pad + 8, x_hat.device)
    with _on_device(x_hat.device):
        t, _b, _keep = _bind(temperature, x_hat.device)
        _lib.check(_lib.load().meclip_lit_fused_forward(x_hat.data_ptr(), y_ext.data_ptr(), rows, cols, d_pad,
                                                        x_hat.stride(0), y_ext.stride(0), t, row_off,
                                                        col_off, u.data_ptr(), u_mode, u.stride(0), workspace.data_ptr(),
                                                        workspace.numel(), _ptr(status), _stream(x_hat)))


def lit_fused_stats(x_hat, y_ext, u, d_pad):
    """(row_sum, diag_s) of the rows of u: row_sum = u[:, d_pad], diag_s[i] = <x_i, y_i>."""
    b = x_hat.shape[0]
    row_sum = torch.empty(b, dtype=torch.float32, device=u.device)
    diag_s = torch.empty(b, dtype=torch.float32, device=u.device)
    with _on_device(u.device):
        _lib.check(_lib.load().meclip_lit_fused_stats(x_hat.data_ptr(), x_hat.stride(0), y_ext.data_ptr(), y_ext.stride(0),
                                                      u.data_ptr(), u.stride(0), b, d_pad, row_sum.data_ptr(),
                                                      diag_s.data_ptr(), _stream(u)))
    return row_sum, diag_s


def lit_fused_forward(x_hat, y_ext, d_pad, temperature, status=None):
    """LiT forward that also does the gradient's contraction: x_hat [b, d_pad], y_ext [b, d_pad + 8] whose
    column d_pad gets the ones.  Returns (loss, u fp32 [b, d_pad + 8], row_sum)."""
    b = x_hat.shape[0]
    dev = x_hat.device
    u = torch.empty(b, d_pad + 8, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    lit_extend(y_ext, d_pad)
    lit_fused_block(x_hat, y_ext, d_pad, temperature, u, _lib.STORE_F32, 0, 0, None, status)
    row_sum, diag_s = lit_fused_stats(x_hat, y_ext, u, d_pad)
    loss_finalize(_lib.LIT, row_sum, None, diag_s, temperature, 1.0 / b, loss)
    return loss, u, row_sum


def lit_fused_backward(u, y_ext, row_sum, grad_out, grad_scale_, d_out, out_dtype, temperature=None,
                       scale_rule=GSCALE_FIXED):
    """dx [b, d_out] in out_dtype from the saved u (meclip_lit_fused_backward).  temperature: only needed
    when it is a tensor (grad_scale_ is then the scale for T = 1, completed on the device by scale_rule)."""
    b = u.shape[0]
    dx = torch.empty(b, d_out, dtype=out_dtype, device=u.device)
    with _on_device(u.device):
        if is_dev(temperature):
            _t, _b, _keep = _bind(temperature, u.device, scale_rule)
        _lib.check(_lib.load().meclip_lit_fused_backward(u.data_ptr(), u.stride(0), y_ext.data_ptr(), y_ext.stride(0),
                                                         row_sum.data_ptr(), _ptr(grad_out), float(grad_scale_), b, d_out,
                                                         dx.data_ptr(), _DT[out_dtype], dx.stride(0), _stream(u)))
    return dx


# ---- whole-step entry points (small batches) --------------------------------------------------------------
_step_ws = {}
_step_saved_bytes = {}


def step_workspace(batch: int, d: int, device) -> torch.Tensor:
    """Backward workspace of the small-batch step path, cached per (device, stream, shape): it is scratch that
    lives only inside one library call, and calls on one stream are ordered."""
    key = (device.index, torch._C._cuda_getCurrentRawStream(device.index), batch, d)
    need = _lib.load().meclip_step_workspace_bytes(batch, d)      # depends on the blocking (a test hook can change it)
    ws = _step_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = _step_ws[key] = torch.empty(need, dtype=torch.uint8, device=device)
    return ws


def step_forward(kind, x, y, normalize, temperature, status=None):
    """(loss, saved): the module's forward in one library call (meclip_step_forward)."""
    b, d = x.shape
    lib = _lib.load()
    n_saved = _step_saved_bytes.get((b, d))
    if n_saved is None:
        n_saved = _step_saved_bytes[(b, d)] = lib.meclip_step_saved_bytes(b, d)
    saved = torch.empty(n_saved, dtype=torch.uint8, device=x.device)
    loss = torch.empty((), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        t, _b, _keep = _bind(temperature, x.device)
        _lib.check(lib.meclip_step_forward(kind, x.data_ptr(), y.data_ptr(), _DT[x.dtype], b, d, x.stride(0), y.stride(0),
                                           int(normalize), t, saved.data_ptr(), saved.numel(), loss.data_ptr(),
                                           _ptr(status), _stream(x)))
    return loss, saved


def step_backward(kind, saved, batch, d, normalize, temperature, grad_out, grad_scale_, scale_rule, out_dtype,
                  need_dx=True, need_dy=True, status=None):
    """(dx, dy) in out_dtype from the buffer step_forward saved (meclip_step_backward)."""
    dev = saved.device
    dx = torch.empty(batch, d, dtype=out_dtype, device=dev) if need_dx else None
    dy = torch.empty(batch, d, dtype=out_dtype, device=dev) if need_dy else None
    ws = step_workspace(batch, d, dev)
    with _on_device(dev):
        t, _b, _keep = _bind(temperature, dev, scale_rule)
        _lib.check(_lib.load().meclip_step_backward(kind, saved.data_ptr(), saved.numel(), batch, d, int(normalize), t,
                                                    _ptr(grad_out), float(grad_scale_), _ptr(dx), _ptr(dy),
                                                    _DT[out_dtype], d, d, ws.data_ptr(), ws.numel(), _ptr(status),
                                                    torch._C._cuda_getCurrentRawStream(dev.index)))
    return dx, dy


def grad_scale(batch: int, temperature: float, stable: bool) -> float:
    """1/(B T) (reference clip_loss.py:182, 235) or, for the Stable variants,
    sqrt(B/T)/B = 1/sqrt(B T) (clip_loss.py:299, 352)."""
    return 1.0 / math.sqrt(batch * temperature) if stable else 1.0 / (batch * temperature)


def grad_scale_args(batch: int, temperature, stable: bool):
    """(grad_scale, scale_rule) for the backward entry points.  A float temperature gives the finished
    scale and GSCALE_FIXED.  A tensor temperature stays on the device: the scale is formed for T = 1 and
    the kernels divide by T (or sqrt(T) for the Stable variants) themselves."""
    if is_dev(temperature):
        return grad_scale(batch, 1.0, stable), (GSCALE_OVER_SQRT_T if stable else GSCALE_OVER_T)
    return grad_scale(batch, float(temperature), stable), GSCALE_FIXED


def debug_wait_probe(status: torch.Tensor, limit_ns: int = 1_000_000) -> None:
    """Test hook: one tiny kernel whose bounded wait is meant to run out (it sets the status word)."""
    with _on_device(status.device):
        _lib.check(_lib.load().meclip_debug_wait_probe(int(limit_ns), status.data_ptr(), _stream(status)))


def debug_gemm(a, b, a_mn_major, b_mn_major, m, n, k, tile_n=0, c_in=None, status=None) -> torch.Tensor:
    c = torch.empty(m, n, dtype=torch.float32, device=a.device) if c_in is None else c_in.clone()
    with _on_device(a.device):
        _lib.check(_lib.load().meclip_debug_gemm(a.data_ptr(), a.stride(0), int(a_mn_major), b.data_ptr(), b.stride(0),
                                                 int(b_mn_major), m, n, k, tile_n, c.data_ptr(), c.stride(0),
                                                 _ptr(c_in) and c.data_ptr(), _ptr(status), _stream(a)))
    return c


class RingCall:
    """One rank's view of the ring for meclip_ring_sum_exp / meclip_ring_grad (include/meclip.h): the addresses
    of every rank's shard of the second argument as this device sees them, two local receive buffers and the
    copy stream.  The compute stream is the current stream at call time."""

    def __init__(self, rank: int, world: int, x_hat: torch.Tensor, shard_addresses, y_own: torch.Tensor, copy_stream):
        import ctypes
        assert len(shard_addresses) == world and x_hat.shape == y_own.shape
        self.rank, self.world, self.x_hat, self.y_own = rank, world, x_hat, y_own
        self.copy_stream = copy_stream
        self.recv = [torch.empty_like(y_own) for _ in range(2)] if world > 1 else [None, None]
        self._shards = (ctypes.c_void_p * world)(*[int(a) for a in shard_addresses])
        self.desc = _lib.RingDesc(rank, world, x_hat.shape[0], x_hat.shape[1], x_hat.stride(0), y_own.stride(0),
                                  ctypes.cast(self._shards, ctypes.POINTER(ctypes.c_void_p)),
                                  (ctypes.c_void_p * 2)(_ptr(self.recv[0]), _ptr(self.recv[1])), None,
                                  copy_stream.cuda_stream)

    def _ref(self):
        import ctypes
        self.desc.compute_stream = _stream(self.x_hat)
        return ctypes.byref(self.desc)


def ring_sum_exp(call: RingCall, kind, temperature, status=None):
    """Forward sums of one rank over the whole ring in one library call.  Returns (row_sum [b], col_part
    [world, b] or None, diag [b]); the caller reduce-scatters col_part over the ranks."""
    x = call.x_hat
    b, dev = x.shape[0], x.device
    row_sum = torch.empty(b, dtype=torch.float32, device=dev)
    diag = torch.empty(b, dtype=torch.float32, device=dev)
    col_part = torch.empty(call.world, b, dtype=torch.float32, device=dev) if kind == _lib.CLIP else None
    counters = torch.empty(call.world, dtype=torch.int32, device=dev)
    with _on_device(dev):
        t, _b, _keep = _bind(temperature, dev)
        _lib.check(_lib.load().meclip_ring_sum_exp(call._ref(), kind, x.data_ptr(), t, row_sum.data_ptr(),
                                                   _ptr(col_part), diag.data_ptr(), counters.data_ptr(), _ptr(status)))
    return row_sum, col_part, diag


def ring_grad(call: RingCall, kind, temperature, row_sum, col_sum_all, grad_out, grad_scale, inbox_addresses,
              status=None, scale_rule=GSCALE_FIXED):
    """Backward of one rank over the whole ring in one library call.  Returns (dx fp32 [b, d], dy_own fp32
    [b, d] or None); for CLIP the partial gradients of the other ranks' shards are on their way into the
    owners' inboxes (inbox_addresses[p]: rank p's inbox as this device sees it) on the copy stream."""
    import ctypes
    x = call.x_hat
    b, d = x.shape
    dev = x.device
    clip = kind == _lib.CLIP
    dx = torch.empty(b, d, dtype=torch.float32, device=dev)
    dy = torch.empty(b, d, dtype=torch.float32, device=dev) if clip else None
    part = [torch.empty(b, d, dtype=torch.float32, device=dev) for _ in range(2)] if clip and call.world > 1 else [None, None]
    inbox = None
    if clip and call.world > 1:
        inbox = (ctypes.c_void_p * call.world)(*[int(a) if a else None for a in inbox_addresses])
    ws = grad_workspace(b, b, d, dev)
    with _on_device(dev):
        t, _b, _keep = _bind(temperature, dev, scale_rule)
        _lib.check(_lib.load().meclip_ring_grad(call._ref(), kind, x.data_ptr(), t, row_sum.data_ptr(),
                                                _ptr(col_sum_all), _ptr(grad_out), float(grad_scale), dx.data_ptr(),
                                                dx.stride(0), _ptr(dy), _ptr(part[0]), _ptr(part[1]), inbox,
                                                ws.data_ptr(), ws.numel(), _ptr(status)))
    # part, ws and the receive buffers are in use on the copy / compute streams: the caching allocator must not
    # hand them out to another stream's tensors before this work has run
    for t_ in part:
        if t_ is not None:
            t_.record_stream(call.copy_stream)
    return dx, dy
