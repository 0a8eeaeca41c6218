"""Torch-tensor front end of the C ABI: every function here launches CUDA kernels from
libmeclip_sm100.so on the current stream of the tensors' device.  Torch is used for
device memory and streams only; no arithmetic of the loss path happens in torch.
"""
from __future__ import annotations

import math

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32, torch.float16: _lib.F16}


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


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
    with torch.cuda.device(status.device):
        _lib.check(_lib.load().meclip_read_status(status.data_ptr(), _stream(status)))


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
    with torch.cuda.device(x.device):
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
    with torch.cuda.device(g.device):
        _lib.check(_lib.load().meclip_normalize_bwd(g.data_ptr(), _DT[g.dtype], g.stride(0), _ptr(x_hat),
                                                    x_hat.stride(0) if x_hat is not None else 0, _ptr(inv_norm),
                                                    rows, d, dx.data_ptr(), _DT[out_dtype], d, _stream(g)))
    return dx


def accumulate_f32(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst += src (fp32, contiguous, same shape) on the current stream."""
    assert dst.dtype == torch.float32 and src.dtype == torch.float32 and dst.numel() == src.numel()
    with torch.cuda.device(dst.device):
        _lib.check(_lib.load().meclip_accumulate_f32(dst.data_ptr(), src.data_ptr(), dst.numel(), _stream(dst)))


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


def sum_exp(kind, x_hat, y_hat, temperature, row_sum, col_sum, diag_s, row_off=0, col_off=0, status=None):
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    counter = torch.zeros(1, dtype=torch.int32, device=x_hat.device)     # dynamic tile hand-out
    with torch.cuda.device(x_hat.device):
        _lib.check(_lib.load().meclip_sum_exp(kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                              y_hat.stride(0), float(temperature), row_off, col_off, row_sum.data_ptr(),
                                              _ptr(col_sum), diag_s.data_ptr(), counter.data_ptr(), _ptr(status),
                                              _stream(x_hat)))


def loss_finalize(kind, row_sum, col_sum, diag_s, temperature, scale, loss_out, accumulate=False):
    with torch.cuda.device(row_sum.device):
        _lib.check(_lib.load().meclip_loss_finalize(kind, row_sum.data_ptr(), _ptr(col_sum), diag_s.data_ptr(),
                                                    row_sum.numel(), float(temperature), float(scale), int(accumulate),
                                                    loss_out.data_ptr(), _stream(row_sum)))


def loss_forward(kind, x_hat, y_hat, temperature, status=None):
    """Returns (loss 0-dim fp32, row_sum, col_sum or None, diag_s)."""
    b, d = x_hat.shape
    assert y_hat.shape == x_hat.shape
    dev = x_hat.device
    row_sum = torch.empty(b, dtype=torch.float32, device=dev)
    col_sum = torch.empty(b, dtype=torch.float32, device=dev) if kind == _lib.CLIP else None
    diag_s = torch.empty(b, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    counter = torch.empty(1, dtype=torch.int32, device=dev)              # cleared by the call
    with torch.cuda.device(dev):
        _lib.check(_lib.load().meclip_loss_forward(kind, x_hat.data_ptr(), y_hat.data_ptr(), b, d, x_hat.stride(0),
                                                   y_hat.stride(0), float(temperature), row_sum.data_ptr(),
                                                   _ptr(col_sum), diag_s.data_ptr(), loss.data_ptr(),
                                                   counter.data_ptr(), _ptr(status), _stream(x_hat)))
    return loss, row_sum, col_sum, diag_s


_MODE = {torch.bfloat16: _lib.STORE_BF16, torch.float32: _lib.STORE_F32}


def grad_workspace(rows, cols, d, device) -> torch.Tensor:
    n = _lib.load().meclip_grad_workspace_bytes(rows, cols, d)
    return torch.empty(n, dtype=torch.uint8, device=device)


def grad_block(kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, dx, dx_mode, dy, dy_mode,
               row_off=0, col_off=0, workspace=None, status=None, sum_g_s=None):
    """One rows x cols block of the backward (see meclip_grad in include/meclip.h).
    sum_g_s: optional fp32 pair; its first element gets sum_ij G_ij S_ij of the block ADDED (meclip_grad_t)."""
    rows, d = x_hat.shape
    cols = y_hat.shape[0]
    if workspace is None:
        workspace = grad_workspace(rows, cols, d, x_hat.device)
    head = (kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0), y_hat.stride(0), float(temperature),
            row_off, col_off, row_sum.data_ptr(), _ptr(col_sum), _ptr(grad_out), float(grad_scale), dx.data_ptr(), dx_mode,
            dx.stride(0), _ptr(dy), dy_mode, dy.stride(0) if dy is not None else 0)
    tail = (workspace.data_ptr(), workspace.numel(), _ptr(status), _stream(x_hat))
    with torch.cuda.device(x_hat.device):
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
    with torch.cuda.device(x_hat.device):
        _lib.check(_lib.load().meclip_grad_static(kind, x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d,
                                                  x_hat.stride(0), y_hat.stride(0), float(temperature), row_off,
                                                  col_off, row_sum.data_ptr(), _ptr(col_sum), _ptr(grad_out),
                                                  float(grad_scale), dx.data_ptr(), dx_mode, dx.stride(0), _ptr(dy),
                                                  dy_mode, dy.stride(0) if dy is not None else 0, _ptr(status),
                                                  _stream(x_hat)))


def loss_backward(kind, x_hat, y_hat, temperature, row_sum, col_sum, grad_out, grad_scale, dx_dtype, dy_dtype,
                  status=None, sum_g_s=None, need_dx=True, need_dy=True):
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
    if sum_g_s is not None:
        with torch.cuda.device(dev):
            _lib.check(_lib.load().meclip_grad_t(kind, x_hat.data_ptr(), y_hat.data_ptr(), b, b, d, x_hat.stride(0),
                                                 y_hat.stride(0), float(temperature), 0, 0, row_sum.data_ptr(),
                                                 _ptr(col_sum), _ptr(grad_out), float(grad_scale), _ptr(dx),
                                                 _MODE[dx_dtype], d, _ptr(dy),
                                                 _MODE[dy_dtype] if dy is not None else 0, d, sum_g_s.data_ptr(),
                                                 ws.data_ptr(), ws.numel(), _ptr(status), _stream(x_hat)))
        return dx, dy
    with torch.cuda.device(dev):
        _lib.check(_lib.load().meclip_loss_backward(kind, x_hat.data_ptr(), y_hat.data_ptr(), b, d, x_hat.stride(0),
                                                    y_hat.stride(0), float(temperature), row_sum.data_ptr(),
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
    with torch.cuda.device(x_hat.device):
        _lib.check(_lib.load().meclip_siglip_sum(x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                                 y_hat.stride(0), float(logit_scale), float(logit_bias), row_off, col_off,
                                                 row_sum.data_ptr(), diag_s.data_ptr(), counter.data_ptr(), _ptr(status),
                                                 _stream(x_hat)))


def siglip_loss_finalize(row_sum, diag_s, logit_scale, logit_bias, scale, loss_out, accumulate=False):
    with torch.cuda.device(row_sum.device):
        _lib.check(_lib.load().meclip_siglip_loss_finalize(row_sum.data_ptr(), diag_s.data_ptr(), row_sum.numel(),
                                                           float(logit_scale), float(logit_bias), float(scale),
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
    with torch.cuda.device(x_hat.device):
        _lib.check(_lib.load().meclip_siglip_grad(x_hat.data_ptr(), y_hat.data_ptr(), rows, cols, d, x_hat.stride(0),
                                                  y_hat.stride(0), float(logit_scale), float(logit_bias), row_off,
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
    with torch.cuda.device(dev):
        _lib.check(_lib.load().meclip_siglip_grad(x_hat.data_ptr(), y_hat.data_ptr(), b, b, d, x_hat.stride(0),
                                                  y_hat.stride(0), float(logit_scale), float(logit_bias), 0, 0,
                                                  _ptr(grad_out), float(grad_scale_), _ptr(dx), _MODE[dx_dtype], d,
                                                  _ptr(dy), _MODE[dy_dtype], d, _ptr(sums), ws.data_ptr(), ws.numel(),
                                                  _ptr(status), _stream(x_hat)))
    return dx, dy


def lit_extend(y_ext, d_pad):
    """Writes the ones column (and seven zeros) at column d_pad of y_ext [rows, d_pad + 8]."""
    with torch.cuda.device(y_ext.device):
        _lib.check(_lib.load().meclip_lit_extend(y_ext.data_ptr(), y_ext.shape[0], d_pad, y_ext.stride(0), _stream(y_ext)))


def lit_fused_block(x_hat, y_ext, d_pad, temperature, u, u_mode, row_off=0, col_off=0, workspace=None, status=None):
    """One rows x cols block of the one-pass LiT forward: u (=|+=) E [y_ext] (meclip_lit_fused_forward)."""
    rows, cols = x_hat.shape[0], y_ext.shape[0]
    if workspace is None:
        workspace = grad_workspace(rows, cols, d_pad + 8, x_hat.device)
    with torch.cuda.device(x_hat.device):
        _lib.check(_lib.load().meclip_lit_fused_forward(x_hat.data_ptr(), y_ext.data_ptr(), rows, cols, d_pad,
                                                        x_hat.stride(0), y_ext.stride(0), float(temperature), row_off,
                                                        col_off, u.data_ptr(), u_mode, u.stride(0), workspace.data_ptr(),
                                                        workspace.numel(), _ptr(status), _stream(x_hat)))


def lit_fused_stats(x_hat, y_ext, u, d_pad):
    """(row_sum, diag_s) of the rows of u: row_sum = u[:, d_pad], diag_s[i] = <x_i, y_i>."""
    b = x_hat.shape[0]
    row_sum = torch.empty(b, dtype=torch.float32, device=u.device)
    diag_s = torch.empty(b, dtype=torch.float32, device=u.device)
    with torch.cuda.device(u.device):
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


def lit_fused_backward(u, y_ext, row_sum, grad_out, grad_scale_, d_out, out_dtype):
    """dx [b, d_out] in out_dtype from the saved u (meclip_lit_fused_backward)."""
    b = u.shape[0]
    dx = torch.empty(b, d_out, dtype=out_dtype, device=u.device)
    with torch.cuda.device(u.device):
        _lib.check(_lib.load().meclip_lit_fused_backward(u.data_ptr(), u.stride(0), y_ext.data_ptr(), y_ext.stride(0),
                                                         row_sum.data_ptr(), _ptr(grad_out), float(grad_scale_), b, d_out,
                                                         dx.data_ptr(), _DT[out_dtype], dx.stride(0), _stream(u)))
    return dx


def grad_scale(batch: int, temperature: float, stable: bool) -> float:
    """1/(B T) (reference clip_loss.py:182, 235) or, for the Stable variants,
    sqrt(B/T)/B = 1/sqrt(B T) (clip_loss.py:299, 352)."""
    return 1.0 / math.sqrt(batch * temperature) if stable else 1.0 / (batch * temperature)


def debug_gemm(a, b, a_mn_major, b_mn_major, m, n, k, tile_n=0, c_in=None, status=None) -> torch.Tensor:
    c = torch.empty(m, n, dtype=torch.float32, device=a.device) if c_in is None else c_in.clone()
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().meclip_debug_gemm(a.data_ptr(), a.stride(0), int(a_mn_major), b.data_ptr(), b.stride(0),
                                                 int(b_mn_major), m, n, k, tile_n, c.data_ptr(), c.stride(0),
                                                 _ptr(c_in) and c.data_ptr(), _ptr(status), _stream(a)))
    return c
