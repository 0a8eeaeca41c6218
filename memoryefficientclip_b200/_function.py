"""The one autograd node behind all eight public classes.

forward:  [normalise | convert to bf16] -> tile pass for the sums -> loss
backward: coefficient panels + two contractions -> [normalise Jacobian]
Saved for backward: the bf16 operands, the fp32 row/column sums and, when the node
normalises, the inverse norms - O(B*D) like the reference (clip_loss.py:199).
"""
from __future__ import annotations

import torch

import os

from . import _lib, ops

# Batches up to this many rows take the whole-step entry points (two library calls per step: the step is
# host-bound there); MECLIP_STEP_PATH_ROWS=0 switches that path off.
_STEP_PATH_ROWS = int(os.environ.get("MECLIP_STEP_PATH_ROWS", "4096"))

# MECLIP_LIT_FUSED=0 keeps LiT on the two-pass path (sums, then recomputing backward) for A/B measurements
_LIT_FUSED = os.environ.get("MECLIP_LIT_FUSED", "1") != "0"


class ContrastiveLossFn(torch.autograd.Function):
    """apply(x, y, temperature, kind, stable, normalize) -> 0-dim fp32 loss."""

    @staticmethod
    def run_forward(ctx, x, y, temperature, kind, stable, normalize):
        assert x.is_cuda and y.is_cuda                      # reference clip_loss.py:166
        assert x.shape == y.shape                           # reference clip_loss.py:167
        ops._check_matrix(x, "first input")
        ops._check_matrix(y, "second input")
        assert x.device == y.device
        # A tensor temperature (e.g. an nn.Parameter) stays on the device: the kernels read it there, so a
        # learnable temperature costs no host synchronisation.  It then also receives a gradient, which the
        # reference does not provide (clip_loss.py:256).
        t_is_tensor = isinstance(temperature, torch.Tensor)
        if t_is_tensor:
            assert temperature.numel() == 1, "temperature must be a scalar"
            temperature_value = temperature.detach()
        else:
            temperature_value = float(temperature)
            assert temperature_value > 0.0, "temperature must be positive"
        learn_t = t_is_tensor and temperature.requires_grad
        status = ops.status_word(x.device)
        ops.poll_status(x.device)           # raises if a kernel of an earlier step gave up a bounded wait
        # small batches are host-bound: the whole step in two library calls (LiT too: fewer calls beat fewer FLOPs there)
        # fp32 inputs, on request: S from fp32 operands with tf32 MMAs, as the reference's tl.dot (clip_loss.py:53)
        tf32 = (ops.TF32_OPERANDS and x.dtype == torch.float32 and y.dtype == torch.float32 and not learn_t
                and not ops.DETERMINISTIC and x.stride(1) == 1 and y.stride(1) == 1)
        step_path = (not tf32 and not learn_t and x.shape[0] <= _STEP_PATH_ROWS and x.dtype == y.dtype and not ops.DETERMINISTIC
                     and x.stride(1) == 1 and y.stride(1) == 1 and x.stride(0) >= x.shape[1]
                     and y.stride(0) >= y.shape[1])
        # LiT's coefficients separate (G_ij = g E_ij / r_i - g [i == j]), so when the first input needs a gradient the
        # forward also contracts E with [Y | 1] and the backward is a row kernel: 4 B^2 D FLOPs instead of 6 B^2 D
        if kind == _lib.LIT and _LIT_FUSED and ctx.needs_input_grad[0] and not learn_t and not step_path and not tf32:
            x_hat, inv_x = ops.normalize_fwd(x, True) if normalize else (ops.as_operand(x), None)
            y_ext, _inv_y = ops.normalize_fwd(y, normalize, extra_cols=8)
            d_pad = x_hat.shape[1]
            loss, u, row_sum = ops.lit_fused_forward(x_hat, y_ext, d_pad, temperature_value, status=status)
            ctx.save_for_backward(*([u, y_ext, row_sum] + ([x_hat, inv_x] if normalize else [])))
            ctx.meclip = (temperature_value, kind, bool(stable), bool(normalize), x.dtype, y.dtype, x.shape[1])
            ctx.meclip_t = None
            ctx.meclip_fused = True
            return loss
        ctx.meclip_fused = False
        ctx.meclip_step = False
        if step_path:
            loss, saved = ops.step_forward(kind, x, y, normalize, temperature_value, status=status)
            ctx.save_for_backward(saved)
            ctx.meclip = (temperature_value, kind, bool(stable), bool(normalize), x.dtype, y.dtype, x.shape[1])
            ctx.meclip_t = None
            ctx.meclip_step = True
            ctx.meclip_batch = x.shape[0]
            if not any(ctx.needs_input_grad[:2]):
                ops.post_status(x.device)
            return loss
        if normalize:
            x_hat, inv_x = ops.normalize_fwd(x, True)
            y_hat, inv_y = ops.normalize_fwd(y, True)
        else:
            x_hat, inv_x = ops.as_operand(x), None
            y_hat, inv_y = ops.as_operand(y), None
        f32_ops = (ops.operand_f32(x, inv_x), ops.operand_f32(y, inv_y)) if tf32 else None
        loss, row_sum, col_sum, _diag = ops.loss_forward(kind, x_hat, y_hat, temperature_value, status=status,
                                                         f32_operands=f32_ops)
        if not any(ctx.needs_input_grad[:3]):
            ops.post_status(x.device)       # no backward will follow this forward
        saved = [x_hat, y_hat, row_sum]
        if col_sum is not None:
            saved.append(col_sum)
        if normalize:
            saved += [inv_x, inv_y]
        ctx.meclip_tf32 = tf32
        if tf32:
            saved += list(f32_ops)
        ctx.save_for_backward(*saved)
        ctx.meclip = (temperature_value, kind, bool(stable), bool(normalize), x.dtype, y.dtype, x.shape[1])
        ctx.meclip_t = temperature if t_is_tensor and temperature.requires_grad else None
        return loss

    @staticmethod
    def run_backward(ctx, grad_output):
        temperature, kind, stable, normalize, x_dtype, y_dtype, d = ctx.meclip
        saved = list(ctx.saved_tensors)
        if getattr(ctx, "meclip_fused", False):
            u, y_ext, row_sum = saved[:3]
            go = grad_output.detach().to(device=u.device, dtype=torch.float32).reshape(1).contiguous()
            scale, rule = ops.grad_scale_args(u.shape[0], temperature, stable)
            ctx.meclip_dt = None
            if normalize:
                x_hat, inv_x = saved[3:]
                g32 = ops.lit_fused_backward(u, y_ext, row_sum, go, scale, x_hat.shape[1], torch.float32, temperature,
                                             rule)
                dx = ops.normalize_bwd(g32, x_hat, inv_x, x_dtype, d)
            else:
                dx = ops.lit_fused_backward(u, y_ext, row_sum, go, scale, d, x_dtype, temperature, rule)
            ops.post_status(u.device)
            return dx, None
        if getattr(ctx, "meclip_step", False):
            buf = saved[0]
            go = grad_output
            if go.dtype != torch.float32 or go.device != buf.device or not go.is_contiguous():
                go = go.detach().to(device=buf.device, dtype=torch.float32).reshape(1).contiguous()
            batch = ctx.meclip_batch
            scale, rule = ops.grad_scale_args(batch, temperature, stable)
            need = tuple(ctx.needs_input_grad) + (False, False)
            ctx.meclip_dt = None
            need_dy = bool(need[1]) and kind == _lib.CLIP       # LiT: the second input gets none (lit_loss.py:247)
            if not (need[0] or need_dy):
                return None, None
            dx, dy = ops.step_backward(kind, buf, batch, d, normalize, temperature, go, scale, rule, x_dtype,
                                       need_dx=bool(need[0]), need_dy=need_dy,
                                       status=ops.status_word(buf.device))
            ctx.meclip_dt = None
            ops.post_status(buf.device)
            return dx, dy
        x_hat, y_hat, row_sum = saved[:3]
        rest = saved[3:]
        f32_ops = None
        if getattr(ctx, "meclip_tf32", False):
            f32_ops = (rest[-2], rest[-1])
            rest = rest[:-2]
        col_sum = rest.pop(0) if kind == _lib.CLIP else None
        inv_x, inv_y = (rest if normalize else (None, None))
        batch = x_hat.shape[0]
        # grad_output stays on the device: no host sync (the reference compares it to 1.0 on the host)
        go = grad_output.detach().to(device=x_hat.device, dtype=torch.float32).reshape(1).contiguous()
        scale, rule = ops.grad_scale_args(batch, temperature, stable)
        status = ops.status_word(x_hat.device)
        need = tuple(ctx.needs_input_grad) + (False, False)
        want_dx = bool(need[0])
        want_dy = kind == _lib.CLIP and bool(need[1])      # a frozen tower costs no contraction
        # with the fused Jacobian the contraction output stays fp32 until the Jacobian rounds once; the same
        # row kernel converts when the contraction cannot write the input's dtype or feature count itself
        post_x = normalize or not ops.direct_grad_dtype(x_dtype, d)
        post_y = normalize or not ops.direct_grad_dtype(y_dtype, d)
        dx_t = torch.float32 if post_x else x_dtype
        dy_t = torch.float32 if post_y else y_dtype
        t_param = getattr(ctx, "meclip_t", None)
        sum_g_s = torch.zeros(2, dtype=torch.float32, device=x_hat.device) if t_param is not None else None
        if sum_g_s is not None and not (want_dx or want_dy):
            want_dx = True       # the temperature sum is produced by the coefficient pass of the backward
        dx, dy = ops.loss_backward(kind, x_hat, y_hat, temperature, row_sum, col_sum, go, scale, dx_t, dy_t,
                                   status=status, sum_g_s=sum_g_s, need_dx=want_dx, need_dy=want_dy, scale_rule=rule,
                                   f32_operands=f32_ops)
        ctx.meclip_dt = None
        if sum_g_s is not None:
            # sum_ij G_ij S_ij = g B dL/d(1/T) with g = go * scale, so go * dL/dT = -(sum / (scale B)) / T^2.
            # (The Stable scaling only rescales the feature gradients; the temperature gets the true one.)
            # The temperature is a device tensor here; scale was formed for T = 1 and the kernels completed it
            # with 1/T (Stable: 1/sqrt(T)), so the same factor is applied in tensor arithmetic: no host read.
            t32 = temperature.to(torch.float32).reshape(())
            scale_t = scale / (torch.sqrt(t32) if stable else t32)
            dt = -sum_g_s[0] / (scale_t * batch * t32 * t32)
            ctx.meclip_dt = dt.reshape(t_param.shape).to(t_param.dtype)
        if post_x and dx is not None:
            dx = ops.normalize_bwd(dx, x_hat, inv_x, x_dtype, d)
        if post_y and dy is not None:
            dy = ops.normalize_bwd(dy, y_hat, inv_y, y_dtype, d)
        ops.post_status(x_hat.device)       # looked at by the next forward, without stalling this step
        return (dx if need[0] else None), (dy if want_dy else None)

    @staticmethod
    def forward(ctx, x, y, temperature, kind, stable, normalize):
        return ContrastiveLossFn.run_forward(ctx, x, y, temperature, kind, stable, normalize)

    @staticmethod
    def backward(ctx, grad_output):
        dx, dy = ContrastiveLossFn.run_backward(ctx, grad_output)
        return dx, dy, ctx.meclip_dt, None, None, None
