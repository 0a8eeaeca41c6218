"""Sigmoid (SigLIP) pairwise contrastive loss with O(B*D) memory on B200.

Not part of the reference (which has the softmax CLIP / LiT losses only); it runs on the same
tile kernels with a different elementwise function, needs no row or column sums, and has a
learnable logit scale and bias:

    a_ij = t * <x_i, y_j> + b,    loss = (1/B) * sum_ij softplus(-z_ij * a_ij),   z_ii = +1, z_ij = -1

``MemoryEfficientSigLIPLoss(init_logit_scale=10.0, init_logit_bias=-10.0, normalized_inputs=False)``
keeps ``log_logit_scale`` and ``logit_bias`` as parameters (t = exp(log_logit_scale)) and takes
``forward(image_features, text_features)``; ``MemoryEfficientSigLIPLossFn.apply(x, y, t, b, normalize)``
is the autograd node (gradients for x, y, t and b).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import _lib, ops


class MemoryEfficientSigLIPLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, logit_scale, logit_bias, normalize):
        assert x.is_cuda and y.is_cuda and x.shape == y.shape and x.device == y.device
        ops._check_matrix(x, "first input")
        ops._check_matrix(y, "second input")
        if normalize:
            x_hat, inv_x = ops.normalize_fwd(x, True)
            y_hat, inv_y = ops.normalize_fwd(y, True)
        else:
            x_hat, inv_x = ops.as_operand(x), None
            y_hat, inv_y = ops.as_operand(y), None
        # tensor scale / bias stay on the device (the kernels read them there): no host synchronisation
        t = logit_scale.detach() if isinstance(logit_scale, torch.Tensor) else float(logit_scale)
        b = logit_bias.detach() if isinstance(logit_bias, torch.Tensor) else float(logit_bias)
        status = ops.status_word(x.device)
        ops.poll_status(x.device)
        loss = ops.siglip_forward(x_hat, y_hat, t, b, status=status)
        saved = [x_hat, y_hat] + ([inv_x, inv_y] if normalize else [])
        ctx.save_for_backward(*saved)
        ctx.sig = (t, b, bool(normalize), x.dtype, y.dtype, x.shape[1],
                   (logit_scale.shape, logit_scale.dtype) if isinstance(logit_scale, torch.Tensor) else None,
                   (logit_bias.shape, logit_bias.dtype) if isinstance(logit_bias, torch.Tensor) else None)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        t, b, normalize, x_dtype, y_dtype, d, t_tensor, b_tensor = ctx.sig
        saved = list(ctx.saved_tensors)
        x_hat, y_hat = saved[:2]
        inv_x, inv_y = saved[2:] if normalize else (None, None)
        need = ctx.needs_input_grad
        batch = x_hat.shape[0]
        go = grad_output.detach().to(device=x_hat.device, dtype=torch.float32).reshape(1).contiguous()
        want_tb = bool(need[2] or need[3])
        want_dx, want_dy = bool(need[0]), bool(need[1])
        if want_tb and not (want_dx or want_dy):
            want_dx = True
        sums = torch.zeros(2, dtype=torch.float32, device=x_hat.device) if want_tb else None
        post_x = normalize or not ops.direct_grad_dtype(x_dtype, d)
        post_y = normalize or not ops.direct_grad_dtype(y_dtype, d)
        dx_t = torch.float32 if post_x else x_dtype
        dy_t = torch.float32 if post_y else y_dtype
        # grad_scale = t / B; with a device-resident t the kernel multiplies 1/B by t itself
        gscale = 1.0 / batch if ops.is_dev(t) else t / batch
        dx, dy = ops.siglip_backward(x_hat, y_hat, t, b, go, gscale, dx_t, dy_t, sums, want_dx, want_dy,
                                     status=ops.status_word(x_hat.device))
        if post_x and dx is not None:
            dx = ops.normalize_bwd(dx, x_hat, inv_x, x_dtype, d)
        if post_y and dy is not None:
            dy = ops.normalize_bwd(dy, y_hat, inv_y, y_dtype, d)
        dt = db = None
        if want_tb:
            # G = g (sigmoid(a) - I) with g = grad_out * t / B, so grad_out * dL/dt = sum(G S) / t, dL/db = sum(G) / t
            if need[2] and t_tensor is not None:
                dt = (sums[0] / t).reshape(t_tensor[0]).to(t_tensor[1])
            if need[3] and b_tensor is not None:
                db = (sums[1] / t).reshape(b_tensor[0]).to(b_tensor[1])
        ops.post_status(x_hat.device)
        return (dx if need[0] else None), (dy if need[1] else None), dt, db, None


class MemoryEfficientSigLIPLoss(nn.Module):
    def __init__(self, init_logit_scale=10.0, init_logit_bias=-10.0, normalized_inputs=False, learnable=True):
        super().__init__()
        self.normalized_inputs = normalized_inputs
        ls = torch.tensor(math.log(init_logit_scale), dtype=torch.float32)
        lb = torch.tensor(float(init_logit_bias), dtype=torch.float32)
        if learnable:
            self.log_logit_scale = nn.Parameter(ls)
            self.logit_bias = nn.Parameter(lb)
        else:
            self.register_buffer("log_logit_scale", ls)
            self.register_buffer("logit_bias", lb)

    def forward(self, image_features, text_features):
        t = self.log_logit_scale.exp()
        return MemoryEfficientSigLIPLossFn.apply(image_features, text_features, t, self.logit_bias,
                                                 not self.normalized_inputs)
