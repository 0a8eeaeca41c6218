"""CLIP (bidirectional) contrastive loss with O(B*D) memory on B200.

Same public surface as the reference's clip_loss.py: the autograd Functions
``MemoryEfficientCLIPLossNormed`` / ``StableMemoryEfficientCLIPLossNormed``
(``apply(x_normalized, y_normalized, temperature)``, reference clip_loss.py:159-256,
276-373) and the modules ``MemoryEfficientCLIPLoss`` / ``StableMemoryEfficientCLIPLoss``
(``(temperature=0.07, normalized_inputs=False)``, ``forward(image_features,
text_features)``, reference clip_loss.py:259-273, 376-401).  All arithmetic runs in
the sm_100a kernels of libmeclip_sm100.so.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib, ops
from ._function import ContrastiveLossFn


class MemoryEfficientCLIPLossNormed(torch.autograd.Function):
    """loss = CLIP(x_normalized, y_normalized); gradients for both inputs."""

    @staticmethod
    def forward(ctx, x_normalized, y_normalized, temperature=0.07):
        return ContrastiveLossFn.run_forward(ctx, x_normalized, y_normalized, temperature, _lib.CLIP, False, False)

    @staticmethod
    def backward(ctx, grad_output):
        dx, dy = ContrastiveLossFn.run_backward(ctx, grad_output)
        return dx, dy, ctx.meclip_dt


class StableMemoryEfficientCLIPLossNormed(torch.autograd.Function):
    """Same loss; gradients scaled by 1/sqrt(B*T) instead of 1/(B*T) (reference clip_loss.py:299)."""

    @staticmethod
    def forward(ctx, x_normalized, y_normalized, temperature=0.07):
        return ContrastiveLossFn.run_forward(ctx, x_normalized, y_normalized, temperature, _lib.CLIP, True, False)

    @staticmethod
    def backward(ctx, grad_output):
        dx, dy = ContrastiveLossFn.run_backward(ctx, grad_output)
        return dx, dy, ctx.meclip_dt


class _CLIPLossModule(nn.Module):
    _stable = False

    def __init__(self, temperature=0.07, normalized_inputs=False):
        super().__init__()
        self.temperature = temperature
        self.normalized_inputs = normalized_inputs

    def forward(self, image_features, text_features):
        if self.normalized_inputs:
            fn = StableMemoryEfficientCLIPLossNormed if self._stable else MemoryEfficientCLIPLossNormed
            return fn.apply(image_features, text_features, self.temperature)
        # L2-normalise and its Jacobian run inside the same autograd node (fused prologue / epilogue)
        return ContrastiveLossFn.apply(image_features, text_features, self.temperature, _lib.CLIP, self._stable, True)


class MemoryEfficientCLIPLoss(_CLIPLossModule):
    """Drop-in for the reference module of the same name (clip_loss.py:259-273)."""
    _stable = False


class StableMemoryEfficientCLIPLoss(_CLIPLossModule):
    """Drop-in for the reference module of the same name (clip_loss.py:376-401)."""
    _stable = True
