"""LiT (text -> frozen image tower) contrastive loss with O(B*D) memory on B200.

Same public surface as the reference's lit_loss.py: ``MemoryEfficientLiTLossNormed`` /
``StableMemoryEfficientLiTLossNormed`` (``apply(text_normalized, image_normalized,
temperature)``, reference lit_loss.py:151-247, 266-362) and the modules
``MemoryEfficientLiTLoss`` / ``StableMemoryEfficientLiTLoss`` whose ``forward`` takes
``(text_features, image_features)`` - text FIRST (lit_loss.py:256).  Only the text
features receive a gradient (lit_loss.py:247).  The reference's Stable module calls
``nn.Module.apply`` by mistake (lit_loss.py:387) and raises; here it does what its
docstring says.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from ._function import ContrastiveLossFn


class MemoryEfficientLiTLossNormed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_normalized, y_normalized, temperature=0.07):
        return ContrastiveLossFn.run_forward(ctx, x_normalized, y_normalized, temperature, _lib.LIT, False, False)

    @staticmethod
    def backward(ctx, grad_output):
        dx, _ = ContrastiveLossFn.run_backward(ctx, grad_output)
        return dx, None, ctx.meclip_dt


class StableMemoryEfficientLiTLossNormed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_normalized, y_normalized, temperature=0.07):
        return ContrastiveLossFn.run_forward(ctx, x_normalized, y_normalized, temperature, _lib.LIT, True, False)

    @staticmethod
    def backward(ctx, grad_output):
        dx, _ = ContrastiveLossFn.run_backward(ctx, grad_output)
        return dx, None, ctx.meclip_dt


class _LiTLossModule(nn.Module):
    _stable = False

    def __init__(self, temperature=0.07, normalized_inputs=False):
        super().__init__()
        self.temperature = temperature
        self.normalized_inputs = normalized_inputs

    def forward(self, text_features, image_features):
        if self.normalized_inputs:
            fn = StableMemoryEfficientLiTLossNormed if self._stable else MemoryEfficientLiTLossNormed
            return fn.apply(text_features, image_features, self.temperature)
        return ContrastiveLossFn.apply(text_features, image_features, self.temperature, _lib.LIT, self._stable, True)


class MemoryEfficientLiTLoss(_LiTLossModule):
    """Drop-in for the reference module of the same name (lit_loss.py:250-263)."""
    _stable = False


class StableMemoryEfficientLiTLoss(_LiTLossModule):
    """The sqrt-scaled LiT loss the reference documents at lit_loss.py:365-389."""
    _stable = True
