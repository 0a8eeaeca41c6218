"""B200-native memory-efficient CLIP / LiT contrastive loss.

The public classes mirror b0nce/MemoryEfficientCLIP; the arithmetic lives in
libmeclip_sm100.so (hand-written sm_100a CUDA behind a C ABI, include/meclip.h).
Importing the package does not load the library; the first operation does, and it
raises if the library has not been built (there is no other implementation).
"""
from .clip_loss import (MemoryEfficientCLIPLoss, MemoryEfficientCLIPLossNormed, StableMemoryEfficientCLIPLoss,
                        StableMemoryEfficientCLIPLossNormed)
from .lit_loss import (MemoryEfficientLiTLoss, MemoryEfficientLiTLossNormed, StableMemoryEfficientLiTLoss,
                       StableMemoryEfficientLiTLossNormed)
from .siglip_loss import MemoryEfficientSigLIPLoss, MemoryEfficientSigLIPLossFn

__all__ = [
    "MemoryEfficientSigLIPLoss", "MemoryEfficientSigLIPLossFn",
    "MemoryEfficientCLIPLoss", "MemoryEfficientCLIPLossNormed", "StableMemoryEfficientCLIPLoss",
    "StableMemoryEfficientCLIPLossNormed", "MemoryEfficientLiTLoss", "MemoryEfficientLiTLossNormed",
    "StableMemoryEfficientLiTLoss", "StableMemoryEfficientLiTLossNormed",
]
