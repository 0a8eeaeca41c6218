"""`from lit_loss import MemoryEfficientLiTLoss` keeps working (reference README.md:50)."""
from memoryefficientclip_b200.lit_loss import (MemoryEfficientLiTLoss, MemoryEfficientLiTLossNormed,  # noqa: F401
                                              StableMemoryEfficientLiTLoss, StableMemoryEfficientLiTLossNormed)
