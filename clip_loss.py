"""`from clip_loss import MemoryEfficientCLIPLoss` keeps working (reference README.md:29)."""
from memoryefficientclip_b200.clip_loss import (MemoryEfficientCLIPLoss, MemoryEfficientCLIPLossNormed,  # noqa: F401
                                               StableMemoryEfficientCLIPLoss, StableMemoryEfficientCLIPLossNormed)
