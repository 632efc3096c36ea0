"""B200-native implementation of the CD-SSM scan path (hand-written sm_100a CUDA behind a C ABI).

``ops`` mirrors the reference's cdssm/ops.py and adds the fused scan and the decode step.
"""
from . import _lib, ops  # noqa: F401
from .ops import (CUDAConv1dSiLUOp, DynamicsFusedFn, NormalizeKQFn, IntraChunkScanFn,  # noqa: F401
                  InterChunkScanFn, ExactCorrectionFn, scan_fused, decode_step, CdssmError)

__version__ = "0.1.0"
