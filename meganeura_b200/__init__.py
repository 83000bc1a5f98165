"""B200 (sm_100a) implementation of meganeura's Q4/Q8 dequantize-fused matmul path.

Importing this package loads the in-tree CUDA library (csrc/libmgq.so) and fails if it has
not been built; there is no CPU implementation behind it.
"""
from ._lib import FMT_Q4, FMT_Q8, A_F32, A_BF16, LIB_PATH, MgqError, lib  # noqa: F401
from .graph import (Graph, Session, build_inference_session, ShaderEntry, WeightFormat,  # noqa: F401
                    Dispatch, ExecutionPlan)
from . import ops  # noqa: F401
