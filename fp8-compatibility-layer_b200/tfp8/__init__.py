"""tfp8 for B200: FP8-stored weights (uint8 E4M3FN / E5M2 codes + scales) served by hand-written
sm_100a kernels -- a bandwidth-bound decode GEMV, a tcgen05 tile GEMM that decodes FP8 tiles in
shared memory, and a fused quantizer -- behind the API of the original Turing `tfp8` package.
"""
__version__ = "0.1.0"

from .config import FP8Config
from .formats import E4M3FN, E5M2, decode, encode, lut
from .linear import FP8Linear
from .planner import plan, prepare_model, report, weight_bytes
from .quantize import dequantize_weight, quantize_weight

__all__ = ["FP8Config", "FP8Linear", "prepare_model", "plan", "report", "weight_bytes",
           "quantize_weight", "dequantize_weight", "decode", "encode", "lut", "E4M3FN", "E5M2"]
