"""spark_kernels for B200 (sm_100a): the quantized-weight GEMM path of the reference library --
w4gemm (int4 W4A16), fp8gemm (e4m3) and fp4gemm (NVFP4 / MXFP4) with their quantizers and
packers -- behind the reference's op names. Hand-written CUDA in libspark_b200.so, reached
through its C ABI; torch is used for device memory and streams only."""

from . import _C, formats, ops, quant
from .ops import (W4_GROUP, W4GateUpWeight, W4Weight, w4gemm_swiglu, fp4_quantize, fp4gemm, fp8_quantize, fp8_quantize_block128, fp8gemm,
                  fp8gemm_block128, grouped_gemm_fp8, grouped_gemm_swiglu_fp8, num_variants, w4_quantize, w4_repack, w4gemm)
from .quant import FORMATS, FP4Linear, FP8Linear, Int4Linear, MXFP8Linear, make_linear

__all__ = ["_C", "ops", "quant", "formats", "W4_GROUP", "W4Weight", "num_variants", "w4_quantize", "w4_repack",
           "w4gemm", "W4GateUpWeight", "w4gemm_swiglu", "fp8gemm", "fp8_quantize", "fp4gemm", "fp4_quantize", "fp8_quantize_block128",
           "fp8gemm_block128", "grouped_gemm_fp8", "grouped_gemm_swiglu_fp8", "FORMATS", "Int4Linear", "FP8Linear", "MXFP8Linear", "FP4Linear", "make_linear"]
