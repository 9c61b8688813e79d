"""spark_kernels for B200 (sm_100a): the quantized-weight GEMM path of the reference library --
w4gemm (int4 W4A16), fp8gemm (e4m3) and fp4gemm (NVFP4 / MXFP4) with their quantizers and
packers -- behind the reference's op names. Hand-written CUDA in libspark_b200.so, reached
through its C ABI; torch is used for device memory and streams only."""

from . import _C, ops
from .ops import W4_GROUP, W4Weight, num_variants, w4_quantize, w4_repack, w4gemm

__all__ = ["_C", "ops", "W4_GROUP", "W4Weight", "num_variants", "w4_quantize", "w4_repack", "w4gemm"]
