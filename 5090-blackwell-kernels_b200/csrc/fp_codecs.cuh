// Device codecs of the fp8 / fp4 paths: e4m3 (fn) and e2m1 elements, ue8m0 and e4m3 block scales,
// and the blocked scale layout of the fp4 operands.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace spk::fp {

// e4m3 byte -> float (exact).
__device__ __forceinline__ float e4m3_to_float(unsigned char b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(__half(h));
}

// float -> e4m3 byte, round to nearest even, saturating at +-448 (no infinity in the format).
__device__ __forceinline__ unsigned char float_to_e4m3(float v) {
    return static_cast<unsigned char>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// ue8m0 scale byte -> 2^(b - 127); 0xff is NaN in the format.
__device__ __forceinline__ float ue8m0_to_float(unsigned char b) {
    return b == 0xff ? __int_as_float(0x7fc00000) : (b == 0 ? __int_as_float(0x00400000) /* 2^-127 */ : __int_as_float(static_cast<int>(b) << 23));
}

// e2m1 code -> float: magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign.
__device__ __forceinline__ float e2m1_to_float(unsigned code) {
    const unsigned m = code & 7u;
    // 0, .5, 1, 1.5, 2, 3, 4, 6 == (m < 2 ? m * .5 : (2 + (m & 1)) * 2^((m >> 1) - 2) ... ) written as a table in a register
    const float mag = m == 0 ? 0.f : m == 1 ? 0.5f : m == 2 ? 1.f : m == 3 ? 1.5f : m == 4 ? 2.f : m == 5 ? 3.f : m == 6 ? 4.f : 6.f;
    return (code & 8u) ? -mag : mag;
}

// float -> e2m1 code, round to nearest even, saturating at 6: the code counts the rounding
// boundaries below |v|, ties to the even code, hence the alternating > and >= (reference
// src/kernels/fp4quant.cu:28-39, python/spark_kernels/reference.py:131-141). Sign set for v < 0.
__device__ __forceinline__ unsigned float_to_e2m1(float v) {
    const float a = fabsf(v);
    const unsigned c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
    return c | (v < 0.f ? 8u : 0u);
}

// Byte offset of the scale of (row r, k-block j) in the blocked layout with `cols` scale columns
// per row (cols a multiple of 4): 128-row x 4-column tiles of 512 bytes, the tiles of a 128-row
// block consecutive along K, and inside a tile (r % 32) * 16 + (r / 32) * 4 + j % 4
// (reference src/kernels/fp4quant.cu:41-45, include/spark/kernels.h:304-309).
__host__ __device__ __forceinline__ size_t sf_offset(int r, int j, int cols) {
    const size_t tile = static_cast<size_t>(r / 128) * (cols / 4) + j / 4;
    return tile * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4 + (j % 4);
}

}  // namespace spk::fp
