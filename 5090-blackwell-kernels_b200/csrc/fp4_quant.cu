// bf16 -> fp4 (e2m1) quantizers with block scales written straight into the blocked layout the
// tensor core reads (contract: reference include/spark/kernels.h:296-347; arithmetic:
// python/spark_kernels/reference.py:131-225). NVFP4: one e4m3 scale per 16 values over a per-tensor
// decode scale; MXFP4: one ue8m0 scale per 32 values, exponent floor(log2 max|x|) - 2. Bit-exact
// contract: the tests compare every byte with the CPU oracle.
//
// Shape of the work, chosen for the blocked scale layout. That layout stores the scales of rows
// r, r + 32, r + 64, r + 96 of a 128-row block and four consecutive k-blocks as 16 contiguous bytes.
// A warp therefore takes those four rows and 128 consecutive k of each: eight lanes per row, sixteen
// values (two 16-byte loads, 32 contiguous bytes) per lane, 256 contiguous bytes per row. The codes
// leave as one 8-byte store per lane; the scale bytes are gathered with a few shuffles and leave as
// 16-byte stores (two per warp for NVFP4, one for MXFP4), so the scale tiles are written in whole
// 16-byte pieces and every byte of the padded layout exactly once (rows past `rows` get zero bytes).
// The element conversion is the hardware's paired e2m1 cvt (round to nearest even, saturating at 6).
#include <cuda_fp4.h>

#include <algorithm>

#include "fp_codecs.cuh"
#include "spk_common.cuh"

// 1: cvt.rn.satfinite.e2m1x2.f32; 0: the seven comparisons of fp::float_to_e2m1 (same bytes, more instructions)
#ifndef SPK_FP4_HW_CVT
#define SPK_FP4_HW_CVT 1
#endif

namespace spk {
namespace {

constexpr int kThreads = 256;
constexpr int kValuesPerLane = 16, kLanesPerRow = 8, kWarpCols = kValuesPerLane * kLanesPerRow;  // 128 k per warp and row

// Two values -> one byte, element 0 in the low nibble. The reference sets the sign bit for v < 0 only,
// so a negative zero encodes as +0: adding +0.0 turns -0.0 into +0.0 and changes nothing else.
__device__ __forceinline__ uint32_t e2m1_pair(float a, float b) {
#if SPK_FP4_HW_CVT
    return __nv_cvt_float2_to_fp4x2(make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f)), __NV_E2M1, cudaRoundNearest) & 0xFFu;
#else
    return fp::float_to_e2m1(a) | (fp::float_to_e2m1(b) << 4);
#endif
}

struct Lane16 {
    float f[kValuesPerLane];
};

__device__ __forceinline__ void widen(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
}

// FORMAT 0 NVFP4, 1 MXFP4. Warp job = (128-row block R, row rb of each quarter, 128-k column group cg).
template <int FORMAT>
__global__ void __launch_bounds__(kThreads)
fp4_quantize_rows4_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ q, unsigned char* __restrict__ sf,
                          int rows, int K, int col_groups, long long jobs, const float* __restrict__ scale,
                          const unsigned* __restrict__ amax_bits, float* __restrict__ scale_out) {
    constexpr int V = FORMAT == 0 ? 16 : 32;            // values per scale
    constexpr int kScalesPerWarpRow = kWarpCols / V;    // 8 or 4 scale bytes per row and warp
    const int lane = threadIdx.x & 31, rsub = lane >> 3, jl = lane & 7;
    const long long job = (static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    float s = 1.0f;
    if (FORMAT == 0) {
        // with a |max| cell the decode scale is max|x| / (6 * 448), at least the smallest normal float
        s = amax_bits != nullptr ? fmaxf(__fdiv_rn(__uint_as_float(*amax_bits), 6.0f * 448.0f), 1.17549435e-38f)
            : scale != nullptr   ? *scale
                                 : 1.0f;
        if (amax_bits != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = s;
    }
    if (job >= jobs) return;
    const int cg = static_cast<int>(job % col_groups);
    const int rb = static_cast<int>((job / col_groups) & 31);
    const int R = static_cast<int>(job / (static_cast<long long>(col_groups) * 32));
    const int r = R * 128 + rb + 32 * rsub;
    const int k0 = cg * kWarpCols + jl * kValuesPerLane;
    const bool live = r < rows && k0 < K;

    Lane16 v;
    float amax = 0.f;
    if (live) {
        const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * K + k0);
        const uint4 a = src[0], b = src[1];
        widen(a, v.f);
        widen(b, v.f + 8);
#pragma unroll
        for (int i = 0; i < kValuesPerLane; ++i) amax = fmaxf(amax, fabsf(v.f[i]));
    }
    if (FORMAT == 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // two lanes share a 32-value block

    uint32_t sbyte = 0;
    uint32_t codes[2] = {0u, 0u};
    if (live) {
        if (FORMAT == 0) {
            sbyte = fp::float_to_e4m3(fminf(__fdiv_rn(__fdiv_rn(amax, 6.0f), s), 448.0f));
            const float denom = fp::e4m3_to_float(static_cast<unsigned char>(sbyte)) * s;
            if (denom > 0.f) {
#pragma unroll
                for (int i = 0; i < kValuesPerLane; i += 2)
                    codes[i >> 3] |= e2m1_pair(__fdiv_rn(v.f[i], denom), __fdiv_rn(v.f[i + 1], denom)) << (4 * (i & 7));
            }
        } else {
            int e = amax > 0.f ? ilogbf(amax) - 2 : -127;
            e = max(-127, min(127, e));
            sbyte = static_cast<uint32_t>(e + 127);
#pragma unroll
            for (int i = 0; i < kValuesPerLane; i += 2)
                codes[i >> 3] |= e2m1_pair(scalbnf(v.f[i], -e), scalbnf(v.f[i + 1], -e)) << (4 * (i & 7));
        }
        *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * (K / 2) + (k0 >> 1)) = make_uint2(codes[0], codes[1]);
    }

    // Scale bytes. Lane -> scale column inside the warp's row: NVFP4 jl (one per lane), MXFP4 jl / 2 (even lanes).
    // First every group of four scale columns becomes one 32-bit word (byte j % 4), then the four row
    // quarters' words become the 16 contiguous bytes of the blocked layout.
    const int jw = FORMAT == 0 ? jl : (jl >> 1);
    uint32_t word = (FORMAT == 0 || (jl & 1) == 0) ? sbyte << (8 * (jw & 3)) : 0u;
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if (FORMAT == 1) word |= __shfl_xor_sync(0xffffffffu, word, 4);
    const int h = FORMAT == 0 ? (jl >> 2) : 0;  // which group of four scale columns this lane sits in
    uint4 piece;
    piece.x = __shfl_sync(0xffffffffu, word, 4 * h);
    piece.y = __shfl_sync(0xffffffffu, word, 8 + 4 * h);
    piece.z = __shfl_sync(0xffffffffu, word, 16 + 4 * h);
    piece.w = __shfl_sync(0xffffffffu, word, 24 + 4 * h);
    const int groups_per_row = K / V / 4;                       // 4-column scale groups (512-byte tiles) per row block
    const int group = cg * (kScalesPerWarpRow / 4) + h;
    if (rsub == 0 && (jl & 3) == 0 && (FORMAT == 0 || jl == 0) && group < groups_per_row)
        *reinterpret_cast<uint4*>(sf + (static_cast<size_t>(R) * groups_per_row + group) * 512 + rb * 16) = piece;
}

}  // namespace
}  // namespace spk

extern "C" size_t spk_fp4_scale_bytes(int rows, int K, int format) {
    const int V = format == SPK_FP4_MXFP4 ? 32 : 16;
    return static_cast<size_t>(spk::cdiv(rows, 128)) * 128 * (K / V);
}

extern "C" int spk_fp4_quantize(const void* x_, unsigned char* q, unsigned char* sf, int rows, int K, const float* scale,
                                int format, void* stream_, unsigned* work, float* scale_out) {
    using namespace spk;
    SPK_REQUIRE(format == SPK_FP4_NVFP4 || format == SPK_FP4_MXFP4, "fp4_quantize: format %d is neither NVFP4 nor MXFP4", format);
    SPK_REQUIRE(x_ != nullptr && q != nullptr && sf != nullptr, "fp4_quantize: x, q and sf are required");
    SPK_REQUIRE(rows > 0 && K > 0, "fp4_quantize: rows=%d and K=%d must be positive", rows, K);
    const int granule = format == SPK_FP4_MXFP4 ? 128 : 64;  // four scale columns
    SPK_REQUIRE(K % granule == 0, "fp4_quantize: K=%d must be a multiple of %d for this format", K, granule);
    SPK_REQUIRE(aligned16(x_) && aligned16(q) && aligned16(sf), "fp4_quantize: x, q and sf must be 16-byte aligned");
    SPK_REQUIRE(work == nullptr || (format == SPK_FP4_NVFP4 && scale_out != nullptr),
                "fp4_quantize: a decode scale computed on the device needs NVFP4 and a scale_out");
    const auto* x = static_cast<const __nv_bfloat16*>(x_);
    auto stream = static_cast<cudaStream_t>(stream_);
    if (work != nullptr)
        if (int rc = spk_absmax_bits(x, static_cast<long long>(rows) * K, work, stream_)) return rc;
    const int col_groups = cdiv(K, kWarpCols);
    const long long jobs = static_cast<long long>(cdiv(rows, 128)) * 32 * col_groups;  // warps
    const unsigned grid = static_cast<unsigned>(cdiv64(jobs * 32, kThreads));
    if (format == SPK_FP4_NVFP4)
        fp4_quantize_rows4_kernel<0><<<grid, kThreads, 0, stream>>>(x, q, sf, rows, K, col_groups, jobs, scale, work, scale_out);
    else
        fp4_quantize_rows4_kernel<1><<<grid, kThreads, 0, stream>>>(x, q, sf, rows, K, col_groups, jobs, nullptr, nullptr, nullptr);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
