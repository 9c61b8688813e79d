// bf16 -> e4m3 activation quantizers of the fp8 GEMM (contract: reference include/spark/kernels.h:349-364;
// arithmetic: python/spark_kernels/reference.py:46-106). Scales: per tensor and per row the smallest
// power of two s with max|x| / s <= 448; MX one ue8m0 byte per 32 values with exponent
// floor(log2 max|x|) - 8; and, as an addition that the reference does not have, fp32 scales per
// 1 x 128 or 128 x 128 block. Every output byte is a bit-exact contract checked against the CPU oracle.
//
// How the work is laid out (all of it is one pass over HBM, 16-byte accesses, full sectors):
//   |max|    bf16x2 abs / max on packed registers (no widening), one redux.sync per warp on the float
//            bits (non-negative floats order like their bit patterns), one atomicMax per warp
//   tensor   after the |max| launch: 16 values per thread, two 16-byte loads -> one 16-byte store,
//            paired hardware conversions (two e4m3 bytes per cvt)
//   row      the row stays in REGISTERS between the |max| pass and the conversion (up to 64 values per
//            thread), so it is read once; a warp per row for short rows, a CTA per row for long ones
//   mx       four lanes per 32-value block: the block |max| is two shuffles, every lane converts its 8
//            values, loads and stores of a warp are contiguous 512- and 256-byte runs
#include <algorithm>

#include "fp_codecs.cuh"
#include "spk_common.cuh"

namespace spk {
namespace {

constexpr int kThreads = 256;
constexpr float kE4m3Max = 448.0f;
constexpr float kFltMin = 1.17549435e-38f;

// ---- packed helpers --------------------------------------------------------------------------------

// max(|a|, |b|, m) per bf16 lane of the 32-bit words
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t v) {
    __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v));
    a = __hmax2(a, *reinterpret_cast<const __nv_bfloat162*>(&m));
    return *reinterpret_cast<const uint32_t*>(&a);
}
__device__ __forceinline__ uint32_t absmax_chunk(uint32_t m, const uint4& v) {
    return absmax2(absmax2(absmax2(absmax2(m, v.x), v.y), v.z), v.w);
}
// the larger half of a packed non-negative bf16 pair, as fp32 bits
__device__ __forceinline__ uint32_t pair_max_f32_bits(uint32_t m) {
    const uint32_t lo = m << 16, hi = m & 0xFFFF0000u;
    return lo > hi ? lo : hi;
}
__device__ __forceinline__ float warp_max_nonneg(float a) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(a)));
}
// Eight bf16 -> eight e4m3 bytes of x * inv (round to nearest even, saturating at 448).
__device__ __forceinline__ uint2 convert_chunk(const uint4& v, float inv) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t out[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t pair = w[2 * h + j];
            const float2 f = make_float2(__uint_as_float(pair << 16) * inv, __uint_as_float(pair & 0xFFFF0000u) * inv);
            packed |= static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3)) << (16 * j);
        }
        out[h] = packed;
    }
    return make_uint2(out[0], out[1]);
}

// Smallest power of two >= max(amax, FLT_MIN) / 448, exponent held to [-126, 127] so that 1 / s is a
// normal float even for an all-zero input.
__device__ __forceinline__ float pow2_at_least(float amax) {
    const float r = __fdiv_rn(fmaxf(amax, kFltMin), kE4m3Max);
    int e = ilogbf(r);
    if (scalbnf(1.0f, e) < r) ++e;
    e = max(-126, min(127, e));
    return scalbnf(1.0f, e);
}

// ---- |max| over a tensor ------------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads)
absmax_bits_kernel(const uint4* __restrict__ x, long long chunks, unsigned* __restrict__ cell) {
    uint32_t m0 = 0, m1 = 0;
    const long long stride = static_cast<long long>(gridDim.x) * kThreads * 2;
    for (long long c = (static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x) * 2; c < chunks; c += stride) {
        m0 = absmax_chunk(m0, x[c]);
        if (c + 1 < chunks) m1 = absmax_chunk(m1, x[c + 1]);
    }
    const uint32_t bits = __reduce_max_sync(0xffffffffu, pair_max_f32_bits(absmax2(m0, m1)));
    if ((threadIdx.x & 31) == 0 && bits != 0) atomicMax(cell, bits);
}

// ---- per-tensor conversion -----------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads)
quantize_by_cell_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, long long chunks, const unsigned* __restrict__ cell,
                        float* __restrict__ scale) {
    const float s = pow2_at_least(__uint_as_float(*cell));
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale = s;
    const float inv = __fdiv_rn(1.0f, s);
    const long long c = (static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x) * 2;
    if (c + 1 < chunks) {
        const uint4 a = x[c], b = x[c + 1];
        const uint2 qa = convert_chunk(a, inv), qb = convert_chunk(b, inv);
        if ((reinterpret_cast<uintptr_t>(q) & 15u) == 0) {
            *reinterpret_cast<uint4*>(q + c) = make_uint4(qa.x, qa.y, qb.x, qb.y);
        } else {  // q only 8-byte aligned
            q[c] = qa;
            q[c + 1] = qb;
        }
    } else if (c < chunks) {
        q[c] = convert_chunk(x[c], inv);
    }
}

// ---- per-row: TPR threads per row, the row kept in registers ----------------------------------------------

constexpr int kRowRegs = 8;  // 16-byte chunks a thread keeps (64 values)

template <int TPR>
__global__ void __launch_bounds__(kThreads)
quantize_rows_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, int rows, int chunks_per_row, float* __restrict__ scales) {
    __shared__ float warp_max[kThreads / 32];
    constexpr int kRowsPerCta = kThreads / TPR;
    const int row = blockIdx.x * kRowsPerCta + threadIdx.x / TPR, t = threadIdx.x % TPR;
    const bool live = row < rows;
    const uint4* xr = x + static_cast<size_t>(live ? row : 0) * chunks_per_row;
    uint4 keep[kRowRegs];
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < kRowRegs; ++i) {
        const int c = t + i * TPR;
        if (live && c < chunks_per_row) {
            keep[i] = xr[c];
            m = absmax_chunk(m, keep[i]);
        }
    }
    for (int c = t + kRowRegs * TPR; live && c < chunks_per_row; c += TPR) m = absmax_chunk(m, xr[c]);  // rows beyond the registers
    float a = warp_max_nonneg(__uint_as_float(pair_max_f32_bits(m)));
    if (TPR > 32) {
        if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = a;
        __syncthreads();
        a = warp_max[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) a = fmaxf(a, warp_max[w]);
    }
    if (!live) return;
    const float s = pow2_at_least(a);
    if (t == 0) scales[row] = s;
    const float inv = __fdiv_rn(1.0f, s);
    uint2* qr = q + static_cast<size_t>(row) * chunks_per_row;
#pragma unroll
    for (int i = 0; i < kRowRegs; ++i) {
        const int c = t + i * TPR;
        if (c < chunks_per_row) qr[c] = convert_chunk(keep[i], inv);
    }
    for (int c = t + kRowRegs * TPR; c < chunks_per_row; c += TPR) qr[c] = convert_chunk(xr[c], inv);
}

// ---- MX: one ue8m0 scale per 32 values --------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads)
quantize_mx_quads_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, unsigned char* __restrict__ sf, long long chunks) {
    const long long c = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;  // chunk = 8 values; 4 chunks = 1 block
    const bool live = c < chunks;  // chunks is a multiple of 4, so a quad is all in or all out
    const uint4 v = live ? x[c] : make_uint4(0, 0, 0, 0);
    uint32_t bits = pair_max_f32_bits(absmax_chunk(0, v));
    bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 1));
    bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 2));
    if (!live) return;
    // e = floor(log2 |max|) - 8, the smallest exponent for an all-zero block, held to the ue8m0 range
    const float amax = __uint_as_float(bits);
    int e = amax > 0.f ? ilogbf(amax) - 8 : -127;
    e = max(-127, min(127, e));
    q[c] = convert_chunk(v, scalbnf(1.0f, -e));
    if ((threadIdx.x & 3) == 0) sf[c >> 2] = static_cast<unsigned char>(e + 127);
}

// ---- fp32 block scales (not in the reference) ---------------------------------------------------------------
// One warp per (block of `block_rows` rows, 128 k): s = |max| / 448 (1 for an all-zero block),
// q = e4m3(x / s). x is fp32 here: this quantizer also serves weights.
__global__ void __launch_bounds__(kThreads)
quantize_block128_kernel(const float* __restrict__ x, unsigned char* __restrict__ q, float* __restrict__ scales,
                         int rows, int K, int block_rows) {
    const int KB = K / 128;
    const long long warp = (static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int RB = (rows + block_rows - 1) / block_rows;
    if (warp >= static_cast<long long>(RB) * KB) return;
    const int rb = static_cast<int>(warp / KB), kb = static_cast<int>(warp % KB);
    const int r0 = rb * block_rows, r1 = min(rows, r0 + block_rows);
    float a = 0.f;
    for (int r = r0; r < r1; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * K + 128 * kb + 4 * lane);
        a = fmaxf(a, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    a = warp_max_nonneg(a);
    const float s = a > 0.f ? __fdiv_rn(a, kE4m3Max) : 1.0f;
    if (lane == 0) scales[static_cast<size_t>(rb) * KB + kb] = s;
    for (int r = r0; r < r1; ++r) {
        const size_t off = static_cast<size_t>(r) * K + 128 * kb + 4 * lane;
        const float4 v = *reinterpret_cast<const float4*>(x + off);
        const unsigned w = fp::float_to_e4m3(__fdiv_rn(v.x, s)) | (fp::float_to_e4m3(__fdiv_rn(v.y, s)) << 8) |
                           (fp::float_to_e4m3(__fdiv_rn(v.z, s)) << 16) | (fp::float_to_e4m3(__fdiv_rn(v.w, s)) << 24);
        *reinterpret_cast<unsigned*>(q + off) = w;
    }
}

int sm_multiple(const DeviceState* dev, long long wanted, int per_sm) {
    return static_cast<int>(std::max<long long>(1, std::min<long long>(wanted, static_cast<long long>(per_sm) * dev->sm_count)));
}

}  // namespace
}  // namespace spk

extern "C" int spk_absmax_bits(const void* x, long long n, unsigned* work, void* stream) {
    using namespace spk;
    SPK_REQUIRE(x != nullptr && work != nullptr, "absmax_bits: x and work are required");
    SPK_REQUIRE(n > 0 && n % 8 == 0, "absmax_bits: n must be a positive multiple of 8, got %lld", n);
    SPK_REQUIRE(aligned16(x), "absmax_bits: x must be 16-byte aligned");
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    const long long chunks = n / 8;
    const int grid = sm_multiple(dev, cdiv64(chunks, 2 * kThreads), 8);
    absmax_bits_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(x), chunks, work);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_fp8_quantize(const void* x, unsigned char* q, void* scale, unsigned* work, int rows, int K,
                                int mode, void* stream_) {
    using namespace spk;
    SPK_REQUIRE(mode == SPK_FP8Q_TENSOR || mode == SPK_FP8Q_ROW || mode == SPK_FP8Q_MX, "fp8_quantize: mode %d is not tensor, row or mx", mode);
    SPK_REQUIRE(x != nullptr && q != nullptr && scale != nullptr, "fp8_quantize: x, q and scale are required");
    SPK_REQUIRE(rows > 0 && K > 0, "fp8_quantize: rows=%d and K=%d must be positive", rows, K);
    const int granule = mode == SPK_FP8Q_MX ? 32 : 8;
    SPK_REQUIRE(K % granule == 0, "fp8_quantize: K=%d must be a multiple of %d in this mode", K, granule);
    SPK_REQUIRE(aligned16(x) && reinterpret_cast<uintptr_t>(q) % 8 == 0, "fp8_quantize: x must be 16-byte and q 8-byte aligned");
    auto stream = static_cast<cudaStream_t>(stream_);
    const auto* xv = static_cast<const uint4*>(x);
    auto* qv = reinterpret_cast<uint2*>(q);
    const long long chunks = static_cast<long long>(rows) * K / 8;
    if (mode == SPK_FP8Q_TENSOR) {
        SPK_REQUIRE(work != nullptr, "fp8_quantize: the tensor mode needs a zeroed work cell");
        if (int rc = spk_absmax_bits(x, chunks * 8, work, stream_)) return rc;
        quantize_by_cell_kernel<<<static_cast<unsigned>(cdiv64(chunks, 2 * kThreads)), kThreads, 0, stream>>>(
            xv, qv, chunks, work, static_cast<float*>(scale));
    } else if (mode == SPK_FP8Q_ROW) {
        const int cpr = K / 8;
        if (cpr <= 32 * kRowRegs)  // a warp holds the row in registers
            quantize_rows_kernel<32><<<cdiv(rows, kThreads / 32), kThreads, 0, stream>>>(xv, qv, rows, cpr, static_cast<float*>(scale));
        else
            quantize_rows_kernel<kThreads><<<rows, kThreads, 0, stream>>>(xv, qv, rows, cpr, static_cast<float*>(scale));
    } else {
        quantize_mx_quads_kernel<<<static_cast<unsigned>(cdiv64(chunks, kThreads)), kThreads, 0, stream>>>(
            xv, qv, static_cast<unsigned char*>(scale), chunks);
    }
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_fp8_quantize_block128(const float* x, unsigned char* q, float* scales, int rows, int K,
                                         int block_rows, void* stream) {
    using namespace spk;
    SPK_REQUIRE(x && q && scales, "fp8_quantize_block128: null pointer");
    SPK_REQUIRE(rows > 0 && K > 0 && K % 128 == 0, "fp8_quantize_block128: K must be a positive multiple of 128, got %d", K);
    SPK_REQUIRE(block_rows == 1 || block_rows == 128, "fp8_quantize_block128: block_rows must be 1 or 128, got %d", block_rows);
    SPK_REQUIRE(aligned16(x) && reinterpret_cast<uintptr_t>(q) % 4 == 0, "fp8_quantize_block128: x must be 16-byte, q 4-byte aligned");
    const long long warps = static_cast<long long>((rows + block_rows - 1) / block_rows) * (K / 128);
    quantize_block128_kernel<<<static_cast<unsigned>(cdiv64(warps * 32, kThreads)), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        x, q, scales, rows, K, block_rows);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
