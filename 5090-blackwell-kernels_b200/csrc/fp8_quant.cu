// bf16 -> e4m3 activation quantizers of the fp8 GEMM (reference include/spark/kernels.h:349-364,
// src/kernels/fp8quant.cu): per tensor and per row with the smallest power-of-two scale that keeps
// max|x| / scale <= 448, the OCP MX recipe (one ue8m0 byte per 32 values), and, as an addition
// that the reference does not have, fp32 scales per 1 x 128 or 128 x 128 block.
// Every output byte is a bit-exact contract: the tests compare with the CPU oracle byte for byte.
#include "fp_codecs.cuh"
#include "spk_common.cuh"

namespace spk {
namespace {

constexpr int kThreads = 256;

struct alignas(16) Bf16x8 {
    __nv_bfloat162 h[4];
};

__device__ __forceinline__ void load8(float (&f)[8], const __nv_bfloat16* p) {
    const Bf16x8 v = *reinterpret_cast<const Bf16x8*>(p);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(v.h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
    }
}

__device__ __forceinline__ float amax8(const float (&f)[8]) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(f[i]));
    return a;
}

__device__ __forceinline__ void store8(unsigned char* q, const float (&f)[8], float inv) {
    unsigned w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i / 4] |= static_cast<unsigned>(fp::float_to_e4m3(f[i] * inv)) << (8 * (i % 4));
    *reinterpret_cast<uint2*>(q) = make_uint2(w[0], w[1]);
}

// The smallest power of two s with amax / s <= 448, exponent clamped to [-126, 127] so that 1 / s
// is a normal float even for an all-zero input.
__device__ __forceinline__ float pow2_scale(float amax) {
    const float r = __fdiv_rn(fmaxf(amax, 1.17549435e-38f), 448.0f);
    int p = 0;
    const float m = frexpf(r, &p);
    int e = m == 0.5f ? p - 1 : p;  // ceil(log2 r)
    e = max(-126, min(127, e));
    return ldexpf(1.0f, e);
}

__device__ __forceinline__ float block_max(float a, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = a;
    __syncthreads();
    a = threadIdx.x < (blockDim.x >> 5) ? smem[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (threadIdx.x == 0) smem[0] = a;
    }
    __syncthreads();
    a = smem[0];
    __syncthreads();
    return a;
}

// Grid-stride amax; non-negative floats order like their bit patterns, so one atomicMax of the
// bits per block into a cell that starts at zero gives max|x|.
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const __nv_bfloat16* __restrict__ x, long long chunks, unsigned* __restrict__ cell) {
    __shared__ float smem[32];
    float a = 0.f;
    for (long long c = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; c < chunks;
         c += static_cast<long long>(gridDim.x) * kThreads) {
        float f[8];
        load8(f, x + 8 * c);
        a = fmaxf(a, amax8(f));
    }
    a = block_max(a, smem);
    if (threadIdx.x == 0) atomicMax(cell, __float_as_uint(a));
}

__global__ void __launch_bounds__(kThreads)
quantize_tensor_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ q, long long chunks,
                       const unsigned* __restrict__ cell, float* __restrict__ scale) {
    const float s = pow2_scale(__uint_as_float(*cell));
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale = s;
    const long long c = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    if (c >= chunks) return;
    float f[8];
    load8(f, x + 8 * c);
    store8(q + 8 * c, f, __fdiv_rn(1.0f, s));
}

// One block per row: amax pass, then the conversion pass re-reads the row from L1/L2.
__global__ void __launch_bounds__(kThreads)
quantize_row_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ q, int K,
                    float* __restrict__ scales) {
    __shared__ float smem[32];
    const size_t base = static_cast<size_t>(blockIdx.x) * K;
    const int chunks = K / 8;
    float a = 0.f;
    for (int c = threadIdx.x; c < chunks; c += kThreads) {
        float f[8];
        load8(f, x + base + 8 * c);
        a = fmaxf(a, amax8(f));
    }
    const float s = pow2_scale(block_max(a, smem));
    if (threadIdx.x == 0) scales[blockIdx.x] = s;
    const float inv = __fdiv_rn(1.0f, s);
    for (int c = threadIdx.x; c < chunks; c += kThreads) {
        float f[8];
        load8(f, x + base + 8 * c);
        store8(q + base + 8 * c, f, inv);
    }
}

// OCP MX: one thread per block of 32 values; e = floor(log2 amax) - 8 through frexp (exact at
// powers of two), an all-zero block gets the smallest scale; scale byte e + 127.
__global__ void __launch_bounds__(kThreads)
quantize_mx_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ q, unsigned char* __restrict__ sf,
                   long long blocks) {
    const long long b = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    if (b >= blocks) return;
    float f[4][8];
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        load8(f[i], x + 32 * b + 8 * i);
        a = fmaxf(a, amax8(f[i]));
    }
    int p = 0;
    (void)frexpf(a, &p);
    int e = a > 0.f ? p - 1 - 8 : -127;
    e = max(-127, min(127, e));
    const float inv = ldexpf(1.0f, -e);
#pragma unroll
    for (int i = 0; i < 4; ++i) store8(q + 32 * b + 8 * i, f[i], inv);
    sf[b] = static_cast<unsigned char>(e + 127);
}

// fp32 block scales (not in the reference): one warp per (block of `block_rows` rows, 128 k):
// s = amax / 448 (1 for an all-zero block), q = e4m3(x / s). x is fp32 here: this quantizer also
// serves weights.
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
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    const float s = a > 0.f ? __fdiv_rn(a, 448.0f) : 1.0f;
    if (lane == 0) scales[static_cast<size_t>(rb) * KB + kb] = s;
    for (int r = r0; r < r1; ++r) {
        const size_t off = static_cast<size_t>(r) * K + 128 * kb + 4 * lane;
        const float4 v = *reinterpret_cast<const float4*>(x + off);
        const unsigned w = fp::float_to_e4m3(__fdiv_rn(v.x, s)) | (fp::float_to_e4m3(__fdiv_rn(v.y, s)) << 8) |
                           (fp::float_to_e4m3(__fdiv_rn(v.z, s)) << 16) | (fp::float_to_e4m3(__fdiv_rn(v.w, s)) << 24);
        *reinterpret_cast<unsigned*>(q + off) = w;
    }
}

}  // namespace
}  // namespace spk

extern "C" int spk_absmax_bits(const void* x, long long n, unsigned* work, void* stream) {
    using namespace spk;
    SPK_REQUIRE(x != nullptr && work != nullptr, "absmax_bits: null pointer");
    SPK_REQUIRE(n > 0 && n % 8 == 0 && aligned16(x), "absmax_bits: n must be a positive multiple of 8 and x 16-byte aligned");
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    const long long chunks = n / 8;
    const int grid = static_cast<int>(std::min<long long>(cdiv64(chunks, kThreads), 8LL * dev->sm_count));
    absmax_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), chunks, work);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_fp8_quantize(const void* x_, unsigned char* q, void* scale, unsigned* work, int rows, int K,
                                int mode, void* stream_) {
    using namespace spk;
    SPK_REQUIRE(x_ != nullptr && q != nullptr && scale != nullptr, "fp8_quantize: null pointer");
    SPK_REQUIRE(rows > 0 && K > 0, "fp8_quantize: rows and K must be positive");
    SPK_REQUIRE(mode >= SPK_FP8Q_TENSOR && mode <= SPK_FP8Q_MX, "fp8_quantize: unknown mode %d", mode);
    SPK_REQUIRE(K % (mode == SPK_FP8Q_MX ? 32 : 8) == 0, "fp8_quantize: K must be a multiple of 8 (32 for mx), got %d", K);
    SPK_REQUIRE(aligned16(x_), "fp8_quantize: x must be 16-byte aligned");
    SPK_REQUIRE(reinterpret_cast<uintptr_t>(q) % 8 == 0, "fp8_quantize: q must be 8-byte aligned");
    auto stream = static_cast<cudaStream_t>(stream_);
    const auto* x = static_cast<const __nv_bfloat16*>(x_);
    const long long n = static_cast<long long>(rows) * K;
    if (mode == SPK_FP8Q_TENSOR) {
        SPK_REQUIRE(work != nullptr, "fp8_quantize: the tensor mode needs a zeroed work cell");
        if (int rc = spk_absmax_bits(x, n, work, stream_)) return rc;
        const long long chunks = n / 8;
        quantize_tensor_kernel<<<static_cast<unsigned>(cdiv64(chunks, kThreads)), kThreads, 0, stream>>>(
            x, q, chunks, work, static_cast<float*>(scale));
    } else if (mode == SPK_FP8Q_ROW) {
        quantize_row_kernel<<<rows, kThreads, 0, stream>>>(x, q, K, static_cast<float*>(scale));
    } else {
        const long long blocks = n / 32;
        quantize_mx_kernel<<<static_cast<unsigned>(cdiv64(blocks, kThreads)), kThreads, 0, stream>>>(
            x, q, static_cast<unsigned char*>(scale), blocks);
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
