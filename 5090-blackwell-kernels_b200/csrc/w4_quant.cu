// int4 weight quantizer and the repack into the layout w4gemm streams. Both run once per weight
// at load time and both are bit-exact contracts: the arithmetic of the quantizer and the layout
// of the repack are what the reference defines (include/spark/kernels.h:375-390,
// python/spark_kernels/reference.py:262-286,323-367); how the work is laid onto the GPU is not.
//
// Quantizer: one CTA per (128-k group, 128 columns). The TMA engine brings the 128 x 128 bf16 tile
// into shared memory with one bulk copy per k row (256 contiguous bytes each, all on one mbarrier),
// so W is read from HBM exactly once, in full rows. A thread takes two adjacent columns (one 32-bit
// shared-memory load gives both, and min / max / |max| run as packed bf16 operations) and a quarter of
// the k range; the four quarters exchange their ranges through shared memory, every thread derives the
// scale and zero point of its two columns and emits its four GPTQ words of each; a warp's stores of one
// k-octet are 256 contiguous bytes. The per-weight division of the definition is replaced by a
// multiplication with the reciprocal plus an exact treatment of ties (see the kernel).
//
// Repack: a warp per 512-byte output block (16 columns x 64 k). Its 8 x 16 source words arrive as one
// 16-byte load per lane and are staged in shared memory; each lane then builds its four output
// words with masks and shifts (every output word is an interleave of two source half-words) and
// writes them with one 16-byte store, so a warp writes its block as one contiguous 512-byte run.
// A CTA takes eight neighbouring strips of one k unit, which makes its reads eight 512-byte rows.
#include <algorithm>

#include "spk_common.cuh"
#include "w4_layout.cuh"

namespace spk {
namespace {

constexpr int kQCols = 128;     // columns per quantizer CTA
constexpr int kQThreads = 256;  // two threads per column

template <bool ASYM>
__global__ void __launch_bounds__(kQThreads)
w4_quantize_tile_kernel(const __nv_bfloat16* __restrict__ W, uint32_t* __restrict__ qweight,
                        __nv_bfloat16* __restrict__ scales, uint8_t* __restrict__ zeros, int N, int bulk, int* status) {
    __shared__ __align__(128) __nv_bfloat16 tile[w4::kGroup][kQCols];
    __shared__ uint3 quarter_range[4][kQCols / 2];  // (min, max, |max|) of a column pair over one k quarter, as bf16 pairs
    __shared__ uint64_t bar;
    const int n0 = blockIdx.x * kQCols, g = blockIdx.y;
    const int cols = min(kQCols, N - n0);  // a multiple of 16
    const __nv_bfloat16* src = W + static_cast<size_t>(g) * w4::kGroup * N + n0;

    if (bulk) {
        if (threadIdx.x == 0) {
            ptx::mbar_init(&bar, 1);
            ptx::fence_mbar_init();
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            if (threadIdx.x == 0) ptx::mbar_arrive_expect_tx(&bar, static_cast<unsigned>(w4::kGroup * cols * 2));
            __syncwarp();
            for (int k = threadIdx.x; k < w4::kGroup; k += 32)
                ptx::bulk_g2s(&tile[k][0], src + static_cast<size_t>(k) * N, static_cast<unsigned>(cols * 2), &bar);
        }
        // bounded; the status word says why the output is missing. The block leaves together or not at all.
        if (!__syncthreads_and(ptx::mbar_wait(&bar, 0, status))) return;
    } else {
        // W not 16-byte aligned: element loads, same tile
        for (int i = threadIdx.x; i < w4::kGroup * cols; i += kQThreads) {
            const int k = i / cols, c = i - k * cols;
            tile[k][c] = src[static_cast<size_t>(k) * N + c];
        }
        __syncthreads();
    }

    // A thread takes two adjacent columns (one 32-bit shared-memory load gives both) and a quarter of the k range.
    const int cp = threadIdx.x & 63, kq = threadIdx.x >> 6;   // column pair, k quarter (32 k)
    const int k0 = kq * (w4::kGroup / 4);
    const uint32_t* tile32 = reinterpret_cast<const uint32_t*>(&tile[0][0]) + cp;   // row pitch kQCols / 2 words
    __nv_bfloat162 lo2 = __float2bfloat162_rn(0.f), hi2 = lo2, am2 = lo2;  // the ranges include 0, as the definition's do
    if (2 * cp < cols) {
#pragma unroll 8
        for (int k = 0; k < w4::kGroup / 4; ++k) {
            const uint32_t u = tile32[(k0 + k) * (kQCols / 2)];
            const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&u);
            lo2 = __hmin2(lo2, x), hi2 = __hmax2(hi2, x), am2 = __hmax2(am2, __habs2(x));
        }
    }
    quarter_range[kq][cp] = make_uint3(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2), *reinterpret_cast<uint32_t*>(&am2));
    __syncthreads();
    if (2 * cp >= cols) return;
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // every thread folds the four quarters itself: no second barrier
        const uint3 o = quarter_range[j][cp];
        lo2 = __hmin2(lo2, *reinterpret_cast<const __nv_bfloat162*>(&o.x));
        hi2 = __hmax2(hi2, *reinterpret_cast<const __nv_bfloat162*>(&o.y));
        am2 = __hmax2(am2, *reinterpret_cast<const __nv_bfloat162*>(&o.z));
    }

    // Per column, fp32 throughout: the codes are computed against the bf16-rounded scale, the number the GEMM will
    // multiply by. The definition divides (IEEE) and rounds half to even. w and s are both bf16, so w / s is a ratio of
    // two 8-bit integers times a power of two: unless it is exactly k + 1/2 it is at least 1 / 2040 away from every such
    // tie, and w * (1 / s) lands within 3e-6 of it. So rint(w * r) is the definition's code except on exact ties, which
    // show as a distance within 1e-4 of 1/2 and are then resolved to the even neighbour: no division per weight.
    float s_col[2], r_col[2], z_col[2];
    bool live_col[2], divide_col[2];  // divide: a scale so small that its reciprocal overflows keeps the division
    __nv_bfloat16 sbf_col[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const float lo = c ? __high2float(lo2) : __low2float(lo2), hi = c ? __high2float(hi2) : __low2float(hi2);
        const float amax = c ? __high2float(am2) : __low2float(am2);
        sbf_col[c] = __float2bfloat16_rn(ASYM ? __fdiv_rn(hi - lo, 15.0f) : __fdiv_rn(amax, 7.0f));
        s_col[c] = __bfloat162float(sbf_col[c]);
        live_col[c] = s_col[c] > 0.f;
        divide_col[c] = live_col[c] && s_col[c] < 1e-30f;
        r_col[c] = live_col[c] && !divide_col[c] ? __frcp_rn(s_col[c]) : 0.f;
        z_col[c] = 8.f;
        if (ASYM) z_col[c] = live_col[c] ? fminf(fmaxf(rintf(__fdiv_rn(-lo, s_col[c])), 0.f), 15.f) : 0.f;
    }
    const float qmin = ASYM ? 0.f : -8.f, qmax = ASYM ? 15.f : 7.f;
    // Rounding and the conversion to an integer go through the adder, not the conversion unit (rint and float -> int
    // run at a quarter of the rate): x + 1.5 * 2^23 rounds x to an integer, half to even, for |x| < 2^22, and the
    // integer then sits in the low mantissa bits.
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
    auto code = [&](float w, int c) -> uint32_t {  // symmetric: clamp(rint(w / s), -8, 7) + 8; asym: clamp(rint(w / s) + z, 0, 15)
        float rn, d;
        if (divide_col[c]) {
            const float t = __fdiv_rn(w, s_col[c]);
            rn = rintf(t), d = t - rn;
        } else {
            rn = __fadd_rn(__fmaf_rn(w, r_col[c], kMagic), -kMagic);   // rint of the product
            d = __fmaf_rn(w, r_col[c], -rn);                           // the product's distance from it
            if (fabsf(fabsf(d) - 0.5f) < 1e-4f) rn = 2.0f * rintf(0.25f * rintf(2.0f * w * r_col[c]));  // an exact tie: the even neighbour
        }
        const float q = fminf(fmaxf(rn + (ASYM ? z_col[c] : 0.f), qmin), qmax) + (ASYM ? 0.f : 8.f);
        const uint32_t bits = static_cast<uint32_t>(__float_as_int(q + kMagic)) & 0xFu;   // q is an integer in 0 .. 15
        return live_col[c] ? bits : static_cast<uint32_t>(z_col[c]);
    };
    const size_t n = static_cast<size_t>(n0) + 2 * cp;
#pragma unroll 2
    for (int o = 0; o < w4::kGroup / 32; ++o) {  // this thread's four k-octets
        uint32_t word0 = 0, word1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t u = tile32[(k0 + 8 * o + i) * (kQCols / 2)];
            word0 |= code(__uint_as_float(u << 16), 0) << (4 * i);
            word1 |= code(__uint_as_float(u & 0xFFFF0000u), 1) << (4 * i);
        }
        *reinterpret_cast<uint2*>(qweight + (static_cast<size_t>(g) * (w4::kGroup / 8) + kq * 4 + o) * N + n) = make_uint2(word0, word1);
    }
    if (kq == 0) {
        *reinterpret_cast<__nv_bfloat162*>(scales + static_cast<size_t>(g) * N + n) = __halves2bfloat162(sbf_col[0], sbf_col[1]);
        if (ASYM) *reinterpret_cast<uchar2*>(zeros + static_cast<size_t>(g) * N + n) = make_uchar2(static_cast<uint8_t>(z_col[0]), static_cast<uint8_t>(z_col[1]));
    }
}

constexpr int kRepackWarps = 8;

// Output word j of lane (g, c) of block (strip, unit) interleaves the nibbles of two source half-words:
// rows k/8 = 4 (j >> 1) + c of the unit, columns g and g + 8 of the strip, half-word j & 1. With those
// as a = a3 a2 a1 a0 and b = b3 b2 b1 b0 the word is b3 a3 b1 a1 b2 a2 b0 a0 (most significant first).
__device__ __forceinline__ uint32_t interleave_halfwords(uint32_t a, uint32_t b) {
    const uint32_t even = (a & 0x0F0Fu) | ((b & 0x0F0Fu) << 4);
    const uint32_t odd = ((a >> 4) & 0x0F0Fu) | (((b >> 4) & 0x0F0Fu) << 4);
    return even | (odd << 16);
}

__global__ void __launch_bounds__(kRepackWarps * 32)
w4_repack_blocks_kernel(const uint32_t* __restrict__ qweight, uint4* __restrict__ packed, int N, int strips, int units,
                        long long jobs) {
    __shared__ __align__(16) uint32_t stage[kRepackWarps][8][24];  // 24-word rows: the gather below is conflict free
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    for (long long job = blockIdx.x; job < jobs; job += gridDim.x) {  // job = (octet of strips, unit)
        const int u = static_cast<int>(job % units);
        const int t = static_cast<int>(job / units) * kRepackWarps + warp;
        if (t < strips) {
            const uint4 v = *reinterpret_cast<const uint4*>(qweight + static_cast<size_t>(8 * u + g) * N + 16 * t + 4 * c);
            *reinterpret_cast<uint4*>(&stage[warp][g][4 * c]) = v;
        }
        __syncwarp();
        if (t < strips) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = 4 * (j >> 1) + c, sh = 16 * (j & 1);
                w[j] = interleave_halfwords((stage[warp][row][g] >> sh) & 0xFFFFu, (stage[warp][row][g + 8] >> sh) & 0xFFFFu);
            }
            packed[(static_cast<size_t>(t) * units + u) * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncwarp();
    }
}

}  // namespace
}  // namespace spk

extern "C" int spk_w4_quantize_bf16(const void* W, int32_t* qweight, void* scales, uint8_t* zeros,
                                    int K, int N, void* stream) {
    using namespace spk;
    SPK_REQUIRE(K > 0 && N > 0 && K % w4::kGroup == 0 && N % 16 == 0,
                "w4_quantize: K must be a positive multiple of 128 and N of 16 (K=%d, N=%d)", K, N);
    SPK_REQUIRE(W != nullptr && qweight != nullptr && scales != nullptr, "w4_quantize: W, qweight and scales are required");
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    const dim3 grid(cdiv(N, kQCols), K / w4::kGroup);
    auto st = static_cast<cudaStream_t>(stream);
    const int bulk = aligned16(W) ? 1 : 0;  // rows are N * 2 bytes apart, a multiple of 32
    auto* q = reinterpret_cast<uint32_t*>(qweight);
    if (zeros)
        w4_quantize_tile_kernel<true><<<grid, kQThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(W), q,
                                                                  static_cast<__nv_bfloat16*>(scales), zeros, N, bulk, dev->status);
    else
        w4_quantize_tile_kernel<false><<<grid, kQThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(W), q,
                                                                   static_cast<__nv_bfloat16*>(scales), nullptr, N, bulk, dev->status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_w4_repack(const int32_t* qweight, int32_t* packed, int K, int N, void* stream) {
    using namespace spk;
    SPK_REQUIRE(K > 0 && N > 0 && K % 64 == 0 && N % 16 == 0,
                "w4_repack: K must be a positive multiple of 64 and N of 16 (K=%d, N=%d)", K, N);
    SPK_REQUIRE(qweight != nullptr && packed != nullptr && qweight != packed, "w4_repack: two distinct buffers are required");
    SPK_REQUIRE(aligned16(qweight) && aligned16(packed), "w4_repack: qweight and packed must be 16-byte aligned");
    const int strips = N / 16, units = K / 64;
    const long long jobs = static_cast<long long>(cdiv(strips, kRepackWarps)) * units;
    const unsigned grid = static_cast<unsigned>(std::min<long long>(jobs, 148LL * 16));
    w4_repack_blocks_kernel<<<grid, kRepackWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<uint4*>(packed), N, strips, units, jobs);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
