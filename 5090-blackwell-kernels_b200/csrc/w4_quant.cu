// int4 weight quantizer and the repack into the layout w4gemm streams. Both run once per weight
// at load time and both are bit-exact contracts: the arithmetic of the quantizer and the layout
// of the repack are what the reference defines (include/spark/kernels.h:375-390,
// python/spark_kernels/reference.py:262-286,323-367); how the work is laid onto the GPU is not.
//
// Quantizer: one CTA per (128-k group, 128 columns). The TMA engine brings the 128 x 128 bf16 tile
// into shared memory with one bulk copy per k row (256 contiguous bytes each, all on one mbarrier),
// so W is read from HBM exactly once, in full rows. Two threads share a column (64 k each): they
// reduce min / max / |max| from shared memory, exchange them, derive scale and zero point, and each
// emits its 8 GPTQ words; a warp's stores of one k-octet are 128 contiguous bytes.
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

struct ColumnRange {
    float lo, hi, amax;
};

template <bool ASYM>
__global__ void __launch_bounds__(kQThreads)
w4_quantize_tile_kernel(const __nv_bfloat16* __restrict__ W, uint32_t* __restrict__ qweight,
                        __nv_bfloat16* __restrict__ scales, uint8_t* __restrict__ zeros, int N, int bulk, int* status) {
    __shared__ __align__(128) __nv_bfloat16 tile[w4::kGroup][kQCols];
    __shared__ ColumnRange other[kQCols];  // the upper half's range of every column
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

    const int col = threadIdx.x & (kQCols - 1), half = threadIdx.x >> 7;
    const int k0 = half * (w4::kGroup / 2);
    ColumnRange r = {0.f, 0.f, 0.f};
    if (col < cols) {
#pragma unroll 16
        for (int k = 0; k < w4::kGroup / 2; ++k) {
            const float w = __bfloat162float(tile[k0 + k][col]);
            r.lo = fminf(r.lo, w);
            r.hi = fmaxf(r.hi, w);
            r.amax = fmaxf(r.amax, fabsf(w));
        }
    }
    if (half == 1) other[col] = r;
    __syncthreads();
    if (half == 0) {
        const ColumnRange o = other[col];
        r.lo = fminf(r.lo, o.lo), r.hi = fmaxf(r.hi, o.hi), r.amax = fmaxf(r.amax, o.amax);
        other[col] = r;
    }
    __syncthreads();
    if (col >= cols) return;
    r = other[col];

    // fp32 throughout; the codes are computed against the bf16-rounded scale, the number the GEMM will
    // multiply by, with IEEE division and round-half-even
    const __nv_bfloat16 s_bf = __float2bfloat16_rn(ASYM ? __fdiv_rn(r.hi - r.lo, 15.0f) : __fdiv_rn(r.amax, 7.0f));
    const float s = __bfloat162float(s_bf);
    const bool live = s > 0.f;
    float zf = 8.f, qmin = -8.f, qmax = 7.f, shift = 8.f;  // symmetric: q = clamp(rint(w / s), -8, 7) + 8
    if (ASYM) {
        zf = live ? fminf(fmaxf(rintf(__fdiv_rn(-r.lo, s)), 0.f), 15.f) : 0.f;
        qmin = 0.f, qmax = 15.f, shift = 0.f;  // q = clamp(rint(w / s) + z, 0, 15)
    }
    const size_t n = static_cast<size_t>(n0) + col;
#pragma unroll 2
    for (int o = 0; o < w4::kGroup / 16; ++o) {  // this thread's eight k-octets
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float q = zf;
            if (live) {
                const float w = __bfloat162float(tile[k0 + 8 * o + i][col]);
                const float t = rintf(__fdiv_rn(w, s)) + (ASYM ? zf : 0.f);
                q = fminf(fmaxf(t, qmin), qmax) + shift;
            }
            word |= static_cast<uint32_t>(static_cast<int>(q)) << (4 * i);
        }
        qweight[(static_cast<size_t>(g) * (w4::kGroup / 8) + half * 8 + o) * N + n] = word;
    }
    if (half == 0) {
        scales[static_cast<size_t>(g) * N + n] = s_bf;
        if (ASYM) zeros[static_cast<size_t>(g) * N + n] = static_cast<uint8_t>(zf);
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
