// W4A16 GEMM: C[M,N] = A[M,K] * bf16((q - z) * s), int4 codes in the repacked layout, one bf16
// scale (and optional zero point) per 128 k of a column, fp32 accumulation, bf16 out.
// Contract: reference include/spark/kernels.h:366-416. Variants:
//   0  one thread per output, scalar decode through w4::locate (the arithmetic of the
//      reference's w4_naive_kernel, src/kernels/w4gemm.cu:46-67)
//   1  one warp per 16-column strip and 8 tokens, codes and activations straight from global
//      memory into registers, register dequant, warp-level MMA
//   2  the B200 weight stream (default): every warp owns a private ring of bulk asynchronous
//      copies (TMA engine) that brings whole 1 KiB groups of codes plus their scales into
//      shared memory; the (strips x groups) work is cut into equal contiguous ranges, one per
//      CTA, so all SMs stream the same number of bytes; a strip whose K is shared by two CTAs
//      is finished through fp32 atomics into a scratch that the last arriver converts and
//      leaves zeroed
//   3  batch invariant: the stream kernel with whole strips per CTA and a fixed K order, no
//      atomics, so row i of C has the same bits for every M
//
// Why this shape on B200: the M <= 64 GEMM is a read-once stream of N*K/2 bytes. What bounds it
// is HBM, then the instruction issue rate of the exact dequant (15 ALU instructions per 8
// weights). Bulk copies keep >100 KiB per SM in flight without costing registers or issue
// slots, and the flat split keeps 148 SMs busy on shapes whose strip count does not divide.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "spk_common.cuh"
#include "w4_layout.cuh"

namespace spk {
namespace {

using ptx::bulk_g2s;
using ptx::mbar_arrive;
using ptx::mbar_arrive_expect_tx;
using ptx::mbar_init;
using ptx::mbar_wait;

// ---- variant 0 ----------------------------------------------------------------------------------

__global__ void w4_naive_kernel(const __nv_bfloat16* __restrict__ A, const uint32_t* __restrict__ packed,
                                const __nv_bfloat16* __restrict__ scales, const uint8_t* __restrict__ zeros,
                                __nv_bfloat16* __restrict__ C, int M, int N, int K) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y;
    if (n >= N || m >= M) return;
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
        size_t word;
        int p;
        w4::locate(n, k, K, word, p);
        const int q = (packed[word] >> (4 * p)) & 15;
        const size_t si = static_cast<size_t>(k / w4::kGroup) * N + n;
        const int z = zeros ? zeros[si] : 8;
        const float w = __bfloat162float(__float2bfloat16_rn(static_cast<float>(q - z) * __bfloat162float(scales[si])));
        acc = fmaf(__bfloat162float(A[static_cast<size_t>(m) * K + k]), w, acc);
    }
    C[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(acc);
}

// ---- shared by variants 1-3 -----------------------------------------------------------------------

// The lane's activations for one 128-k group of one 8-token tile: four 16-byte chunks, chunk i
// holding k = 32 i + 8 c .. + 7 of token (lane / 4), which is what steps 2i and 2i + 1 need.
struct ActGroup {
    uint4 v[4];
};

__device__ __forceinline__ ActGroup load_acts(const __nv_bfloat16* __restrict__ A, int tok, int M, int K, int g,
                                              int c) {
    ActGroup a;
    if (tok < M) {
        const __nv_bfloat16* p = A + static_cast<size_t>(tok) * K + g * w4::kGroup + 8 * c;
#pragma unroll
        for (int i = 0; i < 4; ++i) a.v[i] = ptx::ldg_cached(p + 32 * i);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) a.v[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    return a;
}

// One 64-k unit (a lane's uint4 of four words) of one strip against MT token tiles.
template <int MT>
__device__ __forceinline__ void unit_mma(float (&acc)[MT][4], const uint4& q, int half, uint32_t off_lo,
                                         uint32_t off_hi, uint32_t s_lo, uint32_t s_hi,
                                         const ActGroup (&act)[MT]) {
    const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t x[4];
        w4::dequant_word(qs[j], off_lo, off_hi, s_lo, s_hi, x);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const uint4& a = act[mt].v[2 * half + (j >> 1)];
            if (j & 1)
                ptx::mma_bf16_16816(acc[mt], x, a.z, a.w);
            else
                ptx::mma_bf16_16816(acc[mt], x, a.x, a.y);
        }
    }
}

// Fragment -> C: acc[0], acc[1] are (column g, tokens 2c, 2c+1); acc[2], acc[3] column g + 8.
__device__ __forceinline__ void store_tile(__nv_bfloat16* __restrict__ C, const float (&acc)[4], int tok0, int M,
                                           int N, int n0, int lane) {
    const int gl = lane >> 2, c = lane & 3;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int tok = tok0 + 2 * c + (e & 1);
        const int n = n0 + gl + 8 * (e >> 1);
        if (tok < M) C[static_cast<size_t>(tok) * N + n] = __float2bfloat16_rn(acc[e]);
    }
}

// ---- variant 1 ----------------------------------------------------------------------------------

template <bool ASYM>
__global__ void __launch_bounds__(128)
w4_strip_kernel(const __nv_bfloat16* __restrict__ A, const uint4* __restrict__ packed,
                const __nv_bfloat16* __restrict__ scales, const uint8_t* __restrict__ zeros,
                __nv_bfloat16* __restrict__ C, int M, int N, int K) {
    const int lane = threadIdx.x & 31, gl = lane >> 2, c = lane & 3;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int tok0 = blockIdx.y * 8;
    if (t >= N / 16) return;
    const int G = K / w4::kGroup;
    const uint4* wp = packed + static_cast<size_t>(t) * G * 64 + lane;
    const unsigned short* sp = reinterpret_cast<const unsigned short*>(scales) + 16 * t + gl;
    const uint8_t* zp = zeros + 16 * t + gl;
    float acc[1][4] = {{0.f, 0.f, 0.f, 0.f}};
    for (int g = 0; g < G; ++g) {
        ActGroup act[1] = {load_acts(A, tok0 + gl, M, K, g, c)};
        const uint4 q0 = ptx::ldg_stream(wp + (2 * g) * 32), q1 = ptx::ldg_stream(wp + (2 * g + 1) * 32);
        const uint32_t s_lo = w4::splat16(sp[static_cast<size_t>(g) * N]);
        const uint32_t s_hi = w4::splat16(sp[static_cast<size_t>(g) * N + 8]);
        uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
        if (ASYM) {
            o_lo = w4::offset_pair(zp[static_cast<size_t>(g) * N]);
            o_hi = w4::offset_pair(zp[static_cast<size_t>(g) * N + 8]);
        }
        unit_mma<1>(acc, q0, 0, o_lo, o_hi, s_lo, s_hi, act);
        unit_mma<1>(acc, q1, 1, o_lo, o_hi, s_lo, s_hi, act);
    }
    store_tile(C, acc[0], tok0, M, N, 16 * t, lane);
}

// ---- variants 2 and 3: the weight stream ------------------------------------------------------------

constexpr int kStreamWarps = 8;  // warps per CTA, one strip set each, along N

struct StreamParams {
    const __nv_bfloat16* A;
    const unsigned char* packed;
    const unsigned char* scales;  // bf16 [G][N]
    const unsigned char* zeros;   // u8 [G][N] or null
    __nv_bfloat16* C;
    int M, N, K, G, T;
    int super_strips;       // cdiv(T, kStreamWarps * NS)
    long long total_units;  // super_strips * G
    int whole;              // CTA ranges end on super-strip boundaries (no shared strips)
    float* partials;        // fp32 [M][N] scratch, zero on entry and on exit
    unsigned* counters;     // [gridDim.y][T], zero on entry and on exit
    int* status;
};

// Bytes of one ring slot of one warp.
template <int NS, bool ASYM>
struct Slot {
    static constexpr int kCodes = NS * w4::kGroupBytes;
    static constexpr int kScales = NS * 32;
    static constexpr int kZeros = ASYM ? NS * 16 : 0;
    static constexpr int kBytes = kCodes + kScales + kZeros;
};

template <int MT, int NS, int ST, bool ASYM>
constexpr int stream_smem_bytes() {
    return kStreamWarps * (ST * Slot<NS, ASYM>::kBytes + ST * 8);
}

template <int MT, int NS, int ST, bool ASYM>
__global__ void __launch_bounds__(kStreamWarps * 32)
w4_stream_kernel(const StreamParams p) {
    using S = Slot<NS, ASYM>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gl = lane >> 2, c = lane & 3;
    unsigned char* ring = smem + warp * (ST * S::kBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStreamWarps * ST * S::kBytes) + warp * ST;

    // This CTA's contiguous range of (super-strip, group) units.
    long long f0, f1;
    if (p.whole) {
        f0 = static_cast<long long>(blockIdx.x) * p.super_strips / gridDim.x * p.G;
        f1 = static_cast<long long>(blockIdx.x + 1) * p.super_strips / gridDim.x * p.G;
    } else {
        f0 = blockIdx.x * p.total_units / gridDim.x;
        f1 = (blockIdx.x + 1) * p.total_units / gridDim.x;
    }
    const int n_units = static_cast<int>(f1 - f0);
    if (n_units <= 0) return;
    const int tok0 = blockIdx.y * (8 * MT);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < ST; ++s) mbar_init(&bars[s], 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();

    // Lane 0 arms slot (i % ST) with unit i: per strip of this warp one 1 KiB bulk copy of codes,
    // 32 bytes of scales and, with zero points, 16 bytes of zeros.
    auto issue = [&](int i) {
        const long long f = f0 + i;
        const int ts = static_cast<int>(f / p.G);
        const int g = static_cast<int>(f - static_cast<long long>(ts) * p.G);
        unsigned char* slot = ring + (i % ST) * S::kBytes;
        uint64_t* bar = &bars[i % ST];
        const int t_first = (ts * kStreamWarps + warp) * NS;
        int valid = p.T - t_first;
        valid = valid < 0 ? 0 : (valid > NS ? NS : valid);
        if (valid == 0) {
            mbar_arrive(bar);
            return;
        }
        mbar_arrive_expect_tx(bar, valid * (w4::kGroupBytes + 32 + (ASYM ? 16 : 0)));
        for (int s = 0; s < valid; ++s) {
            const int t = t_first + s;
            bulk_g2s(slot + s * w4::kGroupBytes,
                     p.packed + (static_cast<size_t>(t) * p.G + g) * w4::kGroupBytes, w4::kGroupBytes, bar);
            bulk_g2s(slot + S::kCodes + s * 32, p.scales + (static_cast<size_t>(g) * p.N + 16 * t) * 2, 32, bar);
            if (ASYM)
                bulk_g2s(slot + S::kCodes + S::kScales + s * 16, p.zeros + static_cast<size_t>(g) * p.N + 16 * t,
                         16, bar);
        }
    };

    if (lane == 0) {
        const int pre = n_units < ST ? n_units : ST;
        for (int i = 0; i < pre; ++i) issue(i);
    }

    int ts = static_cast<int>(f0 / p.G);
    int g = static_cast<int>(f0 - static_cast<long long>(ts) * p.G);
    int seg_g0 = g;  // first group of the segment being accumulated
    float acc[NS][MT][4];
#pragma unroll
    for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[s][mt][e] = 0.f;

    // Ends the segment [seg_g0, g] of super-strip ts: a whole K goes straight to C, a part of K
    // goes through the scratch, and whoever completes the strip converts it.
    auto flush = [&](int ts_, int g_last) {
        const bool whole_k = seg_g0 == 0 && g_last == p.G - 1;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const int t = (ts_ * kStreamWarps + warp) * NS + s;
            if (t < p.T) {
                if (whole_k) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) store_tile(p.C, acc[s][mt], tok0 + 8 * mt, p.M, p.N, 16 * t, lane);
                } else {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int tok = tok0 + 8 * mt + 2 * c + (e & 1);
                            const int n = 16 * t + gl + 8 * (e >> 1);
                            if (tok < p.M) atomicAdd(p.partials + static_cast<size_t>(tok) * p.N + n, acc[s][mt][e]);
                        }
                    __threadfence();
                    __syncwarp();
                    unsigned done = 0;
                    if (lane == 0)
                        done = atomicAdd(p.counters + static_cast<size_t>(blockIdx.y) * p.T + t,
                                         static_cast<unsigned>(g_last - seg_g0 + 1));
                    done = __shfl_sync(0xffffffffu, done, 0);
                    if (done + static_cast<unsigned>(g_last - seg_g0 + 1) == static_cast<unsigned>(p.G)) {
                        __threadfence();
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int tok = tok0 + 8 * mt + 2 * c + (e & 1);
                                const int n = 16 * t + gl + 8 * (e >> 1);
                                if (tok < p.M) {
                                    float* cell = p.partials + static_cast<size_t>(tok) * p.N + n;
                                    p.C[static_cast<size_t>(tok) * p.N + n] = __float2bfloat16_rn(__ldcg(cell));
                                    __stcg(cell, 0.f);
                                }
                            }
                        if (lane == 0) p.counters[static_cast<size_t>(blockIdx.y) * p.T + t] = 0u;
                    }
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[s][mt][e] = 0.f;
        }
        seg_g0 = 0;
    };

    bool ok = true;
    for (int i = 0; i < n_units; ++i) {
        // activations first: their latency overlaps the wait on the ring
        ActGroup act[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) act[mt] = load_acts(p.A, tok0 + 8 * mt + gl, p.M, p.K, g, c);

        ok = __all_sync(0xffffffffu, mbar_wait(&bars[i % ST], (i / ST) & 1, p.status));
        if (!ok) {
            // Drain: give the copies already issued a bounded chance to land, then leave.
            for (int j = i + 1; j < n_units && j < i + ST; ++j) (void)mbar_wait(&bars[j % ST], (j / ST) & 1, nullptr);
            break;
        }
        const unsigned char* slot = ring + (i % ST) * S::kBytes;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const int t = (ts * kStreamWarps + warp) * NS + s;
            if (t < p.T) {
                const unsigned short* sc = reinterpret_cast<const unsigned short*>(slot + S::kCodes + s * 32);
                const uint32_t s_lo = w4::splat16(sc[gl]), s_hi = w4::splat16(sc[gl + 8]);
                uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
                if (ASYM) {
                    const unsigned char* zp = slot + S::kCodes + S::kScales + s * 16;
                    o_lo = w4::offset_pair(zp[gl]);
                    o_hi = w4::offset_pair(zp[gl + 8]);
                }
                const uint4* codes = reinterpret_cast<const uint4*>(slot + s * w4::kGroupBytes);
                const uint4 q0 = codes[lane], q1 = codes[32 + lane];
                unit_mma<MT>(acc[s], q0, 0, o_lo, o_hi, s_lo, s_hi, act);
                unit_mma<MT>(acc[s], q1, 1, o_lo, o_hi, s_lo, s_hi, act);
            }
        }
        __syncwarp();  // every lane has consumed the slot before it is re-armed
        if (lane == 0 && i + ST < n_units) issue(i + ST);

        if (g == p.G - 1 || i == n_units - 1) {
            flush(ts, g);
            g = (g == p.G - 1) ? 0 : g + 1;
            ts += (g == 0);
        } else {
            ++g;
        }
    }
}

// ---- host side --------------------------------------------------------------------------------------

struct StreamShape {
    int mt, ns, st;
};

// Environment override for sweeps: SPK_W4_CFG="mt,ns,st[,ctas_per_sm[,min_units]]".
struct StreamTuning {
    int mt = 0, ns = 0, st = 0, ctas_per_sm = 0, min_units = 0;
};

StreamTuning read_tuning() {
    StreamTuning t;
    const char* e = std::getenv("SPK_W4_CFG");
    if (e && *e) std::sscanf(e, "%d,%d,%d,%d,%d", &t.mt, &t.ns, &t.st, &t.ctas_per_sm, &t.min_units);
    return t;
}

template <int MT, int NS, int ST, bool ASYM>
int launch_stream_t(const StreamParams& base, bool whole, int ctas_per_sm_cap, int min_units,
                    const DeviceState& dev, cudaStream_t stream) {
    StreamParams p = base;
    auto kernel = w4_stream_kernel<MT, NS, ST, ASYM>;
    constexpr int smem = stream_smem_bytes<MT, NS, ST, ASYM>();
    static bool configured[16] = {};
    if (!configured[dev.device & 15]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev.device & 15] = true;
    }
    int per_sm = 0;
    SPK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kStreamWarps * 32, smem));
    if (per_sm < 1) return fail(SPK_CUDA_ERROR, "w4gemm: stream kernel does not fit an SM (smem %d)", smem);
    if (ctas_per_sm_cap > 0) per_sm = std::min(per_sm, ctas_per_sm_cap);
    p.super_strips = cdiv(p.T, kStreamWarps * NS);
    p.total_units = static_cast<long long>(p.super_strips) * p.G;
    const int m_chunks = cdiv(p.M, 8 * MT);
    // Partial strips need the scratch: fall back to whole strips when it does not cover [M][N].
    if (static_cast<int64_t>(p.M) * p.N > kPartialFloats || static_cast<int64_t>(m_chunks) * p.T > kCounters)
        whole = true;
    p.whole = whole ? 1 : 0;
    const long long slots = static_cast<long long>(dev.sm_count) * per_sm;
    // One CTA per `min_units` units at least (a unit is 8 KiB x NS of codes), at most what is
    // resident at once; token chunks beyond the first share the slots.
    const long long want = whole ? p.super_strips : std::max<long long>(1, p.total_units / std::max(1, min_units));
    const long long ctas = std::min(want, std::max<long long>(1, slots / m_chunks));
    const dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(m_chunks));
    kernel<<<grid, kStreamWarps * 32, smem, stream>>>(p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

template <bool ASYM>
int launch_stream(const StreamParams& p, bool whole, const DeviceState& dev, cudaStream_t stream) {
    static const StreamTuning tune = read_tuning();
    int mt = p.M <= 8 ? 1 : p.M <= 16 ? 2 : p.M <= 32 ? 4 : 8;
    int ns = mt >= 2 ? 2 : 1;
    if (tune.mt > 0 && (p.M <= 8 * tune.mt || tune.mt == 8)) mt = tune.mt;  // never fewer tiles than M needs per chunk
    if (tune.ns > 0) ns = tune.ns;
    if (mt == 8) ns = 1;  // 8 token tiles x 2 strips would spill
    const int cap = tune.ctas_per_sm, min_units = tune.min_units > 0 ? tune.min_units : 2;
#define SPK_W4_CASE(MT_, NS_, ST_)                                                       \
    if (mt == MT_ && ns == NS_) return launch_stream_t<MT_, NS_, ST_, ASYM>(p, whole, cap, min_units, dev, stream)
    SPK_W4_CASE(1, 1, 8);
    SPK_W4_CASE(1, 2, 4);
    SPK_W4_CASE(2, 1, 8);
    SPK_W4_CASE(2, 2, 4);
    SPK_W4_CASE(4, 1, 8);
    SPK_W4_CASE(4, 2, 4);
    SPK_W4_CASE(8, 1, 8);
#undef SPK_W4_CASE
    return fail(SPK_INVALID, "w4gemm: no stream kernel for mt=%d ns=%d", mt, ns);
}

}  // namespace
}  // namespace spk

extern "C" int spk_w4gemm_num_variants(void) { return 4; }
extern "C" int spk_w4gemm_default_variant(void) { return 2; }
extern "C" int spk_w4gemm_supports(int M, int N, int K, int variant) {
    return variant >= 0 && variant < 4 && M >= 1 && N > 0 && K > 0 && N % 16 == 0 && K % spk::w4::kGroup == 0;
}

extern "C" int spk_w4gemm_bf16(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros,
                               void* C, int M, int N, int K, int variant, void* stream_) {
    using namespace spk;
    SPK_REQUIRE(variant >= 0 && variant < spk_w4gemm_num_variants(), "w4gemm: variant %d out of range [0, %d)",
                variant, spk_w4gemm_num_variants());
    SPK_REQUIRE(M >= 1 && N > 0 && K > 0, "w4gemm: M, N, K must be positive, got %d %d %d", M, N, K);
    SPK_REQUIRE(N % 16 == 0 && K % w4::kGroup == 0, "w4gemm: needs N %% 16 == 0 and K %% 128 == 0, got N=%d K=%d",
                N, K);
    SPK_REQUIRE(A && packed && scales && C, "w4gemm: null pointer");
    SPK_REQUIRE(aligned16(A) && aligned16(packed) && aligned16(scales) && (!zeros || aligned16(zeros)),
                "w4gemm: A, packed, scales and zeros must be 16-byte aligned");
    auto stream = static_cast<cudaStream_t>(stream_);
    const auto* a = static_cast<const __nv_bfloat16*>(A);
    const auto* sc = static_cast<const __nv_bfloat16*>(scales);
    auto* c = static_cast<__nv_bfloat16*>(C);
    if (variant == 0) {
        const dim3 grid(cdiv(N, 128), M);
        w4_naive_kernel<<<grid, 128, 0, stream>>>(a, reinterpret_cast<const uint32_t*>(packed), sc, zeros, c, M, N, K);
        SPK_CHECK_LAUNCH();
        return SPK_OK;
    }
    if (variant == 1) {
        const dim3 grid(cdiv(N / 16, 4), cdiv(M, 8));
        if (zeros)
            w4_strip_kernel<true><<<grid, 128, 0, stream>>>(a, reinterpret_cast<const uint4*>(packed), sc, zeros, c, M, N, K);
        else
            w4_strip_kernel<false><<<grid, 128, 0, stream>>>(a, reinterpret_cast<const uint4*>(packed), sc, zeros, c, M, N, K);
        SPK_CHECK_LAUNCH();
        return SPK_OK;
    }
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    StreamParams p{};
    p.A = a;
    p.packed = reinterpret_cast<const unsigned char*>(packed);
    p.scales = static_cast<const unsigned char*>(scales);
    p.zeros = zeros;
    p.C = c;
    p.M = M;
    p.N = N;
    p.K = K;
    p.G = K / w4::kGroup;
    p.T = N / 16;
    p.partials = dev->partials;
    p.counters = dev->counters;
    p.status = dev->status;
    const bool whole = variant == 3;
    return zeros ? launch_stream<true>(p, whole, *dev, stream) : launch_stream<false>(p, whole, *dev, stream);
}
