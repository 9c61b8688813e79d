// W4A16 GEMM: C[M,N] = A[M,K] * bf16((q - z) * s), int4 codes in the repacked layout, one bf16
// scale (and optional zero point) per 128 k of a column, fp32 accumulation, bf16 out.
// Contract: reference include/spark/kernels.h:366-416. Variants:
//   0  the plain rung, walking the packed layout: a CTA per (strip, token), every lane decodes its own 16-byte
//      pieces nibble by nibble with scalar arithmetic, fixed-order sum through shared memory
//   1  the first tensor-core rung: a CTA per (strip, 32 tokens), the strip's codes staged in shared memory by
//      double-buffered bulk copies and shared by four warps with an 8-token tile each, register dequant, warp-level MMA
//   2  (default) by token count: up to 16 tokens the B200 weight stream described next, up to a few hundred
//      the tcgen05 kernel with the weights in TMEM (w4gemm_tmem.cu), above that dequantize once + dense
//      bf16 tcgen05 GEMM (w4_prefill.cu). The weight stream: every warp owns a private ring of bulk asynchronous
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
// The plain rung, organised by the PACKED layout rather than by output element: a CTA per (strip, token). Warp w walks
// the strip's 64-k units w, w + 4, ...; a lane reads its own 16-byte piece of the unit (the piece of lane (g, c) holds
// 16 k of columns g and g + 8), decodes the 32 codes one at a time with scalar arithmetic (w4::slot_source says which
// column and k a nibble is) and accumulates the two columns' dot products in fp32. The 16 threads that hold the same
// column pair are then summed in a fixed order through shared memory. No tensor cores, no asynchronous copies.
__global__ void __launch_bounds__(128)
w4_scalar_kernel(const __nv_bfloat16* __restrict__ A, const uint4* __restrict__ packed, const __nv_bfloat16* __restrict__ scales,
                 const uint8_t* __restrict__ zeros, __nv_bfloat16* __restrict__ C, int M, int N, int K) {
    __shared__ float part[128][2];
    const int t = blockIdx.x, m = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
    const int units = K / 64;
    const __nv_bfloat16* a_row = A + static_cast<size_t>(m) * K;
    float acc[2] = {0.f, 0.f};  // columns g and g + 8 of the strip
    for (int u = warp; u < units; u += 4) {
        const uint4 piece = packed[(static_cast<size_t>(t) * units + u) * 32 + lane];
        const uint32_t words[4] = {piece.x, piece.y, piece.z, piece.w};
        const size_t row = static_cast<size_t>(u >> 1) * N + 16 * t + g;  // the unit's group, this lane's first column
        const float sc[2] = {__bfloat162float(scales[row]), __bfloat162float(scales[row + 8])};
        const int zp[2] = {zeros ? zeros[row] : 8, zeros ? zeros[row + 8] : 8};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int nib = 0; nib < 8; ++nib) {
                int dn, dk;
                w4::slot_source(lane, u, j, nib, dn, dk);
                const int hi = dn >> 3;  // 0: column g, 1: column g + 8
                const int q = static_cast<int>((words[j] >> (4 * nib)) & 15u);
                const float w = __bfloat162float(__float2bfloat16_rn(static_cast<float>(q - zp[hi]) * sc[hi]));
                acc[hi] = fmaf(__bfloat162float(a_row[64 * u + dk]), w, acc[hi]);
            }
    }
    part[threadIdx.x][0] = acc[0], part[threadIdx.x][1] = acc[1];
    __syncthreads();
    if (threadIdx.x < 16) {  // column threadIdx.x of the strip: the 4 warps x 4 lanes (g, c = 0..3) that hold it, in order
        const int gg = threadIdx.x & 7, hi = threadIdx.x >> 3;
        float sum = 0.f;
        for (int w = 0; w < 4; ++w)
            for (int c = 0; c < 4; ++c) sum += part[w * 32 + 4 * gg + c][hi];
        C[static_cast<size_t>(m) * N + 16 * t + threadIdx.x] = __float2bfloat16_rn(sum);
    }
}

// ---- shared by variants 1-3 -----------------------------------------------------------------------

// The lane's activations for one 128-k group of one 8-token tile: four 16-byte chunks, chunk i
// holding k = 32 i + 8 c .. + 7 of token (lane / 4), which is what steps 2i and 2i + 1 need.
struct ActGroup {
    uint4 v[4];
};

// Rows past M re-read row M - 1: an MMA column only ever feeds its own output column, and the
// stores skip tok >= M, so the duplicate is never seen; this keeps the load free of divergence.
__device__ __forceinline__ ActGroup load_acts(const __nv_bfloat16* __restrict__ A, int tok, int M, int K, int g,
                                              int c) {
    ActGroup a;
    tok = tok < M ? tok : M - 1;
    const __nv_bfloat16* p = A + static_cast<size_t>(tok) * K + g * w4::kGroup + 8 * c;
#pragma unroll
    for (int i = 0; i < 4; ++i) a.v[i] = ptx::ldg_cached(p + 32 * i);
    return a;
}

// One 64-k unit (a lane's uint4 of four words) of one strip against MT token tiles. NA = 2
// alternates two accumulators over the k16 steps so consecutive MMAs do not depend on each other.
template <int MT, int NA>
__device__ __forceinline__ void unit_mma(float (&acc)[MT][NA][4], const uint4& q, int half, uint32_t off_lo,
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
                ptx::mma_bf16_16816(acc[mt][j % NA], x, a.z, a.w);
            else
                ptx::mma_bf16_16816(acc[mt][j % NA], x, a.x, a.y);
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
// The first tensor-core rung: a CTA per (strip, 32 tokens). The strip's codes are brought into shared memory by the TMA
// engine, four groups (4 KiB) per bulk copy, double buffered, and are shared by the CTA's four warps, each of which
// takes its own 8-token tile (one legacy MMA per 16 x 16 weights); scales and zero points come straight from global
// memory. One bounded barrier wait and one block barrier per 4 KiB.
constexpr int kStripChunkGroups = 4;

template <bool ASYM>
__global__ void __launch_bounds__(128)
w4_strip_kernel(const __nv_bfloat16* __restrict__ A, const unsigned char* __restrict__ packed,
                const __nv_bfloat16* __restrict__ scales, const uint8_t* __restrict__ zeros,
                __nv_bfloat16* __restrict__ C, int M, int N, int K, int* status) {
    __shared__ __align__(128) unsigned char codes[2][kStripChunkGroups * w4::kGroupBytes];
    __shared__ uint64_t landed[2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gl = lane >> 2, c = lane & 3;
    const int t = blockIdx.x, G = K / w4::kGroup;
    const int tok0 = blockIdx.y * 32 + warp * 8;          // this warp's token tile
    const bool has_tokens = tok0 < M;                      // a warp without tokens still keeps the barriers' count
    const int chunks = (G + kStripChunkGroups - 1) / kStripChunkGroups;
    const unsigned char* strip = packed + static_cast<size_t>(t) * G * w4::kGroupBytes;
    auto fetch = [&](int chunk) {  // thread 0 only
        const int g0 = chunk * kStripChunkGroups, n = min(kStripChunkGroups, G - g0);
        mbar_arrive_expect_tx(&landed[chunk & 1], static_cast<unsigned>(n * w4::kGroupBytes));
        bulk_g2s(codes[chunk & 1], strip + static_cast<size_t>(g0) * w4::kGroupBytes, static_cast<unsigned>(n * w4::kGroupBytes),
                 &landed[chunk & 1]);
    };
    if (threadIdx.x == 0) {
        mbar_init(&landed[0], 1);
        mbar_init(&landed[1], 1);
        ptx::fence_mbar_init();
        fetch(0);
    }
    __syncthreads();
    const unsigned short* sp = reinterpret_cast<const unsigned short*>(scales) + 16 * t + gl;
    const uint8_t* zp = zeros + 16 * t + gl;
    float acc[1][1][4] = {{{0.f, 0.f, 0.f, 0.f}}};
    for (int chunk = 0; chunk < chunks; ++chunk) {
        if (threadIdx.x == 0 && chunk + 1 < chunks) fetch(chunk + 1);  // its buffer was released by the barrier below
        // bounded; the block leaves together or not at all
        if (!__syncthreads_and(mbar_wait(&landed[chunk & 1], (chunk >> 1) & 1, status))) return;
        const int g0 = chunk * kStripChunkGroups, n = min(kStripChunkGroups, G - g0);
        if (has_tokens) {
            const uint4* cw = reinterpret_cast<const uint4*>(codes[chunk & 1]) + lane;
            for (int gi = 0; gi < n; ++gi) {
                const int g = g0 + gi;
                ActGroup act[1] = {load_acts(A, tok0 + gl, M, K, g, c)};
                const uint4 q0 = cw[(2 * gi) * 32], q1 = cw[(2 * gi + 1) * 32];
                const uint32_t s_lo = w4::splat16(sp[static_cast<size_t>(g) * N]);
                const uint32_t s_hi = w4::splat16(sp[static_cast<size_t>(g) * N + 8]);
                uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
                if (ASYM) {
                    o_lo = w4::offset_pair(zp[static_cast<size_t>(g) * N]);
                    o_hi = w4::offset_pair(zp[static_cast<size_t>(g) * N + 8]);
                }
                unit_mma<1, 1>(acc, q0, 0, o_lo, o_hi, s_lo, s_hi, act);
                unit_mma<1, 1>(acc, q1, 1, o_lo, o_hi, s_lo, s_hi, act);
            }
        }
        __syncthreads();  // every warp is done with this buffer before the copy after next overwrites it
    }
    if (has_tokens) store_tile(C, acc[0][0], tok0, M, N, 16 * t, lane);
}

// ---- variants 2 and 3: the weight stream ------------------------------------------------------------
//
// Arithmetic. Every weight is dequantized exactly as the reference defines it, w = bf16((q - z) * s):
// an exact bf16 subtraction and one rounding multiplication per pair (15 instructions per 8 weights).
// Applying the scale once per 128-k group to the fp32 group sum would save the multiplications, and it
// was built and measured here: it is a DIFFERENT function. The reference's result contains the bf16
// rounding of every single weight; without it outputs move by ~1e-3 of the output range (sqrt(K) terms
// of relative error 2^-9 each), which fails the parity tolerance on every output that is small against
// the range. It also did not run faster: the kernel is not bound by its instruction count.
//
// Work decomposition. A super-strip is kStreamWarps * NS strips (128 * NS columns); a chunk is CG
// groups of one super-strip. Chunks are numbered super-strip major and every CTA takes an equal
// contiguous range of them, so every SM streams the same amount whatever the shape. Warp w owns
// strips (super * 8 + w) * NS .. + NS - 1 of each super-strip the range touches.
// A K segment that covers a whole strip goes straight to C. A partial one is added to an fp32
// scratch with fire-and-forget reductions; at the very end of the warp one fence publishes them,
// a per-strip counter is advanced, and whoever completes a strip converts it to bf16 and leaves
// scratch and counter zeroed. Variant 3 cuts the ranges at super-strip boundaries instead: no
// scratch, a fixed summation order.
//
// Data movement per consumer warp, private to the warp (no block-level barrier anywhere in the loop):
//   codes   one bulk asynchronous copy (TMA engine, untiled) per strip per chunk: CG KiB,
//           contiguous in the repacked layout (2 KiB or more per request: smaller requests
//           measured well below the HBM rate)
//   scales  16-byte cp.async copies (one per half row of 16 bf16), zero points likewise
// all landing in ring slot (chunk % ST) and all signalled on that slot's mbarrier: the bulk copy
// through its transaction count, the cp.async copies through one deferred arrive per lane.

// Development aid, compiled in only with -DSPK_W4_TRACE: device clock stamps of a few CTAs' warps,
// written to a buffer set with spk_debug_w4s_trace (layout [cta slot][warp][kTraceEvents]).
#ifdef SPK_W4_TRACE
constexpr int kTraceEvents = 256;
__device__ unsigned long long* g_w4s_trace = nullptr;
__device__ __forceinline__ void trace_stamp(int warp, int lane, int& n) {
    const int slot = blockIdx.x == 0 ? 0 : blockIdx.x == 1 ? 1 : blockIdx.x == gridDim.x / 2 ? 2 : blockIdx.x == gridDim.x - 1 ? 3 : -1;
    if (lane == 0 && slot >= 0 && blockIdx.y == 0 && g_w4s_trace != nullptr && n < kTraceEvents)
        g_w4s_trace[(static_cast<size_t>(slot) * 32 + warp) * kTraceEvents + n] = clock64();
    ++n;
}
#define W4S_TRACE() trace_stamp(warp, lane, trace_n)
// grid-level schedule: chip-wide nanosecond timer at entry / after the dependency wait / at the end of
// warp 0 of EVERY CTA, for successive launches: g_w4s_grid[(launch * 1024 + cta) * 4 + event]
__device__ unsigned long long* g_w4s_grid = nullptr;
__device__ unsigned g_w4s_seq[1024];
__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define W4S_GRID(ev)                                                                                              \
    do {                                                                                                          \
        if (threadIdx.x == 0 && blockIdx.y == 0 && g_w4s_grid != nullptr && blockIdx.x < 1024 && grid_seq < 64)   \
            g_w4s_grid[(static_cast<size_t>(grid_seq) * 1024 + blockIdx.x) * 4 + (ev)] = globaltimer();         \
    } while (0)
#else
#define W4S_TRACE() ((void)0)
#define W4S_GRID(ev) ((void)0)
#endif

#ifndef SPK_STREAM_WARPS
#define SPK_STREAM_WARPS 8
#endif
constexpr int kStreamWarps = SPK_STREAM_WARPS;          // consumer warps per CTA, one strip set each, along N
constexpr int kStreamThreads = (kStreamWarps + 1) * 32;  // + the activation warp

struct StreamParams {
    const __nv_bfloat16* A;
    const unsigned char* packed;
    const unsigned char* scales;  // bf16 [G][N]
    const unsigned char* zeros;   // u8 [G][N] or null
    __nv_bfloat16* C;
    int M, N, K, G, T;
    int whole;           // 1: CTA ranges end on super-strip boundaries (no scratch, fixed order)
    int super_strips;    // cdiv(T, kStreamWarps * NS)
    int rows_max;        // min(M, 8 MT): token rows the activation ring is sized for
    float* partials;     // fp32 [M][N] scratch, zero on entry and on exit
    unsigned* counters;  // [gridDim.y][T], zero on entry and on exit
    int* status;
};

template <int NS, int CG, bool ASYM>
struct Slot {
    static constexpr int kCodes = NS * CG * w4::kGroupBytes;
    static constexpr int kScales = NS * CG * 32;
    static constexpr int kZeros = ASYM ? NS * CG * 16 : 0;
    static constexpr int kBytes = kCodes + kScales + kZeros;
};

// Activation ring (shared by the CTA): stage j holds, for every token row of this CTA's chunk of
// tokens, the CG * 128 activations of chunk j.
// The activation warp streams the rows in with one bulk copy per row; the consumer warps read their
// MMA B operands from the ring with LDS.128. Activations must live in shared memory: the codes
// stream through L2 at the HBM rate, and activation loads that miss the small L1 left beside
// ~200 KiB of shared memory then queue behind that stream (measured: 25% L1 misses doubled the
// kernel time).
template <int MT>
struct ActRing {
    static constexpr int kStages = MT <= 2 ? 4 : (MT == 4 ? 3 : 2);
};
// Row pitch: chunk bytes + 64, so that the eight lanes of a quarter warp (two token rows x four
// 16-byte columns) fall into distinct 16-byte bank groups.
__host__ __device__ constexpr int act_pitch(int cg) { return cg * 256 + 64; }
__host__ __device__ constexpr int act_stage_bytes(int rows, int cg) { return rows * act_pitch(cg); }

template <int MT, int NS, int CG, int ST, bool ASYM>
constexpr int stream_smem_bytes(int rows) {
    return kStreamWarps * ST * Slot<NS, CG, ASYM>::kBytes + ActRing<MT>::kStages * act_stage_bytes(rows, CG) +
           (2 * ActRing<MT>::kStages + kStreamWarps * ST) * 8;
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(dst)), "l"(src) : "memory");
}
// Arrive on `bar` once every cp.async this thread issued so far has landed (the arrival is
// already part of the barrier's expected count).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(ptx::smem_u32(bar)) : "memory");
}

// Resident CTAs the register budget is held to: two CTAs (18 warps) per SM for the one- and two-tile
// shapes, each with three 4 KiB slots per warp (192 KiB in flight per SM). Measured on the Llama
// shapes at one token, graph-timed: three CTAs with two slots each run gate|up in the same 20.8 us
// and 4096 x 4096 in 7.2 us against 6.2 us.
template <int MT, int NS>
struct StreamOcc {
#ifdef SPK_STREAM_MINCTAS
    static constexpr int kMinCtas = MT * NS <= 2 ? SPK_STREAM_MINCTAS : 1;
#else
    static constexpr int kMinCtas = MT * NS <= 2 ? 2 : 1;
#endif
};


template <int MT, int NS, int CG, int ST, bool ASYM, bool DUAL>
__global__ void __launch_bounds__(kStreamThreads, StreamOcc<MT, NS>::kMinCtas)
w4_stream_kernel(const StreamParams p) {
    using S = Slot<NS, CG, ASYM>;
    constexpr int NA = DUAL ? 2 : 1;  // accumulators a tile alternates between, so that consecutive MMAs do not depend on each other
    constexpr int kPitch = act_pitch(CG);
    constexpr int kActStages = ActRing<MT>::kStages;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gl = lane >> 2, c = lane & 3;
#ifdef SPK_W4_TRACE
    int trace_n = 0;
    unsigned grid_seq = 0;
    if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x < 1024) grid_seq = atomicAdd(&g_w4s_seq[blockIdx.x], 1u);
#endif
    W4S_TRACE();  // 0: entry
    W4S_GRID(0);

    // This CTA's range [f0, f1) of chunks, numbered super-strip major (G % CG == 0).
    const int chunks = p.G / CG;
    int f0, f1;
    if (p.whole) {
        f0 = static_cast<int>(static_cast<long long>(blockIdx.x) * p.super_strips / gridDim.x) * chunks;
        f1 = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * p.super_strips / gridDim.x) * chunks;
    } else {
        const long long total = static_cast<long long>(p.super_strips) * chunks;
        f0 = static_cast<int>(blockIdx.x * total / gridDim.x);
        f1 = static_cast<int>((blockIdx.x + 1) * total / gridDim.x);
    }
    const int n_chunks = f1 - f0;
    const int ss0 = f0 / chunks, ch0 = f0 - ss0 * chunks;
    const int tok0 = blockIdx.y * (8 * MT);
    int rows = p.M - tok0;  // token rows this CTA really has
    rows = rows > 8 * MT ? 8 * MT : rows;

    // shared memory: [8 warps][ST slots] codes+scales(+zeros) | act ring | barriers
    unsigned char* act_ring = smem + kStreamWarps * ST * S::kBytes;
    const int act_stage = act_stage_bytes(p.rows_max, CG);
    uint64_t* bar_base = reinterpret_cast<uint64_t*>(act_ring + kActStages * act_stage);
    uint64_t* a_landed = bar_base;              // [stages] the rows' bulk copies have landed
    uint64_t* a_empty = bar_base + kActStages;  // [stages] the eight consumer warps are done with it
    uint64_t* bars = bar_base + 2 * kActStages + (warp < kStreamWarps ? warp : 0) * ST;  // a consumer's code ring

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < kActStages; ++s) {
            mbar_init(&a_landed[s], 1);
            mbar_init(&a_empty[s], kStreamWarps);
        }
        ptx::fence_mbar_init();
    }
    if (lane == 0 && warp < kStreamWarps) {
#pragma unroll
        for (int s = 0; s < ST; ++s) mbar_init(&bars[s], 33);  // 1 expect_tx arrive + 32 cp.async arrives
        ptx::fence_mbar_init();
    }
    __syncthreads();  // the only block-wide barrier: barrier objects are ready
    pdl_release();  // a chained kernel behind this one may become resident as this grid's CTAs exit
    W4S_TRACE();  // 1: set-up done
    if (n_chunks <= 0) return;

    // this lane's activation rows (token tiles mt); rows past the CTA's last re-read that one
    int act_off[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int r = 8 * mt + gl;
        r = r < rows ? r : rows - 1;
        act_off[mt] = r * kPitch + 16 * c;
    }

    if (warp == kStreamWarps) {
        // ================= activation warp =================
        // Chunk j goes to stage j % kActStages: one bulk copy per token row (lane r issues row r),
        // signalled on the stage's barrier, which the consumers wait on. A stage is reused once the
        // eight consumer warps have released it.
        pdl_wait();  // the activations may be the output of the kernel in front of a chained launch
        W4S_TRACE();  // act warp 2: predecessor complete
        const unsigned char* a_row = reinterpret_cast<const unsigned char*>(p.A) +
                                     static_cast<size_t>(tok0 + (lane < rows ? lane : 0)) * p.K * 2;
        int i_ch = ch0, stage = 0;
        unsigned phase = 0;
        for (int j = 0; j < n_chunks; ++j) {
            if (j >= kActStages && !__all_sync(0xffffffffu, mbar_wait(&a_empty[stage], phase ^ 1u, p.status))) break;
            if (lane == 0) mbar_arrive_expect_tx(&a_landed[stage], rows * (CG * 256));
            __syncwarp();
            for (int r = lane; r < rows; r += 32)
                bulk_g2s(act_ring + stage * act_stage + r * kPitch,
                         a_row + static_cast<size_t>(r - lane) * p.K * 2 + static_cast<size_t>(i_ch) * (CG * 256), CG * 256,
                         &a_landed[stage]);
            i_ch = i_ch + 1 == chunks ? 0 : i_ch + 1;
            if (++stage == kActStages) stage = 0, phase ^= 1u;
        }
        return;  // copies still in flight complete on barriers the consumers wait on before they leave
    }

    // ================= consumer warps =================
    unsigned char* ring = smem + warp * (ST * S::kBytes);
    const size_t strip_bytes = static_cast<size_t>(p.G) * w4::kGroupBytes;
    auto valid_of = [&](int t_first) {
        int v = p.T - t_first;
        return v < 0 ? 0 : (v > NS ? NS : v);
    };

    // ---- code producer (warp-collective; runs ST chunks ahead of the consumer) ----
    // lane roles for the small copies: half a scale row (row = strip s x group gi), a zero-point row
    const int sc_row = lane >> 1, sc_s = sc_row / CG, z_s = lane / CG;
    int p_left = n_chunks, p_slot = 0, p_ch = ch0;
    int p_t = (ss0 * kStreamWarps + warp) * NS, p_valid = valid_of(p_t);
    const unsigned char* code_src = p.packed + static_cast<size_t>(p_t) * strip_bytes +
                                    static_cast<size_t>(ch0) * (CG * w4::kGroupBytes);
    const unsigned char* sc_src =
        p.scales + (static_cast<size_t>(ch0 * CG + sc_row % CG) * p.N + 16 * (p_t + sc_s)) * 2 + (lane & 1) * 16;
    const unsigned char* z_src =
        ASYM ? p.zeros + static_cast<size_t>(ch0 * CG + lane % CG) * p.N + 16 * (p_t + z_s) : nullptr;
    const size_t sc_step = static_cast<size_t>(CG) * p.N * 2, z_step = static_cast<size_t>(CG) * p.N;
    auto issue = [&]() {
        if (p_left <= 0) return;
        unsigned char* slot = ring + p_slot * S::kBytes;
        uint64_t* bar = &bars[p_slot];
        if (lane == 0) {
            if (p_valid == 0) {
                mbar_arrive(bar);
            } else {
                mbar_arrive_expect_tx(bar, p_valid * (CG * w4::kGroupBytes));
#pragma unroll
                for (int s = 0; s < NS; ++s)
                    if (s < p_valid)
                        bulk_g2s(slot + s * (CG * w4::kGroupBytes), code_src + s * strip_bytes, CG * w4::kGroupBytes, bar);
            }
        }
        if (sc_row < NS * CG && sc_s < p_valid) cp_async16(slot + S::kCodes + lane * 16, sc_src);
        if (ASYM && lane < NS * CG && z_s < p_valid) cp_async16(slot + S::kCodes + S::kScales + lane * 16, z_src);
        cp_async_arrive(bar);
        --p_left;
        p_slot = p_slot + 1 == ST ? 0 : p_slot + 1;
        if (++p_ch == chunks) {
            // next super-strip: same warp, strips 8 NS further on, K back to 0
            p_ch = 0;
            p_t += kStreamWarps * NS;
            p_valid = valid_of(p_t);
            code_src += CG * w4::kGroupBytes + (kStreamWarps * NS - 1) * strip_bytes;
            sc_src += sc_step + kStreamWarps * NS * 32 - static_cast<size_t>(p.G) * p.N * 2;
            if (ASYM) z_src += z_step + kStreamWarps * NS * 16 - static_cast<size_t>(p.G) * p.N;
        } else {
            code_src += CG * w4::kGroupBytes;
            sc_src += sc_step;
            if (ASYM) z_src += z_step;
        }
    };
#pragma unroll 1
    for (int s = 0; s < ST; ++s) issue();
    W4S_TRACE();  // 2: first copies requested

    // The weight stream is under way; everything below touches the output and the split-K scratch, which
    // the kernel in front of a chained launch may still be using.
    pdl_wait();
    W4S_TRACE();  // 3: predecessor complete
    W4S_GRID(1);

    // ---- consumer ----
    float acc[NS][MT][NA][4];
#pragma unroll
    for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int a = 0; a < NA; ++a)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[s][mt][a][e] = 0.f;

    // Partial K segments this warp has added to the scratch: at most the first and the last of
    // its range. (first strip, chunks added); completed at the end of the kernel.
    int pend_t[2] = {0, 0}, pend_n[2] = {0, 0}, n_pend = 0;

    // Ends the K segment that began at chunk seg0 of the strips at t_first and ends before ch_end.
    auto flush = [&](int t_first, int seg0, int ch_end) {
        const int valid = valid_of(t_first);
        const bool whole_k = seg0 == 0 && ch_end == chunks;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            float v[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[mt][e] = NA == 2 ? acc[s][mt][0][e] + acc[s][mt][NA - 1][e] : acc[s][mt][0][e];
#pragma unroll
                    for (int a = 0; a < NA; ++a) acc[s][mt][a][e] = 0.f;
                }
            if (s >= valid) continue;
            const int t = t_first + s;
            if (whole_k) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) store_tile(p.C, v[mt], tok0 + 8 * mt, p.M, p.N, 16 * t, lane);
            } else {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int tok = tok0 + 8 * mt + 2 * c + (e & 1);
                        const int n = 16 * t + gl + 8 * (e >> 1);
                        if (tok < p.M) atomicAdd(p.partials + static_cast<size_t>(tok) * p.N + n, v[mt][e]);
                    }
            }
        }
        if (!whole_k && valid > 0) {
            pend_t[n_pend] = t_first;
            pend_n[n_pend] = ch_end - seg0;
            ++n_pend;
        }
    };

    int slot_i = 0, a_stage = 0, ch = ch0, seg0 = ch0;
    int t_first = (ss0 * kStreamWarps + warp) * NS, valid = valid_of(t_first);
    unsigned phase = 0, a_phase = 0;
    for (int left = n_chunks; left > 0; --left) {
        bool ok = mbar_wait(&a_landed[a_stage], a_phase, p.status);
        ok = __all_sync(0xffffffffu, ok && mbar_wait(&bars[slot_i], phase, p.status));
        if (!ok) {
            // Drain: give the copies already issued a bounded chance to land, then leave.
            for (int j = 1; j < ST; ++j) {
                const int sj = (slot_i + j) % ST;
                (void)mbar_wait(&bars[sj], sj > slot_i ? phase : phase ^ 1u, nullptr);
            }
            return;
        }
        W4S_TRACE();  // 4 + 2 chunk: chunk and activations are in
        const unsigned char* slot = ring + slot_i * S::kBytes;
        const unsigned char* acts = act_ring + a_stage * act_stage;
#pragma unroll
        for (int gi = 0; gi < CG; ++gi) {
            ActGroup act[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    act[mt].v[i] = *reinterpret_cast<const uint4*>(acts + act_off[mt] + gi * 256 + i * 64);
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                if (s < valid) {
                    const unsigned short* sc =
                        reinterpret_cast<const unsigned short*>(slot + S::kCodes + (s * CG + gi) * 32);
                    const uint32_t s_lo = w4::splat16(sc[gl]), s_hi = w4::splat16(sc[gl + 8]);
                    uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
                    if (ASYM) {
                        const unsigned char* zp = slot + S::kCodes + S::kScales + (s * CG + gi) * 16;
                        o_lo = w4::offset_pair(zp[gl]);
                        o_hi = w4::offset_pair(zp[gl + 8]);
                    }
                    const uint4* codes = reinterpret_cast<const uint4*>(slot + (s * CG + gi) * w4::kGroupBytes);
                    const uint4 q0 = codes[lane], q1 = codes[32 + lane];
                    unit_mma<MT, NA>(acc[s], q0, 0, o_lo, o_hi, s_lo, s_hi, act);
                    unit_mma<MT, NA>(acc[s], q1, 1, o_lo, o_hi, s_lo, s_hi, act);
                }
            }
        }
        __syncwarp();  // every lane has consumed both slots before they are handed back
        if (lane == 0) mbar_arrive(&a_empty[a_stage]);
        issue();
        W4S_TRACE();  // 5 + 2 chunk: chunk consumed, next copy requested
        if (++slot_i == ST) {
            slot_i = 0;
            phase ^= 1u;
        }
        if (++a_stage == kActStages) {
            a_stage = 0;
            a_phase ^= 1u;
        }
        if (++ch == chunks || left == 1) {
            flush(t_first, seg0, ch);
            if (ch == chunks) {
                ch = 0;
                t_first += kStreamWarps * NS;
                valid = valid_of(t_first);
            }
            seg0 = ch;
        }
    }

    // ---- completion of the partial segments: one fence, then the per-strip counters ----
    W4S_TRACE();  // loop done (all flushes issued)
    W4S_GRID(2);
    if (n_pend == 0) return;
    __threadfence();
    __syncwarp();
    W4S_TRACE();  // fence done
    for (int i = 0; i < n_pend; ++i) {
        const int nv = valid_of(pend_t[i]);
        for (int s = 0; s < nv; ++s) {
            const int t = pend_t[i] + s;
            unsigned done = 0;
            unsigned* counter = p.counters + static_cast<size_t>(blockIdx.y) * p.T + t;
            if (lane == 0) done = atomicAdd(counter, static_cast<unsigned>(pend_n[i]));
            done = __shfl_sync(0xffffffffu, done, 0);
            if (done + static_cast<unsigned>(pend_n[i]) == static_cast<unsigned>(chunks)) {
                __threadfence();
                // every load first, so the tail costs one round trip and not MT * 4 of them
                float v[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int tok = tok0 + 8 * mt + 2 * c + (e & 1);
                        const int n = 16 * t + gl + 8 * (e >> 1);
                        v[mt][e] = tok < p.M ? __ldcg(p.partials + static_cast<size_t>(tok) * p.N + n) : 0.f;
                    }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int tok = tok0 + 8 * mt + 2 * c + (e & 1);
                        const int n = 16 * t + gl + 8 * (e >> 1);
                        if (tok < p.M) {
                            p.C[static_cast<size_t>(tok) * p.N + n] = __float2bfloat16_rn(v[mt][e]);
                            __stcg(p.partials + static_cast<size_t>(tok) * p.N + n, 0.f);
                        }
                    }
                if (lane == 0) *counter = 0u;
            }
        }
    }
    W4S_TRACE();  // completion done
    W4S_GRID(3);
}

#ifdef SPK_W4_TRACE
}  // namespace
}  // namespace spk
extern "C" __attribute__((visibility("default"))) int spk_debug_w4s_trace(unsigned long long* buf) {
    return cudaMemcpyToSymbol(spk::g_w4s_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : 2;
}
extern "C" __attribute__((visibility("default"))) int spk_debug_w4s_grid(unsigned long long* buf) {
    static unsigned zeros[1024] = {};
    if (cudaMemcpyToSymbol(spk::g_w4s_seq, zeros, sizeof(zeros)) != cudaSuccess) return 2;
    return cudaMemcpyToSymbol(spk::g_w4s_grid, &buf, sizeof(buf)) == cudaSuccess ? 0 : 2;
}
namespace spk {
namespace {
#endif

// ---- host side --------------------------------------------------------------------------------------

// Environment override for sweeps: SPK_W4_CFG="mt,ns,cg,st[,ctas_per_sm[,min_units]]" (0 = rule).
struct StreamTuning {
    int mt = 0, ns = 0, cg = 0, st = 0, ctas_per_sm = 0, min_units = 0;
};

constexpr int kDefaultCg = 4, kDefaultSt2 = 4;  // default chunk of the one- and two-tile shapes; slots of 2-group chunks

StreamTuning read_tuning() {
    StreamTuning t;
    const char* e = std::getenv("SPK_W4_CFG");
    if (e && *e) std::sscanf(e, "%d,%d,%d,%d,%d,%d", &t.mt, &t.ns, &t.cg, &t.st, &t.ctas_per_sm, &t.min_units);
    return t;
}

template <int MT, int NS, int CG, int ST, bool ASYM, bool DUAL>
int launch_stream_t(const StreamParams& base, bool whole, int ctas_per_sm_target, int min_chunks,
                    const DeviceState& dev, cudaStream_t stream) {
    StreamParams p = base;
    auto kernel = w4_stream_kernel<MT, NS, CG, ST, ASYM, DUAL>;
    constexpr int smem_max = stream_smem_bytes<MT, NS, CG, ST, ASYM>(8 * MT);
    if constexpr (smem_max > 227 * 1024) return fail(SPK_INVALID, "w4gemm: this stream kernel shape needs %d bytes of shared memory", smem_max);
    static bool configured[kMaxDevices] = {};
    if (!configured[dev.device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max));
        configured[dev.device] = true;
    }
    p.rows_max = std::min(p.M, 8 * MT);
    const int smem = stream_smem_bytes<MT, NS, CG, ST, ASYM>(p.rows_max);
    p.super_strips = cdiv(p.T, kStreamWarps * NS);
    const int chunks = p.G / CG;
    const int m_chunks = cdiv(p.M, 8 * MT);
    // Shared strips need the scratch: whole strips when it does not cover [M][N].
    if (static_cast<int64_t>(p.M) * p.N > kPartialFloats || static_cast<int64_t>(m_chunks) * p.T > kCounters)
        whole = true;
    p.whole = whole ? 1 : 0;
    static int occupancy[kMaxDevices][8 * MT + 1] = {};  // per device and activation-ring height
    int& occ = occupancy[dev.device][p.rows_max];
    if (occ == 0) {
        SPK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, kStreamThreads, smem));
        if (occ < 1) return fail(SPK_CUDA_ERROR, "w4gemm: stream kernel does not fit an SM (smem %d)", smem);
    }
    int per_sm = occ;
    if (ctas_per_sm_target > 0) per_sm = std::min(per_sm, ctas_per_sm_target);
    // Equal ranges over exactly the CTAs that are resident at once, but at least `min_chunks`
    // chunks each; token chunks beyond the first share the slots.
    const long long slots = std::max<long long>(1, static_cast<long long>(dev.sm_count) * per_sm / m_chunks);
    const long long total = static_cast<long long>(p.super_strips) * chunks;
    const long long want = whole ? p.super_strips : std::max<long long>(1, total / std::max(1, min_chunks));
    const dim3 grid(static_cast<unsigned>(std::min(want, slots)), static_cast<unsigned>(m_chunks));
    SPK_CUDA(launch_chained(kernel, grid, dim3(kStreamThreads), smem, stream, p));
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

// Block shapes (Llama-3-8B projections, CUDA-graph chained launches on B200):
//   M <= 8   one token tile, one strip per warp
//   M <= 16  two token tiles
//   M <= 32 / 64  four / eight token tiles on 2-group chunks (registers); these two are the
//            warp-level-MMA fallback for shapes the tcgen05 path does not take
// SPK_W4_CFG="mt,ns,cg,st[,ctas_per_sm[,min_chunks]]" overrides the rule for sweeps (0 = rule);
// only the shapes instantiated below exist.
template <bool ASYM>
int launch_stream(const StreamParams& p, bool whole, const DeviceState& dev, cudaStream_t stream) {
    static const StreamTuning tune = read_tuning();
    int mt = p.M <= 8 ? 1 : p.M <= 16 ? 2 : p.M <= 32 ? 4 : 8;
    int ns = 1, cg = mt <= 2 ? kDefaultCg : 2;
    if (tune.mt > 0 && (p.M <= 8 * tune.mt || tune.mt == 8)) mt = tune.mt;
    if (tune.ns > 0) ns = tune.ns;
    if (tune.cg > 0) cg = tune.cg;
    if (mt >= 4) ns = 1, cg = std::min(cg, 2);
    while (cg > 1 && p.G % cg != 0) cg >>= 1;  // a chunk must not straddle a strip
    int st = tune.st > 0 ? tune.st : (cg == 4 ? 3 : cg == 2 ? (mt <= 2 ? kDefaultSt2 : 4) : 8);
    const bool dual = !whole && mt * ns <= 2;  // variant 3 keeps one accumulation chain for every M
    const int cap = tune.ctas_per_sm, min_chunks = tune.min_units > 0 ? tune.min_units : 1;
#define SPK_W4_CASE(MT_, NS_, CG_, ST_)                                                                       \
    if (mt == MT_ && ns == NS_ && cg == CG_ && st == ST_) {                                                   \
        if (dual) return launch_stream_t<MT_, NS_, CG_, ST_, ASYM, (MT_ * NS_ <= 2)>(p, whole, cap, min_chunks, dev, stream); \
        return launch_stream_t<MT_, NS_, CG_, ST_, ASYM, false>(p, whole, cap, min_chunks, dev, stream);      \
    }
    SPK_W4_CASE(1, 1, 1, 8)
    SPK_W4_CASE(1, 1, 2, 3)
    SPK_W4_CASE(1, 1, 2, 4)
    SPK_W4_CASE(1, 1, 4, 2)
    SPK_W4_CASE(1, 1, 4, 3)
    SPK_W4_CASE(1, 1, 4, 4)
    SPK_W4_CASE(1, 2, 2, 2)
    SPK_W4_CASE(2, 1, 1, 8)
    SPK_W4_CASE(2, 1, 2, 3)
    SPK_W4_CASE(2, 1, 2, 4)
    SPK_W4_CASE(2, 1, 4, 2)
    SPK_W4_CASE(2, 1, 4, 3)
    SPK_W4_CASE(2, 2, 2, 2)
    SPK_W4_CASE(4, 1, 1, 8)
    SPK_W4_CASE(4, 1, 2, 4)
    SPK_W4_CASE(8, 1, 1, 8)
    SPK_W4_CASE(8, 1, 2, 4)
#undef SPK_W4_CASE
    return fail(SPK_INVALID, "w4gemm: no stream kernel for mt=%d ns=%d cg=%d st=%d", mt, ns, cg, st);
}

}  // namespace
}  // namespace spk

namespace spk {
// defined in w4gemm_tmem.cu
int w4gemm_tmem_try(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                    int K, cudaStream_t stream, bool* taken);
// defined in w4_prefill.cu
int w4gemm_prefill_try(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                       int K, cudaStream_t stream, bool* taken);
// defined in w4gemm_umma.cu
int w4gemm_umma_try(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                    int K, cudaStream_t stream, bool* taken);
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
        SPK_REQUIRE(M <= 65535, "w4gemm: variant 0 takes at most 65535 tokens, got %d", M);
        const dim3 grid(N / 16, M);
        w4_scalar_kernel<<<grid, 128, 0, stream>>>(a, reinterpret_cast<const uint4*>(packed), sc, zeros, c, M, N, K);
        SPK_CHECK_LAUNCH();
        return SPK_OK;
    }
    if (variant == 1) {
        DeviceState* dev = nullptr;
        if (int rc = device_state(&dev)) return rc;
        const dim3 grid(N / 16, cdiv(M, 32));
        SPK_REQUIRE(grid.y <= 65535, "w4gemm: variant 1 takes at most 2097120 tokens, got %d", M);
        const auto* codes = reinterpret_cast<const unsigned char*>(packed);
        if (zeros)
            w4_strip_kernel<true><<<grid, 128, 0, stream>>>(a, codes, sc, zeros, c, M, N, K, dev->status);
        else
            w4_strip_kernel<false><<<grid, 128, 0, stream>>>(a, codes, sc, zeros, c, M, N, K, dev->status);
        SPK_CHECK_LAUNCH();
        return SPK_OK;
    }
    if (variant == 2) {  // the tensor-core routes: dense bf16 GEMM on dequantized weights for many tokens, TMEM weights for few
        bool taken = false;
        const int rcp = w4gemm_prefill_try(A, packed, scales, zeros, C, M, N, K, stream, &taken);
        if (taken || rcp != SPK_OK) return rcp;
        const int rc0 = w4gemm_tmem_try(A, packed, scales, zeros, C, M, N, K, stream, &taken);
        if (taken || rc0 != SPK_OK) return rc0;
        const int rc = w4gemm_umma_try(A, packed, scales, zeros, C, M, N, K, stream, &taken);
        if (taken || rc != SPK_OK) return rc;
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

// ---- w4gemm without any allocation ---------------------------------------------------------------
//
// Some callers must not allocate device memory at all: a serving engine that has handed the whole
// HBM budget to its own pool (a cudaMalloc there fails or eats into the pool's headroom), a process
// that runs under a hard device-memory cap, and latency-critical loops that cannot afford the
// device-wide synchronisation cudaMalloc implies.
// spk_w4gemm_bf16 allocates its split-K scratch lazily through the per-device arena; this entry
// point runs the same stream kernel (variant 2) with the scratch in a fixed array that is part of
// the library image instead, so nothing is ever allocated or freed, here or in any routine it calls.
//
// The array is file-scope device memory: every GPU that loads the library holds its
// kNoAllocBytes (8 MiB + 8 KiB + 256 B) until the process exits. That size fixes the limits of this
// entry point: M <= 64, N <= 32768 (so M * N <= 2 Mi fp32 partials and N / 16 <= 2048 strip
// counters). Larger problems are refused with SPK_INVALID; use spk_w4gemm_bf16 for them.
//
// All calls on a device share the one array. A call clears the part it is going to use before its
// kernel runs (a memset on the same stream), because the array keeps whatever the previous call
// left; two calls that overlap on the GPU (different streams, no dependency) race on it and must
// be ordered by the caller.
//
// Errors on the device: a bounded wait that gives up inside this entry point's kernel records
// SPK_TIMEOUT in a status word that also lives in the fixed array. spk_device_status() does not see
// that word (it reads the arena's, and creating the arena allocates); spk_w4gemm_noalloc_status()
// reads and clears it without allocating anything. The per-call clearing leaves the status word
// alone, so a timeout stays visible until it is read.
namespace spk {
namespace {

constexpr int kNoAllocMaxM = 64;
constexpr int kNoAllocMaxN = 32768;
constexpr size_t kNoAllocPartialBytes = static_cast<size_t>(kNoAllocMaxM) * kNoAllocMaxN * sizeof(float);
constexpr size_t kNoAllocCounterBytes = (kNoAllocMaxN / 16) * sizeof(unsigned);
constexpr size_t kNoAllocStatusBytes = 256;
constexpr size_t kNoAllocBytes = kNoAllocPartialBytes + kNoAllocCounterBytes + kNoAllocStatusBytes;

// In host code this name is only a handle for the runtime, not a device address: the address is
// looked up once per device with cudaGetSymbolAddress and that pointer is what kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

struct NoAllocDevice {
    unsigned char* base = nullptr;  // device address of g_noalloc_scratch on this device
    int sm_count = 0;
};
NoAllocDevice g_noalloc[kMaxDevices];

// Set-up of the current device (first call on it): resolve the array's device address and read the
// SM count. No allocation; cudaGetSymbolAddress may initialise the context and load the module,
// which is why the first call on a device should happen before any stream capture.
int noalloc_device(int* dev_out, NoAllocDevice** out) {
    int dev = 0;
    SPK_CUDA(cudaGetDevice(&dev));
    SPK_REQUIRE(dev >= 0 && dev < kMaxDevices, "w4gemm_noalloc: device ordinal %d not supported (max %d)", dev, kMaxDevices);
    NoAllocDevice& d = g_noalloc[dev];
    if (d.base == nullptr) {
        int major = 0, sms = 0;
        SPK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return fail(SPK_UNSUPPORTED, "this library is built for sm_100a only (device %d is sm_%dx)", dev, major);
        SPK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        void* ptr = nullptr;
        SPK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        SPK_REQUIRE(ptr != nullptr, "w4gemm_noalloc: the scratch array has no device address");
        d.sm_count = sms;
        d.base = static_cast<unsigned char*>(ptr);
    }
    *dev_out = dev;
    *out = &d;
    return SPK_OK;
}

}  // namespace
}  // namespace spk

extern "C" int spk_w4gemm_bf16_noalloc(const void* A, const int32_t* packed, const void* scales,
                                       const uint8_t* zeros, void* C, int M, int N, int K, void* stream_) {
    using namespace spk;
    SPK_REQUIRE(M >= 1 && N > 0 && K > 0, "w4gemm_noalloc: M, N, K must be positive, got %d %d %d", M, N, K);
    SPK_REQUIRE(N % 16 == 0 && K % w4::kGroup == 0,
                "w4gemm_noalloc: needs N %% 16 == 0 and K %% 128 == 0, got N=%d K=%d", N, K);
    SPK_REQUIRE(M <= kNoAllocMaxM && N <= kNoAllocMaxN,
                "w4gemm_noalloc: M=%d N=%d exceed the fixed scratch of this entry point (M <= %d, N <= %d); "
                "use spk_w4gemm_bf16 for larger problems",
                M, N, kNoAllocMaxM, kNoAllocMaxN);
    SPK_REQUIRE(A && packed && scales && C, "w4gemm_noalloc: null pointer");
    SPK_REQUIRE(aligned16(A) && aligned16(packed) && aligned16(scales) && (!zeros || aligned16(zeros)),
                "w4gemm_noalloc: A, packed, scales and zeros must be 16-byte aligned");
    auto stream = static_cast<cudaStream_t>(stream_);
    int dev = 0;
    NoAllocDevice* nd = nullptr;
    if (int rc = noalloc_device(&dev, &nd)) return rc;

    // A local description of the device for the launcher: the fixed array instead of the arena.
    DeviceState state;
    state.device = dev;
    state.sm_count = nd->sm_count;
    state.partials = reinterpret_cast<float*>(nd->base);
    state.counters = reinterpret_cast<unsigned*>(nd->base + kNoAllocPartialBytes);
    state.status = reinterpret_cast<int*>(nd->base + kNoAllocPartialBytes + kNoAllocCounterBytes);
    state.ready = true;

    // The array keeps the last call's contents: clear what this call will accumulate into.
    SPK_CUDA(cudaMemsetAsync(state.partials, 0, static_cast<size_t>(M) * N * sizeof(float), stream));
    SPK_CUDA(cudaMemsetAsync(state.counters, 0, kNoAllocCounterBytes, stream));  // not the status word behind them

    StreamParams p{};
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.packed = reinterpret_cast<const unsigned char*>(packed);
    p.scales = static_cast<const unsigned char*>(scales);
    p.zeros = zeros;
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M;
    p.N = N;
    p.K = K;
    p.G = K / w4::kGroup;
    p.T = N / 16;
    p.partials = state.partials;
    p.counters = state.counters;
    p.status = state.status;
    return zeros ? launch_stream<true>(p, false, state, stream) : launch_stream<false>(p, false, state, stream);
}

// Reads the status word of the fixed array on the current device (SPK_OK, or SPK_TIMEOUT after a
// bounded wait of spk_w4gemm_bf16_noalloc's kernel gave up), waits for `stream`, and clears the word
// if it was set. Like the GEMM entry point it allocates nothing: the word is copied straight from
// the array's device address. A result produced by a call that timed out is incomplete; run it again.
extern "C" int spk_w4gemm_noalloc_status(void* stream_, int* code) {
    using namespace spk;
    SPK_REQUIRE(code != nullptr, "w4gemm_noalloc_status: null code");
    int dev = 0;
    NoAllocDevice* nd = nullptr;
    if (int rc = noalloc_device(&dev, &nd)) return rc;
    auto stream = static_cast<cudaStream_t>(stream_);
    int* word = reinterpret_cast<int*>(nd->base + kNoAllocPartialBytes + kNoAllocCounterBytes);
    int host = 0;
    SPK_CUDA(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, stream));
    SPK_CUDA(cudaStreamSynchronize(stream));
    if (host != 0) SPK_CUDA(cudaMemsetAsync(word, 0, sizeof(int), stream));
    *code = host;
    return SPK_OK;
}
