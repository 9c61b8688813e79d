// W4A16 GEMM on the tcgen05 tensor cores with the dequantized weights held in TENSOR MEMORY
// (operand A of tcgen05.mma read from TMEM), for M <= 64.
//
//   D[n][token] (TMEM, 128 x NT fp32)  +=  W^T[n][k] (TMEM, bf16)  *  A[token][k] (smem, bf16, K-major)
//
// Compared with staging the dequantized weights in shared memory this drops the 16-byte shared
// stores, their bank traffic and the generic->async proxy fence from the dequant warps (a
// tcgen05.st plus tcgen05.wait::st takes their place), and it frees 96 KiB of shared memory. TMEM
// also holds six 128-k groups of weights instead of three, so a dequant warp can take a whole
// 2-group chunk (one 2 KiB bulk copy, one barrier wait, one hand-off) per iteration.
//
// A dequant lane (g, c) of the packed layout holds, for columns g and g + 8 of its strip, the k
// quads 8c + 4(r & 1) + 32(r >> 1) + {0..3}, r = 0..3, of a 64-k unit. tcgen05.st.16x256b places
// lane (g, c)'s registers at rows g / g + 8 and 32-bit columns 2c, 2c + 1 of each 8-column block,
// i.e. block r (one K = 16 MMA step) position 4c + i holds k = 8c + 4(r & 1) + 32(r >> 1) + i.
// The activations are therefore put in the same order: a small kernel in front re-orders the
// 8-byte pieces of every 128-byte unit row into the per-device scratch (16 k-steps of a unit become
// 4 (r) x 4 (c) quads), tiled TMA loads bring the re-ordered rows in, and the tensor core contracts
// position against position. (Re-ordering inside the GEMM with 8-byte cp.async copies was measured:
// two producer warps became the bound above 24 tokens.)
//
// The two launches are chained programmatically (spk_common.cuh): the GEMM's CTAs become resident,
// set up and start streaming weights while the re-ordering kernel (and, SM by SM, the tail of the
// GEMM before it) is still running; only the activation producer, the MMA and the epilogue warps wait for it.
//
// One persistent CTA per SM owns a contiguous range of (128-column super-strip, 2-group chunk)
// units. Roles (23 warps):
//   warps 0-15  dequant: strip 2 (w % 4) + (w / 4) % 2 (its 16 TMEM lanes lie in the lane quarter
//               w % 4 that the warp may access), chunks of parity w / 8 (the warp's set) of the CTA's sequence
//   warps 16-19 epilogue (TMEM lane quarter w % 4): adds the two sets' accumulators of a K segment
//   warps 20-21 MMA, one per set: loop warp-wide, one elected lane issues the 16 tcgen05.mma of a chunk
//               of its set into the set's accumulator
//   warp 22     activation producer (one elected lane, four TMA loads per chunk)
// TMEM columns: accumulator (set s, buffer b) at (s * bufs + b) * NT (two buffers per set up to 32
// tokens, one at 64), weights at 128 + 128 cs + 64 sub + 32 h + 8 r for chunk stage cs (3), group sub,
// unit h, MMA step r. The activations of a chunk live in shared-memory stage cs as well, so one commit
// of the chunk's MMAs frees both.
#include <algorithm>

#include "spk_common.cuh"
#include "umma_sm100.cuh"
#include "w4_layout.cuh"

namespace spk {
namespace {

using ptx::bulk_g2s;
using ptx::mbar_arrive;
using ptx::mbar_arrive_expect_tx;
using ptx::mbar_init;
using ptx::mbar_test_wait;
using ptx::mbar_wait;

constexpr int kStrips = 8;        // 16-column strips per super-strip
constexpr int kChunkGroups = 2;   // groups per chunk
constexpr int kSets = 2;          // dequant warps per strip; set s takes chunks of parity s
constexpr int DW = kStrips * kSets;
constexpr int kChunkStages = 3;   // chunks of dequantized weights resident in TMEM
constexpr int kStageBars = kSets * kChunkStages;  // barrier sets of the chunk stages (see the kernel)
// Per-warp ring of one-chunk code pieces (2 KiB each): 2 slots per warp are 64 KiB per SM in flight, enough for the
// HBM rate; deeper rings were measured and change nothing (the kernel is not bound by the stream).
#ifndef SPK_TMEM_CODE_SLOTS
#define SPK_TMEM_CODE_SLOTS 2
#endif
constexpr int kCodeSlots = SPK_TMEM_CODE_SLOTS;
// One MMA warp per dequant set. The MMA issuer is a serial instruction stream in which every barrier wait, fence and
// commit costs 100-300 cycles (device-clock traces: ~2000 cycles per chunk with one issuer, which was the whole kernel's
// pace: removing the dequant arithmetic, the activation loads or the weight stream changed nothing). Two issuers on two
// schedulers, each with its own accumulator (summed by the epilogue), halve that, and the activations of a chunk share
// the chunk's stage barriers (one wait and one commit per chunk instead of three each).
constexpr int kEpilogueWarp0 = DW, kMmaWarp0 = DW + 4, kProducerWarp0 = DW + 4 + kSets;
constexpr int kThreadsT = (DW + 5 + kSets) * 32;
constexpr int kTmemColsT = 512;
constexpr int kWeightCol0 = 128;  // first TMEM column of the weight stages
// accumulators per set: double buffered where the 128 columns in front of the weights allow
template <int NT>
constexpr int acc_bufs() { return 2 * kSets * NT <= kWeightCol0 ? 2 : 1; }

// Development aid, compiled in only with -DSPK_W4_TRACE: device clock stamps of the roles of a few CTAs,
// written to a buffer set with spk_debug_w4_trace (layout [cta slot][warp][kTraceEvents]).
#ifdef SPK_W4_TRACE
constexpr int kTraceEvents = 256, kTraceCtas = 4;
__device__ unsigned long long* g_w4_trace = nullptr;
__device__ __forceinline__ void trace_stamp(int warp, int lane, int& n) {
    const int slot = blockIdx.x == 0 ? 0 : blockIdx.x == 1 ? 1 : blockIdx.x == gridDim.x / 2 ? 2 : blockIdx.x == gridDim.x - 1 ? 3 : -1;
    if (lane == 0 && slot >= 0 && g_w4_trace != nullptr && n < kTraceEvents)
        g_w4_trace[(static_cast<size_t>(slot) * 32 + warp) * kTraceEvents + n] = clock64();
    ++n;
}
#define W4_TRACE() trace_stamp(warp, lane, trace_n)
#else
#define W4_TRACE() ((void)0)
#endif

struct W4TmemParams {
    const unsigned char* packed;
    const unsigned char* scales;
    const unsigned char* zeros;
    __nv_bfloat16* C;
    int M, N, K, G, super_strips;
    float* partials;
    unsigned* counters;
    int* status;
    int swiglu;  // 1: the strips alternate gate / up columns and C is [M][N / 2] = silu(gate) * up
};

// The final sums of this lane's column n (TMEM lane = column) for tokens t0 .. t0 + TB - 1 -> C. Plain form: one bf16 per
// token. SwiGLU form (the weight was built with its 16-column strips alternating gate, up, gate, up, ...): lanes
// 0-15 of a warp hold 16 gate columns and lanes 16-31 the matching up columns, so one shuffle pairs them, and
// lanes 0-15 store silu(gate) * up, computed in fp32 from the unrounded sums, to column
// 64 * super-strip + 16 * quarter + lane of the half-width output.
template <int TB>
__device__ __forceinline__ void store_outputs(const W4TmemParams& p, const float (&v)[TB], int t0, int ss, int quarter, int lane) {
    if (!p.swiglu) {
        const int n = ss * 128 + quarter * 32 + lane;
#pragma unroll
        for (int t = 0; t < TB; ++t)
            if (t0 + t < p.M) p.C[static_cast<size_t>(t0 + t) * p.N + n] = __float2bfloat16_rn(v[t]);
        return;
    }
    const int half_n = p.N / 2, col = ss * 64 + quarter * 16 + (lane & 15);
    // (A form in which the upper half-warp takes half of the tokens through one exchange per token pair halves this
    // arithmetic and brought the fused launch from 36.5 to 35.0 us at 64 tokens, but the plain kernel, which shares
    // this kernel's register allocation and schedule, then ran 6 % slower at 64 tokens, 24.7 -> 26.2 us; making the
    // epilogue a template parameter or an out-of-line function was slower still. Not kept.)
    // Every lane computes (the upper half's results are unused): with the arithmetic under the `lane < 16` branch the
    // shuffle -> exp -> reciprocal chains ran one after another, ~100 cycles each, on this warp's tail.
    // Hardware exp2 / reciprocal: a few ulp of fp32, far below the bf16 rounding of the result.
    __nv_bfloat16 h[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) {
        const float up = __shfl_down_sync(0xffffffffu, v[t], 16), gate = v[t];
        h[t] = __float2bfloat16_rn(__fdividef(gate, 1.0f + __expf(-gate)) * up);
    }
    if (lane < 16) {
#pragma unroll
        for (int t = 0; t < TB; ++t)
            if (t0 + t < p.M) p.C[static_cast<size_t>(t0 + t) * half_n + col] = h[t];
    }
}

template <int NT, bool ASYM>
struct W4TmemSmem {
    static constexpr int kActBytes = 2 * NT * 128;  // one group: two 64-k units of NT token rows
    static constexpr int kCodeBytes = kChunkGroups * w4::kGroupBytes;
    static constexpr int kSlotBytes = kCodeBytes + kChunkGroups * 32 + (ASYM ? kChunkGroups * 16 : 0);
    static constexpr int kCodeRing = DW * kCodeSlots * kSlotBytes;
    static constexpr int kCodeArrivals = 1 + 2 * kChunkGroups + (ASYM ? kChunkGroups : 0);
    static constexpr int kBarriers = 1024;
    static constexpr int kActChunkBytes = kChunkGroups * kActBytes;  // a chunk's activations: one stage per TMEM chunk stage
    static constexpr int kTotal = 1024 + kChunkStages * kActChunkBytes + kCodeRing + kBarriers;
};

__device__ __forceinline__ void cp_async16_t(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_t(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(ptx::smem_u32(bar)) : "memory");
}

// 16 TMEM lanes x 32 columns: registers 4r..4r+3 of lane (g, c) go to rows g (first two) and
// g + 8 (last two), columns 8r + 2c and 8r + 2c + 1.
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Four fp32 additions to consecutive, 16-byte-aligned words of global memory in one reduction.
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem], bf16 operands, K = 16.
__device__ __forceinline__ void mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

// The order in which a CTA visits the chunks [f0, f1) of its range. A range is up to three pieces: the
// rest of the super-strip it starts in (a partial K segment), whole super-strips, and the beginning of
// the super-strip it ends in (partial again). Partial segments end in reductions into the scratch and a
// completion step whose latency is several round trips to L2; whole ones end in plain stores. The
// partial pieces are therefore visited FIRST, so their completion overlaps the streaming of the rest,
// and the last thing a CTA does is, whenever it owns a whole super-strip, a plain store.
struct Visit {
    int f0, h_end, t_start, lt, lh, n;
    __device__ Visit(int f0_, int f1, int chunks) : f0(f0_), n(f1 - f0_) {
        h_end = f0 % chunks == 0 ? f0 : min(f1, (f0 / chunks + 1) * chunks);
        t_start = f1 % chunks == 0 ? f1 : max(h_end, (f1 / chunks) * chunks);
        lt = f1 - t_start;
        lh = h_end - f0;
    }
    __device__ __forceinline__ int at(int i) const { return i < lt ? t_start + i : (i < lt + lh ? f0 + (i - lt) : h_end + (i - lt - lh)); }
    // the chunk visited i-th ends a K segment (the next one visited is not its successor in the same super-strip)
    __device__ __forceinline__ bool ends_segment(int i, int ch, int chunks) const {
        return ch == chunks - 1 || i == n - 1 || i == lt - 1 || i == lt + lh - 1;
    }
};

__device__ __forceinline__ uint64_t make_desc(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
// D[tmem] += A[tmem] * B[smem] (accumulating form: the predicate is a constant)
__device__ __forceinline__ void mma_f16_ta_acc(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc)
        : "memory");
}

template <int NT, bool ASYM>
__global__ void __launch_bounds__(kThreadsT, 1) w4_tmem_kernel(const __grid_constant__ CUtensorMap map_act, const W4TmemParams p) {
    using L = W4TmemSmem<NT, ASYM>;
    constexpr int kAccBufs = acc_bufs<NT>();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    unsigned char* acts = base;
    unsigned char* codes = acts + kChunkStages * L::kActChunkBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(codes + L::kCodeRing);
    // The barriers of the chunk visited i-th are those of index i % kStageBars (its stage is i % kChunkStages): with one
    // barrier per stage the two sets would each see only every other phase of it, and a parity test cannot tell
    // "phase k complete" from "phase k - 1 not yet complete" (a set that ran one chunk ahead of the other took stale
    // weights that way). Indexed by i % 6 every waiter sees consecutive phases of the barriers it waits on.
    uint64_t* act_full = bars;                            // [SB] TMA: the chunk's activations have landed
    uint64_t* a_ready = act_full + kStageBars;            // [SB] the 8 dequant warps of the chunk's set
    uint64_t* a_free = a_ready + kStageBars;              // [SB] MMA commit: TMEM stage and activation stage may be refilled
    uint64_t* acc_ready = a_free + kStageBars;            // [sets][bufs] MMA commit
    uint64_t* acc_free = acc_ready + kSets * kAccBufs;    // [sets][bufs] 4 epilogue warps
    uint64_t* code_bar = acc_free + kSets * kAccBufs;     // [DW][kCodeSlots]
    uint64_t* drain_bar = code_bar + DW * kCodeSlots;     // [sets] MMA commit on the error path only
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + kSets);

    pdl_release();  // a chained kernel behind this one may become resident as this grid's CTAs exit
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef SPK_W4_TRACE
    int trace_n = 0;
#endif
    W4_TRACE();  // 0: kernel entry
    const int chunks = p.G / kChunkGroups;  // chunks per super-strip
    const long long total = static_cast<long long>(p.super_strips) * chunks;
    const int f0 = static_cast<int>(blockIdx.x * total / gridDim.x);
    const int f1 = static_cast<int>((blockIdx.x + 1) * total / gridDim.x);
    const Visit visit(f0, f1, chunks);
    const int n_chunks = visit.n;

    // The dequant warps' code rings are requested before the rest of the set-up (TMEM allocation, the other barriers,
    // the block-wide barrier: ~2 us from kernel entry in device-clock traces of an isolated launch), so the first
    // round trip to HBM runs under it; a warp needs only its own ring barriers for that. (In a chain of launches
    // the set-up already overlaps the kernel in front and the change does not show.)
    const int strip = 2 * (warp & 3) + ((warp >> 2) & 1), set = warp >> 3;  // of a dequant warp
    unsigned char* ring = codes + warp * (kCodeSlots * L::kSlotBytes);
    uint64_t* my_bar = code_bar + warp * kCodeSlots;
    // next chunk to fetch: this warp takes the chunks visited set-th, (set + 2)-th, ...
    int pi = set, p_slot = 0, n_issued = 0;
    auto issue = [&]() {
        if (pi >= n_chunks) return;
        ++n_issued;
        const int f = visit.at(pi), ss = f / chunks, ch = f - ss * chunks;
        const int t = ss * kStrips + strip, g0 = ch * kChunkGroups;
        unsigned char* slot = ring + p_slot * L::kSlotBytes;
        uint64_t* bar = &my_bar[p_slot];
        if (lane == 0) {
            mbar_arrive_expect_tx(bar, L::kCodeBytes);
            bulk_g2s(slot, p.packed + (static_cast<size_t>(t) * p.G + g0) * w4::kGroupBytes, L::kCodeBytes, bar);
        } else if (lane <= 2 * kChunkGroups) {
            const int j = lane - 1;  // scale row j / 2 of the chunk, 16-byte half j % 2
            cp_async16_t(slot + L::kCodeBytes + j * 16,
                         p.scales + (static_cast<size_t>(g0 + (j >> 1)) * p.N + 16 * t) * 2 + (j & 1) * 16);
            cp_async_arrive_t(bar);
        } else if (ASYM && lane <= 3 * kChunkGroups) {
            const int j = lane - 1 - 2 * kChunkGroups;
            cp_async16_t(slot + L::kCodeBytes + kChunkGroups * 32 + j * 16, p.zeros + static_cast<size_t>(g0 + j) * p.N + 16 * t);
            cp_async_arrive_t(bar);
        }
        pi += kSets;
        p_slot = p_slot + 1 == kCodeSlots ? 0 : p_slot + 1;
    };

    // barrier set-up spread over lanes: every dequant warp its own code barriers, one epilogue warp the rest
    if (warp < DW) {
        if (lane < kCodeSlots) {
            mbar_init(&code_bar[warp * kCodeSlots + lane], L::kCodeArrivals);
            ptx::fence_mbar_init();
        }
        __syncwarp();
        for (int i = 0; i < kCodeSlots; ++i) issue();
    } else if (warp == kEpilogueWarp0) {
        if (lane < kStageBars) {
            mbar_init(&act_full[lane], 1);
            mbar_init(&a_ready[lane], kStrips);
            mbar_init(&a_free[lane], 1);
        }
        if (lane < kSets * kAccBufs) {
            mbar_init(&acc_ready[lane], 1);
            mbar_init(&acc_free[lane], 4);
        }
        if (lane < kSets) mbar_init(&drain_bar[lane], 1);
        ptx::fence_mbar_init();
        if (lane == 0) umma::prefetch_tensormap(&map_act);
    }
    if (warp == kMmaWarp0) umma::tmem_alloc(tmem_slot, kTmemColsT);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    W4_TRACE();  // 1: set-up done

    if (warp < DW) {
        // ================= dequant warps =================
        const int gl = lane >> 2;
        const uint32_t my_tmem = tmem_base + (static_cast<uint32_t>(16 * strip) << 16) + kWeightCol0;
        const int n_mine = n_chunks > set ? (n_chunks - set + 1) / 2 : 0;
        int slot_i = 0, cs = set, bi = set;  // chunk stage and barrier index of the chunks visited set-th, (set + 2)-th, ...
        unsigned code_ph = 0, bph = 0;
        // The waits of an iteration are probed early without blocking (mbarrier.test_wait: the next chunk's codes at
        // the end of the iteration before, the TMEM stage before the first group's arithmetic) and the blocking wait
        // runs only if the probe said no. Measured: no difference in time either way; kept because a warp that
        // finds its data there never enters the suspend path.
        bool ok = true, chained = false, codes_in = false;
        int it = 0;
        for (; it < n_mine && ok; ++it) {
            W4_TRACE();  // dequant 2 + 5 it: iteration start
            if (!codes_in) ok = __all_sync(0xffffffffu, mbar_wait(&my_bar[slot_i], code_ph, p.status));
            if (!ok) break;
            W4_TRACE();  // + 1: codes landed
            const bool reused = set + kSets * it >= kChunkStages;  // the stage was used before: wait for those MMAs
            uint64_t* free_bar = &a_free[bi >= kChunkStages ? bi - kChunkStages : bi + kChunkStages];
            const unsigned free_ph = bi >= kChunkStages ? bph : bph ^ 1u;  // chunk j - 3: barrier (j - 3) % 6, phase (j - 3) / 6
            const bool free_early = reused ? mbar_test_wait(free_bar, free_ph) : true;
            const unsigned char* slot = ring + slot_i * L::kSlotBytes;
            const uint4* cw = reinterpret_cast<const uint4*>(slot);
#pragma unroll
            for (int sub = 0; sub < kChunkGroups; ++sub) {
                const unsigned short* sc = reinterpret_cast<const unsigned short*>(slot + L::kCodeBytes + sub * 32);
                const uint32_t s_lo = w4::splat16(sc[gl]), s_hi = w4::splat16(sc[gl + 8]);
                uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
                if (ASYM) {
                    const unsigned char* zp = slot + L::kCodeBytes + kChunkGroups * 32 + sub * 16;
                    o_lo = w4::offset_pair(zp[gl]);
                    o_hi = w4::offset_pair(zp[gl + 8]);
                }
                uint32_t x[2][4][4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 q = cw[(sub * 2 + h) * 32 + lane];
                    w4::dequant_word(q.x, o_lo, o_hi, s_lo, s_hi, x[h][0]);
                    w4::dequant_word(q.y, o_lo, o_hi, s_lo, s_hi, x[h][1]);
                    w4::dequant_word(q.z, o_lo, o_hi, s_lo, s_hi, x[h][2]);
                    w4::dequant_word(q.w, o_lo, o_hi, s_lo, s_hi, x[h][3]);
                }
                if (sub == 0) {  // the stage is free once the MMAs of three chunks ago have read it
                    // The first kChunkStages chunks find their stage fresh. From then on the wait depends on
                    // the MMA warp, which needs activations that exist only once the kernel in front of a
                    // chained launch has completed: wait for that first, so that the poll budget below
                    // measures this kernel's pipeline and not how long the predecessor still runs.
                    if (!chained && reused) {
                        pdl_wait();
                        chained = true;
                    }
                    W4_TRACE();  // + 2: first group dequantized
                    if (!__all_sync(0xffffffffu, free_early)) ok = __all_sync(0xffffffffu, mbar_wait(free_bar, free_ph, p.status));
                    if (!ok) break;
                    umma::fence_after_sync();
                    W4_TRACE();  // + 3: TMEM stage free
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t v[16];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        v[4 * r + 0] = x[h][r][0];
                        v[4 * r + 1] = x[h][r][2];
                        v[4 * r + 2] = x[h][r][1];
                        v[4 * r + 3] = x[h][r][3];
                    }
                    tmem_st_16x256b_x4(my_tmem + cs * 128 + sub * 64 + h * 32, v);
                }
            }
            if (!ok) break;
            __syncwarp();
            issue();
            if (++slot_i == kCodeSlots) slot_i = 0, code_ph ^= 1u;
            const bool next_codes = it + 1 < n_mine && mbar_test_wait(&my_bar[slot_i], code_ph);
            W4_TRACE();  // + 4: stores issued, next copy requested
            tmem_st_wait();
            umma::fence_before_sync();
            codes_in = __all_sync(0xffffffffu, next_codes);
            if (lane == 0) mbar_arrive(&a_ready[bi]);
            cs += kSets;
            if (cs >= kChunkStages) cs -= kChunkStages;
            bi += kSets;
            if (bi >= kStageBars) bi -= kStageBars, bph ^= 1u;
        }
        if (!ok) {
            // A wait gave up: let the code copies still in flight into this warp's ring land (bounded,
            // no status) before the CTA may exit and its shared memory be handed to another CTA.
            const int outstanding = n_issued - it;
            for (int j = 1; j < outstanding && j < kCodeSlots; ++j) {
                const int sj = slot_i + j < kCodeSlots ? slot_i + j : slot_i + j - kCodeSlots;
                (void)mbar_wait(&my_bar[sj], sj > slot_i ? code_ph : code_ph ^ 1u, nullptr);
            }
        }
    } else if (warp == kProducerWarp0) {
        // ================= activation producer: a chunk's groups go to the chunk's stage =================
        pdl_wait();  // the re-ordered activations are written by the kernel in front of this one
        int cs = 0, bi = 0;
        unsigned bph = 0;
        for (int i = 0; i < n_chunks; ++i) {
            const int ch = visit.at(i) % chunks;
            // the stage is free once the MMAs of three chunks ago have read it (the first three find it fresh)
            if (i >= kChunkStages &&
                !__all_sync(0xffffffffu, mbar_wait(&a_free[bi >= kChunkStages ? bi - kChunkStages : bi + kChunkStages],
                                                   bi >= kChunkStages ? bph : bph ^ 1u, p.status)))
                break;
            if (umma::elect_one()) {
                mbar_arrive_expect_tx(&act_full[bi], L::kActChunkBytes);
#pragma unroll
                for (int sub = 0; sub < kChunkGroups; ++sub) {
                    const int x = (ch * kChunkGroups + sub) * 256;  // byte offset of the group in a token row
                    unsigned char* dst = acts + cs * L::kActChunkBytes + sub * L::kActBytes;
                    umma::tma_load_2d(dst, &map_act, x, 0, &act_full[bi]);
                    umma::tma_load_2d(dst + NT * 128, &map_act, x + 128, 0, &act_full[bi]);
                }
            }
            __syncwarp();
            if (++cs == kChunkStages) cs = 0;
            if (++bi == kStageBars) bi = 0, bph ^= 1u;
        }
    } else if (warp >= kMmaWarp0) {
        // ================= MMA issuers: warp kMmaWarp0 + s takes the chunks of set s into accumulator s =================
        // The loop runs warp-wide, one elected lane issues. Descriptors are built once and advanced with 32-bit adds;
        // only the first MMA of this set's part of a K segment carries a run-time predicate.
        const int set = warp - kMmaWarp0;
        constexpr uint32_t idesc = umma::instr_desc(128, NT, 1, 1);  // bf16 x bf16 -> f32
        const uint64_t bdesc0 = umma::smem_desc_k128(acts);
        const uint32_t bd_lo0 = static_cast<uint32_t>(bdesc0), bd_hi = static_cast<uint32_t>(bdesc0 >> 32);
        int segn = 0, cs = set, bi = set;  // K segments this set has contributed to; stage i % 3 and barriers i % 6 of chunk i
        unsigned bph = 0;
        bool ok = true, fresh = true;
        // Everything this warp waits for needs the activations, which the producer requests only after the
        // kernel in front of a chained launch has completed; its bounded waits start counting from there.
        pdl_wait();
        for (int i = set; i < n_chunks && ok; i += kSets) {
            const int ch = visit.at(i) % chunks;
            const int buf = segn % kAccBufs;
            uint64_t* my_ready = &acc_ready[set * kAccBufs + buf];
            if (fresh) {
                ok = __all_sync(0xffffffffu, mbar_wait(&acc_free[set * kAccBufs + buf], ((segn / kAccBufs) & 1) ^ 1, p.status));
                if (!ok) break;
            }
            const uint32_t acc = tmem_base + (set * kAccBufs + buf) * NT;
            W4_TRACE();  // MMA 2 + 2 chunk: waiting for the chunk's weights and activations
            ok = __all_sync(0xffffffffu, mbar_wait(&a_ready[bi], bph, p.status) && mbar_wait(&act_full[bi], bph, p.status));
            if (!ok) break;
            W4_TRACE();  // + 1: both ready
            umma::fence_after_sync();
            // this set's last chunk of the segment: the segment ends here or with the other set's next chunk
            bool seg_end = visit.ends_segment(i, ch, chunks) || i + kSets >= n_chunks;
            if (!seg_end) seg_end = visit.ends_segment(i + 1, visit.at(i + 1) % chunks, chunks);
            if (umma::elect_one()) {
                const uint32_t bd = bd_lo0 + static_cast<uint32_t>(cs) * (L::kActChunkBytes >> 4);
                const uint32_t wa = tmem_base + kWeightCol0 + cs * 128;
                mma_f16_ta(acc, wa, make_desc(bd, bd_hi), idesc, !fresh);
#pragma unroll
                for (int j = 1; j < 8 * kChunkGroups; ++j) {  // group j / 8, MMA step j % 8 (unit (j / 4) % 2, step j % 4 of it)
                    const int sub = j >> 3, hr = j & 7;
                    mma_f16_ta_acc(acc, wa + sub * 64 + (hr >> 2) * 32 + (hr & 3) * 8,
                                   make_desc(bd + sub * (L::kActBytes >> 4) + (hr >> 2) * (NT * 128 >> 4) + 2 * (hr & 3), bd_hi), idesc);
                }
                umma::mma_commit(&a_free[bi]);
                if (seg_end) umma::mma_commit(my_ready);
            }
            __syncwarp();
            cs += kSets;
            if (cs >= kChunkStages) cs -= kChunkStages;
            bi += kSets;
            if (bi >= kStageBars) bi -= kStageBars, bph ^= 1u;
            fresh = seg_end;
            if (seg_end) ++segn;
        }
        if (!ok) {
            // MMAs already issued may still be reading TMEM and shared memory: one more commit, and a
            // bounded wait for it, before the CTA frees them.
            if (umma::elect_one()) umma::mma_commit(&drain_bar[set]);
            __syncwarp();
            (void)mbar_wait(&drain_bar[set], 0, nullptr);
        }
    } else {
        // ================= epilogue warps: TMEM lane quarter = warp % 4 =================
        const int quarter = warp & 3;
        pdl_wait();  // C and the split-K scratch may still be in use by the kernels in front
        int segn[kSets] = {}, seg_ch0 = -1, i0 = 0;  // segments each set has contributed to; first chunk of the open segment
        bool ok = true;
        for (int i = 0; i < n_chunks && ok; ++i) {
            const int f = visit.at(i), ss = f / chunks, ch = f - ss * chunks;
            if (seg_ch0 < 0) seg_ch0 = ch;
            if (!visit.ends_segment(i, ch, chunks)) continue;
            // The segment is the chunks visited i0 .. i; set s holds the partial sum of those of parity s (if any).
            W4_TRACE();  // epilogue 2 + 3 seg: waiting for a segment
            int slots[kSets], n_slots = 0;
#pragma unroll
            for (int s = 0; s < kSets; ++s) {
                const int mine = (i + 2 - s) / 2 - (i0 + 1 - s) / 2;  // chunks of parity s among i0 .. i
                if (mine == 0 || !ok) continue;
                const int slot = s * kAccBufs + segn[s] % kAccBufs;
                ok = __all_sync(0xffffffffu, mbar_wait(&acc_ready[slot], (segn[s] / kAccBufs) & 1, p.status));
                slots[n_slots++] = slot;
                ++segn[s];
            }
            if (!ok) break;
            i0 = i + 1;
            umma::fence_after_sync();
            W4_TRACE();  // + 1: accumulators ready
            const int n = ss * 128 + quarter * 32 + lane;  // TMEM lane = column of the super-strip
            const int seg_chunks = ch - seg_ch0 + 1;
            const bool whole = seg_chunks == chunks;
            // The scratch of this kernel is [32-column block][NT / 4][lane][4 tokens]: a lane's partial sums go
            // out as NT / 4 vector reductions and a warp's reduction covers 512 contiguous bytes (a scalar
            // reduction per token row cost ~100 cycles each here).
            float4* mine = reinterpret_cast<float4*>(p.partials) + static_cast<size_t>(n >> 5) * (NT / 4) * 32 + lane;
            constexpr int TB = NT < 32 ? NT : 32;  // tokens per pass: the sums of 64 tokens do not fit the registers
#pragma unroll
            for (int t0 = 0; t0 < NT; t0 += TB) {
                float v[TB];
#pragma unroll
                for (int k = 0; k < kSets; ++k) {
                    if (k >= n_slots) continue;
#pragma unroll
                    for (int c0 = 0; c0 < TB; c0 += 16) {
                        uint32_t r[16];
                        umma::tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + slots[k] * NT + t0 + c0, r);
                        umma::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[c0 + j] = k == 0 ? __uint_as_float(r[j]) : v[c0 + j] + __uint_as_float(r[j]);
                    }
                }
                if (t0 + TB == NT) {  // everything is in registers: the MMA warps may overwrite the accumulators
                    umma::fence_before_sync();
                    __syncwarp();
                    if (lane == 0)
                        for (int k = 0; k < n_slots; ++k) mbar_arrive(&acc_free[slots[k]]);
                }
                if (whole) {
                    store_outputs<TB>(p, v, t0, ss, quarter, lane);
                } else {
#pragma unroll
                    for (int t = 0; t < TB; t += 4)
                        if (t0 + t < p.M) red_add_v4(reinterpret_cast<float*>(mine + ((t0 + t) / 4) * 32), v[t], v[t + 1], v[t + 2], v[t + 3]);
                }
            }
            if (!whole) {
                // Completion right away (this warp has nothing else to do until the next segment ends): one fence,
                // then the per-(super-strip, quarter) counter; whoever brings it to `chunks` owns the sums.
                __threadfence();
                __syncwarp();
                unsigned done = 0;
                unsigned* counter = p.counters + ss * 4 + quarter;
                if (lane == 0) done = atomicAdd(counter, static_cast<unsigned>(seg_chunks));
                done = __shfl_sync(0xffffffffu, done, 0);
                if (done + static_cast<unsigned>(seg_chunks) == static_cast<unsigned>(chunks)) {
                    __threadfence();
                    // this lane's sums, TB tokens at a time: vector loads in one round trip, re-zero, store bf16
#pragma unroll
                    for (int t0 = 0; t0 < NT; t0 += TB) {
                        float4 w[TB / 4];
#pragma unroll
                        for (int j = 0; j < TB / 4; ++j) w[j] = t0 + 4 * j < p.M ? __ldcg(mine + (t0 / 4 + j) * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int j = 0; j < TB / 4; ++j)
                            if (t0 + 4 * j < p.M) __stcg(mine + (t0 / 4 + j) * 32, make_float4(0.f, 0.f, 0.f, 0.f));
                        float sums[TB];
#pragma unroll
                        for (int j = 0; j < TB / 4; ++j) sums[4 * j] = w[j].x, sums[4 * j + 1] = w[j].y, sums[4 * j + 2] = w[j].z, sums[4 * j + 3] = w[j].w;
                        store_outputs<TB>(p, sums, t0, ss, quarter, lane);
                    }
                    if (lane == 0) *counter = 0u;
                }
            }
            seg_ch0 = -1;
            W4_TRACE();  // + 2: stored or reduced and completed
        }
    }
    W4_TRACE();  // role finished
    umma::fence_before_sync();
    __syncthreads();
    W4_TRACE();  // CTA finished
    if (warp == kMmaWarp0) umma::tmem_dealloc(tmem_base, kTmemColsT);
}

// Re-orders the 8-byte pieces of every 128-byte unit row: destination piece 4 r + c (MMA step r,
// quad c) comes from source piece 8 (r >> 1) + 2 c + (r & 1). One thread per destination 16 bytes.
__global__ void __launch_bounds__(256)
w4_permute_acts_kernel(const uint2* __restrict__ src, uint4* __restrict__ dst, int chunks16) {
    pdl_release();  // the GEMM behind this kernel may start its set-up and weight stream now
    pdl_wait();     // the source may be the output of the kernel before; the scratch may still be read by it
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= chunks16) return;
    const int m = i & 7, unit = i >> 3;           // 16-byte chunk of the unit row; unit row index
    const int r = m >> 1, c = (m & 1) * 2;         // destination pieces 2m, 2m + 1 = (r, c), (r, c + 1)
    const uint2* u = src + static_cast<size_t>(unit) * 16 + 8 * (r >> 1) + 2 * c + (r & 1);
    const uint2 a = u[0], b = u[2];
    dst[i] = make_uint4(a.x, a.y, b.x, b.y);
}

template <int NT, bool ASYM>
int launch_w4_tmem(const void* A, W4TmemParams p, DeviceState* dev, cudaStream_t stream) {
    using L = W4TmemSmem<NT, ASYM>;
    static_assert(L::kTotal <= 227 * 1024, "w4 tmem kernel exceeds shared memory");
    static_assert(L::kSlotBytes % 16 == 0 && (NT * 128) % 1024 == 0, "slot alignment");
    static_assert(kSets * acc_bufs<NT>() * NT <= kWeightCol0 && kWeightCol0 + kChunkStages * 128 <= kTmemColsT, "TMEM column budget");
    const int chunks16 = p.M * (p.K / 8);
    SPK_CUDA(launch_chained(w4_permute_acts_kernel, dim3(cdiv(chunks16, 256)), dim3(256), 0, stream, static_cast<const uint2*>(A),
                            reinterpret_cast<uint4*>(dev->act_scratch), chunks16));
    CUtensorMap map_act;
    if (!umma::make_map_2d_u8(&map_act, dev->act_scratch, static_cast<uint64_t>(p.K) * 2, static_cast<uint64_t>(p.M), NT))
        return fail(SPK_CUDA_ERROR, "w4gemm: cuTensorMapEncodeTiled failed for M=%d K=%d", p.M, p.K);
    auto kernel = w4_tmem_kernel<NT, ASYM>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[dev->device] = true;
    }
    p.super_strips = p.N / 128;
    const long long total = static_cast<long long>(p.super_strips) * (p.G / kChunkGroups);
    const int grid = static_cast<int>(std::min<long long>(dev->sm_count, total));
    SPK_CUDA(launch_chained(kernel, dim3(grid), dim3(kThreadsT), L::kTotal, stream, map_act, p));
    return SPK_OK;
}

}  // namespace

// Takes M >= 16 (in passes of 64 tokens) with N a multiple of 128, an even number of groups, 16-byte-aligned activations
// and M * K within the activation scratch; at exactly 16 tokens only weights of 16 MiB and more (below
// that the stream kernel's smaller fixed cost wins: 4096 x 4096 13.0 us against 14.9 us). `taken` says
// whether it ran. Measured on B200, 28672 x 4096 weights, graph-timed, including the re-ordering
// launch: 16 tokens 32.7 us (stream kernel 37.0), 32 tokens 36.1 (shared-memory-operand kernel 45.7),
// 64 tokens 46.5 (53.0). SPK_W4_TMEM=0 turns the route off, SPK_W4_TMEM_MIN_M moves the lower bound.
int w4gemm_tmem_run(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N, int K,
                    cudaStream_t stream, bool* taken, int min_m, bool swiglu);

int w4gemm_tmem_try(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                    int K, cudaStream_t stream, bool* taken) {
    static const int min_m = [] {
        const char* e = std::getenv("SPK_W4_TMEM_MIN_M");
        return e && *e ? std::atoi(e) : 16;
    }();
    return w4gemm_tmem_run(A, packed, scales, zeros, C, M, N, K, stream, taken, min_m, false);
}

// The fused gate|up + SwiGLU form: N counts the interleaved gate and up columns (C is [M][N / 2]); every token count.
int w4gemm_tmem_swiglu(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                       int K, cudaStream_t stream, bool* taken) {
    return w4gemm_tmem_run(A, packed, scales, zeros, C, M, N, K, stream, taken, 1, true);
}

int w4gemm_tmem_run(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N, int K,
                    cudaStream_t stream, bool* taken, int min_m, bool swiglu) {
    *taken = false;
    static const int enabled = [] {
        const char* e = std::getenv("SPK_W4_TMEM");
        return e && *e ? std::atoi(e) : 1;
    }();
    if ((!enabled && !swiglu) || M < min_m || N % 128 != 0 || (K / w4::kGroup) % kChunkGroups != 0) return SPK_OK;
    if (!swiglu && M == 16 && min_m == 16 && static_cast<int64_t>(K) * N < (int64_t{1} << 25)) return SPK_OK;
    if (static_cast<int64_t>(64) * N > kPartialFloats || (N / 128) * 4 > kCounters) return SPK_OK;  // scratch is [N][NT]
    if (reinterpret_cast<uintptr_t>(A) % 16 != 0 || static_cast<int64_t>(std::min(M, 64)) * K * 2 > kActScratchBytes) return SPK_OK;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    *taken = true;
    // More than 64 tokens run as consecutive 64-token passes (each re-reads the weights): 42 us per pass
    // on 28672 x 4096 against 123 us per 64-token chunk of the stream kernel.
    for (int m0 = 0; m0 < M; m0 += 64) {
        const int mc = std::min(64, M - m0);
        W4TmemParams p{};
        p.packed = reinterpret_cast<const unsigned char*>(packed);
        p.scales = static_cast<const unsigned char*>(scales);
        p.zeros = zeros;
        p.C = static_cast<__nv_bfloat16*>(C) + static_cast<size_t>(m0) * (swiglu ? N / 2 : N);
        p.M = mc, p.N = N, p.K = K, p.G = K / w4::kGroup;
        p.swiglu = swiglu ? 1 : 0;
        p.partials = dev->partials, p.counters = dev->counters, p.status = dev->status;
        const void* a = static_cast<const __nv_bfloat16*>(A) + static_cast<size_t>(m0) * K;
        const int nt = mc <= 16 ? 16 : mc <= 32 ? 32 : 64;
        int rc;
        if (zeros)
            rc = nt == 16 ? launch_w4_tmem<16, true>(a, p, dev, stream)
                 : nt == 32 ? launch_w4_tmem<32, true>(a, p, dev, stream)
                            : launch_w4_tmem<64, true>(a, p, dev, stream);
        else
            rc = nt == 16 ? launch_w4_tmem<16, false>(a, p, dev, stream)
                 : nt == 32 ? launch_w4_tmem<32, false>(a, p, dev, stream)
                            : launch_w4_tmem<64, false>(a, p, dev, stream);
        if (rc != SPK_OK) return rc;
    }
    return SPK_OK;
}

#ifdef SPK_W4_TRACE
extern "C" __attribute__((visibility("default"))) int spk_debug_w4_trace(unsigned long long* buf) {
    return cudaMemcpyToSymbol(g_w4_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : 2;
}
#endif

}  // namespace spk
