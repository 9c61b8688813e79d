// W4A16 GEMM on the tcgen05 tensor cores for 16 < M <= 64 (the tensor-core route of variant 2).
//
// The warp-level MMA of the stream kernel runs out at M = 16..64: every extra 8 tokens cost one more
// legacy MMA and more activation reads per packed word, and the legacy tensor rate binds before
// HBM does. Here the dequantized weights become the 128-row operand of a tcgen05.mma whose other
// operand is the token tile, so the cost per weight no longer depends on M:
//
//   D[n][tok] (TMEM, 128 x NT fp32)  +=  W^T[n][k] (smem, bf16, K-major)  *  A[tok][k] (smem, bf16)
//
// One persistent CTA per SM owns a contiguous range of (128-column super-strip, 2-group chunk)
// units; every CTA gets the same number of chunks. Three rings, each as deep as its latency needs:
//   codes       per dequant warp, 3-4 slots of one group (1 KiB of codes + the group's scales / zeros
//               for the warp's strip), filled by a bulk copy plus 16-byte cp.async copies
//   activations CTA-wide, 4 slots of one group (2 units of NT tokens x 128 B, tiled TMA, 128-byte swizzle)
//   operand     CTA-wide, 3 slots of one 128-k group of dequantized bf16 weights (2 x 128 rows x 128 B)
// Roles:
//   warps 0-15  dequant: warp w streams strip w % 8 of the super-strip and takes group w / 8 of
//               every chunk, so two groups are always being dequantized side by side. A dequant
//               warp is a chain of latencies (shared loads, half-rate bf16x2 / logic pipes, shared
//               stores, the proxy fence); measured with 8 warps the chain, not a pipe, set the pace,
//               hence four of them per scheduler. Each dequantizes exactly (bf16((q - z) * s) per
//               weight) and writes its 16 rows of the operand slot in the 128-byte-swizzled K-major
//               layout the tensor core reads. Row r of a strip's 8-row swizzle group holds column
//               ((r & 3) << 1) | (r >> 2), which spreads a quarter-warp's 16-byte stores over all
//               banks; the epilogue undoes the permutation.
//   warp 16     activation producer (one thread)
//   warp 17     MMA: the loop runs warp-wide and one elected lane issues per group 2 x 4
//               tcgen05.mma.kind::f16 (128 x NT x 16); commits release the activation and operand slots; at the end of a K segment the accumulator is handed over
//   warps 18-21 epilogue: read the accumulator (double buffered in TMEM), then either store bf16
//               (segment = whole K) or add fp32 partials to the scratch; partial tiles are completed
//               at the end as in the stream kernel (one fence, per-quarter counters, last arriver
//               converts and re-zeroes, loads batched so the tail is one round trip per 16 rows)
// The k order inside a 64-k unit is the natural one on both operands: a lane's two words for
// k16 steps 2i, 2i+1 hold eight consecutive k of one column, i.e. one 16-byte chunk of the row.
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
using ptx::mbar_wait;

constexpr int kStrips = 8;      // 16-column strips per super-strip
constexpr int kChunkGroups = 2; // groups per chunk = dequant warps per strip
constexpr int DW = kStrips * kChunkGroups;  // dequant warps
constexpr int kStagesU = 3;     // operand slots (one 128-k group each)
constexpr int kProducerWarp = DW, kMmaWarp = DW + 1, kEpilogueWarp0 = DW + 2;
constexpr int kUnitBytes = 128 * 128;          // 128 columns x 64 k of bf16
constexpr int kOperandStage = 2 * kUnitBytes;  // one group
constexpr int kThreadsU = (DW + 6) * 32;
// arrivals that complete a code slot: the lane that posts the bulk copy, and one per cp.async lane
template <bool ASYM>
constexpr int kCodeArrivals = 1 + 2 + (ASYM ? 1 : 0);

struct W4UmmaParams {
    const unsigned char* packed;
    const unsigned char* scales;
    const unsigned char* zeros;
    __nv_bfloat16* C;
    int M, N, K, G, super_strips;
    float* partials;
    unsigned* counters;
    int* status;
};

template <int NT, bool ASYM>
struct W4UmmaSmem {
    static constexpr int kActStages = 4;            // one group (two 64-k units) per slot
    static constexpr int kActBytes = 2 * NT * 128;
    static constexpr int kCodeSlots = NT <= 32 ? 4 : 3;  // per-warp ring of one-group code pieces
    static constexpr int kCodeBytes = w4::kGroupBytes;
    static constexpr int kSlotBytes = kCodeBytes + 32 + (ASYM ? 16 : 0);
    static constexpr int kCodeRing = DW * kCodeSlots * kSlotBytes;
    static constexpr int kBarriers = 1024;
    static constexpr int kTotal = 1024 + kStagesU * kOperandStage + kActStages * kActBytes + kCodeRing + kBarriers;
    static constexpr int kTmemCols = 2 * NT < 32 ? 32 : 2 * NT;
};

__device__ __forceinline__ void cp_async16_u(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_u(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(ptx::smem_u32(bar)) : "memory");
}

template <int NT, bool ASYM>
__global__ void __launch_bounds__(kThreadsU, 1)
w4_umma_kernel(const __grid_constant__ CUtensorMap map_act, const W4UmmaParams p) {
    using L = W4UmmaSmem<NT, ASYM>;
    constexpr int AS = L::kActStages, kCodeSlots = L::kCodeSlots;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    unsigned char* operand = base;
    unsigned char* acts = operand + kStagesU * kOperandStage;
    unsigned char* codes = acts + AS * L::kActBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(codes + L::kCodeRing);
    uint64_t* act_full = bars;                 // [AS] TMA
    uint64_t* act_empty = act_full + AS;       // [AS] MMA commit
    uint64_t* a_ready = act_empty + AS;        // [S] the 8 dequant warps of the group's set
    uint64_t* a_free = a_ready + kStagesU;     // [S] MMA commit
    uint64_t* acc_ready = a_free + kStagesU;   // [2] MMA commit
    uint64_t* acc_free = acc_ready + 2;        // [2] 4 epilogue warps
    uint64_t* code_bar = acc_free + 2;         // [DW][kCodeSlots] 1 expect_tx arrive + the cp.async lanes' arrives
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(code_bar + DW * kCodeSlots);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = p.G / kChunkGroups;  // chunks per super-strip
    const long long total = static_cast<long long>(p.super_strips) * chunks;
    const int f0 = static_cast<int>(blockIdx.x * total / gridDim.x);
    const int f1 = static_cast<int>((blockIdx.x + 1) * total / gridDim.x);
    const int n_chunks = f1 - f0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < AS; ++s) {
            mbar_init(&act_full[s], 1);
            mbar_init(&act_empty[s], 1);
        }
        for (int s = 0; s < kStagesU; ++s) {
            mbar_init(&a_ready[s], kStrips);
            mbar_init(&a_free[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_ready[b], 1);
            mbar_init(&acc_free[b], 4);
        }
        for (int i = 0; i < DW * kCodeSlots; ++i) mbar_init(&code_bar[i], kCodeArrivals<ASYM>);
        ptx::fence_mbar_init();
        umma::prefetch_tensormap(&map_act);
    }
    if (warp == kMmaWarp) umma::tmem_alloc(tmem_slot, L::kTmemCols);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DW) {
        // ================= dequant warps =================
        const int gl = lane >> 2, c = lane & 3;
        const int strip = warp & (kStrips - 1), set = warp >> 3;  // set = which group of each chunk
        unsigned char* ring = codes + warp * (kCodeSlots * L::kSlotBytes);
        uint64_t* my_bar = code_bar + warp * kCodeSlots;
        // source of the next piece to fetch: codes of (strip t, group g), scales / zeros row g
        int pf = f0, p_slot = 0, p_ss = f0 / chunks, p_ch = f0 - p_ss * chunks;
        auto issue = [&]() {
            if (pf >= f1) return;
            const int t = p_ss * kStrips + strip, g = p_ch * kChunkGroups + set;
            unsigned char* slot = ring + p_slot * L::kSlotBytes;
            uint64_t* bar = &my_bar[p_slot];
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, L::kCodeBytes);
                bulk_g2s(slot, p.packed + (static_cast<size_t>(t) * p.G + g) * w4::kGroupBytes, L::kCodeBytes, bar);
            } else if (lane < 3) {
                cp_async16_u(slot + L::kCodeBytes + (lane - 1) * 16,
                             p.scales + (static_cast<size_t>(g) * p.N + 16 * t) * 2 + (lane - 1) * 16);
                cp_async_arrive_u(bar);
            } else if (ASYM && lane == 3) {
                cp_async16_u(slot + L::kCodeBytes + 32, p.zeros + static_cast<size_t>(g) * p.N + 16 * t);
                cp_async_arrive_u(bar);
            }
            ++pf;
            if (++p_ch == chunks) p_ch = 0, ++p_ss;
            p_slot = p_slot + 1 == kCodeSlots ? 0 : p_slot + 1;
        };
        for (int i = 0; i < kCodeSlots; ++i) issue();

        // This lane's rows of the operand tile: columns gl and gl + 8 of the strip sit in rows r8 and
        // r8 + 8 of the strip's 16, r8 = ((gl & 1) << 2) | (gl >> 1); both swizzle with r8. Chunk c of
        // a row holds k 8c..8c+7 of the unit, chunk 4 + c holds k 32+8c..
        const int r8 = ((gl & 1) << 2) | (gl >> 1);
        const uint32_t row_off = (16 * strip + r8) * 128;
        const uint32_t off_a = row_off + ((c ^ r8) << 4), off_b = row_off + (((4 + c) ^ r8) << 4);
        int slot_i = 0, s = set;  // this warp's groups are set, set + 2, ... of the CTA's sequence
        unsigned code_ph = 0, ph = 0;
        bool ok = true;
        for (int cidx = 0; cidx < n_chunks && ok; ++cidx) {
            ok = __all_sync(0xffffffffu, mbar_wait(&my_bar[slot_i], code_ph, p.status));
            if (!ok) break;
            const unsigned char* slot = ring + slot_i * L::kSlotBytes;
            const uint4* cw = reinterpret_cast<const uint4*>(slot);
            const unsigned short* sc = reinterpret_cast<const unsigned short*>(slot + L::kCodeBytes);
            const uint32_t s_lo = w4::splat16(sc[gl]), s_hi = w4::splat16(sc[gl + 8]);
            uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
            if (ASYM) {
                const unsigned char* zp = slot + L::kCodeBytes + 32;
                o_lo = w4::offset_pair(zp[gl]);
                o_hi = w4::offset_pair(zp[gl + 8]);
            }
            // dequantize both units of the group into registers, then hand the slot back
            uint32_t x[2][4][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q = cw[h * 32 + lane];
                w4::dequant_word(q.x, o_lo, o_hi, s_lo, s_hi, x[h][0]);
                w4::dequant_word(q.y, o_lo, o_hi, s_lo, s_hi, x[h][1]);
                w4::dequant_word(q.z, o_lo, o_hi, s_lo, s_hi, x[h][2]);
                w4::dequant_word(q.w, o_lo, o_hi, s_lo, s_hi, x[h][3]);
            }
            __syncwarp();
            issue();
            if (++slot_i == kCodeSlots) slot_i = 0, code_ph ^= 1u;

            ok = __all_sync(0xffffffffu, mbar_wait(&a_free[s], ph ^ 1u, p.status));
            if (!ok) break;
            unsigned char* op = operand + s * kOperandStage;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                unsigned char* u = op + h * kUnitBytes;
                *reinterpret_cast<uint4*>(u + off_a) = make_uint4(x[h][0][0], x[h][0][2], x[h][1][0], x[h][1][2]);
                *reinterpret_cast<uint4*>(u + off_b) = make_uint4(x[h][2][0], x[h][2][2], x[h][3][0], x[h][3][2]);
                *reinterpret_cast<uint4*>(u + off_a + 1024) = make_uint4(x[h][0][1], x[h][0][3], x[h][1][1], x[h][1][3]);
                *reinterpret_cast<uint4*>(u + off_b + 1024) = make_uint4(x[h][2][1], x[h][2][3], x[h][3][1], x[h][3][3]);
            }
            ptx::fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_ready[s]);
            s += kChunkGroups;
            if (s >= kStagesU) s -= kStagesU, ph ^= 1u;
        }
    } else if (warp == kProducerWarp) {
        // ================= activation producer: one 128-k group (two units) per slot =================
        if (lane == 0) {
            int s = 0, ch = f0 % chunks;
            unsigned ph = 0;
            bool ok = true;
            for (int f = f0; f < f1 && ok; ++f) {
                for (int sub = 0; sub < kChunkGroups && ok; ++sub) {
                    ok = mbar_wait(&act_empty[s], ph ^ 1u, p.status);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&act_full[s], L::kActBytes);
                    const int x = (ch * kChunkGroups + sub) * 256;  // byte offset of the group in a token row
                    umma::tma_load_2d(acts + s * L::kActBytes, &map_act, x, 0, &act_full[s]);
                    umma::tma_load_2d(acts + s * L::kActBytes + NT * 128, &map_act, x + 128, 0, &act_full[s]);
                    if (++s == AS) s = 0, ph ^= 1u;
                }
                if (++ch == chunks) ch = 0;
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer: the loop runs warp-wide, one elected lane issues =================
        constexpr uint32_t idesc = umma::instr_desc(128, NT, 1, 1);  // bf16 x bf16 -> f32
        const uint64_t adesc0 = umma::smem_desc_k128(operand), bdesc0 = umma::smem_desc_k128(acts);
        int seg = 0, s = 0, as = 0, ch = f0 % chunks;
        unsigned ph = 0, aph = 0;
        bool ok = true, fresh = true;
        for (int f = f0; f < f1 && ok; ++f) {
            const int buf = seg & 1;
            if (fresh) {
                ok = __all_sync(0xffffffffu, mbar_wait(&acc_free[buf], ((seg >> 1) & 1) ^ 1, p.status));
                if (!ok) break;
            }
            const uint32_t acc = tmem_base + buf * NT;
            for (int sub = 0; sub < kChunkGroups && ok; ++sub) {
                ok = __all_sync(0xffffffffu, mbar_wait(&a_ready[s], ph, p.status) && mbar_wait(&act_full[as], aph, p.status));
                if (!ok) break;
                umma::fence_after_sync();
                const uint64_t ad = adesc0 + static_cast<uint64_t>(s) * (kOperandStage >> 4);
                const uint64_t bd = bdesc0 + static_cast<uint64_t>(as) * (L::kActBytes >> 4);
                if (umma::elect_one()) {
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma::mma_f16(acc, ad + h * (kUnitBytes >> 4) + 2 * k, bd + h * (NT * 128 >> 4) + 2 * k, idesc,
                                          !fresh || h > 0 || k > 0);
                    umma::mma_commit(&act_empty[as]);
                    umma::mma_commit(&a_free[s]);
                }
                __syncwarp();
                fresh = false;
                if (++as == AS) as = 0, aph ^= 1u;
                if (++s == kStagesU) s = 0, ph ^= 1u;
            }
            if (ok && (ch == chunks - 1 || f == f1 - 1)) {  // end of this K segment
                if (umma::elect_one()) umma::mma_commit(&acc_ready[buf]);
                __syncwarp();
                ++seg;
                fresh = true;
            }
            if (++ch == chunks) ch = 0;
        }
    } else {
        // ================= epilogue warps: TMEM lane quarter = warp % 4 =================
        const int quarter = warp & 3;
        // TMEM lane 32 quarter + lane = operand row R: strip R / 16, swizzle-group row R & 7, upper half R & 8
        const int n_in_tile = 16 * (2 * quarter + (lane >> 4)) + (((lane & 3) << 1) | ((lane >> 2) & 1)) + (lane & 8);
        int pend_ss[2] = {0, 0}, pend_n[2] = {0, 0}, n_pend = 0;
        int seg = 0, seg_ch0 = f0 % chunks;
        bool ok = true;
        for (int f = f0; f < f1 && ok; ++f) {
            const int ss = f / chunks, ch = f - ss * chunks;
            if (!(ch == chunks - 1 || f == f1 - 1)) continue;
            const int buf = seg & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_ready[buf], (seg >> 1) & 1, p.status));
            if (!ok) break;
            umma::fence_after_sync();
            uint32_t v[NT];
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 16) {
                uint32_t r[16];
                umma::tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * NT + c0, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[c0 + i] = r[i];
            }
            umma::tmem_ld_wait();
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free[buf]);
            const int n = ss * 128 + n_in_tile;
            const bool whole_k = seg_ch0 == 0 && ch == chunks - 1;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (t < p.M) {
                    if (whole_k)
                        p.C[static_cast<size_t>(t) * p.N + n] = __float2bfloat16_rn(__uint_as_float(v[t]));
                    else
                        atomicAdd(p.partials + static_cast<size_t>(t) * p.N + n, __uint_as_float(v[t]));
                }
            }
            if (!whole_k) {
                pend_ss[n_pend] = ss;
                pend_n[n_pend] = ch - seg_ch0 + 1;
                ++n_pend;
            }
            ++seg;
            seg_ch0 = 0;
        }
        // completion of the partial segments: one fence, then the per-(tile, quarter) counters
        if (n_pend > 0) {
            __threadfence();
            __syncwarp();
            for (int i = 0; i < n_pend; ++i) {
                unsigned done = 0;
                unsigned* counter = p.counters + pend_ss[i] * 4 + quarter;
                if (lane == 0) done = atomicAdd(counter, static_cast<unsigned>(pend_n[i]));
                done = __shfl_sync(0xffffffffu, done, 0);
                if (done + static_cast<unsigned>(pend_n[i]) == static_cast<unsigned>(chunks)) {
                    __threadfence();
                    const int n = pend_ss[i] * 128 + n_in_tile;
                    for (int t0 = 0; t0 < p.M; t0 += 16) {  // all loads of a batch in flight together
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[j] = t0 + j < p.M ? __ldcg(p.partials + static_cast<size_t>(t0 + j) * p.N + n) : 0.f;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (t0 + j < p.M) {
                                p.C[static_cast<size_t>(t0 + j) * p.N + n] = __float2bfloat16_rn(v[j]);
                                __stcg(p.partials + static_cast<size_t>(t0 + j) * p.N + n, 0.f);
                            }
                    }
                    if (lane == 0) *counter = 0u;
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) umma::tmem_dealloc(tmem_base, L::kTmemCols);
}

template <int NT, bool ASYM>
int launch_w4_umma(const void* A, W4UmmaParams p, DeviceState* dev, cudaStream_t stream) {
    using L = W4UmmaSmem<NT, ASYM>;
    static_assert(L::kTotal <= 227 * 1024, "w4 umma kernel exceeds shared memory");
    static_assert(L::kSlotBytes % 16 == 0 && L::kActBytes % 1024 == 0, "slot alignment");
    CUtensorMap map_act;
    if (!umma::make_map_2d_u8(&map_act, A, static_cast<uint64_t>(p.K) * 2, static_cast<uint64_t>(p.M), NT))
        return fail(SPK_CUDA_ERROR, "w4gemm: cuTensorMapEncodeTiled failed for M=%d K=%d", p.M, p.K);
    auto kernel = w4_umma_kernel<NT, ASYM>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        configured[dev->device] = true;
    }
    p.super_strips = p.N / 128;
    const long long total = static_cast<long long>(p.super_strips) * (p.G / kChunkGroups);
    const int grid = static_cast<int>(std::min<long long>(dev->sm_count, total));
    kernel<<<grid, kThreadsU, L::kTotal, stream>>>(map_act, p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace

// Takes min_m <= M <= 64 with N a multiple of 128 and an even number of groups; `taken` says whether
// it ran. SPK_W4_UMMA_MIN_M moves the lower bound. Default 17, measured on B200 (28672 x 4096 weights):
// 16 tokens 37 us on the stream kernel against 43 us here, 32 tokens 69 against 45, 64 tokens 123 against 53.
int w4gemm_umma_try(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                    int K, cudaStream_t stream, bool* taken) {
    *taken = false;
    static const int min_m = [] {
        const char* e = std::getenv("SPK_W4_UMMA_MIN_M");
        return e && *e ? std::atoi(e) : 17;
    }();
    if (M < min_m || M > 64 || N % 128 != 0 || (K / w4::kGroup) % kChunkGroups != 0) return SPK_OK;
    if (static_cast<int64_t>(M) * N > kPartialFloats || (N / 128) * 4 > kCounters) return SPK_OK;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    W4UmmaParams p{};
    p.packed = reinterpret_cast<const unsigned char*>(packed);
    p.scales = static_cast<const unsigned char*>(scales);
    p.zeros = zeros;
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M, p.N = N, p.K = K, p.G = K / w4::kGroup;
    p.partials = dev->partials, p.counters = dev->counters, p.status = dev->status;
    *taken = true;
    const int nt = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    if (zeros)
        return nt == 16 ? launch_w4_umma<16, true>(A, p, dev, stream)
               : nt == 32 ? launch_w4_umma<32, true>(A, p, dev, stream)
                          : launch_w4_umma<64, true>(A, p, dev, stream);
    return nt == 16 ? launch_w4_umma<16, false>(A, p, dev, stream)
           : nt == 32 ? launch_w4_umma<32, false>(A, p, dev, stream)
                      : launch_w4_umma<64, false>(A, p, dev, stream);
}

}  // namespace spk
