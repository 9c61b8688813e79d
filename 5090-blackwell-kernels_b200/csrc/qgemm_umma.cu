// Tensor-core route of the fp8 and fp4 GEMMs: one TMA-fed tcgen05 kernel, accumulator in TMEM,
// in four operand modes
//   kFp8     e4m3 x e4m3, per-tensor scales              tcgen05.mma.kind::f8f6f4
//   kFp8Mx   e4m3 x e4m3, ue8m0 scale per 32 k           kind::mxf8f6f4.block_scale
//   kNvfp4   e2m1 x e2m1, e4m3 scale per 16 k            kind::mxf4nvf4.block_scale.scale_vec::4X
//   kMxfp4   e2m1 x e2m1, ue8m0 scale per 32 k           kind::mxf4nvf4.block_scale.scale_vec::2X
//   kBf16    bf16 x bf16 (the prefill route of the int4 GEMM: activations times dequantized weights)   kind::f16
//
// A persistent CTA computes 128 x BN tiles of C one after another. Roles, one warp each unless noted:
//   warp 0   producer: per K block (128 bytes of K per row) one thread issues two tiled TMA loads
//            (A 128 x 128 B, Bt BN x 128 B, 128-byte swizzle) and, in the block-scaled modes, bulk
//            copies of the 512-byte scale tiles (128 rows x 4 scales, the blocked layout of the
//            API, which is the layout the tensor core wants) into a ring of kStages stages
//   warp 1   MMA: allocates TMEM; one thread copies the stage's scale tiles shared -> TMEM
//            (tcgen05.cp), issues four MMAs (128 x BN x 32 bytes of K) and commits them to the
//            stage's "empty" barrier, and at the end to the "accumulator ready" barrier
//   warps 2-5  epilogue: each reads the 32 accumulator rows of its TMEM quarter (tcgen05.ld), applies
//            scale_a * scale_b in fp32, rounds once to bf16 and stores
// Rows past M, columns past N and k past K are zero-filled by TMA, so any shape the API accepts
// runs; the stores are predicated. Every barrier wait is bounded; on a timeout the roles stop,
// the status word is set, and TMEM is still released.
#include <algorithm>

#include "qgemm_simt.cuh"
#include "umma_sm100.cuh"

#ifndef UMMA_FP8_TWO_CTAS
#define UMMA_FP8_TWO_CTAS 1
#endif

namespace spk {
namespace {

using ptx::bulk_g2s;
using ptx::mbar_arrive_expect_tx;
using ptx::mbar_init;
using ptx::mbar_wait;

enum UmmaMode { kFp8 = 0, kFp8Mx = 1, kNvfp4 = 2, kMxfp4 = 3, kBf16 = 4 };

constexpr int kBM = 128, kBKBytes = 128;
constexpr int kSfTile = 512;             // 128 rows x 4 scale bytes
constexpr int kSfColsPerStage = 16 + 32;  // TMEM columns kept for one stage's scales (A: <= 16, B: <= 32)

// Tile order: groups of kTileGroup row tiles, inside a group the column tiles outermost. The A rows of
// a group (16 x 128 rows) stay in L2 while Bt streams through once per group; with the plain order
// (rows fastest over all of M) an 8192^3 problem read its 134 MB of operands 6 times from DRAM.
constexpr int kTileGroup = 16;
__device__ __forceinline__ void grouped_tile(int tiles_m, int tiles_n, int bid, int& tile_m, int& tile_n) {
    const int per_group = kTileGroup * tiles_n;
    const int first_m = (bid / per_group) * kTileGroup;
    const int rows = tiles_m - first_m < kTileGroup ? tiles_m - first_m : kTileGroup;
    const int r = bid % per_group;
    tile_m = first_m + r % rows;
    tile_n = r / rows;
}

template <int MODE>
struct ModeTraits {
    static constexpr bool kScaled = MODE != kFp8 && MODE != kBf16;
    // scale tiles per 128-row block per stage: MXFP8 1 (4 scales = 128 k), NVFP4 4 (one per MMA),
    // MXFP4 2 (one per two MMAs)
    static constexpr int kTiles = MODE == kFp8Mx ? 1 : MODE == kNvfp4 ? 4 : MODE == kMxfp4 ? 2 : 0;
    static constexpr int kElemsPerByte = (MODE == kNvfp4 || MODE == kMxfp4) ? 2 : 1;
    static constexpr int kBytesPerElem = MODE == kBf16 ? 2 : 1;  // K in elements -> bytes: K * kBytesPerElem / kElemsPerByte
};

template <int BN, int MODE>
struct UmmaCfg {
    using T = ModeTraits<MODE>;
    static constexpr int kABytes = kBM * kBKBytes, kBBytes = BN * kBKBytes;
    static constexpr int kSfABytes = T::kTiles * kSfTile, kSfBBytes = (BN / 128) * T::kTiles * kSfTile;
    static constexpr int kTxBytes = kABytes + kBBytes + kSfABytes + kSfBBytes;  // what lands per stage
    static constexpr int kStageBytes = (kTxBytes + 1023) / 1024 * 1024;           // stages keep the tile alignment
    // Per-tensor fp8 runs two CTAs per SM with two stages each: one CTA's epilogue (TMEM -> bf16
    // stores) and prologue then overlap the other's MMAs. The block-scaled modes need their TMEM
    // columns for scales and keep one CTA per SM with four stages.
    static constexpr int kCtasPerSm = ((MODE == kFp8 || MODE == kBf16) && UMMA_FP8_TWO_CTAS) ? 2 : 1;
    static constexpr int kStages = kCtasPerSm == 2 ? 2 : 4;
    static constexpr int kSmem = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr int kTmemCols = T::kScaled ? 512 : BN;
    static constexpr int kSfColBase = BN;  // scale columns follow the accumulator
};

struct UmmaParams {
    __nv_bfloat16* C;
    int M, N, K;  // K in elements
    const float* scale_a;
    const float* scale_b;
    const unsigned char* sfa;  // blocked layout (all block-scaled modes)
    const unsigned char* sfb;
    int sf_tiles_per_rowblock;  // 512-byte tiles per 128-row block (K / 128, K / 64, K / 128)
    int* status;
};

// Shared-memory descriptor of one 512-byte scale tile for tcgen05.cp: 32 rows of 16 bytes, no
// swizzle (8-row core matrices of 128 contiguous bytes, 128 bytes apart).
__device__ __forceinline__ uint64_t sf_desc(const void* tile) {
    const uint64_t addr = (ptx::smem_u32(tile) & 0x3FFFFu) >> 4;
    return addr | (uint64_t{128 >> 4} << 32) | (uint64_t{1} << 46);
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Block-scaled instruction descriptor: formats at [7,10) and [10,13), N >> 3 at [17,23), scale
// format (0 e4m3, 1 ue8m0) at bit 23, M >> 4 at [24,29), scale ids of B at [4,6) and of A at [29,31).
__host__ __device__ constexpr uint32_t instr_desc_scaled(int m, int n, int fmt, int scale_fmt, int sf_id) {
    return (static_cast<uint32_t>(sf_id) << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(scale_fmt) << 23) |
           (static_cast<uint32_t>(m >> 4) << 24) | (static_cast<uint32_t>(sf_id) << 29);
}

template <int MODE>
__device__ __forceinline__ void mma_scaled(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa,
                                           uint32_t tsfb, bool accumulate) {
    const uint32_t acc = accumulate;
    if (MODE == kFp8Mx)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(tmem_d),
                     "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(tsfa), "r"(tsfb)
                     : "memory");
    else if (MODE == kNvfp4)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(
                         tmem_d),
                     "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(tsfa), "r"(tsfb)
                     : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(
                         tmem_d),
                     "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(tsfa), "r"(tsfb)
                     : "memory");
}

template <int BN, int MODE>
__global__ void __launch_bounds__(192, UmmaCfg<BN, MODE>::kCtasPerSm)
qgemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const UmmaParams p) {
    using Cfg = UmmaCfg<BN, MODE>;
    using T = ModeTraits<MODE>;
    constexpr int NB = BN / 128;  // 128-row blocks of Bt per tile
    constexpr int kStages = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    // 128-byte-swizzled tiles must start on a 1024-byte boundary
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + kStages * Cfg::kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* acc_ready = empty + kStages;  // MMA commit: the tile's accumulator is complete
    uint64_t* acc_free = acc_ready + 1;     // the 4 epilogue warps have read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
    volatile uint32_t* mma_failed = tmem_slot + 1;  // set before the MMA warp releases the epilogue after a failed wait

    // Persistent: CTA b computes tiles b, b + gridDim.x, ... (grouped order). The stage ring runs on
    // across tiles, so the producer fills the next tile's first stages while the epilogue drains the
    // accumulator, and set-up (barriers, TMEM, tensor maps) is paid once per CTA.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + kBM - 1) / kBM, tiles_n = (p.N + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n;
    const int k_bytes = p.K * T::kBytesPerElem / T::kElemsPerByte;
    const int k_blocks = (k_bytes + kBKBytes - 1) / kBKBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        mbar_init(acc_free, 4);
        *mma_failed = 0u;
        ptx::fence_mbar_init();
        umma::prefetch_tensormap(&map_a);
        umma::prefetch_tensormap(&map_b);
    }
    if (warp == 1) umma::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            int tile_m, tile_n;
            grouped_tile(tiles_m, tiles_n, tile, tile_m, tile_n);
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                // a fresh barrier passes a wait on the opposite parity, so the first lap does not block
                ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, p.status));
                if (!ok) break;
                if (umma::elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::kTxBytes);
                    unsigned char* st = tiles + s * Cfg::kStageBytes;
                    umma::tma_load_2d(st, &map_a, kb * kBKBytes, tile_m * kBM, &full[s]);
                    umma::tma_load_2d(st + Cfg::kABytes, &map_b, kb * kBKBytes, tile_n * BN, &full[s]);
                    if (T::kScaled) {
                        unsigned char* sf = st + Cfg::kABytes + Cfg::kBBytes;
                        const size_t tile0 = static_cast<size_t>(kb) * T::kTiles;
                        bulk_g2s(sf, p.sfa + (static_cast<size_t>(tile_m) * p.sf_tiles_per_rowblock + tile0) * kSfTile,
                                 Cfg::kSfABytes, &full[s]);
#pragma unroll
                        for (int i = 0; i < NB; ++i)
                            bulk_g2s(sf + Cfg::kSfABytes + i * (T::kTiles * kSfTile),
                                     p.sfb + (static_cast<size_t>(tile_n * NB + i) * p.sf_tiles_per_rowblock + tile0) * kSfTile,
                                     T::kTiles * kSfTile, &full[s]);
                    }
                }
                __syncwarp();
                if (++s == kStages) s = 0, ph ^= 1u;
            }
        }
    } else if (warp == 1) {
        // The loop runs warp-wide so that stage indices and descriptors stay uniform; one elected lane
        // issues the tcgen05 instructions (always the same lane, so its commits cover its MMAs).
        bool ok = true;
        int s = 0, it = 0;
        unsigned ph = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            // the epilogue must have read the previous tile's accumulator
            ok = __all_sync(0xffffffffu, mbar_wait(acc_free, (it & 1) ^ 1, p.status));
            if (!ok) break;
            umma::fence_after_sync();
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, p.status));
                if (!ok) break;
                umma::fence_after_sync();
                if (umma::elect_one()) {
                    const unsigned char* st = tiles + s * Cfg::kStageBytes;
                    const uint64_t adesc = umma::smem_desc_k128(st), bdesc = umma::smem_desc_k128(st + Cfg::kABytes);
                    if (MODE == kBf16) {
                        constexpr uint32_t idesc = umma::instr_desc(kBM, BN, 1, 1);  // bf16 x bf16 -> f32, K = 16 per MMA
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma::mma_f16(tmem_acc, umma::desc_advance(adesc, 32 * k), umma::desc_advance(bdesc, 32 * k), idesc,
                                          kb > 0 || k > 0);
                    } else if (!T::kScaled) {
                        constexpr uint32_t idesc = umma::instr_desc(kBM, BN, 0, 0);  // e4m3 x e4m3 -> f32
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma::mma_f8f6f4(tmem_acc, umma::desc_advance(adesc, 32 * k), umma::desc_advance(bdesc, 32 * k), idesc,
                                             kb > 0 || k > 0);
                    } else {
                        // this stage's scale tiles, shared -> TMEM: A tile t at columns sfa + 4 t; Bt row block i of
                        // tile t at sfb + 4 (NB t + i), so the NB row blocks of one MMA sit side by side
                        const unsigned char* sf = st + Cfg::kABytes + Cfg::kBBytes;
                        const uint32_t sfa_col = tmem_acc + Cfg::kSfColBase + s * kSfColsPerStage, sfb_col = sfa_col + 16;
#pragma unroll
                        for (int t = 0; t < T::kTiles; ++t) {
                            tmem_cp_sf(sfa_col + 4 * t, sf_desc(sf + t * kSfTile));
#pragma unroll
                            for (int i = 0; i < NB; ++i)
                                tmem_cp_sf(sfb_col + 4 * (NB * t + i), sf_desc(sf + Cfg::kSfABytes + (i * T::kTiles + t) * kSfTile));
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // which scale tile and which bytes of its 32-bit words MMA k uses
                            const int t = MODE == kNvfp4 ? k : MODE == kMxfp4 ? (k >> 1) : 0;
                            const int sf_id = MODE == kNvfp4 ? 0 : MODE == kMxfp4 ? 2 * (k & 1) : k;
                            const uint32_t idesc = instr_desc_scaled(kBM, BN, MODE == kFp8Mx ? 0 : 1, MODE == kNvfp4 ? 0 : 1, sf_id);
                            mma_scaled<MODE>(tmem_acc, umma::desc_advance(adesc, 32 * k), umma::desc_advance(bdesc, 32 * k), idesc,
                                             sfa_col + 4 * t, sfb_col + 4 * NB * t, kb > 0 || k > 0);
                        }
                    }
                    umma::mma_commit(&empty[s]);  // the stage is free once these MMAs have read it
                    if (kb == k_blocks - 1) umma::mma_commit(acc_ready);  // the tile's accumulator is complete
                }
                __syncwarp();
                if (++s == kStages) s = 0, ph ^= 1u;
            }
        }
        if (!ok) {  // release the epilogue on a failed wait
            *mma_failed = 1u;
            __threadfence_block();
            if (umma::elect_one()) umma::mma_commit(acc_ready);
        }
        __syncwarp();
    } else {
        // ---- epilogue: warps 2..5 -> TMEM lane quarters 2, 3, 0, 1 ----
        const int quarter = warp & 3;
        const float s = (p.scale_a ? *p.scale_a : 1.0f) * (p.scale_b ? *p.scale_b : 1.0f);
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            int tile_m, tile_n;
            grouped_tile(tiles_m, tiles_n, tile, tile_m, tile_n);
            ok = __all_sync(0xffffffffu, mbar_wait(acc_ready, it & 1, p.status)) && *mma_failed == 0u;
            umma::fence_after_sync();
            if (!ok) break;
            const int row = tile_m * kBM + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                umma::tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, r);
                umma::tmem_ld_wait();
                if (c0 + 32 == BN) {  // every column has been read: the next tile may overwrite the accumulator
                    umma::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_free);
                }
                const int col = tile_n * BN + c0;
                if (row < p.M && col < p.N) {  // N % 64 == 0 and c0 % 32 == 0: a 32-column run is all in or all out
                    uint4 out[4];
                    uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * s, __uint_as_float(r[2 * j + 1]) * s);
                        o[j] = *reinterpret_cast<const uint32_t*>(&v);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.C + static_cast<size_t>(row) * p.N + col);
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = out[j];
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 1) umma::tmem_dealloc(tmem_acc, Cfg::kTmemCols);
}

template <int BN, int MODE>
int launch_umma(const simt::Params& q, const unsigned char* sfa, const unsigned char* sfb, DeviceState* dev,
                cudaStream_t stream) {
    using Cfg = UmmaCfg<BN, MODE>;
    using T = ModeTraits<MODE>;
    static_assert(Cfg::kStageBytes % 1024 == 0, "stages must keep the 1024-byte tile alignment");
    static_assert(Cfg::kSmem <= 227 * 1024, "stage ring exceeds shared memory");
    const uint64_t row_bytes = static_cast<uint64_t>(q.K) * T::kBytesPerElem / T::kElemsPerByte;
    CUtensorMap map_a, map_b;
    if (!umma::make_map_2d_u8(&map_a, q.A, row_bytes, static_cast<uint64_t>(q.M), kBM) ||
        !umma::make_map_2d_u8(&map_b, q.Bt, row_bytes, static_cast<uint64_t>(q.N), BN))
        return fail(SPK_CUDA_ERROR, "umma gemm: cuTensorMapEncodeTiled failed for %dx%dx%d", q.M, q.N, q.K);
    auto kernel = qgemm_umma_kernel<BN, MODE>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        configured[dev->device] = true;
    }
    UmmaParams p{};
    p.C = q.C, p.M = q.M, p.N = q.N, p.K = q.K;
    p.scale_a = q.scale_a, p.scale_b = q.scale_b;
    p.sfa = sfa, p.sfb = sfb;
    p.sf_tiles_per_rowblock = MODE == kNvfp4 ? q.K / 64 : q.K / 128;
    p.status = dev->status;
    const int grid = std::min(cdiv(q.M, kBM) * cdiv(q.N, BN), dev->sm_count * Cfg::kCtasPerSm);
    kernel<<<grid, 192, Cfg::kSmem, stream>>>(map_a, map_b, p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

// ---- decode shapes (M <= 64): weights as the 128-row operand, split-K ------------------------------
//
// D[n][m] (TMEM, 128 x NT fp32) += Bt[n][k] (smem) * A[m][k] (smem): the weight rows fill the 128
// lanes of the MMA and the few tokens are its N (16 / 32 / 64, rows past M zero-filled by TMA), so
// no tensor-core work is spent on padding tokens. The GEMM is a read-once stream of the weights:
// K is split over as many CTAs as fill the SMs once, every CTA keeps kDecodeStages stages of TMA
// loads in flight, and the partial tiles are summed in the fp32 scratch (atomics, per-(tile,
// quarter) counters, the last arriver converts and re-zeroes). The output is written transposed:
// a lane holds one n for all m, and for each m a warp stores 32 consecutive n.
constexpr int kDecodeStages = 6;

template <int NT, int MODE>
struct DecodeCfg {
    using T = ModeTraits<MODE>;
    static constexpr int kWBytes = kBM * kBKBytes, kXBytes = NT * kBKBytes;
    static constexpr int kSfBytes = T::kTiles * kSfTile;  // per operand
    static constexpr int kTxBytes = kWBytes + kXBytes + 2 * kSfBytes;
    static constexpr int kStageBytes = (kTxBytes + 1023) / 1024 * 1024;
    static constexpr int kSmem = kDecodeStages * kStageBytes + 1024 + 256;
    static constexpr int kSfColBase = 64, kSfColsPerStage = 32;  // weights' scales at +0, tokens' at +16
    static constexpr int kTmemCols = T::kScaled ? 256 : (NT < 32 ? 32 : NT);
    static_assert(!T::kScaled || kSfColBase + kDecodeStages * kSfColsPerStage <= 256, "TMEM columns");
};

struct DecodeParams {
    __nv_bfloat16* C;
    int M, N, K;  // K in elements
    const float* scale_a;
    const float* scale_b;
    const unsigned char* sfw;  // blocked scales of the weights (Bt) and of the tokens (A)
    const unsigned char* sfx;
    int sf_tiles_per_rowblock;
    int n_tiles, split;
    float* partials;
    unsigned* counters;
    int* status;
};

template <int NT, int MODE>
__global__ void __launch_bounds__(192, 1)
qgemm_umma_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const DecodeParams p) {
    using Cfg = DecodeCfg<NT, MODE>;
    using T = ModeTraits<MODE>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + kDecodeStages * Cfg::kStageBytes);
    uint64_t* empty = full + kDecodeStages;
    uint64_t* acc_ready = empty + kDecodeStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

    pdl_release();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x % p.n_tiles, sk = blockIdx.x / p.n_tiles;
    const int k_bytes = p.K * T::kBytesPerElem / T::kElemsPerByte;
    const int k_blocks_all = (k_bytes + kBKBytes - 1) / kBKBytes;
    const int kb0 = static_cast<int>(static_cast<long long>(sk) * k_blocks_all / p.split);
    const int kb1 = static_cast<int>(static_cast<long long>(sk + 1) * k_blocks_all / p.split);

    if (threadIdx.x < 2 * kDecodeStages) mbar_init(&full[threadIdx.x], 1);  // full[] and empty[] are contiguous
    if (threadIdx.x == 2 * kDecodeStages) {
        mbar_init(acc_ready, 1);
        umma::prefetch_tensormap(&map_w);
        umma::prefetch_tensormap(&map_x);
    }
    ptx::fence_mbar_init();
    if (warp == 1) umma::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        // The launch is chained: the weight tiles of the first stages are requested at once, everything a
        // kernel in front may still be writing (tokens, their scales, repacked MX scales) after pdl_wait().
        auto load_weights = [&](int kb, int s) {
            mbar_arrive_expect_tx(&full[s], Cfg::kTxBytes);
            umma::tma_load_2d(tiles + s * Cfg::kStageBytes, &map_w, kb * kBKBytes, tile_n * kBM, &full[s]);
        };
        auto load_rest = [&](int kb, int s) {
            unsigned char* st = tiles + s * Cfg::kStageBytes;
            umma::tma_load_2d(st + Cfg::kWBytes, &map_x, kb * kBKBytes, 0, &full[s]);
            if (T::kScaled) {
                unsigned char* sf = st + Cfg::kWBytes + Cfg::kXBytes;
                const size_t tile0 = static_cast<size_t>(kb) * T::kTiles;
                bulk_g2s(sf, p.sfw + (static_cast<size_t>(tile_n) * p.sf_tiles_per_rowblock + tile0) * kSfTile, Cfg::kSfBytes,
                         &full[s]);
                bulk_g2s(sf + Cfg::kSfBytes, p.sfx + tile0 * kSfTile, Cfg::kSfBytes, &full[s]);
            }
        };
        const int early = kb1 - kb0 < kDecodeStages ? kb1 - kb0 : kDecodeStages;
        if (umma::elect_one())
            for (int i = 0; i < early; ++i) load_weights(kb0 + i, i);
        __syncwarp();
        pdl_wait();
        if (umma::elect_one())
            for (int i = 0; i < early; ++i) load_rest(kb0 + i, i);
        __syncwarp();
        int s = early == kDecodeStages ? 0 : early;
        unsigned ph = early == kDecodeStages ? 1u : 0u;
        bool ok = true;
        for (int kb = kb0 + early; kb < kb1 && ok; ++kb) {
            ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, p.status));
            if (!ok) break;
            if (umma::elect_one()) {
                load_weights(kb, s);
                load_rest(kb, s);
            }
            __syncwarp();
            if (++s == kDecodeStages) s = 0, ph ^= 1u;
        }
    } else if (warp == 1) {
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        // a stage is complete only once the tokens are in, and those are requested after the kernel in front
        // of a chained launch has completed: the bounded waits below start counting from there
        pdl_wait();
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
            ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, p.status));
            if (!ok) break;
            umma::fence_after_sync();
            if (umma::elect_one()) {
                const unsigned char* st = tiles + s * Cfg::kStageBytes;
                const uint64_t wdesc = umma::smem_desc_k128(st), xdesc = umma::smem_desc_k128(st + Cfg::kWBytes);
                if (!T::kScaled) {
                    constexpr uint32_t idesc = umma::instr_desc(kBM, NT, 0, 0);  // e4m3 x e4m3 -> f32
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma::mma_f8f6f4(tmem_acc, umma::desc_advance(wdesc, 32 * k), umma::desc_advance(xdesc, 32 * k), idesc,
                                         kb > kb0 || k > 0);
                } else {
                    const unsigned char* sf = st + Cfg::kWBytes + Cfg::kXBytes;
                    const uint32_t sfw_col = tmem_acc + Cfg::kSfColBase + s * Cfg::kSfColsPerStage, sfx_col = sfw_col + 16;
#pragma unroll
                    for (int t = 0; t < T::kTiles; ++t) {
                        tmem_cp_sf(sfw_col + 4 * t, sf_desc(sf + t * kSfTile));
                        tmem_cp_sf(sfx_col + 4 * t, sf_desc(sf + Cfg::kSfBytes + t * kSfTile));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int t = MODE == kNvfp4 ? k : MODE == kMxfp4 ? (k >> 1) : 0;
                        const int sf_id = MODE == kNvfp4 ? 0 : MODE == kMxfp4 ? 2 * (k & 1) : k;
                        const uint32_t idesc = instr_desc_scaled(kBM, NT, MODE == kFp8Mx ? 0 : 1, MODE == kNvfp4 ? 0 : 1, sf_id);
                        mma_scaled<MODE>(tmem_acc, umma::desc_advance(wdesc, 32 * k), umma::desc_advance(xdesc, 32 * k), idesc,
                                         sfw_col + 4 * t, sfx_col + 4 * t, kb > kb0 || k > 0);
                    }
                }
                umma::mma_commit(&empty[s]);
            }
            __syncwarp();
            if (++s == kDecodeStages) s = 0, ph ^= 1u;
        }
        if (umma::elect_one()) umma::mma_commit(acc_ready);
        __syncwarp();
    } else {
        // ---- epilogue: warps 2..5 -> TMEM lane quarters 2, 3, 0, 1; lane = weight row n ----
        const int quarter = warp & 3;
        pdl_wait();  // C, the scale scalars and the split-K scratch may still be in use by the kernel in front
        const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_ready, 0, p.status));
        umma::fence_after_sync();
        if (ok && kb1 > kb0) {
            const float s = (p.scale_a ? *p.scale_a : 1.0f) * (p.scale_b ? *p.scale_b : 1.0f);
            const int n = tile_n * kBM + quarter * 32 + lane;
            uint32_t v[NT];
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 16) {
                uint32_t r[16];
                umma::tmem_ld_32x16(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[c0 + i] = r[i];
            }
            umma::tmem_ld_wait();
            if (p.split == 1) {
                if (n < p.N) {
#pragma unroll
                    for (int m = 0; m < NT; ++m)
                        if (m < p.M) p.C[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(__uint_as_float(v[m]) * s);
                }
            } else {
                // Split-K scratch laid out [32-column block][NT / 4][lane][4 tokens]: NT / 4 vector reductions per
                // lane, each warp-wide reduction 512 contiguous bytes (rows past M are exact zeros).
                float* mine = p.partials + (static_cast<size_t>(tile_n * 4 + quarter) * (NT / 4) * 32 + lane) * 4;
#pragma unroll
                for (int m = 0; m < NT; m += 4)
                    if (m < p.M)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mine + m * 32), "f"(__uint_as_float(v[m]) * s),
                                     "f"(__uint_as_float(v[m + 1]) * s), "f"(__uint_as_float(v[m + 2]) * s),
                                     "f"(__uint_as_float(v[m + 3]) * s)
                                     : "memory");
                __threadfence();
                __syncwarp();
                unsigned done = 0;
                unsigned* counter = p.counters + tile_n * 4 + quarter;
                if (lane == 0) done = atomicAdd(counter, 1u);
                done = __shfl_sync(0xffffffffu, done, 0);
                if (done + 1 == static_cast<unsigned>(p.split)) {
                    __threadfence();
                    float4* all = reinterpret_cast<float4*>(p.partials) + static_cast<size_t>(tile_n * 4 + quarter) * (NT / 4) * 32 + lane;
                    float4 w[NT / 4];
#pragma unroll
                    for (int j = 0; j < NT / 4; ++j) w[j] = 4 * j < p.M ? __ldcg(all + j * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < NT / 4; ++j)
                        if (4 * j < p.M) __stcg(all + j * 32, make_float4(0.f, 0.f, 0.f, 0.f));
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < NT / 4; ++j) {
                            const float e[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                if (4 * j + q < p.M) p.C[static_cast<size_t>(4 * j + q) * p.N + n] = __float2bfloat16_rn(e[q]);
                        }
                    }
                    if (lane == 0) *counter = 0u;
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 1) umma::tmem_dealloc(tmem_acc, Cfg::kTmemCols);
}

// sfw / sfx: blocked scales of Bt and A (null in the per-tensor mode); partials: M * N zeroed floats.
template <int NT, int MODE>
int launch_decode(const simt::Params& q, const unsigned char* sfw, const unsigned char* sfx, float* partials,
                  DeviceState* dev, cudaStream_t stream) {
    using Cfg = DecodeCfg<NT, MODE>;
    using T = ModeTraits<MODE>;
    static_assert(Cfg::kSmem <= 227 * 1024, "stage ring exceeds shared memory");
    const uint64_t row_bytes = static_cast<uint64_t>(q.K) * T::kBytesPerElem / T::kElemsPerByte;
    CUtensorMap map_w, map_x;
    if (!umma::make_map_2d_u8(&map_w, q.Bt, row_bytes, static_cast<uint64_t>(q.N), kBM) ||
        !umma::make_map_2d_u8(&map_x, q.A, row_bytes, static_cast<uint64_t>(q.M), NT))
        return fail(SPK_CUDA_ERROR, "umma decode gemm: cuTensorMapEncodeTiled failed for %dx%dx%d", q.M, q.N, q.K);
    auto kernel = qgemm_umma_decode_kernel<NT, MODE>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        configured[dev->device] = true;
    }
    DecodeParams p{};
    p.C = q.C, p.M = q.M, p.N = q.N, p.K = q.K;
    p.scale_a = q.scale_a, p.scale_b = q.scale_b;
    p.sfw = sfw, p.sfx = sfx;
    p.sf_tiles_per_rowblock = MODE == kNvfp4 ? q.K / 64 : q.K / 128;
    p.n_tiles = cdiv(q.N, kBM);
    const int k_blocks = cdiv(static_cast<int>(row_bytes), kBKBytes);
    // one wave of one CTA per SM: as many K slices as fit, at least two K blocks per slice. Two CTAs
    // per SM (SPK_QDECODE_CTAS_PER_SM=2) measured slower at N = 4096: 9 slices instead of 4 more than
    // double the partial-sum traffic and the completion tail (fp8 64 x 4096 x 14336: 24.9 us against 19.7).
    static const int per_sm = [] {
        const char* e = std::getenv("SPK_QDECODE_CTAS_PER_SM");
        return e && *e ? std::max(1, std::atoi(e)) : 1;
    }();
    p.split = std::max(1, std::min(per_sm * dev->sm_count / p.n_tiles, k_blocks / 2));
    p.partials = partials, p.counters = dev->counters, p.status = dev->status;
    SPK_CUDA(launch_chained(kernel, dim3(p.n_tiles * p.split), dim3(192), Cfg::kSmem, stream, map_w, map_x, p));
    return SPK_OK;
}

template <int MODE>
int launch_decode_nt(const simt::Params& q, const unsigned char* sfw, const unsigned char* sfx, float* partials,
                     DeviceState* dev, cudaStream_t stream) {
    if (q.M <= 16) return launch_decode<16, MODE>(q, sfw, sfx, partials, dev, stream);
    if (q.M <= 32) return launch_decode<32, MODE>(q, sfw, sfx, partials, dev, stream);
    return launch_decode<64, MODE>(q, sfw, sfx, partials, dev, stream);
}

bool decode_fits(const simt::Params& p, size_t scratch_bytes_before) {
    // split-K scratch: 128 columns x up to 64 token slots per tile
    return static_cast<int64_t>(cdiv(p.N, kBM)) * 128 * 64 + static_cast<int64_t>(scratch_bytes_before / 4) <= kPartialFloats &&
           cdiv(p.N, kBM) * 4 <= kCounters;
}

// ---- fp8 with fp32 block scales (1 x 128 of A, 128 x 128 of Bt) ------------------------------------
//
// The tensor core has no fp32 block scaling, so every 128-k block is contracted on its own into a
// TMEM buffer (4 MMAs of K = 32, the first one overwriting) and the epilogue warps fold it into fp32
// register accumulators with the block's two scales: acc += (sA[m][kb] * sB[n / 128][kb]) * block.
// Two TMEM buffers let the folding of block kb overlap the MMAs of block kb + 1. A folding thread
// owns one row of one 128-column half of the tile (one sB per block and half) and its 128 accumulators.
struct Block128Params {
    __nv_bfloat16* C;
    int M, N, K;
    const float* sA;  // [M][K / 128]
    const float* sB;  // [cdiv(N, 128)][K / 128]
    int* status;
};

constexpr int kBlkStages = 4;

template <int BN>
struct BlkCfg {
    static constexpr int kHalves = BN / 128;                 // 128-column halves of the tile = sB blocks per k-block
    static constexpr int kThreads = 64 + 128 * kHalves;      // producer, MMA, 4 epilogue warps per half
    static constexpr int kStageBytes = (kBM + BN) * kBKBytes;
    static constexpr int kSmem = kBlkStages * kStageBytes + 1024 + 256;
    static constexpr int kTmemCols = 2 * BN;                  // two buffers
};

// One CTA per 128 x BN tile, BN = 128 or 256. Epilogue warp e (0 .. 4 kHalves - 1) owns the 32 rows of
// TMEM lane quarter (e + 2) % 4 and the 128 columns of half e / 4: 128 fp32 accumulators per thread.
// (Packed f32x2 FMAs in the fold were tried and changed nothing: the fold waits on its four
// tcgen05.ld round trips per block, not on the FMA pipe.)
template <int BN>
__global__ void __launch_bounds__(BlkCfg<BN>::kThreads, 1)
qgemm_umma_block128_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const Block128Params p) {
    using Cfg = BlkCfg<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + kBlkStages * Cfg::kStageBytes);
    uint64_t* empty = full + kBlkStages;
    uint64_t* tfull = empty + kBlkStages;  // [2] MMA commit: a block's sum is complete in TMEM buffer b
    uint64_t* tfree = tfull + 2;           // [2] every epilogue warp has read buffer b
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfree + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int tile_m, tile_n;
    grouped_tile((p.M + kBM - 1) / kBM, (p.N + BN - 1) / BN, blockIdx.x, tile_m, tile_n);
    const int KB = p.K / 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kBlkStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tfree[b], 4 * Cfg::kHalves);
        }
        ptx::fence_mbar_init();
        umma::prefetch_tensormap(&map_a);
        umma::prefetch_tensormap(&map_b);
    }
    if (warp == 1) umma::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int kb = 0; kb < KB && ok; ++kb) {
            ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, p.status));
            if (!ok) break;
            if (umma::elect_one()) {
                mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
                unsigned char* st = tiles + s * Cfg::kStageBytes;
                umma::tma_load_2d(st, &map_a, kb * kBKBytes, tile_m * kBM, &full[s]);
                umma::tma_load_2d(st + kBM * kBKBytes, &map_b, kb * kBKBytes, tile_n * BN, &full[s]);
            }
            __syncwarp();
            if (++s == kBlkStages) s = 0, ph ^= 1u;
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = umma::instr_desc(kBM, BN, 0, 0);  // e4m3 x e4m3 -> f32
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int kb = 0; kb < KB && ok; ++kb) {
            const int buf = kb & 1;
            ok = __all_sync(0xffffffffu,
                            mbar_wait(&full[s], ph, p.status) && mbar_wait(&tfree[buf], ((kb >> 1) & 1) ^ 1, p.status));
            if (!ok) break;
            umma::fence_after_sync();
            if (umma::elect_one()) {
                const unsigned char* st = tiles + s * Cfg::kStageBytes;
                const uint64_t adesc = umma::smem_desc_k128(st), bdesc = umma::smem_desc_k128(st + kBM * kBKBytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma::mma_f8f6f4(tmem_acc + buf * BN, umma::desc_advance(adesc, 32 * k), umma::desc_advance(bdesc, 32 * k), idesc,
                                     k > 0);
                umma::mma_commit(&empty[s]);
                umma::mma_commit(&tfull[buf]);
            }
            __syncwarp();
            if (++s == kBlkStages) s = 0, ph ^= 1u;
        }
    } else {
        // ---- epilogue warps: TMEM lane quarter = warp % 4; a thread owns one row of one 128-column half ----
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = tile_m * kBM + quarter * 32 + lane;
        const int nb = tile_n * Cfg::kHalves + half;  // 128-column block of Bt
        const bool nb_ok = nb * 128 < p.N;
        const float* sa_row = p.sA + static_cast<size_t>(row < p.M ? row : 0) * KB;
        const float* sb_row = p.sB + static_cast<size_t>(nb_ok ? nb : 0) * KB;
        float acc[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) acc[i] = 0.f;
        bool ok = true;
        float f_next = KB > 0 ? __ldg(sa_row) * __ldg(sb_row) : 0.f;
        for (int kb = 0; kb < KB && ok; ++kb) {
            const int buf = kb & 1;
            const float f = f_next;
            if (kb + 1 < KB) f_next = __ldg(sa_row + kb + 1) * __ldg(sb_row + kb + 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&tfull[buf], (kb >> 1) & 1, p.status));
            if (!ok) break;
            umma::fence_after_sync();
            const uint32_t t0 = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + half * 128;
#pragma unroll
            for (int c0 = 0; c0 < 128; c0 += 32) {
                uint32_t r0[32];
                umma::tmem_ld_32x32(t0 + c0, r0);
                umma::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[c0 + i] = fmaf(__uint_as_float(r0[i]), f, acc[c0 + i]);
            }
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tfree[buf]);
        }
        if (ok && row < p.M && nb_ok) {
#pragma unroll
            for (int c0 = 0; c0 < 128; c0 += 32) {
                const int col = nb * 128 + c0;
                if (col < p.N) {  // N % 64 == 0: a 32-column run is all in or all out
                    uint4 out[4];
                    uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const __nv_bfloat162 v = __floats2bfloat162_rn(acc[c0 + 2 * j], acc[c0 + 2 * j + 1]);
                        o[j] = *reinterpret_cast<const uint32_t*>(&v);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.C + static_cast<size_t>(row) * p.N + col);
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = out[j];
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 1) umma::tmem_dealloc(tmem_acc, Cfg::kTmemCols);
}

template <int BN>
int launch_block128(const simt::Params& q, DeviceState* dev, cudaStream_t stream) {
    using Cfg = BlkCfg<BN>;
    static_assert(Cfg::kSmem <= 227 * 1024, "stage ring exceeds shared memory");
    CUtensorMap map_a, map_b;
    if (!umma::make_map_2d_u8(&map_a, q.A, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.M), kBM) ||
        !umma::make_map_2d_u8(&map_b, q.Bt, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.N), BN))
        return fail(SPK_CUDA_ERROR, "fp8gemm_block128: cuTensorMapEncodeTiled failed for %dx%dx%d", q.M, q.N, q.K);
    auto kernel = qgemm_umma_block128_kernel<BN>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        configured[dev->device] = true;
    }
    Block128Params p{};
    p.C = q.C, p.M = q.M, p.N = q.N, p.K = q.K;
    p.sA = q.blk_a, p.sB = q.blk_b;
    p.status = dev->status;
    kernel<<<cdiv(q.M, kBM) * cdiv(q.N, BN), Cfg::kThreads, Cfg::kSmem, stream>>>(map_a, map_b, p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

// Row-major ue8m0 scales [rows][K/32] (the fp8 MX API layout) -> the blocked layout the tensor core
// reads, rows padded to 128 with zero bytes. One thread per 4 scales (one 32-bit word).
__global__ void __launch_bounds__(256)
mx_scales_to_blocked_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, int rows, int cols,
                            long long words) {
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= words) return;
    const int wpr = cols / 4;
    const int r = static_cast<int>(i / wpr), jw = static_cast<int>(i % wpr);
    const unsigned v = r < rows ? *reinterpret_cast<const unsigned*>(src + static_cast<size_t>(r) * cols + 4 * jw) : 0u;
    *reinterpret_cast<unsigned*>(dst + fp::sf_offset(r, 4 * jw, cols)) = v;
}

bool umma_disabled() {
    const char* e = std::getenv("SPK_NO_UMMA");
    return e && *e == '1';
}

// 128 x 256 tiles when they fill the SMs once, 128 x 128 tiles otherwise (twice the CTAs on small problems).
bool wide_tiles(int M, int N, int sms) { return N % 256 == 0 && static_cast<long long>(cdiv(M, kBM)) * (N / 256) >= sms; }

}  // namespace

// Which tensor-core kernel variant 3 (and 2) of fp8gemm runs for a shape, or nullptr when the shape stays on
// the CUDA cores. One predicate for the launcher and for fp8gemm_v3_route_name.
const char* fp8gemm_umma_plan(int M, int N, int K, bool mx, int variant, bool c_aligned, int sms) {
    if (umma_disabled()) return nullptr;
    const bool decode = M <= 64;
    if (decode ? variant != 3 : !c_aligned) return nullptr;  // variant 2 keeps the reference's tile rule
    simt::Params p{};
    p.M = M, p.N = N, p.K = K;
    size_t sf_bytes = 0;
    if (mx) {
        const int cols = K / 32;
        sf_bytes = (static_cast<size_t>(cdiv(M, 128)) + cdiv(N, 128)) * 128 * cols;
        if (sf_bytes > static_cast<size_t>(kPartialFloats) * sizeof(float)) return nullptr;  // scratch too small
    }
    if (decode) return decode_fits(p, sf_bytes) ? "umma_decode_splitk" : nullptr;
    return wide_tiles(M, N, sms) ? "umma_128x256" : "umma_128x128";
}

// Variant 3 (and 2) of fp8gemm: every shape with M > 64 runs on the tensor cores as 128 x BN tiles, and
// variant 3 takes M <= 64 with the weights as the 128-row operand and K split over the SMs. In MX mode the
// row-major scales are first rewritten into the blocked layout inside the per-device scratch.
int fp8gemm_umma_try(const simt::Params& p, bool mx, int variant, cudaStream_t stream, bool* taken) {
    *taken = false;
    if (umma_disabled()) return SPK_OK;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    if (fp8gemm_umma_plan(p.M, p.N, p.K, mx, variant, aligned16(p.C), dev->sm_count) == nullptr) return SPK_OK;
    const bool decode = p.M <= 64;
    const bool wide = wide_tiles(p.M, p.N, dev->sm_count);
    *taken = true;
    if (!mx) {
        if (decode) return launch_decode_nt<kFp8>(p, nullptr, nullptr, dev->partials, dev, stream);
        return wide ? launch_umma<256, kFp8>(p, nullptr, nullptr, dev, stream) : launch_umma<128, kFp8>(p, nullptr, nullptr, dev, stream);
    }
    const int cols = p.K / 32;
    const size_t a_bytes = static_cast<size_t>(cdiv(p.M, 128)) * 128 * cols, b_bytes = static_cast<size_t>(cdiv(p.N, 128)) * 128 * cols;
    unsigned char* sfa = reinterpret_cast<unsigned char*>(dev->partials);
    unsigned char* sfb = sfa + a_bytes;
    const long long wa = static_cast<long long>(a_bytes / 4), wb = static_cast<long long>(b_bytes / 4);
    mx_scales_to_blocked_kernel<<<static_cast<unsigned>(cdiv64(wa, 256)), 256, 0, stream>>>(p.sfa, sfa, p.M, cols, wa);
    mx_scales_to_blocked_kernel<<<static_cast<unsigned>(cdiv64(wb, 256)), 256, 0, stream>>>(p.sfb, sfb, p.N, cols, wb);
    SPK_CHECK_LAUNCH();
    int rc;
    if (decode)  // the split-K partials live behind the repacked scales
        rc = launch_decode_nt<kFp8Mx>(p, sfb, sfa, dev->partials + (a_bytes + b_bytes) / 4, dev, stream);
    else
        rc = wide ? launch_umma<256, kFp8Mx>(p, sfa, sfb, dev, stream) : launch_umma<128, kFp8Mx>(p, sfa, sfb, dev, stream);
    if (rc != SPK_OK) return rc;
    // the scratch is shared with the split-K kernels, which expect it zeroed
    SPK_CUDA(cudaMemsetAsync(sfa, 0, a_bytes + b_bytes, stream));
    return SPK_OK;
}

// C bf16 [M][N] = A bf16 [M][K] * Bt bf16 [N][K]^T on the tile kernel (the second half of the int4 prefill route).
// Needs N % 64 == 0, K % 8 == 0 and 16-byte aligned operands and output.
int bf16gemm_umma(const void* A, const void* Bt, void* C, int M, int N, int K, cudaStream_t stream) {
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    simt::Params p{};
    p.A = static_cast<const unsigned char*>(A);
    p.Bt = static_cast<const unsigned char*>(Bt);
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M, p.N = N, p.K = K;
    return wide_tiles(M, N, dev->sm_count) ? launch_umma<256, kBf16>(p, nullptr, nullptr, dev, stream)
                                           : launch_umma<128, kBf16>(p, nullptr, nullptr, dev, stream);
}

// fp4gemm on the tensor cores: variants 1 and 2 at every M > 64 (TMA zero-fills the rows past M and the
// blocked scale layout is padded to 128 rows already, so ragged shapes need nothing special), and the
// split-K decode kernel for M <= 64 (reached through variant 1).
int fp4gemm_umma_try(const simt::Params& p, int format, cudaStream_t stream, bool* taken) {
    *taken = false;
    if (umma_disabled()) return SPK_OK;
    DeviceState* dev = nullptr;
    if (p.M <= 64) {
        if (!decode_fits(p, 0)) return SPK_OK;
        if (int rc = device_state(&dev)) return rc;
        *taken = true;
        return format == SPK_FP4_NVFP4 ? launch_decode_nt<kNvfp4>(p, p.sfb, p.sfa, dev->partials, dev, stream)
                                       : launch_decode_nt<kMxfp4>(p, p.sfb, p.sfa, dev->partials, dev, stream);
    }
    if (!aligned16(p.C)) return SPK_OK;
    if (int rc = device_state(&dev)) return rc;
    *taken = true;
    const bool wide = wide_tiles(p.M, p.N, dev->sm_count);
    if (format == SPK_FP4_NVFP4)
        return wide ? launch_umma<256, kNvfp4>(p, p.sfa, p.sfb, dev, stream) : launch_umma<128, kNvfp4>(p, p.sfa, p.sfb, dev, stream);
    return wide ? launch_umma<256, kMxfp4>(p, p.sfa, p.sfb, dev, stream) : launch_umma<128, kMxfp4>(p, p.sfa, p.sfb, dev, stream);
}

namespace {

// ---- fp32-block-scaled fp8 at decode shapes (M <= 64) -----------------------------------------------
//
// The decode arrangement (weights as the 128-row operand, K split over the SMs) with the per-block
// fold of the block-scaled kernel: one TMA stage is one 128-k block, its four MMAs overwrite one of
// two TMEM buffers, and the epilogue warps fold it into NT fp32 registers per thread,
// acc[m] += block[n][m] * sA[m][kb] * sB[n / 128][kb] (the tile is one 128-row block of Bt, so sB is
// one value per stage). The partial sums of the K slices then go through the scratch as above.
struct DecodeBlkParams {
    __nv_bfloat16* C;
    int M, N, K;
    const float* sA;  // [M][K / 128]
    const float* sB;  // [cdiv(N, 128)][K / 128]
    int n_tiles, split;
    float* partials;
    unsigned* counters;
    int* status;
};

template <int NT>
struct DecodeBlkCfg {
    static constexpr int kStageBytes = (kBM + NT) * kBKBytes;  // multiples of 1024 for NT = 16, 32, 64
    static constexpr int kSmem = kDecodeStages * kStageBytes + 1024 + 256;
    static constexpr int kTmemCols = 2 * NT < 32 ? 32 : 2 * NT;
};

template <int NT>
__global__ void __launch_bounds__(192, 1)
qgemm_umma_decode_block128_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                  const DecodeBlkParams p) {
    using Cfg = DecodeBlkCfg<NT>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + kDecodeStages * Cfg::kStageBytes);
    uint64_t* empty = full + kDecodeStages;
    uint64_t* tfull = empty + kDecodeStages;  // [2]
    uint64_t* tfree = tfull + 2;              // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfree + 2);

    pdl_release();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x % p.n_tiles, sk = blockIdx.x / p.n_tiles;
    const int KB = p.K / 128;
    const int kb0 = static_cast<int>(static_cast<long long>(sk) * KB / p.split);
    const int kb1 = static_cast<int>(static_cast<long long>(sk + 1) * KB / p.split);

    if (threadIdx.x < 2 * kDecodeStages) mbar_init(&full[threadIdx.x], 1);  // full[] and empty[] are contiguous
    if (threadIdx.x >= 32 && threadIdx.x < 34) {
        mbar_init(&tfull[threadIdx.x - 32], 1);
        mbar_init(&tfree[threadIdx.x - 32], 4);
    }
    if (threadIdx.x == 64) {
        umma::prefetch_tensormap(&map_w);
        umma::prefetch_tensormap(&map_x);
    }
    ptx::fence_mbar_init();
    if (warp == 1) umma::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        // weights first (the launch is chained), tokens after the kernel in front has completed
        auto load_weights = [&](int kb, int s) {
            mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
            umma::tma_load_2d(tiles + s * Cfg::kStageBytes, &map_w, kb * kBKBytes, tile_n * kBM, &full[s]);
        };
        auto load_tokens = [&](int kb, int s) {
            umma::tma_load_2d(tiles + s * Cfg::kStageBytes + kBM * kBKBytes, &map_x, kb * kBKBytes, 0, &full[s]);
        };
        const int early = kb1 - kb0 < kDecodeStages ? kb1 - kb0 : kDecodeStages;
        if (umma::elect_one())
            for (int i = 0; i < early; ++i) load_weights(kb0 + i, i);
        __syncwarp();
        pdl_wait();
        if (umma::elect_one())
            for (int i = 0; i < early; ++i) load_tokens(kb0 + i, i);
        __syncwarp();
        int s = early == kDecodeStages ? 0 : early;
        unsigned ph = early == kDecodeStages ? 1u : 0u;
        bool ok = true;
        for (int kb = kb0 + early; kb < kb1 && ok; ++kb) {
            ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, p.status));
            if (!ok) break;
            if (umma::elect_one()) {
                load_weights(kb, s);
                load_tokens(kb, s);
            }
            __syncwarp();
            if (++s == kDecodeStages) s = 0, ph ^= 1u;
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = umma::instr_desc(kBM, NT, 0, 0);  // e4m3 x e4m3 -> f32
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        pdl_wait();  // as in the plain decode kernel: count the bounded waits from the predecessor's completion
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
            const int i = kb - kb0, buf = i & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, p.status) && mbar_wait(&tfree[buf], ((i >> 1) & 1) ^ 1, p.status));
            if (!ok) break;
            umma::fence_after_sync();
            if (umma::elect_one()) {
                const unsigned char* st = tiles + s * Cfg::kStageBytes;
                const uint64_t wdesc = umma::smem_desc_k128(st), xdesc = umma::smem_desc_k128(st + kBM * kBKBytes);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma::mma_f8f6f4(tmem_acc + buf * NT, umma::desc_advance(wdesc, 32 * k), umma::desc_advance(xdesc, 32 * k), idesc, k > 0);
                umma::mma_commit(&empty[s]);
                umma::mma_commit(&tfull[buf]);
            }
            __syncwarp();
            if (++s == kDecodeStages) s = 0, ph ^= 1u;
        }
    } else {
        // ---- epilogue warps: lane = weight row n of the tile; fold every block with its scales ----
        const int quarter = warp & 3;
        pdl_wait();
        const int n = tile_n * kBM + quarter * 32 + lane;
        const float* sb_row = p.sB + static_cast<size_t>(tile_n) * KB;
        float acc[NT];
#pragma unroll
        for (int m = 0; m < NT; ++m) acc[m] = 0.f;
        bool ok = true;
        // Lane l fetches the block scales of tokens l and l + 32 one block ahead (two loads per lane and
        // block instead of NT broadcast loads); the fold gets token m's scale by shuffle.
        constexpr int kPer = NT > 32 ? 2 : 1;
        auto fetch = [&](int kb, float (&out)[kPer]) {
            const float fb = kb < kb1 ? __ldg(sb_row + kb) : 0.f;
#pragma unroll
            for (int h = 0; h < kPer; ++h) {
                const int m = lane + 32 * h;
                out[h] = (kb < kb1 && m < p.M) ? __ldg(p.sA + static_cast<size_t>(m) * KB + kb) * fb : 0.f;
            }
        };
        float nxt[kPer];
        fetch(kb0, nxt);
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
            const int i = kb - kb0, buf = i & 1;
            float cur[kPer];
#pragma unroll
            for (int h = 0; h < kPer; ++h) cur[h] = nxt[h];
            fetch(kb + 1, nxt);
            float fa[NT];
#pragma unroll
            for (int m = 0; m < NT; ++m) fa[m] = __shfl_sync(0xffffffffu, cur[m >> 5], m & 31);
            ok = __all_sync(0xffffffffu, mbar_wait(&tfull[buf], (i >> 1) & 1, p.status));
            if (!ok) break;
            umma::fence_after_sync();
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 16) {
                uint32_t r[16];
                umma::tmem_ld_32x16(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + buf * NT + c0, r);
                umma::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c0 + j] = fmaf(__uint_as_float(r[j]), fa[c0 + j], acc[c0 + j]);
            }
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tfree[buf]);
        }
        if (ok && kb1 > kb0) {
            if (p.split == 1) {
                if (n < p.N) {
#pragma unroll
                    for (int m = 0; m < NT; ++m)
                        if (m < p.M) p.C[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(acc[m]);
                }
            } else {
                float* mine = p.partials + (static_cast<size_t>(tile_n * 4 + quarter) * (NT / 4) * 32 + lane) * 4;
#pragma unroll
                for (int m = 0; m < NT; m += 4)
                    if (m < p.M)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mine + m * 32), "f"(acc[m]), "f"(acc[m + 1]),
                                     "f"(acc[m + 2]), "f"(acc[m + 3])
                                     : "memory");
                __threadfence();
                __syncwarp();
                unsigned done = 0;
                unsigned* counter = p.counters + tile_n * 4 + quarter;
                if (lane == 0) done = atomicAdd(counter, 1u);
                done = __shfl_sync(0xffffffffu, done, 0);
                if (done + 1 == static_cast<unsigned>(p.split)) {
                    __threadfence();
                    float4* all = reinterpret_cast<float4*>(p.partials) + static_cast<size_t>(tile_n * 4 + quarter) * (NT / 4) * 32 + lane;
                    float4 w[NT / 4];
#pragma unroll
                    for (int j = 0; j < NT / 4; ++j) w[j] = 4 * j < p.M ? __ldcg(all + j * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < NT / 4; ++j)
                        if (4 * j < p.M) __stcg(all + j * 32, make_float4(0.f, 0.f, 0.f, 0.f));
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < NT / 4; ++j) {
                            const float e[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                if (4 * j + q < p.M) p.C[static_cast<size_t>(4 * j + q) * p.N + n] = __float2bfloat16_rn(e[q]);
                        }
                    }
                    if (lane == 0) *counter = 0u;
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 1) umma::tmem_dealloc(tmem_acc, Cfg::kTmemCols);
}

template <int NT>
int launch_decode_block128(const simt::Params& q, DeviceState* dev, cudaStream_t stream) {
    using Cfg = DecodeBlkCfg<NT>;
    static_assert(Cfg::kStageBytes % 1024 == 0 && Cfg::kSmem <= 227 * 1024, "stage ring");
    CUtensorMap map_w, map_x;
    if (!umma::make_map_2d_u8(&map_w, q.Bt, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.N), kBM) ||
        !umma::make_map_2d_u8(&map_x, q.A, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.M), NT))
        return fail(SPK_CUDA_ERROR, "fp8gemm_block128: cuTensorMapEncodeTiled failed for %dx%dx%d", q.M, q.N, q.K);
    auto kernel = qgemm_umma_decode_block128_kernel<NT>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        configured[dev->device] = true;
    }
    DecodeBlkParams p{};
    p.C = q.C, p.M = q.M, p.N = q.N, p.K = q.K;
    p.sA = q.blk_a, p.sB = q.blk_b;
    p.n_tiles = cdiv(q.N, kBM);
    p.split = std::max(1, std::min(dev->sm_count / p.n_tiles, (q.K / 128) / 2));
    p.partials = dev->partials, p.counters = dev->counters, p.status = dev->status;
    SPK_CUDA(launch_chained(kernel, dim3(p.n_tiles * p.split), dim3(192), Cfg::kSmem, stream, map_w, map_x, p));
    return SPK_OK;
}

}  // namespace

// The fp32-block-scaled fp8 GEMM on the tensor cores (every shape; C rows must be 16-byte aligned).
int fp8gemm_block128_umma_try(const simt::Params& q, cudaStream_t stream, bool* taken) {
    *taken = false;
    if (umma_disabled() || !aligned16(q.C)) return SPK_OK;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    if (q.M <= 64 && decode_fits(q, 0)) {  // decode: weights as the 128-row operand, K split over the SMs
        *taken = true;
        return q.M <= 16 ? launch_decode_block128<16>(q, dev, stream)
               : q.M <= 32 ? launch_decode_block128<32>(q, dev, stream)
                           : launch_decode_block128<64>(q, dev, stream);
    }
    *taken = true;
    // 128 x 256 tiles (8 folding warps) once they fill the SMs; 128 x 128 for small problems
    const bool wide = q.N % 256 == 0 && static_cast<long long>(cdiv(q.M, kBM)) * (q.N / 256) >= dev->sm_count;
    return wide ? launch_block128<256>(q, dev, stream) : launch_block128<128>(q, dev, stream);
}

}  // namespace spk
