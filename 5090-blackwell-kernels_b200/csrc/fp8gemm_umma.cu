// Tensor-core route of the fp8 GEMM (variants 2 and 3, per-tensor scales): a TMA-fed tcgen05
// kernel with the accumulator in TMEM.
//
// One CTA computes one 128 x BN tile of C. Roles, one warp each unless noted:
//   warp 0   producer: one thread issues two tiled TMA loads per K block (A 128 x 128 B, Bt BN x
//            128 B, 128-byte swizzle) into a ring of kStages shared-memory stages
//   warp 1   MMA: allocates TMEM; one thread issues four tcgen05.mma.kind::f8f6f4 (128 x BN x 32)
//            per K block and commits them to the stage's "empty" barrier, and at the end to the
//            "accumulator ready" barrier
//   warps 2-5  epilogue: each reads the 32 accumulator rows of its TMEM quarter (tcgen05.ld), applies
//            scale_a * scale_b in fp32, rounds once to bf16 and stores
// Rows past M, columns past N and k past K are zero-filled by TMA, so any shape the API accepts
// runs; the stores are predicated. Every barrier wait is bounded; on a timeout the roles stop,
// the status word is set, and TMEM is still released.
#include "qgemm_simt.cuh"
#include "umma_sm100.cuh"

namespace spk {
namespace {

using ptx::mbar_arrive_expect_tx;
using ptx::mbar_init;
using ptx::mbar_wait;

constexpr int kBM = 128, kBKBytes = 128;

template <int BN>
struct UmmaCfg {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = kBM * kBKBytes, kBBytes = BN * kBKBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSmem = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr int kTmemCols = BN;  // power of two >= 32
};

struct UmmaParams {
    __nv_bfloat16* C;
    int M, N, K;
    const float* scale_a;
    const float* scale_b;
    int* status;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
fp8gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const UmmaParams p) {
    using Cfg = UmmaCfg<BN>;
    extern __shared__ unsigned char smem_raw[];
    // 128-byte-swizzled tiles must start on a 1024-byte boundary
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* empty = full + Cfg::kStages;
    uint64_t* acc_ready = empty + Cfg::kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tile_m = blockIdx.x % tiles_m, tile_n = blockIdx.x / tiles_m;
    const int k_blocks = (p.K + kBKBytes - 1) / kBKBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
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
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % Cfg::kStages;
                // a fresh barrier passes a wait on the opposite parity, so the first lap does not block
                if (!mbar_wait(&empty[s], ((kb / Cfg::kStages) & 1) ^ 1, p.status)) break;
                mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
                unsigned char* a_dst = tiles + s * Cfg::kStageBytes;
                umma::tma_load_2d(a_dst, &map_a, kb * kBKBytes, tile_m * kBM, &full[s]);
                umma::tma_load_2d(a_dst + Cfg::kABytes, &map_b, kb * kBKBytes, tile_n * BN, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma::instr_desc(kBM, BN, 0, 0);  // e4m3 x e4m3 -> f32
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % Cfg::kStages;
                ok = mbar_wait(&full[s], (kb / Cfg::kStages) & 1, p.status);
                if (!ok) break;
                umma::fence_after_sync();
                const unsigned char* a_tile = tiles + s * Cfg::kStageBytes;
                const uint64_t adesc = umma::smem_desc_k128(a_tile), bdesc = umma::smem_desc_k128(a_tile + Cfg::kABytes);
#pragma unroll
                for (int k = 0; k < kBKBytes / 32; ++k)
                    umma::mma_f8f6f4(tmem_acc, umma::desc_advance(adesc, 32 * k), umma::desc_advance(bdesc, 32 * k), idesc,
                                     kb > 0 || k > 0);
                umma::mma_commit(&empty[s]);  // the stage is free once these MMAs have read it
            }
            umma::mma_commit(acc_ready);  // fires after every MMA above has completed (also on failure)
        }
    } else {
        // ---- epilogue: warps 2..5 -> TMEM lane quarters 2, 3, 0, 1 ----
        const int quarter = warp & 3;
        const bool ok = mbar_wait(acc_ready, 0, p.status);
        umma::fence_after_sync();
        if (ok) {
            const float s = (p.scale_a ? *p.scale_a : 1.0f) * (p.scale_b ? *p.scale_b : 1.0f);
            const int row = tile_m * kBM + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                umma::tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, r);
                umma::tmem_ld_wait();
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

template <int BN>
int launch_umma(const simt::Params& q, DeviceState* dev, cudaStream_t stream) {
    using Cfg = UmmaCfg<BN>;
    CUtensorMap map_a, map_b;
    if (!umma::make_map_2d_u8(&map_a, q.A, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.M), kBM) ||
        !umma::make_map_2d_u8(&map_b, q.Bt, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.N), BN))
        return fail(SPK_CUDA_ERROR, "fp8gemm: cuTensorMapEncodeTiled failed for %dx%dx%d", q.M, q.N, q.K);
    auto kernel = fp8gemm_umma_kernel<BN>;
    static bool configured[16] = {};
    if (!configured[dev->device & 15]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        configured[dev->device & 15] = true;
    }
    UmmaParams p{q.C, q.M, q.N, q.K, q.scale_a, q.scale_b, dev->status};
    const int grid = cdiv(q.M, kBM) * cdiv(q.N, BN);
    kernel<<<grid, 192, Cfg::kSmem, stream>>>(map_a, map_b, p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace

// Variant 2 takes exactly the shapes its rule names; variant 3 takes whatever has at least one
// M tile of work worth a tensor-core launch (M > 64) in per-tensor mode. MX mode and decode shapes
// stay on the other routes for now.
int fp8gemm_umma_try(const simt::Params& p, bool mx, int variant, cudaStream_t stream, bool* taken) {
    *taken = false;
    if (mx || p.M <= 64 || !aligned16(p.C)) return SPK_OK;
    if (const char* e = std::getenv("SPK_FP8_NO_UMMA"); e && *e == '1') return SPK_OK;
    (void)variant;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    *taken = true;
    return p.N % 256 == 0 ? launch_umma<256>(p, dev, stream) : launch_umma<128>(p, dev, stream);
}

}  // namespace spk
