// Grouped fp8 GEMM for a mixture-of-experts layer: every expert's GEMM in one persistent launch,
//   C[r, :] = scale_a * scale_b[e] * A[r, :] * W[e]^T      for r in offsets[e] .. offsets[e + 1] - 1
// (contract: reference include/spark/kernels.h:459-494, grouped_gemm_fp8 / grouped_gemm_swiglu_fp8). A [T][K]
// e4m3 has its rows sorted by expert, `offsets` is int32 [E + 1] ON THE DEVICE (offsets[0] == 0,
// offsets[E] == T, empty experts allowed), W is [E][N][K] e4m3 (K contiguous), C [T][N] bf16, fp32 accumulate.
// Nothing is read back to the host: every CTA builds the tile list itself from `offsets` (a prefix sum of
// ceil(rows_e / 128) * N / BN over the experts, in shared memory) and takes tiles b, b + grid, ... of it.
//
// The kernel is the tcgen05 tile kernel of qgemm_umma.cu in its plain fp8 form: a producer warp feeds a
// ring of TMA stages (A box 128 rows x 128 bytes starting at the expert's row offset + 128 i, W box BN rows
// of the [E * N][K] view), one warp issues tcgen05.mma.kind::f8f6f4 into a TMEM accumulator, four warps
// drain it. A row tile that runs past its expert's last row reads the next expert's rows (or TMA zero
// fill past T); those rows are simply not stored. The SwiGLU form takes W with its rows alternating
// gate_j, up_j: the two sums of one output sit in adjacent accumulator columns of the same thread, which
// stores silu(gate) * up to C [T][N / 2], computed in fp32 after the scales.
// The summation order of a tile is fixed, so the output is the same bits every run.
#include <algorithm>

#include "spk_common.cuh"
#include "umma_sm100.cuh"

namespace spk {
namespace {

using ptx::mbar_arrive_expect_tx;
using ptx::mbar_init;
using ptx::mbar_wait;

constexpr int kGBM = 128, kGBK = 128, kGStages = 4, kMaxExperts = 512;

struct GroupedParams {
    __nv_bfloat16* C;
    const int32_t* offsets;
    const float* scale_a;  // device scalar or null
    const float* scale_b;  // device [E] or null
    int T, E, N, K, swiglu;
    int* status;
};

template <int BN>
struct GroupedCfg {
    static constexpr int kABytes = kGBM * kGBK, kBBytes = BN * kGBK, kStageBytes = kABytes + kBBytes;
    static constexpr int kPrefixBytes = (kMaxExperts + 1) * 8;  // tile prefix and row offsets
    static constexpr int kSmem = kGStages * kStageBytes + 1024 + 256 + kPrefixBytes;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const GroupedParams p) {
    using Cfg = GroupedCfg<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + kGStages * Cfg::kStageBytes);
    uint64_t* empty = full + kGStages;
    uint64_t* acc_ready = empty + kGStages;
    uint64_t* acc_free = acc_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
    int* prefix = reinterpret_cast<int*>(tiles + kGStages * Cfg::kStageBytes + 256);  // [E + 1] tiles before expert e
    int* row0 = prefix + kMaxExperts + 1;                                             // [E + 1] offsets, in shared memory

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = p.N / BN, k_blocks = p.K / kGBK;

    for (int e = threadIdx.x; e <= p.E; e += blockDim.x) row0[e] = __ldg(p.offsets + e);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kGStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        mbar_init(acc_free, 4);
        ptx::fence_mbar_init();
        umma::prefetch_tensormap(&map_a);
        umma::prefetch_tensormap(&map_w);
    }
    if (warp == 1) umma::tmem_alloc(tmem_slot, BN);
    __syncthreads();
    if (threadIdx.x == 0) {  // E <= 512: a serial prefix is a few hundred cycles, once per CTA
        int acc = 0;
        for (int e = 0; e < p.E; ++e) {
            prefix[e] = acc;
            const int rows = max(0, min(row0[e + 1], p.T) - max(row0[e], 0));
            acc += ((rows + kGBM - 1) / kGBM) * tiles_n;
        }
        prefix[p.E] = acc;
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;
    const int total_tiles = prefix[p.E];

    // tile q -> expert (the last e with prefix[e] <= q), row tile (fastest) and column tile inside it
    auto locate = [&](int q, int& e, int& a_row, int& row_end, int& tile_n) {
        int lo = 0, hi = p.E - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= q) lo = mid; else hi = mid - 1;
        }
        e = lo;
        const int first = max(row0[e], 0);
        row_end = min(row0[e + 1], p.T);
        const int mt = (row_end - first + kGBM - 1) / kGBM, local = q - prefix[e];
        a_row = first + (local % mt) * kGBM;
        tile_n = local / mt;
    };

    if (warp == 0) {
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int q = blockIdx.x; q < total_tiles && ok; q += gridDim.x) {
            int e, a_row, row_end, tile_n;
            locate(q, e, a_row, row_end, tile_n);
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, p.status));
                if (!ok) break;
                if (umma::elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
                    unsigned char* st = tiles + s * Cfg::kStageBytes;
                    umma::tma_load_2d(st, &map_a, kb * kGBK, a_row, &full[s]);
                    umma::tma_load_2d(st + Cfg::kABytes, &map_w, kb * kGBK, e * p.N + tile_n * BN, &full[s]);
                }
                __syncwarp();
                if (++s == kGStages) s = 0, ph ^= 1u;
            }
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = umma::instr_desc(kGBM, BN, 0, 0);  // e4m3 x e4m3 -> f32
        bool ok = true;
        int s = 0, it = 0;
        unsigned ph = 0;
        for (int q = blockIdx.x; q < total_tiles && ok; q += gridDim.x, ++it) {
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
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma::mma_f8f6f4(tmem_acc, umma::desc_advance(adesc, 32 * k), umma::desc_advance(bdesc, 32 * k), idesc, kb > 0 || k > 0);
                    umma::mma_commit(&empty[s]);
                    if (kb == k_blocks - 1) umma::mma_commit(acc_ready);
                }
                __syncwarp();
                if (++s == kGStages) s = 0, ph ^= 1u;
            }
        }
        if (!ok && umma::elect_one()) umma::mma_commit(acc_ready);  // release the epilogue; its own wait fails next
        __syncwarp();
    } else {
        const int quarter = warp & 3;
        const float sa = p.scale_a ? *p.scale_a : 1.0f;
        int it = 0;
        bool ok = true;
        for (int q = blockIdx.x; q < total_tiles && ok; q += gridDim.x, ++it) {
            int e, a_row, row_end, tile_n;
            locate(q, e, a_row, row_end, tile_n);
            const float s = sa * (p.scale_b ? __ldg(p.scale_b + e) : 1.0f);
            ok = __all_sync(0xffffffffu, mbar_wait(acc_ready, it & 1, p.status));
            umma::fence_after_sync();
            if (!ok) break;
            const int row = a_row + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                umma::tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, r);
                umma::tmem_ld_wait();
                if (c0 + 32 == BN) {
                    umma::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_free);
                }
                if (row >= row_end) continue;
                const int col = tile_n * BN + c0;
                if (!p.swiglu) {
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
                } else {
                    uint4 out[2];
                    uint32_t* o = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {  // outputs 2 j, 2 j + 1 of this run of 16: (gate, up) pairs at columns 4 j .. 4 j + 3
                        float h[2];
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const float gate = __uint_as_float(r[4 * j + 2 * i]) * s, up = __uint_as_float(r[4 * j + 2 * i + 1]) * s;
                            h[i] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                        }
                        const __nv_bfloat162 v = __floats2bfloat162_rn(h[0], h[1]);
                        o[j] = *reinterpret_cast<const uint32_t*>(&v);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.C + static_cast<size_t>(row) * (p.N / 2) + col / 2);
                    dst[0] = out[0];
                    dst[1] = out[1];
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 1) umma::tmem_dealloc(tmem_acc, BN);
}

template <int BN>
int launch_grouped(const void* A, const void* W, const GroupedParams& p, DeviceState* dev, cudaStream_t stream) {
    using Cfg = GroupedCfg<BN>;
    static_assert(Cfg::kSmem <= 227 * 1024, "grouped GEMM stage ring exceeds shared memory");
    CUtensorMap map_a, map_w;
    if (!umma::make_map_2d_u8(&map_a, A, static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.T), kGBM) ||
        !umma::make_map_2d_u8(&map_w, W, static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.E) * p.N, BN))
        return fail(SPK_CUDA_ERROR, "grouped_gemm_fp8: cuTensorMapEncodeTiled failed for T=%d E=%d N=%d K=%d", p.T, p.E, p.N, p.K);
    auto kernel = grouped_gemm_fp8_kernel<BN>;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        configured[dev->device] = true;
    }
    // the tile count lives on the device; at most ceil(T / 128) + E row tiles exist
    const long long upper = (static_cast<long long>(cdiv(p.T, kGBM)) + p.E) * (p.N / BN);
    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(upper, dev->sm_count)));
    kernel<<<grid, 192, Cfg::kSmem, stream>>>(map_a, map_w, p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

bool grouped_ok(int E, int N, int K) { return E >= 1 && E <= kMaxExperts && N > 0 && K > 0 && N % 128 == 0 && K % 128 == 0; }

int grouped_run(const void* A, const void* W, const int32_t* offsets, void* C, int T, int E, int N, int K, const float* scale_a,
                const float* scale_b, bool swiglu, void* stream) {
    SPK_REQUIRE(A && W && offsets && C, "grouped_gemm_fp8: null pointer");
    SPK_REQUIRE(T >= 0 && grouped_ok(E, N, K), "grouped_gemm_fp8: needs 1 <= E <= 512, N %% 128 == 0, K %% 128 == 0, got T=%d E=%d N=%d K=%d", T, E, N, K);
    SPK_REQUIRE(aligned16(A) && aligned16(W) && aligned16(C), "grouped_gemm_fp8: A, W and C must be 16-byte aligned");
    if (T == 0) return SPK_OK;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    GroupedParams p{};
    p.C = static_cast<__nv_bfloat16*>(C);
    p.offsets = offsets, p.scale_a = scale_a, p.scale_b = scale_b;
    p.T = T, p.E = E, p.N = N, p.K = K, p.swiglu = swiglu ? 1 : 0;
    p.status = dev->status;
    const bool wide = N % 256 == 0 && static_cast<long long>(cdiv(T, kGBM) + E / 2) * (N / 256) >= dev->sm_count;
    return wide ? launch_grouped<256>(A, W, p, dev, static_cast<cudaStream_t>(stream))
                : launch_grouped<128>(A, W, p, dev, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace spk

extern "C" int spk_grouped_gemm_supports(int E, int N, int K) { return spk::grouped_ok(E, N, K) ? 1 : 0; }

extern "C" int spk_grouped_gemm_fp8(const void* A, const void* W, const int32_t* offsets, void* C, int T, int E, int N, int K,
                                    const float* scale_a, const float* scale_b, void* stream) {
    return spk::grouped_run(A, W, offsets, C, T, E, N, K, scale_a, scale_b, false, stream);
}

extern "C" int spk_grouped_gemm_swiglu_fp8(const void* A, const void* W, const int32_t* offsets, void* C, int T, int E, int N, int K,
                                           const float* scale_a, const float* scale_b, void* stream) {
    return spk::grouped_run(A, W, offsets, C, T, E, N, K, scale_a, scale_b, true, stream);
}
