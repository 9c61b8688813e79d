// Prefill route of the W4A16 GEMM (many tokens): dequantize the weight once into bf16, then run a dense
// bf16 GEMM on the tcgen05 tile kernel. Above a few hundred tokens the GEMM is bound by the tensor
// cores, not by the weight stream, and the per-weight dequant cost has to be paid once per call
// instead of once per 64-token pass (the reference describes the same crossover for its own kernels,
// docs/design/w4gemm.md:303-319: dequant-to-bf16 + dense GEMM above M ~ 128).
//
//   step 1  w4_dequant_kernel: packed [N/16][K/64][32][4] + scales (+ zeros) -> Wd bf16 [N][K], K
//           contiguous in natural k order. A warp takes one 512-byte block (16 columns x 64 k); a
//           lane's four words are 4 x 4 consecutive k of columns g and g + 8, so it writes four 16-byte
//           pieces (two columns x two 32-k halves) and the four lanes of a quad fill 64 contiguous
//           bytes of a row. Every weight is bf16((q - z) * s) exactly as the decode kernels compute it.
//   step 2  C[M][N] = A[M][K] Wd^T: qgemm_umma_kernel in its bf16 mode (TMA-fed tcgen05.mma.kind::f16,
//           accumulators in TMEM), the tokens as the 128-row operand.
//
// Wd lives in a per-device scratch that grows on demand (cudaMalloc, kept until the process exits):
// reserve it with spk_w4_prefill_reserve before capturing a CUDA graph, as with every other scratch here.
#include <algorithm>
#include <mutex>

#include "spk_common.cuh"
#include "w4_layout.cuh"

namespace spk {
// defined in qgemm_umma.cu
int bf16gemm_umma(const void* A, const void* Bt, void* C, int M, int N, int K, cudaStream_t stream);

namespace {

template <bool ASYM>
__global__ void __launch_bounds__(256)
w4_dequant_kernel(const uint4* __restrict__ packed, const unsigned short* __restrict__ scales, const uint8_t* __restrict__ zeros,
                  uint4* __restrict__ wd, int N, int K, long long blocks) {
    const long long blk = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;  // (strip, unit), unit fastest
    if (blk >= blocks) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int units = K / 64;
    const int u = static_cast<int>(blk % units), t = static_cast<int>(blk / units);
    const int grp = u >> 1;
    const int n_lo = 16 * t + g, n_hi = n_lo + 8;
    const uint32_t s_lo = w4::splat16(scales[static_cast<size_t>(grp) * N + n_lo]);
    const uint32_t s_hi = w4::splat16(scales[static_cast<size_t>(grp) * N + n_hi]);
    uint32_t o_lo = w4::kSymOffset, o_hi = w4::kSymOffset;
    if (ASYM) {
        o_lo = w4::offset_pair(zeros[static_cast<size_t>(grp) * N + n_lo]);
        o_hi = w4::offset_pair(zeros[static_cast<size_t>(grp) * N + n_hi]);
    }
    const uint4 q = packed[blk * 32 + lane];
    uint32_t x[4][4];
    w4::dequant_word(q.x, o_lo, o_hi, s_lo, s_hi, x[0]);
    w4::dequant_word(q.y, o_lo, o_hi, s_lo, s_hi, x[1]);
    w4::dequant_word(q.z, o_lo, o_hi, s_lo, s_hi, x[2]);
    w4::dequant_word(q.w, o_lo, o_hi, s_lo, s_hi, x[3]);
    // word j holds k = 64 u + 32 (j >> 1) + 8 c + 4 (j & 1) + {0..3}: x[j][0], x[j][2] column g, x[j][1], x[j][3] column g + 8
    const size_t row_vecs = static_cast<size_t>(K) / 8;  // 16-byte pieces per row
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const size_t piece = static_cast<size_t>(8 * u + 4 * i + c);  // (64 u + 32 i + 8 c) / 8
        wd[n_lo * row_vecs + piece] = make_uint4(x[2 * i][0], x[2 * i][2], x[2 * i + 1][0], x[2 * i + 1][2]);
        wd[n_hi * row_vecs + piece] = make_uint4(x[2 * i][1], x[2 * i][3], x[2 * i + 1][1], x[2 * i + 1][3]);
    }
}

struct PrefillScratch {
    void* ptr = nullptr;
    size_t bytes = 0;
};
PrefillScratch g_scratch[kMaxDevices];
std::mutex g_scratch_mutex;

int scratch_for(size_t bytes, int device, void** out) {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    PrefillScratch& s = g_scratch[device];
    if (s.bytes < bytes) {
        // growth: the old block may still be in use by work in flight, so wait for the device before it is freed
        if (s.ptr != nullptr) {
            SPK_CUDA(cudaDeviceSynchronize());
            SPK_CUDA(cudaFree(s.ptr));
            s.ptr = nullptr, s.bytes = 0;
        }
        SPK_CUDA(cudaMalloc(&s.ptr, bytes));
        s.bytes = bytes;
    }
    *out = s.ptr;
    return SPK_OK;
}

int prefill_min_m() {
    static const int v = [] {
        const char* e = std::getenv("SPK_W4_PREFILL_MIN_M");
        return e && *e ? std::atoi(e) : 256;
    }();
    return v;
}

}  // namespace

// Takes M >= 256 tokens (SPK_W4_PREFILL_MIN_M) when the dense GEMM has at least one 128 x 128 tile per SM (with fewer
// the GEMM leaves SMs idle and consecutive 64-token passes of the TMEM kernel are faster: 4096 x 14336 at 256 tokens
// 99 us against 168), N a multiple of 64 and 16-byte aligned A and C. `taken` says whether it ran.
// Measured on B200 (CUDA events, 10 launches): 28672 x 4096 at 256 / 512 / 2048 tokens 121 / 168 / 430 us against
// 147 / 286 / 1112 us for the passes (1.12 PFLOP/s at 2048 tokens); 4096 x 14336 at 2048 tokens 209 us against 763.
int w4gemm_prefill_try(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N,
                       int K, cudaStream_t stream, bool* taken) {
    *taken = false;
    if (M < prefill_min_m() || N % 64 != 0 || !aligned16(A) || !aligned16(C)) return SPK_OK;
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    if (static_cast<long long>(cdiv(M, 128)) * cdiv(N, 128) < dev->sm_count) return SPK_OK;
    void* wd = nullptr;
    if (int rc = scratch_for(static_cast<size_t>(N) * K * 2, dev->device, &wd)) return rc;
    *taken = true;
    const long long blocks = static_cast<long long>(N / 16) * (K / 64);
    const unsigned grid = static_cast<unsigned>(cdiv64(blocks * 32, 256));
    if (zeros)
        w4_dequant_kernel<true><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint4*>(packed), static_cast<const unsigned short*>(scales),
                                                          zeros, static_cast<uint4*>(wd), N, K, blocks);
    else
        w4_dequant_kernel<false><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint4*>(packed),
                                                           static_cast<const unsigned short*>(scales), nullptr, static_cast<uint4*>(wd), N, K,
                                                           blocks);
    SPK_CHECK_LAUNCH();
    return bf16gemm_umma(A, wd, C, M, N, K, stream);
}

}  // namespace spk

extern "C" int spk_w4_prefill_reserve(long long bytes) {
    using namespace spk;
    SPK_REQUIRE(bytes > 0, "w4_prefill_reserve: bytes must be positive");
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    void* p = nullptr;
    return scratch_for(static_cast<size_t>(bytes), dev->device, &p);
}
