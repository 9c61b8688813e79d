// int4 weight quantizer and the repack into the layout w4gemm streams. Both run once per weight
// at load time; both are bit-exact contracts (reference src/kernels/w4gemm_quant.cu:15-103,
// python/spark_kernels/reference.py:262-286,344-354).
#include "spk_common.cuh"
#include "w4_layout.cuh"

namespace spk {
namespace {

// One thread per (128-k group, column). The 128 reads of a thread are strided by N but
// consecutive threads read consecutive columns, so every warp request is one 64-byte run.
// Arithmetic, in fp32: the scale is rounded to bf16 first and the codes are computed against
// the rounded value, so (q - z) * s reconstructs from the numbers the GEMM will see.
template <bool ASYM>
__global__ void __launch_bounds__(128)
w4_quantize_kernel(const __nv_bfloat16* __restrict__ W, int32_t* __restrict__ qweight,
                   __nv_bfloat16* __restrict__ scales, uint8_t* __restrict__ zeros, int N) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int g = blockIdx.y;
    if (n >= N) return;
    const __nv_bfloat16* col = W + static_cast<size_t>(g) * w4::kGroup * N + n;
    float lo = 0.f, hi = 0.f, amax = 0.f;
#pragma unroll 8
    for (int k = 0; k < w4::kGroup; ++k) {
        const float w = __bfloat162float(col[static_cast<size_t>(k) * N]);
        lo = fminf(lo, w);
        hi = fmaxf(hi, w);
        amax = fmaxf(amax, fabsf(w));
    }
    const __nv_bfloat16 sb = __float2bfloat16_rn(ASYM ? __fdiv_rn(hi - lo, 15.0f) : __fdiv_rn(amax, 7.0f));
    const float s = __bfloat162float(sb);
    int z = 8;
    if (ASYM) z = s > 0.f ? static_cast<int>(fminf(fmaxf(rintf(__fdiv_rn(-lo, s)), 0.f), 15.f)) : 0;
    for (int k8 = 0; k8 < w4::kGroup / 8; ++k8) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float w = __bfloat162float(col[static_cast<size_t>(8 * k8 + i) * N]);
            int q = z;
            if (s > 0.f) {
                const float r = rintf(__fdiv_rn(w, s));
                q = ASYM ? static_cast<int>(fminf(fmaxf(r + static_cast<float>(z), 0.f), 15.f))
                         : static_cast<int>(fminf(fmaxf(r, -8.f), 7.f)) + 8;
            }
            word |= static_cast<uint32_t>(q) << (4 * i);
        }
        qweight[static_cast<size_t>(g * (w4::kGroup / 8) + k8) * N + n] = static_cast<int32_t>(word);
    }
    scales[static_cast<size_t>(g) * N + n] = sb;
    if (ASYM) zeros[static_cast<size_t>(g) * N + n] = static_cast<uint8_t>(z);
}

// One thread per packed word: gathers the eight codes that word holds from qweight.
__global__ void __launch_bounds__(256)
w4_repack_kernel(const int32_t* __restrict__ qweight, int32_t* __restrict__ packed, int K, int N,
                 int64_t total) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int j = static_cast<int>(i & 3);
    const int lane = static_cast<int>((i >> 2) & 31);
    const int64_t blk = i >> 7;
    const int units = K / 64;
    const int u = static_cast<int>(blk % units);
    const int t = static_cast<int>(blk / units);
    uint32_t word = 0;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        int dn, dk;
        w4::slot_source(lane, u, j, p, dn, dk);
        const int n = 16 * t + dn, k = 64 * u + dk;
        const uint32_t src = static_cast<uint32_t>(__ldg(qweight + static_cast<size_t>(k >> 3) * N + n));
        word |= ((src >> (4 * (k & 7))) & 15u) << (4 * p);
    }
    packed[i] = static_cast<int32_t>(word);
}

}  // namespace
}  // namespace spk

extern "C" int spk_w4_quantize_bf16(const void* W, int32_t* qweight, void* scales, uint8_t* zeros,
                                    int K, int N, void* stream) {
    using namespace spk;
    SPK_REQUIRE(K > 0 && N > 0 && K % w4::kGroup == 0 && N % 16 == 0,
                "w4_quantize: needs K %% 128 == 0 and N %% 16 == 0, got K=%d N=%d", K, N);
    SPK_REQUIRE(W && qweight && scales, "w4_quantize: null pointer");
    const dim3 grid(cdiv(N, 128), K / w4::kGroup);
    auto st = static_cast<cudaStream_t>(stream);
    if (zeros)
        w4_quantize_kernel<true><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(W), qweight,
                                                       static_cast<__nv_bfloat16*>(scales), zeros, N);
    else
        w4_quantize_kernel<false><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(W), qweight,
                                                        static_cast<__nv_bfloat16*>(scales), nullptr, N);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_w4_repack(const int32_t* qweight, int32_t* packed, int K, int N, void* stream) {
    using namespace spk;
    SPK_REQUIRE(K > 0 && N > 0 && K % 64 == 0 && N % 16 == 0,
                "w4_repack: needs K %% 64 == 0 and N %% 16 == 0, got K=%d N=%d", K, N);
    SPK_REQUIRE(qweight && packed && qweight != packed, "w4_repack: bad pointers");
    const int64_t total = static_cast<int64_t>(N / 16) * (K / 64) * 128;
    w4_repack_kernel<<<static_cast<unsigned>(cdiv64(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        qweight, packed, K, N, total);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
