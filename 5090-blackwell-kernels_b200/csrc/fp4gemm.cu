// fp4 (e2m1) GEMM, NVFP4 and MXFP4: C = scale_a * scale_b * sum_k (sfa A)(sfb Bt), operands packed
// two to a byte, block scales in the blocked layout, bf16 out, fp32 accumulation.
// Contract: reference include/spark/kernels.h:296-331.
//   0  CUDA-core kernel, M % 16 == 0
//   1  any M: tcgen05 tiles above 64 tokens (ragged M by TMA zero fill), tcgen05 split-K decode below
//   2  the same tile kernel under the reference's shape rule (M, N multiples of 128, a tile per SM)
#include "qgemm_simt.cuh"

namespace spk {
namespace {

bool fp4_base_ok(int M, int N, int K) { return M >= 1 && N > 0 && K > 0 && N % 64 == 0 && K % 256 == 0; }

int fp4_sms() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0) {
        (void)cudaGetLastError();
        return 148;
    }
    return sms;
}

bool fp4_supports(int M, int N, int K, int variant) {
    if (variant < 0 || variant >= 3 || !fp4_base_ok(M, N, K)) return false;
    if (variant == 0) return M % 16 == 0;
    if (variant == 2) return M % 128 == 0 && N % 128 == 0 && static_cast<long long>(M / 128) * (N / 128) >= fp4_sms();
    return true;
}

}  // namespace
// defined in fp4gemm_umma.cu
int fp4gemm_umma_try(const simt::Params& p, int format, cudaStream_t stream, bool* taken);
}  // namespace spk

extern "C" int spk_fp4gemm_num_variants(void) { return 3; }
extern "C" int spk_fp4gemm_supports(int M, int N, int K, int variant) { return spk::fp4_supports(M, N, K, variant); }
extern "C" int spk_fp4gemm_available(void) { return 1; }

extern "C" int spk_fp4gemm(const void* A, const void* Bt, void* C, int M, int N, int K, const unsigned char* sfa,
                           const unsigned char* sfb, const float* scale_a, const float* scale_b, int format, int variant,
                           void* stream_) {
    using namespace spk;
    SPK_REQUIRE(variant >= 0 && variant < 3, "fp4gemm: variant %d out of range [0, 3)", variant);
    SPK_REQUIRE(format == SPK_FP4_NVFP4 || format == SPK_FP4_MXFP4, "fp4gemm: unknown format %d", format);
    SPK_REQUIRE(A && Bt && C && sfa && sfb, "fp4gemm: null pointer");
    SPK_REQUIRE(M >= 1 && N > 0 && K > 0, "fp4gemm: M, N, K must be positive, got %d %d %d", M, N, K);
    SPK_REQUIRE(N % 64 == 0 && K % 256 == 0, "fp4gemm: needs N %% 64 == 0 and K %% 256 == 0, got N=%d K=%d", N, K);
    SPK_REQUIRE((scale_a == nullptr) == (scale_b == nullptr), "fp4gemm: scale_a and scale_b must both be given or both be null");
    SPK_REQUIRE(aligned16(A) && aligned16(Bt) && aligned16(sfa) && aligned16(sfb), "fp4gemm: A, Bt, sfa, sfb must be 16-byte aligned");
    SPK_REQUIRE(fp4_supports(M, N, K, variant), "fp4gemm: variant %d does not take M=%d N=%d K=%d", variant, M, N, K);
    auto stream = static_cast<cudaStream_t>(stream_);
    simt::Params p{};
    p.A = static_cast<const unsigned char*>(A);
    p.Bt = static_cast<const unsigned char*>(Bt);
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M, p.N = N, p.K = K;
    p.scale_a = scale_a, p.scale_b = scale_b;
    p.sfa = sfa, p.sfb = sfb;
    if (variant >= 1) {  // tensor cores for every M: 128-row tiles above 64 tokens, split-K decode below
        bool taken = false;
        const int rc = fp4gemm_umma_try(p, format, stream, &taken);
        if (taken || rc != SPK_OK) return rc;
    }
    return format == SPK_FP4_NVFP4 ? simt::launch<simt::kFp4Nv>(p, stream) : simt::launch<simt::kFp4Mx>(p, stream);
}
