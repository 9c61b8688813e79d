// fp8 (e4m3) GEMM: C = scale_a * scale_b * A Bt^T, A [M][K] and Bt [N][K] K-contiguous, bf16 out,
// fp32 accumulation; per-tensor scales, MX block scales (ue8m0 per 32 k on both operands), and an
// additive mode with fp32 scales per 1 x 128 (A) and 128 x 128 (B) block that the reference does
// not have. Contract: reference include/spark/kernels.h:230-294.
//
// Variants (numbers and shape rules follow the reference's ladder so callers can keep theirs):
//   0  CUDA-core kernel, M % 16 == 0      1  CUDA-core kernel, any M
//   2  tensor-core kernel, M, N, K multiples of 128 and at least one 128 x 128 tile per SM
//   3  default: per shape, the tensor-core kernel where it applies, else variant 1
//   4  batch invariant: the CUDA-core kernel for every M (one fma chain per output)
#include "qgemm_simt.cuh"

namespace spk {
// defined in fp8gemm_umma.cu
int fp8gemm_umma_try(const simt::Params& p, bool mx, int variant, cudaStream_t stream, bool* taken);
const char* fp8gemm_umma_plan(int M, int N, int K, bool mx, int variant, bool c_aligned, int sms);
int fp8gemm_block128_umma_try(const simt::Params& p, cudaStream_t stream, bool* taken);
namespace {

int g_v3_route = -1;  // SPK_FP8GEMM_V3_ROUTE_DEFAULT

bool base_ok(int M, int N, int K) { return M >= 1 && N > 0 && K > 0 && N % 64 == 0 && K % 64 == 0; }

bool tensor_core_shape(int M, int N, int K, int sms) {
    return M % 128 == 0 && N % 128 == 0 && K % 128 == 0 && static_cast<long long>(M / 128) * (N / 128) >= sms;
}

int sm_count_or(int fallback) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return fallback;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        (void)cudaGetLastError();
        return fallback;
    }
    return sms;
}

bool supports(int M, int N, int K, int variant, bool mx) {
    if (variant < 0 || variant >= 5 || !base_ok(M, N, K)) return false;
    if (mx && K % 256 != 0) return false;
    if (variant == 0) return M % 16 == 0;
    if (variant == 2) return tensor_core_shape(M, N, K, sm_count_or(148));
    return true;
}

// The variant that really runs. Variant 3 under the legacy route (-2, reference include/spark/kernels.h:281-294:
// "the old route") is what this library's ladder had before the per-shape rule: variant 2 where its
// tile rule holds, else the CUDA-core kernel.
int effective_variant(int M, int N, int K, int variant) {
    if (variant != 3 || g_v3_route != -2) return variant;
    return tensor_core_shape(M, N, K, sm_count_or(148)) ? 2 : 1;
}

int run(const simt::Params& p, bool mx, int variant, cudaStream_t stream) {
    variant = effective_variant(p.M, p.N, p.K, variant);
    // The tensor-core route (variants 2 and 3) lives in qgemm_umma.cu and is reached through this hook.
    if (variant == 2 || variant == 3) {
        bool taken = false;
        const int rc = fp8gemm_umma_try(p, mx, variant, stream, &taken);
        if (taken || rc != SPK_OK) return rc;
        if (variant == 2) return fail(SPK_INVALID, "fp8gemm: variant 2 does not take %dx%dx%d", p.M, p.N, p.K);
    }
    return mx ? simt::launch<simt::kFp8Mx>(p, stream) : simt::launch<simt::kFp8Tensor>(p, stream);
}

int check_common(const char* op, const void* A, const void* Bt, void* C, int M, int N, int K, int variant, bool mx) {
    SPK_REQUIRE(variant >= 0 && variant < 5, "%s: variant %d out of range [0, 5)", op, variant);
    SPK_REQUIRE(A && Bt && C, "%s: null pointer", op);
    SPK_REQUIRE(M >= 1 && N > 0 && K > 0, "%s: M, N, K must be positive, got %d %d %d", op, M, N, K);
    SPK_REQUIRE(N % 64 == 0 && K % 64 == 0, "%s: needs N %% 64 == 0 and K %% 64 == 0, got N=%d K=%d", op, N, K);
    SPK_REQUIRE(!mx || K % 256 == 0, "%s: block scales need K %% 256 == 0, got %d", op, K);
    SPK_REQUIRE(aligned16(A) && aligned16(Bt), "%s: A and Bt must be 16-byte aligned", op);
    SPK_REQUIRE(supports(M, N, K, variant, mx), "%s: variant %d does not take M=%d N=%d K=%d", op, variant, M, N, K);
    return SPK_OK;
}

}  // namespace
}  // namespace spk

extern "C" int spk_fp8gemm_num_variants(void) { return 5; }
extern "C" int spk_fp8gemm_default_variant(void) { return 3; }
extern "C" int spk_fp8gemm_supports(int M, int N, int K, int variant) { return spk::supports(M, N, K, variant, false); }
extern "C" int spk_fp8gemm_mx_supports(int M, int N, int K, int variant) { return spk::supports(M, N, K, variant, true); }
extern "C" int spk_fp8gemm_mx_available(void) { return 1; }

extern "C" int spk_fp8gemm(const void* A, const void* Bt, void* C, int M, int N, int K, const float* scale_a,
                           const float* scale_b, int variant, void* stream) {
    using namespace spk;
    if (int rc = check_common("fp8gemm", A, Bt, C, M, N, K, variant, false)) return rc;
    SPK_REQUIRE(scale_a && scale_b, "fp8gemm: scale_a and scale_b are required (device fp32 scalars)");
    simt::Params p{};
    p.A = static_cast<const unsigned char*>(A);
    p.Bt = static_cast<const unsigned char*>(Bt);
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M, p.N = N, p.K = K;
    p.scale_a = scale_a, p.scale_b = scale_b;
    return run(p, false, variant, static_cast<cudaStream_t>(stream));
}

extern "C" int spk_fp8gemm_mx(const void* A, const void* Bt, void* C, int M, int N, int K, const float* scale_a,
                              const float* scale_b, const unsigned char* sfa, const unsigned char* sfb, int variant,
                              void* stream) {
    using namespace spk;
    if (int rc = check_common("fp8gemm_mx", A, Bt, C, M, N, K, variant, true)) return rc;
    SPK_REQUIRE(sfa && sfb, "fp8gemm_mx: sfa and sfb are required");
    SPK_REQUIRE((scale_a == nullptr) == (scale_b == nullptr), "fp8gemm_mx: scale_a and scale_b must both be given or both be null");
    SPK_REQUIRE(aligned16(sfa) && aligned16(sfb), "fp8gemm_mx: sfa and sfb must be 16-byte aligned");
    simt::Params p{};
    p.A = static_cast<const unsigned char*>(A);
    p.Bt = static_cast<const unsigned char*>(Bt);
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M, p.N = N, p.K = K;
    p.scale_a = scale_a, p.scale_b = scale_b;
    p.sfa = sfa, p.sfb = sfb;
    return run(p, true, variant, static_cast<cudaStream_t>(stream));
}

extern "C" int spk_fp8gemm_block128(const void* A, const void* Bt, void* C, int M, int N, int K, const float* sA,
                                    const float* sB, void* stream) {
    using namespace spk;
    SPK_REQUIRE(A && Bt && C && sA && sB, "fp8gemm_block128: null pointer");
    SPK_REQUIRE(M >= 1 && N > 0 && K > 0 && N % 64 == 0 && K % 128 == 0,
                "fp8gemm_block128: needs N %% 64 == 0 and K %% 128 == 0, got M=%d N=%d K=%d", M, N, K);
    SPK_REQUIRE(aligned16(A) && aligned16(Bt), "fp8gemm_block128: A and Bt must be 16-byte aligned");
    simt::Params p{};
    p.A = static_cast<const unsigned char*>(A);
    p.Bt = static_cast<const unsigned char*>(Bt);
    p.C = static_cast<__nv_bfloat16*>(C);
    p.M = M, p.N = N, p.K = K;
    p.blk_a = sA, p.blk_b = sB;
    bool taken = false;
    const int rc = fp8gemm_block128_umma_try(p, static_cast<cudaStream_t>(stream), &taken);
    if (taken || rc != SPK_OK) return rc;
    return simt::launch<simt::kFp8Block128>(p, static_cast<cudaStream_t>(stream));
}

// Variant 3's route knob (reference include/spark/kernels.h:281-294): -1 the per-shape rule, -2 the legacy
// route (variant 2 where its tile rule holds, else the CUDA cores). The reference's other values force
// sm_120 tile shapes that do not exist here; they are stored and behave like -1. The name says which
// kernel of THIS library the shape runs on under the current route, from the launcher's own predicate.
extern "C" void spk_fp8gemm_v3_set_route(int route) { spk::g_v3_route = route; }
extern "C" int spk_fp8gemm_v3_route(void) { return spk::g_v3_route; }
extern "C" int spk_fp8gemm_v3_num_tiles(void) { return 2; }  // 128 x 256 and 128 x 128
extern "C" const char* spk_fp8gemm_v3_route_name(int M, int N, int K, int mx) {
    using namespace spk;
    if (!base_ok(M, N, K) || (mx && K % 256 != 0)) return "unsupported";
    const int v = effective_variant(M, N, K, 3);
    if (v == 1) return M <= 64 ? "simt_decode" : "simt";
    const char* plan = fp8gemm_umma_plan(M, N, K, mx != 0, v, true, sm_count_or(148));
    return plan ? plan : (M <= 64 ? "simt_decode" : "simt");
}
extern "C" const char* spk_fp8gemm_v4_route_name(int M, int N, int K) {
    return spk::base_ok(M, N, K) ? "simt_unsplit" : "unsupported";
}
