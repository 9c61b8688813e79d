// Fused gate|up projection + SwiGLU on int4 weights: H[M][I] = silu(A Wg) * (A Wu), one GEMM launch, no
// [M][2 I] intermediate. The reference runs the GEMM and then a separate swiglu kernel on its bf16
// output (python/spark_kernels/engine.py:447-451, docs/design/llm_quant.md:51-68); it names the fusion
// as the first widening of the quantized GEMMs.
//
// The activation needs gate column n and up column n of one token in the same thread block. In the
// fused [gate | up] weight they are I columns apart, so the weight is re-ordered once at load time
// (spk_w4_interleave_gate_up, on the GPTQ-order tensors, before w4_repack): 16-column strips alternate
// gate, up, gate, up. The packed layout and the GEMM kernels are untouched by that; the tcgen05 kernel's
// epilogue then finds 16 gate columns in lanes 0-15 of a warp and the matching up columns in lanes 16-31
// (w4gemm_tmem.cu, store_outputs), pairs them with one shuffle and stores silu(gate) * up, computed in
// fp32 from the unrounded sums (the unfused path rounds gate and up to bf16 in between).
#include "spk_common.cuh"
#include "w4_layout.cuh"

namespace spk {
// defined in w4gemm_tmem.cu
int w4gemm_tmem_swiglu(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* C, int M, int N, int K,
                       cudaStream_t stream, bool* taken);
namespace {

// destination column j of the interleaved order <- source column of the [gate | up] order
__device__ __forceinline__ int source_column(int j, int inter) {
    const int strip = j >> 4, within = j & 15;
    return ((strip & 1) ? inter : 0) + (strip >> 1) * 16 + within;
}

template <typename T>
__global__ void __launch_bounds__(256) interleave_columns_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int N2) {
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= static_cast<long long>(rows) * N2) return;
    const int r = static_cast<int>(i / N2), j = static_cast<int>(i % N2);
    dst[i] = src[static_cast<size_t>(r) * N2 + source_column(j, N2 / 2)];
}

template <typename T>
void interleave(const T* src, T* dst, int rows, int N2, cudaStream_t stream) {
    const long long total = static_cast<long long>(rows) * N2;
    interleave_columns_kernel<T><<<static_cast<unsigned>(cdiv64(total, 256)), 256, 0, stream>>>(src, dst, rows, N2);
}

}  // namespace
}  // namespace spk

extern "C" int spk_w4_interleave_gate_up(const int32_t* qweight, const void* scales, const uint8_t* zeros, int32_t* qweight_out,
                                         void* scales_out, uint8_t* zeros_out, int K, int N2, void* stream_) {
    using namespace spk;
    SPK_REQUIRE(K > 0 && N2 > 0 && K % w4::kGroup == 0 && N2 % 128 == 0,
                "w4_interleave_gate_up: K must be a multiple of 128 and the fused width of 128 (64 gate + 64 up columns per tile), got K=%d N=%d", K, N2);
    SPK_REQUIRE(qweight && scales && qweight_out && scales_out && (zeros == nullptr) == (zeros_out == nullptr),
                "w4_interleave_gate_up: null pointer (zeros and zeros_out go together)");
    SPK_REQUIRE(qweight != qweight_out && scales != scales_out, "w4_interleave_gate_up: not in place");
    auto stream = static_cast<cudaStream_t>(stream_);
    interleave<int32_t>(qweight, qweight_out, K / 8, N2, stream);
    interleave<unsigned short>(static_cast<const unsigned short*>(scales), static_cast<unsigned short*>(scales_out), K / w4::kGroup, N2, stream);
    if (zeros) interleave<uint8_t>(zeros, zeros_out, K / w4::kGroup, N2, stream);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_w4gemm_swiglu_bf16(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros, void* H, int M,
                                      int N2, int K, void* stream) {
    using namespace spk;
    SPK_REQUIRE(M >= 1 && N2 > 0 && K > 0, "w4gemm_swiglu: M, N, K must be positive, got %d %d %d", M, N2, K);
    SPK_REQUIRE(N2 % 128 == 0 && K % (2 * w4::kGroup) == 0, "w4gemm_swiglu: needs the fused width a multiple of 128 and K of 256, got N=%d K=%d", N2, K);
    SPK_REQUIRE(A && packed && scales && H, "w4gemm_swiglu: null pointer");
    SPK_REQUIRE(aligned16(A) && aligned16(packed) && aligned16(scales) && (!zeros || aligned16(zeros)),
                "w4gemm_swiglu: A, packed, scales and zeros must be 16-byte aligned");
    bool taken = false;
    const int rc = w4gemm_tmem_swiglu(A, packed, scales, zeros, H, M, N2, K, static_cast<cudaStream_t>(stream), &taken);
    if (rc != SPK_OK) return rc;
    if (!taken) return fail(SPK_INVALID, "w4gemm_swiglu: shape M=%d N=%d K=%d is outside the fused kernel's scratch (N <= 65536, M * K <= 2 Mi per 64 tokens)", M, N2, K);
    return SPK_OK;
}
