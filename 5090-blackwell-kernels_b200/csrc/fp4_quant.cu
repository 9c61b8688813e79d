// bf16 -> fp4 (e2m1) quantizers with block scales in the blocked layout the fp4 GEMM reads
// (reference include/spark/kernels.h:332-347, src/kernels/fp4quant.cu:80-174). One thread per scale
// block (16 values NVFP4, 32 MXFP4): 16-byte loads, amax, the block scale, the codes, one packed
// store and one scale byte. Bit-exact contract: the tests compare every byte with the CPU oracle.
#include "fp_codecs.cuh"
#include "spk_common.cuh"

namespace spk {
namespace {

constexpr int kThreads = 256;

struct alignas(16) Bf16x8 {
    __nv_bfloat162 h[4];
};

template <int V>
__device__ __forceinline__ void load_block(float (&f)[V], const __nv_bfloat16* p) {
#pragma unroll
    for (int i = 0; i < V / 8; ++i) {
        const Bf16x8 v = reinterpret_cast<const Bf16x8*>(p)[i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 t = __bfloat1622float2(v.h[j]);
            f[8 * i + 2 * j] = t.x;
            f[8 * i + 2 * j + 1] = t.y;
        }
    }
}

// V codes -> V / 8 words (element 2i in the low nibble of byte i), one vector store.
template <int V>
__device__ __forceinline__ void store_codes(unsigned char* q, const unsigned (&c)[V]) {
    unsigned w[V / 8];
#pragma unroll
    for (int i = 0; i < V / 8; ++i) {
        w[i] = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) w[i] |= c[8 * i + j] << (4 * j);
    }
    if constexpr (V == 16)
        *reinterpret_cast<uint2*>(q) = make_uint2(w[0], w[1]);
    else
        *reinterpret_cast<uint4*>(q) = make_uint4(w[0], w[1], w[2], w[3]);
}

// FORMAT 0: NVFP4 (e4m3 scale per 16 over a per-tensor decode scale s); 1: MXFP4 (2^e per 32,
// e = floor(log2 amax) - 2). Threads past `rows` zero the padding rows' scale bytes.
template <int FORMAT>
__global__ void __launch_bounds__(kThreads)
fp4_quantize_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ q, unsigned char* __restrict__ sf,
                    int rows, int padded_rows, int K, const float* __restrict__ scale,
                    const unsigned* __restrict__ amax_bits, float* __restrict__ scale_out) {
    constexpr int V = FORMAT == 0 ? 16 : 32;
    const int cols = K / V;
    const long long idx = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    float s = 1.0f;
    if (FORMAT == 0) {
        // with an amax cell the decode scale is max|x| / (6 * 448), at least the smallest normal
        s = amax_bits != nullptr ? fmaxf(__fdiv_rn(__uint_as_float(*amax_bits), 6.0f * 448.0f), 1.17549435e-38f)
            : scale != nullptr   ? *scale
                                 : 1.0f;
        if (amax_bits != nullptr && idx == 0) *scale_out = s;
    }
    if (idx >= static_cast<long long>(padded_rows) * cols) return;
    const int r = static_cast<int>(idx / cols), j = static_cast<int>(idx % cols);
    if (r >= rows) {
        sf[fp::sf_offset(r, j, cols)] = 0;
        return;
    }
    float f[V];
    load_block<V>(f, x + static_cast<size_t>(r) * K + j * V);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) amax = fmaxf(amax, fabsf(f[i]));
    unsigned c[V];
    unsigned char sbyte;
    if (FORMAT == 0) {
        sbyte = fp::float_to_e4m3(fminf(__fdiv_rn(__fdiv_rn(amax, 6.0f), s), 448.0f));
        const float denom = fp::e4m3_to_float(sbyte) * s;
#pragma unroll
        for (int i = 0; i < V; ++i) c[i] = denom > 0.f ? fp::float_to_e2m1(__fdiv_rn(f[i], denom)) : 0u;
    } else {
        int p = 0;
        (void)frexpf(amax, &p);
        int e = amax > 0.f ? p - 1 - 2 : -127;
        e = max(-127, min(127, e));
#pragma unroll
        for (int i = 0; i < V; ++i) c[i] = fp::float_to_e2m1(ldexpf(f[i], -e));
        sbyte = static_cast<unsigned char>(e + 127);
    }
    store_codes<V>(q + static_cast<size_t>(r) * (K / 2) + j * (V / 2), c);
    sf[fp::sf_offset(r, j, cols)] = sbyte;
}

}  // namespace
}  // namespace spk

extern "C" size_t spk_fp4_scale_bytes(int rows, int K, int format) {
    const int V = format == SPK_FP4_MXFP4 ? 32 : 16;
    return static_cast<size_t>(spk::cdiv(rows, 128)) * 128 * (K / V);
}

extern "C" int spk_fp4_quantize(const void* x_, unsigned char* q, unsigned char* sf, int rows, int K, const float* scale,
                                int format, void* stream_, unsigned* work, float* scale_out) {
    using namespace spk;
    SPK_REQUIRE(x_ != nullptr && q != nullptr && sf != nullptr, "fp4_quantize: null pointer");
    SPK_REQUIRE(format == SPK_FP4_NVFP4 || format == SPK_FP4_MXFP4, "fp4_quantize: unknown format %d", format);
    SPK_REQUIRE(rows > 0 && K > 0, "fp4_quantize: rows and K must be positive");
    SPK_REQUIRE(K % (format == SPK_FP4_MXFP4 ? 128 : 64) == 0,
                "fp4_quantize: K must be a multiple of 64 (NVFP4) or 128 (MXFP4), got %d", K);
    SPK_REQUIRE(aligned16(x_) && aligned16(q) && aligned16(sf), "fp4_quantize: x, q, sf must be 16-byte aligned");
    SPK_REQUIRE(work == nullptr || (format == SPK_FP4_NVFP4 && scale_out != nullptr),
                "fp4_quantize: a scale computed on the device needs NVFP4 and a scale_out");
    const auto* x = static_cast<const __nv_bfloat16*>(x_);
    auto stream = static_cast<cudaStream_t>(stream_);
    const int padded = cdiv(rows, 128) * 128;
    const int cols = K / (format == SPK_FP4_MXFP4 ? 32 : 16);
    const long long threads = static_cast<long long>(padded) * cols;
    const unsigned grid = static_cast<unsigned>(cdiv64(threads, kThreads));
    if (work != nullptr)
        if (int rc = spk_absmax_bits(x, static_cast<long long>(rows) * K, work, stream_)) return rc;
    if (format == SPK_FP4_NVFP4)
        fp4_quantize_kernel<0><<<grid, kThreads, 0, stream>>>(x, q, sf, rows, padded, K, scale, work, scale_out);
    else
        fp4_quantize_kernel<1><<<grid, kThreads, 0, stream>>>(x, q, sf, rows, padded, K, nullptr, nullptr, nullptr);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
