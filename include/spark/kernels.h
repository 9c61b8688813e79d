// C++ host API of the quantized-GEMM path, with the reference's names and signatures
// (namespace spark; the declarations of the reference's include/spark/kernels.h:230-416 and
// :1033-1052), implemented inline over the C ABI of include/spk.h.
//
// Conventions, as in the reference: row-major contiguous matrices, device pointers owned by the
// caller, launches asynchronous on `stream`; a host-side validation failure throws
// std::invalid_argument, anything else std::runtime_error.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>

#include "../spk.h"

namespace spark {

namespace detail {
inline void check(int rc) {
    if (rc == SPK_OK) return;
    if (rc == SPK_INVALID) throw std::invalid_argument(spk_last_error());
    throw std::runtime_error(spk_last_error());
}
}  // namespace detail

// ---- fp8 (e4m3) GEMM: reference kernels.h:260-294 -------------------------------------------
inline void fp8gemm(const __nv_fp8_e4m3* A, const __nv_fp8_e4m3* Bt, __nv_bfloat16* C, int M, int N, int K,
                    const float* scale_a, const float* scale_b, int variant, cudaStream_t stream) {
    detail::check(spk_fp8gemm(A, Bt, C, M, N, K, scale_a, scale_b, variant, stream));
}
inline int fp8gemm_num_variants() { return spk_fp8gemm_num_variants(); }
inline int fp8gemm_default_variant() { return spk_fp8gemm_default_variant(); }
inline bool fp8gemm_supports(int M, int N, int K, int variant) { return spk_fp8gemm_supports(M, N, K, variant) != 0; }
inline void fp8gemm_mx(const __nv_fp8_e4m3* A, const __nv_fp8_e4m3* Bt, __nv_bfloat16* C, int M, int N, int K,
                       const float* scale_a, const float* scale_b, const unsigned char* sfa, const unsigned char* sfb,
                       int variant, cudaStream_t stream) {
    detail::check(spk_fp8gemm_mx(A, Bt, C, M, N, K, scale_a, scale_b, sfa, sfb, variant, stream));
}
inline bool fp8gemm_mx_supports(int M, int N, int K, int variant) { return spk_fp8gemm_mx_supports(M, N, K, variant) != 0; }
inline bool fp8gemm_mx_available() { return spk_fp8gemm_mx_available() != 0; }
enum Fp8gemmV3Route { FP8GEMM_V3_ROUTE_DEFAULT = -1, FP8GEMM_V3_ROUTE_LEGACY = -2 };
inline void fp8gemm_v3_set_route(int route) { spk_fp8gemm_v3_set_route(route); }
inline int fp8gemm_v3_route() { return spk_fp8gemm_v3_route(); }
inline int fp8gemm_v3_num_tiles() { return spk_fp8gemm_v3_num_tiles(); }
inline const char* fp8gemm_v3_route_name(int M, int N, int K, bool mx = false) { return spk_fp8gemm_v3_route_name(M, N, K, mx); }
inline const char* fp8gemm_v4_route_name(int M, int N, int K) { return spk_fp8gemm_v4_route_name(M, N, K); }

// ---- fp4 (e2m1) GEMM and quantizer: reference kernels.h:322-347 -------------------------------
enum Fp4Format { FP4_NVFP4 = 0, FP4_MXFP4 = 1 };
inline void fp4gemm(const unsigned char* A, const unsigned char* Bt, __nv_bfloat16* C, int M, int N, int K,
                    const unsigned char* sfa, const unsigned char* sfb, const float* scale_a, const float* scale_b,
                    int format, int variant, cudaStream_t stream) {
    detail::check(spk_fp4gemm(A, Bt, C, M, N, K, sfa, sfb, scale_a, scale_b, format, variant, stream));
}
inline int fp4gemm_num_variants() { return spk_fp4gemm_num_variants(); }
inline bool fp4gemm_supports(int M, int N, int K, int variant) { return spk_fp4gemm_supports(M, N, K, variant) != 0; }
inline bool fp4gemm_available() { return spk_fp4gemm_available() != 0; }
inline size_t fp4_scale_bytes(int rows, int K, int format) { return spk_fp4_scale_bytes(rows, K, format); }
inline void fp4_quantize(const __nv_bfloat16* x, unsigned char* q, unsigned char* sf, int rows, int K, const float* scale,
                         int format, cudaStream_t stream, unsigned* work = nullptr, float* scale_out = nullptr) {
    detail::check(spk_fp4_quantize(x, q, sf, rows, K, scale, format, stream, work, scale_out));
}

// ---- fp8 activation quantizer: reference kernels.h:359-364 ------------------------------------
enum Fp8QuantMode { FP8Q_TENSOR = 0, FP8Q_ROW = 1, FP8Q_MX = 2 };
inline void absmax_bits(const __nv_bfloat16* x, long long n, unsigned* work, cudaStream_t stream) {
    detail::check(spk_absmax_bits(x, n, work, stream));
}
inline void fp8_quantize(const __nv_bfloat16* x, unsigned char* q, void* scale, unsigned* work, int rows, int K, int mode,
                         cudaStream_t stream) {
    detail::check(spk_fp8_quantize(x, q, scale, work, rows, K, mode, stream));
}

// ---- W4A16: reference kernels.h:373-416 ---------------------------------------------------------
constexpr int kW4GroupSize = 128;
inline void w4_quantize_bf16(const __nv_bfloat16* W, int32_t* qweight, __nv_bfloat16* scales, uint8_t* zeros, int K, int N,
                             cudaStream_t stream) {
    detail::check(spk_w4_quantize_bf16(W, qweight, scales, zeros, K, N, stream));
}
inline void w4_repack(const int32_t* qweight, int32_t* packed, int K, int N, cudaStream_t stream) {
    detail::check(spk_w4_repack(qweight, packed, K, N, stream));
}
inline void w4gemm_bf16(const __nv_bfloat16* A, const int32_t* packed, const __nv_bfloat16* scales, const uint8_t* zeros,
                        __nv_bfloat16* C, int M, int N, int K, int variant, cudaStream_t stream) {
    detail::check(spk_w4gemm_bf16(A, packed, scales, zeros, C, M, N, K, variant, stream));
}
inline int w4gemm_num_variants() { return spk_w4gemm_num_variants(); }
inline int w4gemm_default_variant() { return spk_w4gemm_default_variant(); }
inline bool w4gemm_supports(int M, int N, int K, int variant) { return spk_w4gemm_supports(M, N, K, variant) != 0; }

// ---- launch rules of the decode kernels: reference kernels.h:1033-1052 ---------------------------
inline int device_shape_sm_count() { return spk_device_shape_sm_count(); }
inline int64_t device_shape_l2_bytes() { return spk_device_shape_l2_bytes(); }
inline double device_shape_spec_gbps() { return spk_device_shape_spec_gbps(); }
inline int64_t device_shape_bytes_in_flight() { return spk_device_shape_bytes_in_flight(); }
inline bool device_shape_forced() { return spk_device_shape_forced() != 0; }
enum DecodeDevice { DECODE_DEVICE_CURRENT = 0, DECODE_DEVICE_GB10 = 1, DECODE_DEVICE_RTX5090 = 2, DECODE_DEVICE_B200 = 3 };
inline int decode_split_k(int64_t weight_bytes, int tiles, int max_split, int64_t per_cta_in_flight, int slots,
                          int device = DECODE_DEVICE_CURRENT) {
    return spk_decode_split_k(weight_bytes, tiles, max_split, per_cta_in_flight, slots, device);
}
inline int decode_need_ctas(int64_t per_cta_in_flight, int device = DECODE_DEVICE_CURRENT) {
    return spk_decode_need_ctas(per_cta_in_flight, device);
}
inline bool decode_fits_l2(int64_t bytes, int device = DECODE_DEVICE_CURRENT) { return spk_decode_fits_l2(bytes, device) > 0; }
inline void decode_force_split_k(int split) { spk_decode_force_split_k(split); }
inline int decode_forced_split_k() { return spk_decode_forced_split_k(); }

}  // namespace spark
