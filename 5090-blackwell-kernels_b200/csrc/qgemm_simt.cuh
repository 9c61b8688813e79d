// The CUDA-core GEMM of the fp8 and fp4 paths: C = scale * A Bt^T for K-contiguous quantized
// operands, any M, with every scaling mode of the API folded into the operand decode. It is the
// low rungs of the variant ladders (0 and 1), the route for shapes the tensor-core kernels do not
// take, and the definition the faster kernels are tested against on the GPU. One output is one
// thread's fp32 fma chain over k in ascending order, so its bits do not depend on M or on the
// launch: it is also the batch-invariant route.
#pragma once

#include "fp_codecs.cuh"
#include "spk_common.cuh"

namespace spk::simt {

enum Mode { kFp8Tensor = 0, kFp8Mx = 1, kFp8Block128 = 2, kFp4Nv = 3, kFp4Mx = 4 };

struct Params {
    const unsigned char* A;    // [M][K] e4m3 or [M][K/2] packed e2m1
    const unsigned char* Bt;   // [N][K] or [N][K/2]
    __nv_bfloat16* C;          // [M][N]
    int M, N, K;
    const float* scale_a;      // device scalars or null
    const float* scale_b;
    const unsigned char* sfa;  // fp8 MX: [M][K/32] row-major; fp4: blocked layout
    const unsigned char* sfb;
    const float* blk_a;        // fp8 block128: [M][K/128]
    const float* blk_b;        // fp8 block128: [cdiv(N,128)][K/128]
};

constexpr int kBM = 64, kBN = 64, kBK = 64, kPad = 1;

template <int MODE>
__device__ __forceinline__ float decode(const unsigned char* base, const unsigned char* sf, int row, int rows, int k,
                                        int K) {
    if (row >= rows) return 0.f;
    if (MODE == kFp8Tensor || MODE == kFp8Block128) return fp::e4m3_to_float(base[static_cast<size_t>(row) * K + k]);
    if (MODE == kFp8Mx)
        return fp::e4m3_to_float(base[static_cast<size_t>(row) * K + k]) *
               fp::ue8m0_to_float(sf[static_cast<size_t>(row) * (K / 32) + k / 32]);
    const unsigned char byte = base[static_cast<size_t>(row) * (K / 2) + k / 2];
    const float v = fp::e2m1_to_float((k & 1) ? (byte >> 4) : (byte & 15));
    if (MODE == kFp4Nv) return v * fp::e4m3_to_float(sf[fp::sf_offset(row, k / 16, K / 16)]);
    return v * fp::ue8m0_to_float(sf[fp::sf_offset(row, k / 32, K / 32)]);
}

template <int MODE>
__global__ void __launch_bounds__(256) qgemm_simt_kernel(const Params p) {
    __shared__ float As[kBM][kBK + kPad];
    __shared__ float Bs[kBN][kBK + kPad];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
    float acc[4][4] = {}, part[4][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += kBK) {
        for (int i = threadIdx.x; i < kBM * kBK; i += 256) {
            const int r = i / kBK, k = i % kBK;
            As[r][k] = decode<MODE>(p.A, p.sfa, m0 + r, p.M, k0 + k, p.K);
            Bs[r][k] = decode<MODE>(p.Bt, p.sfb, n0 + r, p.N, k0 + k, p.K);
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < kBK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[ty + 16 * i][k], b[i] = Bs[tx + 16 * i][k];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (MODE == kFp8Block128)
                        part[i][j] = fmaf(a[i], b[j], part[i][j]);
                    else
                        acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                }
        }
        if (MODE == kFp8Block128 && ((k0 + kBK) % 128 == 0)) {
            // end of a 128-k block: fold the block's partial sum in with its two fp32 scales
            const int kb = k0 / 128, KB = p.K / 128;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
                    if (m < p.M && n < p.N)
                        acc[i][j] = fmaf(part[i][j],
                                         p.blk_a[static_cast<size_t>(m) * KB + kb] * p.blk_b[static_cast<size_t>(n / 128) * KB + kb],
                                         acc[i][j]);
                    part[i][j] = 0.f;
                }
        }
        __syncthreads();
    }
    const float s = (p.scale_a != nullptr ? *p.scale_a : 1.0f) * (p.scale_b != nullptr ? *p.scale_b : 1.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
            if (m < p.M && n < p.N)
                p.C[static_cast<size_t>(m) * p.N + n] =
                    __float2bfloat16_rn(MODE == kFp8Block128 ? acc[i][j] : acc[i][j] * s);
        }
}

template <int MODE>
inline int launch(const Params& p, cudaStream_t stream) {
    const dim3 grid(cdiv(p.N, kBN), cdiv(p.M, kBM));
    qgemm_simt_kernel<MODE><<<grid, 256, 0, stream>>>(p);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace spk::simt
