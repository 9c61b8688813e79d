// The int4 weight layouts of the W4A16 path and the register dequantizer.
//
// qweight (GPTQ order): int32 [K/8][N]; word (k/8, n) holds the codes of k = 8 (k/8) + i in bits
// 4i..4i+3 (reference include/spark/kernels.h:380-382).
//
// packed (what w4gemm reads): int32 [N/16][K/64][32][4] = [strip][unit][lane][slot]
// (reference src/kernels/w4gemm_internal.cuh:23-35). One 512-byte block per 16 columns x 64 k;
// a lane's 16 bytes are four words, one per 16-k step; nibble p of a word is the code of
//     column  16 strip + lane/4 + 8 (p & 1)
//     k       128-k group offset given by group_k(step, c = lane % 4, (p >> 1) & 1, p >> 2)
// The k order inside a group is a permutation chosen so that a lane's codes for two steps
// belong to eight consecutive k, 32 (step/2) + 8 c .. + 7. A dot product is free to visit k in
// any order as long as the activations follow the same one.
//
// This layout is an interface contract (the reference's tests compare w4_repack bit for bit),
// so it is kept on B200; the kernels here read it with bulk copies of whole 1 KiB groups.
#pragma once

#include <cuda_bf16.h>

#include <cstdint>

#include "ptx_sm100.cuh"

namespace spk::w4 {

constexpr int kGroup = 128;        // k per scale
constexpr int kStripCols = 16;     // columns per strip
constexpr int kGroupBytes = 1024;  // one strip x one 128-k group of packed codes

// k inside the 128-k group of: step (0..7), lane column c (0..3), upper half of the step's 16 k
// (k_hi) and odd element of the pair (odd).
__host__ __device__ __forceinline__ int group_k(int step, int c, int k_hi, int odd) {
    return 32 * (step >> 1) + 8 * c + 4 * (step & 1) + 2 * k_hi + odd;
}

// Source coordinates of nibble p of word (unit u, lane, slot j): column offset in the strip
// and k offset in the 64-k unit.
__host__ __device__ __forceinline__ void slot_source(int lane, int u, int j, int p, int& dn, int& dk) {
    dn = (lane >> 2) + 8 * (p & 1);
    dk = group_k(4 * (u & 1) + j, lane & 3, (p >> 1) & 1, p >> 2) - 64 * (u & 1);
}

// Where code (n, k) lives: word index into packed and nibble position. Reads the bits of
// a = k % 128 as [6:5] step pair, [4:3] c, [2] step parity, [1] k_hi, [0] odd.
__host__ __device__ __forceinline__ void locate(int n, int k, int K, size_t& word, int& p) {
    const int a = k & 127;
    const int step = 2 * (a >> 5) + ((a >> 2) & 1);
    const int u = 2 * (k >> 7) + (step >> 2);
    const int r = n & 15;
    const int lane = 4 * (r & 7) + ((a >> 3) & 3);
    p = (r >> 3) + 2 * ((a >> 1) & 1) + 4 * (a & 1);
    word = ((static_cast<size_t>(n >> 4) * (K / 64) + u) * 32 + lane) * 4 + (step & 3);
}

// ---- register dequant ------------------------------------------------------------------------
// A packed word holds, for lane (g, c), the four bf16x2 operands of one 16(columns) x 16(k)
// block: x[0] = column g, k pair 2c;  x[1] = column g + 8, k pair 2c;  x[2] = column g, pair
// 2c + 8;  x[3] = column g + 8, pair 2c + 8. Nibbles p and p + 4 land in the low and high half
// of one register: (word >> 4p) & 0x000F000F puts each code in the low mantissa bits of a bf16
// whose exponent field is then set to that of 128, making the halves exactly 128 + q. The
// subtraction of 128 + z is exact and the multiplication by the scale rounds once, which is
// bf16((q - z) * s) bit for bit (reference src/kernels/w4gemm_internal.cuh:96-117 and
// include/spark/kernels.h:369-371).
constexpr uint32_t kNibblePairMask = 0x000F000Fu;
constexpr uint32_t kBias128 = 0x43004300u;   // bf16 128.0 twice
constexpr uint32_t kSymOffset = 0x43084308u; // bf16 136.0 twice = 128 + 8

__device__ __forceinline__ uint32_t offset_pair(uint32_t z) { return kBias128 | z | (z << 16); }
__device__ __forceinline__ uint32_t splat16(uint32_t h) { return h | (h << 16); }

__device__ __forceinline__ void dequant_word(uint32_t q, uint32_t off_lo, uint32_t off_hi,
                                             uint32_t s_lo, uint32_t s_hi, uint32_t (&x)[4]) {
    using namespace spk::ptx;
    x[0] = bf16x2_mul(bf16x2_sub(lop3_and_or(q, kNibblePairMask, kBias128), off_lo), s_lo);
    x[1] = bf16x2_mul(bf16x2_sub(lop3_and_or(q >> 4, kNibblePairMask, kBias128), off_hi), s_hi);
    x[2] = bf16x2_mul(bf16x2_sub(lop3_and_or(q >> 8, kNibblePairMask, kBias128), off_lo), s_lo);
    x[3] = bf16x2_mul(bf16x2_sub(lop3_and_or(q >> 12, kNibblePairMask, kBias128), off_hi), s_hi);
}

}  // namespace spk::w4
