/*
 * spk.h -- C ABI of the B200 (sm_100a) quantized-GEMM library.
 *
 * This is the drop-in boundary: plain C, plain pointers and sizes, no C++ or torch types.
 * Every function that launches work is asynchronous on `stream` (a cudaStream_t passed as
 * void*; NULL is the legacy default stream), takes DEVICE pointers owned by the caller, and
 * returns a status code; spk_last_error() gives the message of the calling thread's last
 * failure. Matrices are row-major and contiguous.
 *
 * Each entry point replaces one function of the reference's host API
 * (include/spark/kernels.h in the reference); the citation beside it names the declaration.
 * The C++ header include/spark/kernels.h of this repository re-exports them under the
 * reference's own names and signatures (namespace spark, exceptions instead of codes).
 */
#ifndef SPK_H_
#define SPK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPK_API __attribute__((visibility("default")))

enum {
    SPK_OK = 0,
    SPK_INVALID = 1,     /* host-side validation failed (reference: std::invalid_argument) */
    SPK_CUDA_ERROR = 2,  /* a CUDA call failed (reference: std::runtime_error) */
    SPK_TIMEOUT = 3,     /* a bounded device-side wait gave up (read by spk_device_status) */
    SPK_UNSUPPORTED = 4  /* the device is not an sm_100 part */
};

/* Message of the last failure on the calling thread ("" if none). */
SPK_API const char* spk_last_error(void);
/* Library version string. */
SPK_API const char* spk_version(void);
/* Allocates the per-device scratch (16 MiB of fp32 partials, counters, a status word) for the
 * current device. Every kernel that needs it calls this lazily; call it yourself before
 * capturing a CUDA graph so that no allocation happens during capture. */
SPK_API int spk_init(void);
/* Synchronizes the stream and reads the device status word: *code is SPK_OK unless a kernel's
 * bounded wait timed out (SPK_TIMEOUT). After a timeout the word is cleared and the shared split-K
 * scratch (which the interrupted kernel may have left half summed) is zeroed again on `stream`;
 * the outputs of the GEMMs launched since the last clean status are not to be trusted: run them
 * again. Does not cover spk_w4gemm_bf16_noalloc, which has its own status call below. */
SPK_API int spk_device_status(void* stream, int* code);
/* Test hook, no counterpart in the reference: launches a one-block kernel that leaves `dirty` words of
 * the split-K scratch non-zero, waits a tenth of a millisecond for a barrier phase nothing completes and
 * records SPK_TIMEOUT, i.e. the state a broken pipeline would leave. No fault, no trap; the context
 * stays usable. */
SPK_API int spk_debug_expire_wait(int dirty, void* stream);

/* ---- int4 W4A16 ------------------------------------------------------------------------- */

/* reference include/spark/kernels.h:384-385 (w4_quantize_bf16). W bf16 [K][N]; qweight int32
 * [K/8][N] (GPTQ order); scales bf16 [K/128][N]; zeros u8 [K/128][N] or NULL (symmetric).
 * K % 128 == 0, N % 16 == 0. */
SPK_API int spk_w4_quantize_bf16(const void* W, int32_t* qweight, void* scales, uint8_t* zeros,
                                 int K, int N, void* stream);
/* reference include/spark/kernels.h:390 (w4_repack): qweight -> int32 [N/16][K/64][32][4].
 * K % 64 == 0, N % 16 == 0. */
SPK_API int spk_w4_repack(const int32_t* qweight, int32_t* packed, int K, int N, void* stream);
/* reference include/spark/kernels.h:411-413 (w4gemm_bf16): C bf16 [M][N] = A bf16 [M][K] times
 * bf16((q - z) * s). N % 16 == 0, K % 128 == 0, M >= 1, 16-byte aligned A, packed, scales,
 * zeros. variant 0 scalar (walks the packed layout), 1 CTA per strip with TMA-staged codes and warp MMA, 2 tuned (default), 3 batch invariant. */
SPK_API int spk_w4gemm_bf16(const void* A, const int32_t* packed, const void* scales,
                            const uint8_t* zeros, void* C, int M, int N, int K, int variant,
                            void* stream);
/* No counterpart in the reference. The same GEMM as spk_w4gemm_bf16 variant 2 for callers that
 * must not allocate device memory (a serving engine whose pool owns all of HBM, a process
 * under a hard device-memory cap, latency-critical loops that cannot take cudaMalloc's
 * device-wide synchronisation): the split-K scratch is a fixed array inside the library image (about 8 MiB,
 * held by every GPU that loads the library until the process exits), nothing is allocated or
 * freed. Limits from that array: M <= 64 and N <= 32768, larger sizes return SPK_INVALID. The
 * first call on a device resolves the array's address (make it before any stream capture). All
 * calls on a device share the array; a call clears the part it uses first, and calls that overlap
 * on the GPU race on it, so order them. */
SPK_API int spk_w4gemm_bf16_noalloc(const void* A, const int32_t* packed, const void* scales,
                                    const uint8_t* zeros, void* C, int M, int N, int K, void* stream);
/* No counterpart in the reference. The status word of spk_w4gemm_bf16_noalloc lives in the same fixed
 * array and is NOT the one spk_device_status reads (that call creates the per-device arena, i.e. it
 * allocates). This call waits for `stream`, returns the word in *code (SPK_OK or SPK_TIMEOUT) and
 * clears it, without allocating. A GEMM call does not clear the word, so a timeout stays visible
 * until it is read here. */
SPK_API int spk_w4gemm_noalloc_status(void* stream, int* code);
/* No counterpart in the reference, which runs the gate|up GEMM and then a separate swiglu kernel
 * (python/spark_kernels/engine.py:447-451); its docs name this fusion as the next step (docs/design/llm_quant.md:51-68).
 * spk_w4_interleave_gate_up re-orders the columns of the GPTQ-order tensors of a fused [gate | up] weight
 * (N2 = 2 I columns, N2 % 128 == 0) so that 16-column strips alternate gate, up; repack the result with
 * spk_w4_repack as usual. spk_w4gemm_swiglu_bf16 then computes H bf16 [M][N2 / 2] = silu(A Wgate) * (A Wup)
 * in one launch per 64 tokens (K % 256 == 0), the activation in fp32 on the unrounded sums. */
SPK_API int spk_w4_interleave_gate_up(const int32_t* qweight, const void* scales, const uint8_t* zeros,
                                      int32_t* qweight_out, void* scales_out, uint8_t* zeros_out, int K, int N2,
                                      void* stream);
SPK_API int spk_w4gemm_swiglu_bf16(const void* A, const int32_t* packed, const void* scales, const uint8_t* zeros,
                                   void* H, int M, int N2, int K, void* stream);
/* No counterpart in the reference (its workspaces grow inside the launchers). From 256 tokens up variant 2
 * dequantizes the weight once into a per-device bf16 scratch of N * K * 2 bytes and runs a dense GEMM; the
 * scratch grows on demand with cudaMalloc. Call this with the largest N * K * 2 you will use before
 * capturing a CUDA graph so that no allocation happens during capture. */
SPK_API int spk_w4_prefill_reserve(long long bytes);
/* reference include/spark/kernels.h:414-416 */
SPK_API int spk_w4gemm_num_variants(void);
SPK_API int spk_w4gemm_default_variant(void);
SPK_API int spk_w4gemm_supports(int M, int N, int K, int variant);

/* ---- fp8 e4m3 ------------------------------------------------------------------------------ */

enum { SPK_FP8Q_TENSOR = 0, SPK_FP8Q_ROW = 1, SPK_FP8Q_MX = 2 };  /* reference kernels.h:359 */

/* reference include/spark/kernels.h:362 (absmax_bits): atomicMax of max|x| over n bf16 values into
 * *work as float bits; *work must hold zero or a smaller amax. n % 8 == 0, x 16-byte aligned. */
SPK_API int spk_absmax_bits(const void* x, long long n, unsigned* work, void* stream);
/* reference include/spark/kernels.h:363-364 (fp8_quantize): x bf16 [rows][K] -> q e4m3 [rows][K]
 * plus scales: TENSOR float[1] (work: one zeroed unsigned), ROW float[rows], MX u8 [rows][K/32]. */
SPK_API int spk_fp8_quantize(const void* x, unsigned char* q, void* scale, unsigned* work, int rows,
                             int K, int mode, void* stream);
/* reference include/spark/kernels.h:260-261 (fp8gemm): C bf16 [M][N] = sa sb A Bt^T, A [M][K] and
 * Bt [N][K] e4m3, scale_a / scale_b device fp32 scalars. N % 64 == 0, K % 64 == 0. */
SPK_API int spk_fp8gemm(const void* A, const void* Bt, void* C, int M, int N, int K,
                        const float* scale_a, const float* scale_b, int variant, void* stream);
/* reference include/spark/kernels.h:273-275 (fp8gemm_mx): ue8m0 scales sfa [M][K/32], sfb [N][K/32]
 * row-major; scale_a / scale_b may both be NULL. K % 256 == 0. */
SPK_API int spk_fp8gemm_mx(const void* A, const void* Bt, void* C, int M, int N, int K,
                           const float* scale_a, const float* scale_b, const unsigned char* sfa,
                           const unsigned char* sfb, int variant, void* stream);
/* reference include/spark/kernels.h:262-265,276,280 */
SPK_API int spk_fp8gemm_num_variants(void);
SPK_API int spk_fp8gemm_default_variant(void);
SPK_API int spk_fp8gemm_supports(int M, int N, int K, int variant);
SPK_API int spk_fp8gemm_mx_supports(int M, int N, int K, int variant);
SPK_API int spk_fp8gemm_mx_available(void);
/* reference include/spark/kernels.h:287-294 (variant 3's route; -1 the rule, -2 CUDA cores only) */
SPK_API void spk_fp8gemm_v3_set_route(int route);
SPK_API int spk_fp8gemm_v3_route(void);
SPK_API int spk_fp8gemm_v3_num_tiles(void);
SPK_API const char* spk_fp8gemm_v3_route_name(int M, int N, int K, int mx);
SPK_API const char* spk_fp8gemm_v4_route_name(int M, int N, int K);
/* No counterpart in the reference (its fp8 modes are per-tensor and MX): fp32 block scales, sA
 * [M][K/128] (1 x 128 blocks of A) and sB [cdiv(N,128)][K/128] (128 x 128 blocks of Bt):
 * C = bf16( sum_kb (sum_{k in kb} a b) sA[m][kb] sB[n/128][kb] ). K % 128 == 0, N % 64 == 0. */
SPK_API int spk_fp8gemm_block128(const void* A, const void* Bt, void* C, int M, int N, int K,
                                 const float* sA, const float* sB, void* stream);
/* No counterpart in the reference: the quantizer of that mode. x fp32 [rows][K]; block_rows 1 or
 * 128; s = amax / 448 per block (1 for an all-zero block), q = e4m3(x / s). */
SPK_API int spk_fp8_quantize_block128(const float* x, unsigned char* q, float* scales, int rows, int K,
                                      int block_rows, void* stream);

/* reference include/spark/kernels.h:476-494 (grouped_gemm_fp8, grouped_gemm_swiglu_fp8, grouped_gemm_supports): every
 * expert's GEMM of a mixture-of-experts layer in one persistent launch. A e4m3 [T][K], rows sorted by expert;
 * offsets int32 [E + 1] on the device (offsets[0] == 0, offsets[E] == T, empty experts allowed); W e4m3 [E][N][K];
 * C bf16 [T][N] = scale_a * scale_b[e] * A W[e]^T (scale_a device fp32 [1], scale_b device fp32 [E], either may be
 * NULL: 1). The SwiGLU form takes W with rows alternating gate_j, up_j and writes C [T][N / 2] = silu(G) * U in
 * fp32 from the two scaled sums. 1 <= E <= 512, N % 128 == 0, K % 128 == 0, 16-byte aligned A, W, C. */
SPK_API int spk_grouped_gemm_supports(int E, int N, int K);
SPK_API int spk_grouped_gemm_fp8(const void* A, const void* W, const int32_t* offsets, void* C, int T, int E, int N, int K,
                                 const float* scale_a, const float* scale_b, void* stream);
SPK_API int spk_grouped_gemm_swiglu_fp8(const void* A, const void* W, const int32_t* offsets, void* C, int T, int E, int N,
                                        int K, const float* scale_a, const float* scale_b, void* stream);

/* ---- fp4 e2m1 (NVFP4, MXFP4) -------------------------------------------------------------- */

enum { SPK_FP4_NVFP4 = 0, SPK_FP4_MXFP4 = 1 };  /* reference kernels.h:322 */

/* reference include/spark/kernels.h:331 (fp4_scale_bytes) */
SPK_API size_t spk_fp4_scale_bytes(int rows, int K, int format);
/* reference include/spark/kernels.h:345-347 (fp4_quantize): x bf16 [rows][K] -> q [rows][K/2] and sf
 * (blocked layout, every byte written). NVFP4: `scale` the decode scale (NULL: 1), or with `work`
 * (a zeroed unsigned) max|x| / (6 * 448) computed on the device and written to *scale_out. */
SPK_API int spk_fp4_quantize(const void* x, unsigned char* q, unsigned char* sf, int rows, int K,
                             const float* scale, int format, void* stream, unsigned* work,
                             float* scale_out);
/* reference include/spark/kernels.h:323-325 (fp4gemm). N % 64 == 0, K % 256 == 0. */
SPK_API int spk_fp4gemm(const void* A, const void* Bt, void* C, int M, int N, int K,
                        const unsigned char* sfa, const unsigned char* sfb, const float* scale_a,
                        const float* scale_b, int format, int variant, void* stream);
/* reference include/spark/kernels.h:326-329 */
SPK_API int spk_fp4gemm_num_variants(void);
SPK_API int spk_fp4gemm_supports(int M, int N, int K, int variant);
SPK_API int spk_fp4gemm_available(void);

/* ---- launch rules of the decode kernels ----------------------------------------------------- */

/* reference include/spark/kernels.h:1044 (DecodeDevice) plus the B200 constants */
enum { SPK_DEVICE_CURRENT = 0, SPK_DEVICE_GB10 = 1, SPK_DEVICE_RTX5090 = 2, SPK_DEVICE_B200 = 3 };

/* reference include/spark/kernels.h:1033-1037 (device_shape_*) */
SPK_API int spk_device_shape_sm_count(void);
SPK_API int64_t spk_device_shape_l2_bytes(void);
SPK_API double spk_device_shape_spec_gbps(void);
SPK_API int64_t spk_device_shape_bytes_in_flight(void);
SPK_API int spk_device_shape_forced(void);
/* reference include/spark/kernels.h:1045-1052 (decode_*): host arithmetic, no CUDA call for a named
 * device; -1 for an unknown device. */
SPK_API int spk_decode_split_k(int64_t weight_bytes, int tiles, int max_split,
                               int64_t per_cta_in_flight, int slots, int device);
SPK_API int spk_decode_need_ctas(int64_t per_cta_in_flight, int device);
SPK_API int spk_decode_fits_l2(int64_t bytes, int device);
SPK_API void spk_decode_force_split_k(int split);
SPK_API int spk_decode_forced_split_k(void);
/* No counterpart in the reference's API (its docs describe the measurement, docs/design/hgemm.md:235-244):
 * a read-only stream of `bytes` (a multiple of 4096) from `src` by `ctas` CTAs, each keeping `depth`
 * 4 KiB bulk copies in flight (1..48). Time it with events: the CTA-count sweep gives the loaded
 * latency and the bytes in flight behind the B200 constants of the launch rule, and it is the floor
 * the decode GEMMs are compared with. */
SPK_API int spk_stream_probe(const void* src, long long bytes, int ctas, int depth, void* stream);

/* ---- push all-reduce for the row-split projections of a tensor-parallel layer ---------------
 * No counterpart in the reference (it is single GPU). One process per GPU of one node: every rank
 * allocates a buffer with spk_comm_alloc (spk_comm_buffer_bytes(world, slot_elems) bytes, zeroed),
 * exports it (64-byte CUDA IPC handle), opens the handles of its peers, and passes the world
 * pointers (its own at index rank) to every call. spk_allreduce_push_bf16 sums `n` bf16 elements
 * (n % 8 == 0, n <= slot_elems) in place over all ranks, in rank order in fp32, one rounding: the
 * same bits on every rank. All ranks must make the same sequence of calls. world <= 8. A wait for
 * a peer that does not arrive within about a second sets the status word read by spk_comm_status
 * (SPK_TIMEOUT) and leaves the data unsummed. */
SPK_API long long spk_comm_buffer_bytes(int world, long long slot_elems);
SPK_API int spk_comm_alloc(long long bytes, void** ptr);
SPK_API int spk_comm_free(void* ptr);
SPK_API int spk_comm_export(void* ptr, unsigned char* handle64);
SPK_API int spk_comm_open(const unsigned char* handle64, void** ptr);
SPK_API int spk_comm_close(void* ptr);
SPK_API int spk_comm_status(void* local_buf, int* code);
SPK_API int spk_allreduce_push_bf16(void* data, long long n, void* const* bufs, int rank, int world,
                                    long long slot_elems, void* stream);
/* The same sum with the form forced: mode 1 one phase (every rank stores its whole tensor into every
 * peer), mode 2 two phases (reduce-scatter then all-gather by peer stores and arrival counters), mode 3
 * the two phases with the sequence number travelling inside every 8-byte store (no fence, no counter:
 * the lowest latency), mode 4 one hop of such flagged words (the whole tensor to every peer, summed where it lands:
 * what two to four ranks get by default), mode 0 what spk_allreduce_push_bf16 picks. Modes 2 and 3 need n % (8 world) == 0.
 * Identical bits on every rank in all forms; they may be mixed as long as all ranks make the same calls. */
SPK_API int spk_allreduce_push_bf16_mode(void* data, long long n, void* const* bufs, int rank, int world,
                                         long long slot_elems, int mode, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPK_H_ */
