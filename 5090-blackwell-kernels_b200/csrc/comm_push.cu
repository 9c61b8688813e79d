// Push all-reduce of a small bf16 tensor across the GPUs of one node, for the row-split
// projections of a tensor-parallel decoder layer (one [tokens, hidden] sum per o / down GEMM).
// At 8 KiB - 512 KiB a ring or tree collective is latency bound; here every rank stores its
// partial tensor straight into a slot of every peer's buffer (plain peer stores over NVLink),
// raises a flag, waits until the flags of all ranks have arrived in ITS OWN memory, and sums the
// slots locally in rank order (fp32, one rounding), so all ranks get identical bits.
//
// Buffer of one rank (the same layout on all, allocated by spk_comm_alloc, opened by the peers
// through CUDA IPC):
//   [0, 1024)      arrival counters, one per source rank, 128 bytes apart; they only ever grow:
//                  every call adds kCtas per source, and call number q waits for kCtas * (q + 1)
//   [1024, 1040)   call counter, finished-CTA counter, status word
//   [4096, ...)    slots [2][world][slot_elems] bf16; call q uses half q % 2, so a rank that is one
//                  call ahead never writes where a slower peer still reads (it cannot be two ahead:
//                  finishing call q + 1 needs the peer's arrival for q + 1, which the peer raises only
//                  after it has left call q)
// No kernel here reads peer memory and none uses multimem; every wait is bounded (about a second),
// then the status word is set and the kernel returns.
#include <cstring>

#include "spk_common.cuh"

namespace spk {
namespace {

constexpr int kCommCtas = 32, kCommThreads = 256, kCommMaxWorld = 8;
constexpr int kCommFlagStride = 128, kCommSeqOffset = 1024, kCommDataOffset = 4096;
constexpr unsigned kCommPolls = 1u << 21;

struct CommParams {
    unsigned char* bufs[kCommMaxWorld];
    __nv_bfloat16* data;
    long long n;           // elements, a multiple of 8
    long long slot_elems;  // capacity of one slot
    int rank, world;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kCommThreads) allreduce_push_kernel(const CommParams p) {
    // Chained launch: the GEMM behind this kernel may start streaming its weights now; this kernel
    // itself starts once the GEMM in front (whose output it sums) has completed.
    pdl_release();
    pdl_wait();
    unsigned char* local = p.bufs[p.rank];
    unsigned* seq_ptr = reinterpret_cast<unsigned*>(local + kCommSeqOffset);
    unsigned* done_ptr = seq_ptr + 1;
    int* status = reinterpret_cast<int*>(seq_ptr + 2);
    const unsigned seq = *reinterpret_cast<volatile unsigned*>(seq_ptr);  // advanced only after every CTA has finished
    const unsigned half = seq & 1u;
    const long long vecs = p.n / 8;  // 16-byte vectors
    const long long v0 = vecs * blockIdx.x / gridDim.x, v1 = vecs * (blockIdx.x + 1) / gridDim.x;
    const size_t slot_bytes = static_cast<size_t>(p.slot_elems) * 2;

    // ---- push this CTA's share of the local tensor into slot [half][rank] of every rank ----
    const uint4* src = reinterpret_cast<const uint4*>(p.data);
    for (long long v = v0 + threadIdx.x; v < v1; v += kCommThreads) {
        const uint4 x = src[v];
        for (int r = 0; r < p.world; ++r)
            *reinterpret_cast<uint4*>(p.bufs[r] + kCommDataOffset + (half * p.world + p.rank) * slot_bytes + v * 16) = x;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // the CTA's stores, ordered before the arrivals
        for (int r = 0; r < p.world; ++r)
            atomicAdd_system(reinterpret_cast<unsigned*>(p.bufs[r] + kCommFlagStride * p.rank), 1u);
    }

    // ---- wait until every rank has delivered all of its CTAs' shares for this call ----
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (threadIdx.x < p.world) {
        const unsigned* flag = reinterpret_cast<const unsigned*>(local + kCommFlagStride * threadIdx.x);
        const unsigned target = static_cast<unsigned>(gridDim.x) * (seq + 1u);
        bool ok = false;
        for (unsigned i = 0; i < kCommPolls && !ok; ++i) {
            ok = static_cast<int>(ld_acquire_sys(flag) - target) >= 0;  // counters wrap together
            if (!ok) __nanosleep(64);
        }
        if (!ok) {
            atomicCAS(status, 0, 3);  // SPK_TIMEOUT
            failed = 1;
        }
    }
    __syncthreads();

    // ---- sum the world slots of this CTA's share in rank order ----
    if (!failed) {
        uint4* dst = reinterpret_cast<uint4*>(p.data);
        for (long long v = v0 + threadIdx.x; v < v1; v += kCommThreads) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < p.world; ++r) {
                const uint4 x = *reinterpret_cast<const uint4*>(local + kCommDataOffset + (half * p.world + r) * slot_bytes + v * 16);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
            uint4 out;
            __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            dst[v] = out;
        }
    }

    // ---- the last CTA to finish opens the next call ----
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done_ptr, 1u) == gridDim.x - 1) {
            *done_ptr = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(seq_ptr) = seq + 1u;
        }
    }
}

}  // namespace
}  // namespace spk

extern "C" long long spk_comm_buffer_bytes(int world, long long slot_elems) {
    if (world < 1 || world > spk::kCommMaxWorld || slot_elems < 8) return -1;
    return spk::kCommDataOffset + 2ll * world * slot_elems * 2;
}

extern "C" int spk_comm_alloc(long long bytes, void** ptr) {
    using namespace spk;
    SPK_REQUIRE(ptr != nullptr && bytes >= kCommDataOffset, "comm_alloc: bad arguments");
    SPK_CUDA(cudaMalloc(ptr, static_cast<size_t>(bytes)));
    SPK_CUDA(cudaMemset(*ptr, 0, static_cast<size_t>(bytes)));
    SPK_CUDA(cudaDeviceSynchronize());
    return SPK_OK;
}

extern "C" int spk_comm_free(void* ptr) {
    using namespace spk;
    SPK_CUDA(cudaFree(ptr));
    return SPK_OK;
}

extern "C" int spk_comm_export(void* ptr, unsigned char* handle64) {
    using namespace spk;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    SPK_REQUIRE(ptr && handle64, "comm_export: null pointer");
    cudaIpcMemHandle_t h;
    SPK_CUDA(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle64, &h, 64);
    return SPK_OK;
}

extern "C" int spk_comm_open(const unsigned char* handle64, void** ptr) {
    using namespace spk;
    SPK_REQUIRE(ptr && handle64, "comm_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    SPK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return SPK_OK;
}

extern "C" int spk_comm_close(void* ptr) {
    using namespace spk;
    SPK_CUDA(cudaIpcCloseMemHandle(ptr));
    return SPK_OK;
}

extern "C" int spk_comm_status(void* local_buf, int* code) {
    using namespace spk;
    SPK_REQUIRE(local_buf && code, "comm_status: null pointer");
    SPK_CUDA(cudaDeviceSynchronize());
    SPK_CUDA(cudaMemcpy(code, static_cast<unsigned char*>(local_buf) + kCommSeqOffset + 8, sizeof(int), cudaMemcpyDeviceToHost));
    return SPK_OK;
}

extern "C" int spk_allreduce_push_bf16(void* data, long long n, void* const* bufs, int rank, int world, long long slot_elems,
                                       void* stream) {
    using namespace spk;
    SPK_REQUIRE(data && bufs, "allreduce_push: null pointer");
    SPK_REQUIRE(world >= 1 && world <= kCommMaxWorld && rank >= 0 && rank < world, "allreduce_push: rank %d of %d", rank, world);
    SPK_REQUIRE(n > 0 && n % 8 == 0 && n <= slot_elems, "allreduce_push: n=%lld must be a multiple of 8 and at most %lld", n,
                slot_elems);
    SPK_REQUIRE(aligned16(data), "allreduce_push: data must be 16-byte aligned");
    CommParams p{};
    for (int r = 0; r < world; ++r) {
        SPK_REQUIRE(bufs[r] != nullptr, "allreduce_push: buffer of rank %d is null", r);
        p.bufs[r] = static_cast<unsigned char*>(bufs[r]);
    }
    p.data = static_cast<__nv_bfloat16*>(data);
    p.n = n, p.slot_elems = slot_elems, p.rank = rank, p.world = world;
    SPK_CUDA(launch_chained(allreduce_push_kernel, dim3(kCommCtas), dim3(kCommThreads), 0, static_cast<cudaStream_t>(stream), p));
    return SPK_OK;
}
