// Push all-reduce of a small bf16 tensor across the GPUs of one node, for the row-split
// projections of a tensor-parallel decoder layer (one [tokens, hidden] sum per o / down GEMM).
// At 8 KiB - 512 KiB a ring or tree collective is latency bound; here every rank stores its
// partial tensor straight into a slot of every peer's buffer (plain peer stores over NVLink),
// raises a flag, waits until the flags of all ranks have arrived in ITS OWN memory, and sums the
// slots locally in rank order (fp32, one rounding), so all ranks get identical bits.
//
// Buffer of one rank (the same layout on all, allocated by spk_comm_alloc, opened by the peers
// through CUDA IPC):
//   [0, 1024)      arrival counters, one pair per source rank, 128 bytes apart; they only ever grow:
//                  every call of a counter form adds kCtas per source to the first, and the c-th such
//                  call waits for kCtas * (c + 1); two-phase calls add kCtas to the second (at +64) as well
//   [1024, 1048)   call counter (all forms: selects the half and the flagged words' sequence number),
//                  finished-CTA counter, status word, two-phase call counter, counter-form call counter
//                  (flagged calls raise no arrival counter, so the counter forms count their own calls)
//   [4096, ...)    slots [2][world][slot_elems] bf16, then the flagged inboxes [2][2][slot_elems / 2] cells; call q uses half q % 2, so a rank that is one
//                  call ahead never writes where a slower peer still reads (it cannot be two ahead:
//                  finishing call q + 1 needs the peer's arrival for q + 1, which the peer raises only
//                  after it has left call q)
//
// Two forms, chosen by payload and world size (spk_allreduce_push_bf16 picks, _mode forces):
//   one phase   every rank stores its whole tensor into every peer (world x the tensor per rank,
//               one hop): best while the sum is latency bound
//   two phases  reduce-scatter then all-gather, both by peer stores: rank r receives slice r of every
//               peer's tensor (slots of its first half-region), sums them in rank order, and stores
//               the summed slice into every peer's second region; every rank then copies the other
//               ranks' slices out of its own memory. 2 (world - 1) / world of the tensor per rank
//               and two hops: the form for [64, 4096] (512 KiB) sums over four and eight ranks.
//   flagged     the two phases without any barrier, fence or arrival counter: every 4 bytes of payload
//               travel in an 8-byte store together with the call's sequence number (NVLink delivers
//               an aligned 8-byte store whole), and the receiver polls the payload itself until the
//               number is the one it expects. A hop costs one store latency instead of
//               store + system fence + counter + poll; the price is twice the bytes on the wire.
//               Inboxes of their own behind the slots: [2][ world slices | whole tensor ] of 8-byte cells.
//   flagged, one hop   every rank stores its whole tensor, as flagged words, into its own inbox in every peer and
//               sums the world inboxes (its own tensor from registers) in rank order: one store latency in all,
//               world - 1 times the doubled tensor on the wire. The form for two to four ranks. Inboxes behind the
//               others: [2][world][slot_elems / 4] cells of 16 bytes.
// Every rank gets identical bits either way (a slice is summed once, by its owner). The call counter
// and the half of the buffer it selects are shared by both forms, so they can be mixed freely as
// long as all ranks make the same sequence of calls.
// No kernel here reads peer memory and none uses multimem; every wait is bounded (about a second),
// then the status word is set and the kernel returns.
#include <cstdlib>
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
    int two_phase;  // 0 one phase, 1 two phases with arrival counters, 2 two phases with flagged words, 3 one hop of flagged words
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
    unsigned* cnt1_ptr = seq_ptr + 4;  // calls that raised the first arrival counter (one phase, two phases)
    const unsigned cnt1 = *reinterpret_cast<volatile unsigned*>(cnt1_ptr);
    const unsigned half = seq & 1u;
    const long long vecs = p.n / 8;  // 16-byte vectors
    const long long v0 = vecs * blockIdx.x / gridDim.x, v1 = vecs * (blockIdx.x + 1) / gridDim.x;
    const size_t slot_bytes = static_cast<size_t>(p.slot_elems) * 2;

    if (p.two_phase == 3) {
        // ---- one hop of flagged words: the whole tensor to every peer, summed in rank order where it lands ----
        const unsigned f = seq + 1u == 0u ? 1u : seq + 1u;
        const long long cells = p.n / 4;  // 16-byte cells of two payload words (four bf16) and two flags
        const size_t one_hop = kCommDataOffset + 2 * static_cast<size_t>(p.world) * slot_bytes + 16 * static_cast<size_t>(p.slot_elems) +
                               static_cast<size_t>(half) * p.world * (4 * static_cast<size_t>(p.slot_elems));
        const size_t inbox_bytes = 4 * static_cast<size_t>(p.slot_elems);  // one source's inbox
        const long long g = static_cast<long long>(blockIdx.x) * kCommThreads + threadIdx.x, stride = static_cast<long long>(gridDim.x) * kCommThreads;
        uint2* words = reinterpret_cast<uint2*>(p.data);
        for (long long c = g; c < cells; c += stride) {
            const uint2 d = words[c];
            for (int r = 0; r < p.world; ++r)
                if (r != p.rank)
                    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p.bufs[r] + one_hop + p.rank * inbox_bytes + c * 16),
                                 "r"(d.x), "r"(f), "r"(d.y), "r"(f)
                                 : "memory");
        }
        bool ok = true;
        for (long long c = g; c < cells && ok; c += stride) {
            const uint2 mine = words[c];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < p.world && ok; ++r) {
                uint32_t a = mine.x, b = mine.y;
                if (r != p.rank) {
                    uint32_t fa = 0, fb = 0;
                    unsigned i = 0;
                    for (; i < kCommPolls; ++i) {
                        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb)
                                     : "l"(local + one_hop + r * inbox_bytes + c * 16)
                                     : "memory");
                        if (fa == f && fb == f) break;
                        if (i > 64) __nanosleep(32);
                    }
                    if (i == kCommPolls) {
                        atomicCAS(status, 0, 3);  // SPK_TIMEOUT
                        ok = false;
                        break;
                    }
                }
                const float2 fa2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
                const float2 fb2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b));
                acc[0] += fa2.x, acc[1] += fa2.y, acc[2] += fb2.x, acc[3] += fb2.y;
            }
            if (!ok) break;
            const __nv_bfloat162 oa = __floats2bfloat162_rn(acc[0], acc[1]), ob = __floats2bfloat162_rn(acc[2], acc[3]);
            words[c] = make_uint2(*reinterpret_cast<const uint32_t*>(&oa), *reinterpret_cast<const uint32_t*>(&ob));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(done_ptr, 1u) == gridDim.x - 1) {
                *done_ptr = 0u;
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(seq_ptr) = seq + 1u;
            }
        }
        return;
    }

    if (p.two_phase == 2) {
        // ---- flagged words: payload and sequence number in the same 8-byte store, no barriers ----
        const unsigned f = seq + 1u == 0u ? 1u : seq + 1u;
        const long long pairs = p.n / 4, spairs = pairs / p.world;  // 16-byte cells (two payload words each), per slice
        const size_t ll_half = kCommDataOffset + 2 * static_cast<size_t>(p.world) * slot_bytes + static_cast<size_t>(half) * (8 * p.slot_elems);
        const size_t inbox_b = ll_half + 4 * static_cast<size_t>(p.slot_elems);
        const long long g = static_cast<long long>(blockIdx.x) * kCommThreads + threadIdx.x, stride = static_cast<long long>(gridDim.x) * kCommThreads;
        uint2* words = reinterpret_cast<uint2*>(p.data);
        bool ok = true;
        auto put = [](unsigned char* base, long long cell, uint32_t a, uint32_t b, unsigned flag) {
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(base + cell * 16), "r"(a), "r"(flag), "r"(b), "r"(flag) : "memory");
        };
        auto take = [&](const unsigned char* base, long long cell, uint32_t& a, uint32_t& b) {
            uint32_t fa, fb;
            for (unsigned i = 0; i < kCommPolls; ++i) {
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb) : "l"(base + cell * 16) : "memory");
                if (fa == f && fb == f) return true;
                if (i > 64) __nanosleep(32);
            }
            atomicCAS(status, 0, 3);  // SPK_TIMEOUT
            return false;
        };
        // slice r of the local tensor -> cell [rank][.] of rank r's first inbox
        for (int r = 0; r < p.world; ++r)
            for (long long c = g; c < spairs; c += stride) {
                const uint2 d = words[r * spairs + c];
                put(p.bufs[r] + ll_half, p.rank * spairs + c, d.x, d.y, f);
            }
        // this rank's slice: wait for every source's cell, sum in rank order, keep, and send to every peer's second inbox
        for (long long c = g; c < spairs && ok; c += stride) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < p.world && ok; ++r) {
                uint32_t a, b;
                ok = take(local + ll_half, r * spairs + c, a, b);
                const float2 fa2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
                const float2 fb2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b));
                acc[0] += fa2.x, acc[1] += fa2.y, acc[2] += fb2.x, acc[3] += fb2.y;
            }
            if (!ok) break;
            const __nv_bfloat162 oa = __floats2bfloat162_rn(acc[0], acc[1]), ob = __floats2bfloat162_rn(acc[2], acc[3]);
            const uint32_t wa = *reinterpret_cast<const uint32_t*>(&oa), wb = *reinterpret_cast<const uint32_t*>(&ob);
            words[p.rank * spairs + c] = make_uint2(wa, wb);
            for (int r = 0; r < p.world; ++r)
                if (r != p.rank) put(p.bufs[r] + inbox_b, p.rank * spairs + c, wa, wb, f);
        }
        // the other ranks' summed slices, as they arrive in the second inbox
        for (int r = 0; r < p.world && ok; ++r) {
            if (r == p.rank) continue;
            for (long long c = g; c < spairs && ok; c += stride) {
                uint32_t a, b;
                ok = take(local + inbox_b, r * spairs + c, a, b);
                if (ok) words[r * spairs + c] = make_uint2(a, b);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(done_ptr, 1u) == gridDim.x - 1) {
                *done_ptr = 0u;
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(seq_ptr) = seq + 1u;
            }
        }
        return;
    }

    if (p.two_phase) {
        unsigned* seq2_ptr = seq_ptr + 3;
        const unsigned seq2 = *reinterpret_cast<volatile unsigned*>(seq2_ptr);
        const long long svecs = vecs / p.world;  // vectors per slice
        const long long s0 = svecs * blockIdx.x / gridDim.x, s1 = svecs * (blockIdx.x + 1) / gridDim.x;
        const size_t region = kCommDataOffset + static_cast<size_t>(half) * p.world * slot_bytes;  // this call's half
        const uint4* src = reinterpret_cast<const uint4*>(p.data);
        uint4* dst = reinterpret_cast<uint4*>(p.data);
        __shared__ int failed2;
        if (threadIdx.x == 0) failed2 = 0;
        // ---- phase 1: slice r of the local tensor goes to slot [rank] of rank r's first region ----
        for (int r = 0; r < p.world; ++r) {
            uint4* inbox = reinterpret_cast<uint4*>(p.bufs[r] + region) + static_cast<size_t>(p.rank) * svecs;
            for (long long v = s0 + threadIdx.x; v < s1; v += kCommThreads) inbox[v] = src[r * svecs + v];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            for (int r = 0; r < p.world; ++r)
                atomicAdd_system(reinterpret_cast<unsigned*>(p.bufs[r] + kCommFlagStride * p.rank), 1u);
        }
        auto wait_all = [&](int flag_off, unsigned target) {  // every source's counter in local memory
            if (threadIdx.x < p.world) {
                const unsigned* flag = reinterpret_cast<const unsigned*>(local + kCommFlagStride * threadIdx.x + flag_off);
                bool ok = false;
                for (unsigned i = 0; i < kCommPolls && !ok; ++i) {
                    ok = static_cast<int>(ld_acquire_sys(flag) - target) >= 0;
                    if (!ok) __nanosleep(64);
                }
                if (!ok) {
                    atomicCAS(status, 0, 3);  // SPK_TIMEOUT
                    failed2 = 1;
                }
            }
            __syncthreads();
        };
        wait_all(0, static_cast<unsigned>(gridDim.x) * (cnt1 + 1u));
        // ---- phase 2: sum the world slots of this CTA's share of the local slice in rank order, keep it, and
        // store it into the second region of every peer ----
        if (!failed2) {
            const uint4* slots = reinterpret_cast<const uint4*>(local + region);
            for (long long v = s0 + threadIdx.x; v < s1; v += kCommThreads) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int r = 0; r < p.world; ++r) {
                    const uint4 x = slots[static_cast<size_t>(r) * svecs + v];
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
                dst[p.rank * svecs + v] = out;
                for (int r = 0; r < p.world; ++r)
                    if (r != p.rank) reinterpret_cast<uint4*>(p.bufs[r] + region + slot_bytes)[p.rank * svecs + v] = out;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            for (int r = 0; r < p.world; ++r)
                atomicAdd_system(reinterpret_cast<unsigned*>(p.bufs[r] + kCommFlagStride * p.rank + 64), 1u);
        }
        wait_all(64, static_cast<unsigned>(gridDim.x) * (seq2 + 1u));
        // ---- the other ranks' summed slices, out of local memory ----
        if (!failed2) {
            const uint4* gathered = reinterpret_cast<const uint4*>(local + region + slot_bytes);
            for (int r = 0; r < p.world; ++r) {
                if (r == p.rank) continue;
                for (long long v = s0 + threadIdx.x; v < s1; v += kCommThreads) dst[r * svecs + v] = gathered[r * svecs + v];
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(done_ptr, 1u) == gridDim.x - 1) {
                *done_ptr = 0u;
                *reinterpret_cast<volatile unsigned*>(seq2_ptr) = seq2 + 1u;
                *reinterpret_cast<volatile unsigned*>(cnt1_ptr) = cnt1 + 1u;
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(seq_ptr) = seq + 1u;
            }
        }
        return;
    }

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
        const unsigned target = static_cast<unsigned>(gridDim.x) * (cnt1 + 1u);
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
            *reinterpret_cast<volatile unsigned*>(cnt1_ptr) = cnt1 + 1u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(seq_ptr) = seq + 1u;
        }
    }
}

}  // namespace
}  // namespace spk

extern "C" long long spk_comm_buffer_bytes(int world, long long slot_elems) {
    if (world < 1 || world > spk::kCommMaxWorld || slot_elems < 8) return -1;
    // slots [2][world][slot_elems] bf16, the flagged-word inboxes [2][2][slot_elems / 2] cells of 8 bytes, and the
    // one-hop inboxes [2][world][slot_elems / 4] cells of 16 bytes
    return spk::kCommDataOffset + 2ll * world * slot_elems * 2 + 16ll * slot_elems + 8ll * world * slot_elems;
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

namespace spk {
namespace {
// 0 one phase, 1 two phases with counters, 2 two phases of flagged words, 3 one hop of flagged words. SPK_PUSH_FORM
// overrides. One hop wins while (world - 1) x the doubled tensor is cheap on the wire (measured on four ranks: 8 KiB
// 5.2 us against 8.1 in two phases, 128 KiB 7.0 against 8.5, 512 KiB 16.0 against 11.8); the two-phase form beyond.
int choose_form(bool can_two, int world, long long n) {
    static const int forced = [] {
        const char* e = std::getenv("SPK_PUSH_FORM");
        return e && *e ? std::atoi(e) : -1;
    }();
    if (forced >= 0 && forced <= 3 && (forced == 0 || forced == 3 || can_two)) return forced;
    // one hop while what a rank puts on the wire, (world - 1) x the doubled tensor, stays within 1 MiB
    if (static_cast<long long>(world - 1) * n * 4 <= (1LL << 20) || !can_two) return 3;
    return 2;
}

// mode: 0 choose, 1 one phase, 2 two phases with arrival counters, 3 two phases with flagged words, 4 one hop of flagged words
int allreduce_push(void* data, long long n, void* const* bufs, int rank, int world, long long slot_elems, int mode, void* stream) {
    SPK_REQUIRE(data && bufs, "allreduce_push: null pointer");
    SPK_REQUIRE(world >= 1 && world <= kCommMaxWorld && rank >= 0 && rank < world, "allreduce_push: rank %d of %d", rank, world);
    SPK_REQUIRE(n > 0 && n % 8 == 0 && n <= slot_elems, "allreduce_push: n=%lld must be a multiple of 8 and at most %lld", n,
                slot_elems);
    SPK_REQUIRE(aligned16(data), "allreduce_push: data must be 16-byte aligned");
    SPK_REQUIRE(mode >= 0 && mode <= 4,
                "allreduce_push: mode %d is not 0 (choose), 1 (one phase), 2 (two phases), 3 (flagged words) or 4 (flagged words, one hop)", mode);
    const bool can_two = world >= 2 && n % (8LL * world) == 0;
    SPK_REQUIRE(mode < 2 || mode == 4 || can_two, "allreduce_push: two phases need n a multiple of 8 * world (n=%lld, world=%d)", n, world);
    const int form = mode == 1 ? 0 : mode == 2 ? 1 : mode == 3 ? 2 : mode == 4 ? 3 : choose_form(can_two, world, n);
    CommParams p{};
    for (int r = 0; r < world; ++r) {
        SPK_REQUIRE(bufs[r] != nullptr, "allreduce_push: buffer of rank %d is null", r);
        p.bufs[r] = static_cast<unsigned char*>(bufs[r]);
    }
    p.data = static_cast<__nv_bfloat16*>(data);
    p.n = n, p.slot_elems = slot_elems, p.rank = rank, p.world = world;
    p.two_phase = form;
    SPK_CUDA(launch_chained(allreduce_push_kernel, dim3(kCommCtas), dim3(kCommThreads), 0, static_cast<cudaStream_t>(stream), p));
    return SPK_OK;
}
}  // namespace
}  // namespace spk

extern "C" int spk_allreduce_push_bf16(void* data, long long n, void* const* bufs, int rank, int world, long long slot_elems,
                                       void* stream) {
    return spk::allreduce_push(data, n, bufs, rank, world, slot_elems, 0, stream);
}

extern "C" int spk_allreduce_push_bf16_mode(void* data, long long n, void* const* bufs, int rank, int world, long long slot_elems,
                                            int mode, void* stream) {
    return spk::allreduce_push(data, n, bufs, rank, world, slot_elems, mode, stream);
}
