// Read-only stream probe: what a weight stream can reach on this GPU with a given number of CTAs and a
// given number of bytes in flight per CTA. It is the measurement behind the launch rule's device
// constants (bytes in flight = bandwidth x loaded latency; the reference obtained its constants the
// same way, docs/design/hgemm.md:235-244: fix the bytes in flight per CTA, sweep the CTA count; GB/s
// per CTA at small counts gives the loaded latency, the knee gives the chip-wide bytes in flight), and
// the floor the decode GEMMs are compared with (a kernel that only reads the same bytes).
//
// Each CTA owns an equal contiguous share of the buffer and keeps `depth` bulk asynchronous copies
// (TMA engine, 4 KiB each) in flight into a shared-memory ring; nothing consumes the data, a copy's
// completion on its mbarrier is all the kernel waits for.
#include <algorithm>

#include "spk_common.cuh"
#include "ptx_sm100.cuh"

namespace spk {
namespace {

constexpr int kProbeCopy = 4096;
constexpr int kProbeMaxDepth = 48;  // 192 KiB of ring

__global__ void __launch_bounds__(32) stream_probe_kernel(const unsigned char* __restrict__ src, long long bytes, int depth, int* status) {
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ uint64_t bars[kProbeMaxDepth];
    pdl_release();
    const int lane = threadIdx.x;
    const long long copies = bytes / kProbeCopy;
    const long long c0 = copies * blockIdx.x / gridDim.x, c1 = copies * (blockIdx.x + 1) / gridDim.x;
    for (int i = lane; i < depth; i += 32) ptx::mbar_init(&bars[i], 1);
    ptx::fence_mbar_init();
    __syncwarp();
    auto issue = [&](long long c, int slot) {
        ptx::mbar_arrive_expect_tx(&bars[slot], kProbeCopy);
        ptx::bulk_g2s(ring + static_cast<size_t>(slot) * kProbeCopy, src + c * kProbeCopy, kProbeCopy, &bars[slot]);
    };
    if (lane == 0)
        for (long long c = c0; c < c1 && c < c0 + depth; ++c) issue(c, static_cast<int>(c - c0));
    __syncwarp();
    int slot = 0;
    unsigned phase = 0;
    for (long long c = c0; c < c1; ++c) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars[slot], phase, status))) return;
        if (lane == 0 && c + depth < c1) issue(c + depth, slot);
        __syncwarp();
        if (++slot == depth) slot = 0, phase ^= 1u;
    }
}

}  // namespace
}  // namespace spk

extern "C" int spk_stream_probe(const void* src, long long bytes, int ctas, int depth, void* stream) {
    using namespace spk;
    SPK_REQUIRE(src != nullptr && aligned16(src), "stream_probe: src must be a 16-byte aligned device pointer");
    SPK_REQUIRE(bytes >= kProbeCopy && bytes % kProbeCopy == 0, "stream_probe: bytes must be a positive multiple of %d", kProbeCopy);
    SPK_REQUIRE(ctas >= 1 && depth >= 1 && depth <= kProbeMaxDepth, "stream_probe: ctas >= 1 and 1 <= depth <= %d", kProbeMaxDepth);
    DeviceState* dev = nullptr;
    if (int rc = device_state(&dev)) return rc;
    static bool configured[kMaxDevices] = {};
    if (!configured[dev->device]) {
        SPK_CUDA(cudaFuncSetAttribute(stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeMaxDepth * kProbeCopy));
        configured[dev->device] = true;
    }
    SPK_CUDA(launch_chained(stream_probe_kernel, dim3(ctas), dim3(32), static_cast<size_t>(depth) * kProbeCopy,
                            static_cast<cudaStream_t>(stream), static_cast<const unsigned char*>(src), bytes, depth, dev->status));
    return SPK_OK;
}
