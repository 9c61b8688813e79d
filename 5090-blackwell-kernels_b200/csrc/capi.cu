// Library-wide pieces of the C-ABI: the error message, per-device state, init and status.
#include <mutex>

#include "ptx_sm100.cuh"
#include "spk_common.cuh"

namespace spk {

namespace {
thread_local char g_error[512] = "";
DeviceState g_devices[kMaxDevices];
std::mutex g_mutex;
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { g_error[0] = '\0'; }

int device_state(DeviceState** out) {
    int dev = 0;
    SPK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(SPK_INVALID, "device ordinal %d not supported (max %d)", dev, kMaxDevices);
    DeviceState& d = g_devices[dev];
    if (!d.ready) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!d.ready) {
            cudaDeviceProp prop;
            SPK_CUDA(cudaGetDeviceProperties(&prop, dev));
            if (prop.major != 10)
                return fail(SPK_UNSUPPORTED, "this library is built for sm_100a only; device %d is sm_%d%d", dev,
                            prop.major, prop.minor);
            d.device = dev;
            d.sm_count = prop.multiProcessorCount;
            d.l2_bytes = prop.l2CacheSize;
            int v = 0;
            if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, dev) == cudaSuccess) d.mem_clock_khz = v;
            if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, dev) == cudaSuccess) d.bus_width_bits = v;
            (void)cudaGetLastError();
            d.max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
            SPK_CUDA(cudaMalloc(&d.partials, kPartialFloats * sizeof(float)));
            SPK_CUDA(cudaMalloc(&d.counters, kCounters * sizeof(unsigned)));
            SPK_CUDA(cudaMalloc(&d.status, kStatusWords * sizeof(int)));
            SPK_CUDA(cudaMalloc(&d.act_scratch, kActScratchBytes));
            SPK_CUDA(cudaMemset(d.partials, 0, kPartialFloats * sizeof(float)));
            SPK_CUDA(cudaMemset(d.counters, 0, kCounters * sizeof(unsigned)));
            SPK_CUDA(cudaMemset(d.status, 0, kStatusWords * sizeof(int)));
            SPK_CUDA(cudaDeviceSynchronize());
            d.ready = true;
        }
    }
    *out = &d;
    return SPK_OK;
}

}  // namespace spk

extern "C" const char* spk_last_error(void) { return spk::g_error; }
extern "C" const char* spk_version(void) { return "spk-b200 0.1 (sm_100a)"; }

extern "C" int spk_init(void) {
    spk::DeviceState* d = nullptr;
    return spk::device_state(&d);
}

extern "C" int spk_device_status(void* stream, int* code) {
    using namespace spk;
    SPK_REQUIRE(code != nullptr, "spk_device_status: null code");
    DeviceState* d = nullptr;
    if (int rc = device_state(&d)) return rc;
    auto st = static_cast<cudaStream_t>(stream);
    int host = 0;
    SPK_CUDA(cudaMemcpyAsync(&host, d->status, sizeof(int), cudaMemcpyDeviceToHost, st));
    SPK_CUDA(cudaStreamSynchronize(st));
    if (host != 0) {
        // A kernel that gave up on a wait returned without its completion step: partial sums and strip
        // counters may be left behind, and every later split-K launch assumes they are zero. Put the
        // scratch back into its clean state together with the status word.
        SPK_CUDA(cudaMemsetAsync(d->partials, 0, kPartialFloats * sizeof(float), st));
        SPK_CUDA(cudaMemsetAsync(d->counters, 0, kCounters * sizeof(unsigned), st));
        SPK_CUDA(cudaMemsetAsync(d->status, 0, sizeof(int), st));
    }
    *code = host;
    return SPK_OK;
}

// ---- a wait that runs out, for tests -------------------------------------------------------------
namespace spk {
namespace {
// One thread waits (a tenth of a millisecond) for a barrier phase that nothing completes,
// exactly as a broken pipeline would make a kernel of this library wait, records SPK_TIMEOUT in the
// status word and returns. Before that it leaves `dirty` floats and counters non-zero, which is the
// state an interrupted split-K kernel leaves behind.
__global__ void expire_wait_kernel(float* partials, unsigned* counters, int dirty, int* status) {
    __shared__ uint64_t bar;
    for (int i = threadIdx.x; i < dirty; i += blockDim.x) {
        partials[i] = 1.0f;
        counters[i] = 1u;
    }
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
        bool done = false;
        const long long t0 = clock64();
        while (!done && clock64() - t0 < 200000) done = ptx::mbar_try_wait(&bar, 0);  // ~0.1 ms, then give up
        if (!done) atomicCAS(status, 0, SPK_TIMEOUT);
    }
}
}  // namespace
}  // namespace spk

extern "C" int spk_debug_expire_wait(int dirty, void* stream) {
    using namespace spk;
    SPK_REQUIRE(dirty >= 0 && dirty <= kCounters, "spk_debug_expire_wait: dirty must be in [0, %d]", kCounters);
    DeviceState* d = nullptr;
    if (int rc = device_state(&d)) return rc;
    expire_wait_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(d->partials, d->counters, dirty, d->status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
