// Library-wide pieces of the C-ABI: the error message, per-device state, init and status.
#include <mutex>

#include "spk_common.cuh"

namespace spk {

namespace {
thread_local char g_error[512] = "";
constexpr int kMaxDevices = 16;
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
    if (host != 0) SPK_CUDA(cudaMemsetAsync(d->status, 0, sizeof(int), st));
    *code = host;
    return SPK_OK;
}
