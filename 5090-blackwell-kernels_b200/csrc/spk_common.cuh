// Shared host-side plumbing of the library: status codes, the thread-local error message,
// per-device state (properties, the scratch arena, the device status word).
//
// Error model of the C-ABI: every entry point returns an int status and leaves a message
// readable through spk_last_error(). The C++ namespace-spark shim turns SPK_INVALID into
// std::invalid_argument and the others into std::runtime_error, which is the error behaviour
// of the reference's host API (reference include/spark/common.cuh:22-37).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <utility>

#include "../../include/spk.h"

namespace spk {

// printf-style; stores the message for spk_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

#define SPK_REQUIRE(cond, ...)                                   \
    do {                                                         \
        if (!(cond)) return ::spk::fail(SPK_INVALID, __VA_ARGS__); \
    } while (0)

#define SPK_CUDA(call)                                                                        \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return ::spk::fail(SPK_CUDA_ERROR, "%s failed: %s (%s:%d)", #call,                \
                               cudaGetErrorString(e__), __FILE__, __LINE__);                  \
    } while (0)

#define SPK_CHECK_LAUNCH() SPK_CUDA(cudaGetLastError())

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }
inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Scratch every split-K kernel shares on one device. Allocated once per device on first use
// (or by spk_init), never moved or freed, so pointers baked into captured CUDA graphs stay
// valid. The kernels leave partials and counters zeroed when they finish.
struct DeviceState {
    int device = -1;
    int sm_count = 0;
    int64_t l2_bytes = 0;
    int mem_clock_khz = 0;
    int bus_width_bits = 0;
    int max_smem_optin = 0;
    float* partials = nullptr;      // kPartialFloats fp32, zero between launches
    unsigned* counters = nullptr;   // kCounters, zero between launches
    int* status = nullptr;          // kStatusWords device ints: [0] first error code of a kernel
    unsigned char* act_scratch = nullptr;  // kActScratchBytes: re-ordered activations of one GEMM
    bool ready = false;
};

// Device ordinals the library keeps state for; device_state() refuses larger ones, so every per-device
// table below is indexed by an ordinal that has passed that check.
constexpr int kMaxDevices = 16;

constexpr int64_t kPartialFloats = int64_t{64} * 65536;  // 64 tokens x 65536 columns, 16 MiB
constexpr int kCounters = 1 << 16;
constexpr int kStatusWords = 8;
constexpr int64_t kActScratchBytes = int64_t{64} * 32768 * 2;  // 64 tokens x 32768 k of bf16, 4 MiB

// Programmatic dependent launch. A kernel launched through launch_chained() may begin while the
// kernel before it in the stream is still running, provided that kernel has executed
// pdl_release() (griddepcontrol.launch_dependents) in all of its blocks; it must then execute
// pdl_wait() (griddepcontrol.wait: the predecessor has completed and its writes are visible)
// before it reads anything the predecessor may write or writes anything the predecessor may read.
// Only kernels of this library release early, so a kernel of this library that follows foreign work
// starts after that work has completed, as usual. SPK_PDL=0 turns the attribute off.
inline bool pdl_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("SPK_PDL");
        return !(e && *e == '0');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// State of the current device; *out stays valid for the life of the process.
int device_state(DeviceState** out);

}  // namespace spk
