// Launch geometry of the decode (weight-stream) kernels as a host-side rule, and its public view
// (reference include/spark/kernels.h:1033-1052, src/kernels/launch_config.cuh:34-198).
//
// A weight stream saturates DRAM once the bytes outstanding across the device cover bandwidth x
// loaded latency (Little's law). The rule turns that into a CTA count and a K split:
//   need  = ceil(bytes_in_flight / per_cta_in_flight), at least 1
//   split = clamp(ceil(need / tiles), 1, max_split)
//   if need exceeds the resident slots, the tail wave is paid anyway: take the first split in
//   [split, 2 split] whose last wave is >= 87.5% full, else the fullest
//   a forced split (decode_force_split_k / SPARK_DECODE_SPLIT) replaces the rule.
// Named shapes make the rule testable without a GPU: the two the reference names (GB10, RTX 5090)
// with its constants, and B200 (148 SMs, 126 MB L2, 7.7 TB/s HBM3e nominal) with the bytes in flight MEASURED here:
// a read-only stream of bulk copies (spk_stream_probe) reaches ~6 TB/s once ~10 MB are outstanding over the
// device (6.5 TB/s x ~1.5 us loaded latency) and 7.2 TB/s with more; less in flight leaves bandwidth unused.
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "spk_common.cuh"

namespace spk {
namespace {

struct Shape {
    int sm_count;
    int64_t l2_bytes;
    double spec_gbps;
    int64_t bytes_in_flight;
    bool forced;
};

constexpr Shape kGB10 = {48, int64_t{24} << 20, 273.0, 273 * 800, false};
constexpr Shape kRTX5090 = {170, int64_t{96} << 20, 1792.0, int64_t{64} * 24 * 1024, false};
constexpr Shape kB200 = {148, int64_t{126} << 20, 7700.0, int64_t{10} << 20, false};
constexpr double kL2ResidentShare = 0.75;

std::atomic<int> g_forced_split{-1};  // -1: SPARK_DECODE_SPLIT not read yet

int env_int(const char* name) {
    const char* e = std::getenv(name);
    const int n = (e && *e) ? std::atoi(e) : 0;
    return n > 0 ? n : 0;
}

int forced_split() {
    int cur = g_forced_split.load(std::memory_order_relaxed);
    if (cur < 0) {
        int expected = -1;
        g_forced_split.compare_exchange_strong(expected, env_int("SPARK_DECODE_SPLIT"), std::memory_order_relaxed);
        cur = g_forced_split.load(std::memory_order_relaxed);
    }
    return cur;
}

// The current device without touching the scratch arena; falls back to the B200 constants for
// whatever the runtime does not report.
Shape current_shape() {
    Shape s = kB200;
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return s;
    }
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) s.sm_count = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) == cudaSuccess && v > 0) s.l2_bytes = v;
    int clk = 0, width = 0;
    if (cudaDeviceGetAttribute(&clk, cudaDevAttrMemoryClockRate, dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&width, cudaDevAttrGlobalMemoryBusWidth, dev) == cudaSuccess && clk > 0 && width > 0)
        s.spec_gbps = 2.0 * clk * 1e3 * (width / 8.0) / 1e9;
    (void)cudaGetLastError();
    // the measured B200 figure scaled by the bandwidth this device reports (1.3 us of its nominal rate)
    s.bytes_in_flight = static_cast<int64_t>(static_cast<double>(kB200.bytes_in_flight) * s.spec_gbps / kB200.spec_gbps);
    const int forced = env_int("SPARK_FORCE_SMS");
    if (forced > 0) {
        s.sm_count = forced;
        s.forced = true;
    }
    return s;
}

bool shape_of(int device, Shape* out) {
    switch (device) {
        case SPK_DEVICE_CURRENT: *out = current_shape(); return true;
        case SPK_DEVICE_GB10: *out = kGB10; return true;
        case SPK_DEVICE_RTX5090: *out = kRTX5090; return true;
        case SPK_DEVICE_B200: *out = kB200; return true;
        default: return false;
    }
}

int need_ctas(int64_t per_cta, const Shape& d) {
    const int64_t per = per_cta > 1 ? per_cta : 1;
    const int64_t n = cdiv64(d.bytes_in_flight, per);
    return static_cast<int>(n > 1 ? n : 1);
}

// ctas CTAs on `slots` resident slots run in ceil(ctas / slots) waves; the last one is what a split can
// waste. Fractions are compared exactly, as integers: fill = ctas / (waves * slots).
struct WaveFill {
    int64_t ctas, capacity;  // capacity = waves * slots
    bool at_least_seven_eighths() const { return 8 * ctas >= 7 * capacity; }
    bool fuller_than(const WaveFill& o) const { return ctas * o.capacity > o.ctas * capacity; }
};

WaveFill wave_fill(int64_t ctas, int slots) { return {ctas, cdiv64(ctas, slots) * slots}; }

// Little's law first: enough CTAs that their copies in flight cover bandwidth x latency, spread over
// the tiles. When that many CTAs do not fit at once anyway (need > slots) the tail wave is paid
// whatever the split, so among the splits up to twice the minimum the first whose waves are at least
// 7/8 full wins, and failing that the fullest. A forced split overrides everything.
int split_rule(int tiles, int max_split, int64_t per_cta, int slots, const Shape& d) {
    tiles = std::max(tiles, 1);
    max_split = std::max(max_split, 1);
    const int need = need_ctas(per_cta, d);
    int split = std::clamp(cdiv(need, tiles), 1, max_split);
    if (slots > 0 && need > slots) {
        const int last = std::min(max_split, 2 * split);
        int chosen = split;
        WaveFill best = wave_fill(static_cast<int64_t>(tiles) * split, slots);
        for (int s = split; s <= last && !best.at_least_seven_eighths(); ++s) {
            const WaveFill f = wave_fill(static_cast<int64_t>(tiles) * s, slots);
            if (f.at_least_seven_eighths() || f.fuller_than(best)) chosen = s, best = f;
        }
        split = chosen;
    }
    if (const int forced = forced_split(); forced > 0) split = std::clamp(forced, 1, max_split);
    return split;
}

}  // namespace
}  // namespace spk

extern "C" int spk_device_shape_sm_count(void) { return spk::current_shape().sm_count; }
extern "C" int64_t spk_device_shape_l2_bytes(void) { return spk::current_shape().l2_bytes; }
extern "C" double spk_device_shape_spec_gbps(void) { return spk::current_shape().spec_gbps; }
extern "C" int64_t spk_device_shape_bytes_in_flight(void) { return spk::current_shape().bytes_in_flight; }
extern "C" int spk_device_shape_forced(void) { return spk::current_shape().forced ? 1 : 0; }

extern "C" int spk_decode_split_k(int64_t weight_bytes, int tiles, int max_split, int64_t per_cta_in_flight, int slots,
                                  int device) {
    (void)weight_bytes;  // kept for the reference's signature; the split does not depend on it
    spk::Shape d;
    if (!spk::shape_of(device, &d)) return -1;
    return spk::split_rule(tiles, max_split, per_cta_in_flight, slots, d);
}
extern "C" int spk_decode_need_ctas(int64_t per_cta_in_flight, int device) {
    spk::Shape d;
    if (!spk::shape_of(device, &d)) return -1;
    return spk::need_ctas(per_cta_in_flight, d);
}
extern "C" int spk_decode_fits_l2(int64_t bytes, int device) {
    spk::Shape d;
    if (!spk::shape_of(device, &d)) return -1;
    return bytes > 0 && static_cast<double>(bytes) <= spk::kL2ResidentShare * static_cast<double>(d.l2_bytes);
}
extern "C" void spk_decode_force_split_k(int split) { spk::g_forced_split.store(split > 0 ? split : 0, std::memory_order_relaxed); }
extern "C" int spk_decode_forced_split_k(void) { return spk::forced_split(); }
