// Library-wide plumbing: version, thread-local error text, cached device facts.
#include <atomic>
#include <climits>
#include <mutex>

#include "common.cuh"

namespace vq {

char *last_error_buf() {
    static thread_local char buf[512] = "";
    return buf;
}

int32_t fail(int32_t code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// Process-wide knobs behind vq_tune(): defaults, and the accepted range of each.
namespace {
struct KnobSpec { int def, lo, hi; };
constexpr KnobSpec kKnobSpec[] = {{2, 2, 4}, {2, 1, 32}, {0, 0, 4}, {0, 0, 1}, {0, 0, 1}};
constexpr int kNumKnobs = sizeof(kKnobSpec) / sizeof(kKnobSpec[0]);
std::atomic<int> g_knobs[kNumKnobs] = {{2}, {2}, {0}, {0}, {0}};
}  // namespace

int knob_get(int knob) { return g_knobs[knob].load(std::memory_order_relaxed); }
int knob_take(int knob) { return g_knobs[knob].exchange(kKnobSpec[knob].def, std::memory_order_relaxed); }

int32_t device_info(DeviceInfo *out) {
    // One entry per device ordinal; filled on first use and read-only afterwards.
    static DeviceInfo cache[64];
    static bool have[64];
    static std::mutex mu;
    int dev = 0;
    VQ_CHECK_CUDA(cudaGetDevice(&dev));
    VQ_REQUIRE(dev >= 0 && dev < 64, VQ_ERR_CUDA, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        cudaDeviceProp p;
        VQ_CHECK_CUDA(cudaGetDeviceProperties(&p, dev));
        cache[dev].sm_count = p.multiProcessorCount;
        cache[dev].cc_major = p.major;
        cache[dev].cc_minor = p.minor;
        cache[dev].smem_optin = p.sharedMemPerBlockOptin;
        have[dev] = true;
    }
    *out = cache[dev];
    VQ_REQUIRE(out->cc_major == 10, VQ_ERR_ARCH,
               "libvqb200 is built for sm_100a only; device %d is sm_%d%d", dev, out->cc_major, out->cc_minor);
    return VQ_OK;
}

}  // namespace vq

extern "C" int32_t vq_version(void) { return 200; }
extern "C" int32_t vq_tune(int32_t knob, int32_t value) {
    using namespace vq;
    if (knob < 0 || knob >= kNumKnobs || value < kKnobSpec[knob].lo || value > kKnobSpec[knob].hi) return INT_MIN;
    return g_knobs[knob].exchange(value, std::memory_order_relaxed);
}
extern "C" const char *vq_last_error(void) { return vq::last_error_buf(); }
