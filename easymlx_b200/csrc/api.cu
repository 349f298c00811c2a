// Host-side plumbing of the C ABI: per-thread error text, launch accounting, status read-back.
#include "common.cuh"

#include <cstring>

namespace emlx {

static thread_local char t_error[512] = "";
std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace emlx

extern "C" {

const char* emlx_last_error(void) { return emlx::t_error; }

int emlx_abi_version(void) { return 1; }

int64_t emlx_launch_count(void) { return emlx::g_launches.load(std::memory_order_relaxed); }

int emlx_selftest_device_once(void) {
    // the bookkeeping behind "once per device" set-up, driven with made-up ordinals: no CUDA call is made
    emlx::DeviceOnce once;
    int bad = 0;
    for (int dev : {0, 1, 63, 64, 127}) {
        bad += once.needs(dev) ? 0 : 1;       // nothing is configured at the start
        once.done(dev);
        bad += once.needs(dev) ? 1 : 0;       // ... and this device is afterwards
    }
    bad += once.needs(2) ? 0 : 1;             // a device nobody configured still needs it
    bad += once.needs(65) ? 0 : 1;
    once.done(-1);
    once.done(emlx::kMaxDevices);             // out-of-range ordinals are never remembered
    bad += once.needs(-1) ? 0 : 1;
    bad += once.needs(emlx::kMaxDevices) ? 0 : 1;
    return bad;
}

int emlx_read_status(const int32_t* status, void* stream) {
    if (!status) return emlx::fail(EMLX_ERR_INVALID, "status pointer is NULL");
    int32_t host = 0;
    EMLX_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    EMLX_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    if (host == 0) return EMLX_OK;
    return emlx::fail(EMLX_ERR_DEVICE, "device status 0x%x:%s%s%s%s%s", host,
                      (host & EMLX_DEV_BAD_SLOT) ? " slot id out of range;" : "",
                      (host & EMLX_DEV_BAD_PAGE) ? " page id out of range inside a live sequence;" : "",
                      (host & EMLX_DEV_OVERFLOW) ? " sequence outgrows its page-table row;" : "",
                      (host & EMLX_DEV_TOKEN_MISMATCH) ? " sum(query_lens) != total_tokens;" : "",
                      (host & EMLX_DEV_WAIT_TIMEOUT) ? " in-kernel wait timed out;" : "");
}

}  // extern "C"
