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
