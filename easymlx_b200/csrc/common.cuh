// Shared host/device helpers for the paged-attention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/easymlx_b200.h"

namespace emlx {

// ---------------------------------------------------------------- host side: errors, accounting
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
extern std::atomic<int64_t> g_launches;

#define EMLX_CUDA_OK(expr)                                                                     \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return ::emlx::fail(EMLX_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                                cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define EMLX_LAUNCHED()                                                                        \
    do {                                                                                       \
        ::emlx::g_launches.fetch_add(1, std::memory_order_relaxed);                            \
        EMLX_CUDA_OK(cudaGetLastError());                                                      \
    } while (0)

// Per-device bookkeeping.  Attributes such as the dynamic shared-memory limit of a kernel and the SM count belong
// to a device, not to the process: a process that drives several GPUs needs them once per device.
constexpr int kMaxDevices = 128;

inline int current_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev;
}

// One flag per device ordinal; `needs(dev)` is true until `done(dev)` has been called for that device.  Ordinals
// outside [0, kMaxDevices) are never remembered (the caller then repeats its set-up on every call, which is correct).
struct DeviceOnce {
    std::atomic<uint64_t> mask[kMaxDevices / 64] = {};
    bool needs(int dev) const {
        if (dev < 0 || dev >= kMaxDevices) return true;
        return ((mask[dev >> 6].load(std::memory_order_acquire) >> (dev & 63)) & 1ull) == 0;
    }
    void done(int dev) {
        if (dev >= 0 && dev < kMaxDevices) mask[dev >> 6].fetch_or(1ull << (dev & 63), std::memory_order_release);
    }
};

// Sets the dynamic shared-memory limit of `kernel` once per device.
template <typename K>
inline cudaError_t allow_dynamic_smem(K kernel, int bytes, DeviceOnce& once) {
    const int dev = current_device();
    if (!once.needs(dev)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) once.done(dev);
    return e;
}

inline int num_sms() {
    static std::atomic<int> cached[kMaxDevices] = {};
    const int dev = current_device();
    const bool slot = dev >= 0 && dev < kMaxDevices;
    int n = slot ? cached[dev].load(std::memory_order_relaxed) : 0;
    if (!n) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (slot) cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Launch with programmatic stream serialisation: the kernel may be scheduled while its predecessor in the stream
// drains; it must execute grid_dep_wait() before touching anything the predecessor wrote.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int kQuantGroup = 64;

// ---------------------------------------------------------------- device side
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// Programmatic dependent launch: wait for the predecessor grid's memory, let the successor grid be scheduled.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void flag_error(int32_t* status, int bits) {
    if (status) atomicOr(status, bits);
}

// Largest s in [0, n) with loc[s] <= token < loc[s+1] for a non-decreasing loc[0..n]; rows of
// zero length are skipped.  Returns -1 when token is outside [loc[0], loc[n]).
__device__ __forceinline__ int find_sequence(const int32_t* __restrict__ loc, int n, int token) {
    if (n <= 0 || token < loc[0] || token >= loc[n]) return -1;
    int lo = 0, hi = n;  // invariant: loc[lo] <= token < loc[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (loc[mid] <= token) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace emlx
