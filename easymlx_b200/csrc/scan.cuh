// Block-wide exclusive prefix sum used by the single-CTA metadata and plan kernels.
#pragma once
#include "common.cuh"

namespace emlx {

constexpr int kMetaThreads = 1024;

// Exclusive prefix sum over data[0..n) in place; returns the total to every thread.
// Each thread owns a contiguous segment; segment totals are scanned through shared memory.
__device__ __forceinline__ int block_exclusive_scan(int32_t* data, int n, int32_t* smem /* [kMetaThreads/32 + 1] */) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (n + kMetaThreads - 1) / kMetaThreads;
    const int begin = min(n, tid * per), end = min(n, begin + per);
    int local = 0;
    for (int i = begin; i < end; ++i) local += data[i];
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) smem[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = smem[lane];
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        smem[lane] = wi - w;  // exclusive offset of each warp
        if (lane == 31) smem[32] = wi;
    }
    __syncthreads();
    int running = smem[warp] + incl - local;
    const int total = smem[32];
    for (int i = begin; i < end; ++i) {
        int v = data[i];
        data[i] = running;
        running += v;
    }
    __syncthreads();
    return total;
}

}  // namespace emlx
