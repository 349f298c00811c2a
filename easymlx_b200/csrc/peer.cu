// Host side of the peer-mapped output gather: buffers that other processes on the node can map, and the table of
// the ranks' buffers that the attention kernels read.  The device side is in peer.cuh / attn_tiled.cu.
#include "peer.cuh"

#include <cstring>

namespace emlx {
static_assert(sizeof(cudaIpcMemHandle_t) == EMLX_PEER_HANDLE_BYTES, "handle size");
}

extern "C" {

int emlx_peer_buffer_create(size_t bytes, void** ptr, void* handle) {
    using namespace emlx;
    if (!ptr || !handle || bytes == 0) return fail(EMLX_ERR_INVALID, "peer buffer: null argument or zero size");
    void* p = nullptr;
    EMLX_CUDA_OK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(EMLX_ERR_CUDA, "peer buffer: %s", cudaGetErrorString(e));
    }
    std::memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return EMLX_OK;
}

int emlx_peer_buffer_open(const void* handle, void** ptr) {
    using namespace emlx;
    if (!ptr || !handle) return fail(EMLX_ERR_INVALID, "peer buffer: null argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    EMLX_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return EMLX_OK;
}

int emlx_peer_buffer_close(void* ptr) {
    using namespace emlx;
    if (ptr) EMLX_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return EMLX_OK;
}

int emlx_peer_buffer_free(void* ptr) {
    using namespace emlx;
    if (ptr) EMLX_CUDA_OK(cudaFree(ptr));
    return EMLX_OK;
}

int emlx_gather_init(void* flag_block, void* const* out_ptrs, void* const* flag_ptrs, int32_t num_ranks, int32_t rank,
                     int32_t poll_limit, void* stream) {
    using namespace emlx;
    if (!flag_block || !out_ptrs || !flag_ptrs) return fail(EMLX_ERR_INVALID, "gather: null argument");
    if (num_ranks < 1 || num_ranks > kMaxPeers || rank < 0 || rank >= num_ranks)
        return fail(EMLX_ERR_INVALID, "gather: need 1 <= num_ranks <= %d and 0 <= rank < num_ranks", kMaxPeers);
    if (flag_ptrs[rank] != flag_block) return fail(EMLX_ERR_INVALID, "gather: flag_ptrs[rank] must be this rank's flag block");
    PeerTable t;
    std::memset(&t, 0, sizeof(t));
    for (int r = 0; r < num_ranks; ++r) {
        if (!out_ptrs[r] || !flag_ptrs[r]) return fail(EMLX_ERR_INVALID, "gather: rank %d has no buffer", r);
        if ((uintptr_t)out_ptrs[r] & 15) return fail(EMLX_ERR_INVALID, "gather: output buffers must be 16-byte aligned");
        t.out[r] = out_ptrs[r];
        t.flags[r] = (int32_t*)flag_ptrs[r];
    }
    t.num_ranks = num_ranks;
    t.rank = rank;
    t.poll_limit = poll_limit > 0 ? poll_limit : (1 << 22);
    // pageable source: the copy is staged before the call returns
    EMLX_CUDA_OK(cudaMemcpyAsync((uint8_t*)flag_block + kPeerTableOffset, &t, sizeof(t), cudaMemcpyHostToDevice,
                                 (cudaStream_t)stream));
    return EMLX_OK;
}

}  // extern "C"
