// Decode attention for callers that cannot allocate device memory: the work list and the split-KV
// workspace live in one file-scope device array instead of caller-provided buffers.
#include "attn_tiled.cuh"
#include "ptx.cuh"

#include <mutex>

namespace {

// Every GPU on which this library runs holds this array from module load until the process exits.
constexpr size_t kStaticScratchBytes = 12u << 20;  // 12 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kStaticMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kStaticMaxDevices] = {};

// In host code the array's name is only a handle; the device address comes from the runtime, once per
// device, with that device current.
int scratch_address(void** out) {
    int dev = 0;
    EMLX_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kStaticMaxDevices) return emlx::fail(EMLX_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        EMLX_CUDA_OK(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        if (!ptr) return emlx::fail(EMLX_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return EMLX_OK;
}

}  // namespace

extern "C" int emlx_attn_decode_static(const emlx_attn_args* args, const emlx_pool* pool, void* stream) {
    using namespace emlx;
    if (!args || !pool) return fail(EMLX_ERR_INVALID, "attention args / pool are NULL");
    if (pool->num_kv_heads <= 0 || args->num_q_heads <= 0 || args->num_q_heads % pool->num_kv_heads)
        return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
    if (args->total_tokens < 0 || args->num_seqs < 0) return fail(EMLX_ERR_INVALID, "total_tokens/num_seqs must be non-negative");
    if (args->total_tokens == 0) return EMLX_OK;
    const int S = args->num_seqs, T = args->total_tokens, Hq = args->num_q_heads, Hkv = pool->num_kv_heads;
    const size_t plan_bytes = (emlx_attn_plan_bytes(S, T, Hq, Hkv) + 255) & ~(size_t)255;
    const WorkspaceLayout W = workspace_layout(S, T, Hq, Hkv, pool->head_dim);
    if (plan_bytes + W.bytes > kStaticScratchBytes)
        return fail(EMLX_ERR_WORKSPACE,
                    "batch too large for the built-in scratch: %d sequences / %d tokens need %zu bytes, the limit is "
                    "%zu; use emlx_attn_decode with caller-provided plan and workspace",
                    S, T, plan_bytes + W.bytes, kStaticScratchBytes);
    void* base = nullptr;
    if (int rc = scratch_address(&base)) return rc;
    unsigned char* plan = (unsigned char*)base;
    unsigned char* workspace = plan + plan_bytes;
    // The array keeps whatever the previous call left: the arrival counters must start at zero.
    EMLX_CUDA_OK(cudaMemsetAsync(workspace + W.counter_off[0], 0, W.bytes - W.counter_off[0], (cudaStream_t)stream));
    if (int rc = emlx_attn_plan(args->query_start_loc, args->kv_lens, S, T, Hq, Hkv, pool->block_size,
                                args->sliding_window, args->max_query_len, 0, plan, plan_bytes, stream))
        return rc;
    emlx_attn_args local = *args;
    // the work list above is built without 128-row units (plan_flags 0), so every row set lands in the classes the
    // decode kernels serve; a caller's row-class hint may speak for a different kind of plan and is dropped
    local.plan_flags = 0;
    local.row_class_mask = 0;
    local.plan = plan;
    local.plan_bytes = plan_bytes;
    local.workspace = workspace;
    local.workspace_bytes = W.bytes;
    return emlx_attn_decode(&local, pool, stream);
}

// ------------------------------------------------------------------------------------------ wait self-test
namespace emlx {
// One warp waits on a barrier that nothing ever completes; the bounded wait gives up after `limit` polls, the
// kernel records EMLX_DEV_WAIT_TIMEOUT and returns normally.  The context stays usable.
__global__ void wait_timeout_selftest_kernel(int32_t* status, uint32_t limit) {
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abort_word = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    const bool done = ptx::mbar_wait(&bar, 0, &abort_word, limit);
    __syncthreads();
    if (threadIdx.x == 0 && (!done || abort_word)) flag_error(status, EMLX_DEV_WAIT_TIMEOUT);
}
}  // namespace emlx

extern "C" int emlx_selftest_wait_timeout(int32_t* status, uint32_t poll_limit, void* stream) {
    using namespace emlx;
    if (!status) return fail(EMLX_ERR_INVALID, "status pointer is NULL");
    if (poll_limit == 0 || poll_limit > (1u << 20)) return fail(EMLX_ERR_INVALID, "poll_limit must be in [1, 2^20]");
    wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, poll_limit);
    EMLX_LAUNCHED();
    return EMLX_OK;
}
