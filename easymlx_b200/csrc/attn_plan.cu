// Builds the tiled kernels' work list on the GPU from query_start_loc / kv_lens: which sequences are
// decode-like, which need 32-row blocks, and how many KV tiles each unit covers.  One CTA.
#include "plan_device.cuh"

namespace emlx {

__global__ void __launch_bounds__(kMetaThreads) attn_plan_kernel(const int32_t* __restrict__ qsl,
                                                                 const int32_t* __restrict__ kv_lens, int S, int G,
                                                                 int window, int class_lo, int class_hi, bool wide,
                                                                 int Hkv, int num_ctas, int32_t* plan, PlanLayout L,
                                                                 int short_ctas) {
    __shared__ int32_t scan_smem[kMetaThreads / 32 + 1];
    grid_dep_wait();
    grid_dep_launch();
    build_plan(qsl, kv_lens, S, G, window, class_lo, class_hi, wide, Hkv, num_ctas, plan, L, scan_smem, nullptr, nullptr, 0,
               short_ctas & 0xff, (short_ctas >> 8) != 0);
}

}  // namespace emlx

extern "C" {

size_t emlx_attn_plan_bytes(int32_t num_seqs, int32_t total_tokens, int32_t num_q_heads, int32_t num_kv_heads) {
    if (num_kv_heads <= 0 || num_q_heads <= 0) return 0;
    return (size_t)emlx::plan_layout(num_seqs, total_tokens, num_q_heads, num_kv_heads).words * sizeof(int32_t);
}

size_t emlx_attn_workspace_bytes(int32_t num_seqs, int32_t total_tokens, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t head_dim) {
    if (num_kv_heads <= 0 || num_q_heads <= 0) return 0;
    return emlx::workspace_layout(num_seqs, total_tokens, num_q_heads, num_kv_heads, head_dim).bytes;
}

int emlx_attn_plan(const int32_t* query_start_loc, const int32_t* kv_lens, int32_t num_seqs, int32_t total_tokens,
                   int32_t num_q_heads, int32_t num_kv_heads, int32_t block_size, int32_t sliding_window,
                   int32_t max_query_len, int32_t plan_flags, void* plan, size_t plan_bytes, void* stream) {
    using namespace emlx;
    if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads)
        return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
    if (!tiled_page_size_ok(block_size, 0)) return fail(EMLX_ERR_UNSUPPORTED, "the attention work list needs page size 16, 32, 64 or 128");
    if (num_seqs < 0 || total_tokens < 0) return fail(EMLX_ERR_INVALID, "num_seqs/total_tokens must be non-negative");
    if (!plan || plan_bytes < emlx_attn_plan_bytes(num_seqs, total_tokens, num_q_heads, num_kv_heads))
        return fail(EMLX_ERR_WORKSPACE, "plan buffer missing or smaller than emlx_attn_plan_bytes()");
    if (num_seqs > 0 && (!query_start_loc || !kv_lens)) return fail(EMLX_ERR_INVALID, "attn_plan: NULL input");
    PlanLayout L = plan_layout(num_seqs, total_tokens, num_q_heads, num_kv_heads);
    int class_lo, class_hi;
    const bool wide = (plan_flags & kPlanWideUnits) != 0;
    class_range(num_q_heads / num_kv_heads, max_query_len, wide, class_lo, class_hi);
    attn_plan_kernel<<<1, kMetaThreads, 0, (cudaStream_t)stream>>>(query_start_loc, kv_lens, num_seqs,
                                                                    num_q_heads / num_kv_heads, sliding_window, class_lo,
                                                                    class_hi, wide, num_kv_heads, min(num_sms(), kMaxGrid),
                                                                    (int32_t*)plan, L,
                                                                    ((plan_flags >> kPlanShortCtasShift) & 0xff) | ((plan_flags & kPlanTwoCtas) ? 0x100 : 0));
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // extern "C"
