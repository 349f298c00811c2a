// Builds the tiled kernels' work list on the GPU from query_start_loc / kv_lens: which sequences are
// decode-like, which need 32-row blocks, and how many KV tiles each unit covers.  One CTA.
#include "attn_tiled.cuh"
#include "scan.cuh"

namespace emlx {

__device__ __forceinline__ int unit_class(int rows) { return rows <= 8 ? 0 : (rows <= 16 ? 1 : 2); }

__global__ void __launch_bounds__(kMetaThreads) attn_plan_kernel(const int32_t* __restrict__ qsl,
                                                                 const int32_t* __restrict__ kv_lens, int S, int G,
                                                                 int window, int32_t* plan, PlanLayout L) {
    __shared__ int32_t scan_smem[kMetaThreads / 32 + 1];
    const int tid = threadIdx.x;
    int32_t* tmp = plan + L.tmp;
    for (int c = 0; c < kNumClasses; ++c) {
        const int rows_c = class_rows(c);
        int32_t* unit_seq = plan + L.unit_seq[c];
        int32_t* unit_row0 = plan + L.unit_row0[c];
        int32_t* unit_tile_lo = plan + L.unit_tile_lo[c];
        int32_t* unit_cum = plan + L.unit_cum[c];
        for (int s = tid; s < S; s += kMetaThreads) {
            const int q_len = qsl[s + 1] - qsl[s];
            const int rows = q_len * G;
            int n = 0;
            if (q_len > 0 && unit_class(rows) == c) n = (rows + rows_c - 1) / rows_c;
            tmp[s] = n;
        }
        __syncthreads();
        const int num_units = block_exclusive_scan(tmp, S, scan_smem);
        for (int s = tid; s < S; s += kMetaThreads) {
            const int q_len = qsl[s + 1] - qsl[s];
            const int rows = q_len * G;
            if (q_len <= 0 || unit_class(rows) != c) continue;
            const int kv_len = kv_lens[s], ctx = kv_len - q_len;
            const int n = (rows + rows_c - 1) / rows_c;
            for (int u = 0; u < n; ++u) {
                const int row0 = u * rows_c, row1 = min(rows, row0 + rows_c);
                const int i_min = row0 / G, i_max = (row1 - 1) / G;
                const int hi = min(kv_len, ctx + i_max + 1);                       // exclusive end of the last row's keys
                const int lo = window > 0 ? max(0, min(kv_len - 1, ctx + i_min) - window + 1) : 0;
                int tile_lo = 0, ntiles = 1;  // a unit without keys still gets one (fully masked) tile: its rows become 0
                if (hi > 0 && hi > lo) {
                    tile_lo = lo / kTile;
                    ntiles = (hi + kTile - 1) / kTile - tile_lo;
                }
                const int idx = tmp[s] + u;
                unit_seq[idx] = s;
                unit_row0[idx] = row0;
                unit_tile_lo[idx] = tile_lo;
                unit_cum[idx] = ntiles;
            }
        }
        __syncthreads();
        const int total_tiles = block_exclusive_scan(unit_cum, num_units, scan_smem);
        if (tid == 0) {
            unit_cum[num_units] = total_tiles;
            plan[4 * c + 0] = num_units;
            plan[4 * c + 1] = total_tiles;
        }
        __syncthreads();
    }
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
                   int32_t num_q_heads, int32_t num_kv_heads, int32_t block_size, int32_t sliding_window, void* plan,
                   size_t plan_bytes, void* stream) {
    using namespace emlx;
    if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads)
        return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
    if (block_size != kTile) return fail(EMLX_ERR_UNSUPPORTED, "the tiled kernels need page size %d", kTile);
    if (num_seqs < 0 || total_tokens < 0) return fail(EMLX_ERR_INVALID, "num_seqs/total_tokens must be non-negative");
    if (!plan || plan_bytes < emlx_attn_plan_bytes(num_seqs, total_tokens, num_q_heads, num_kv_heads))
        return fail(EMLX_ERR_WORKSPACE, "plan buffer missing or smaller than emlx_attn_plan_bytes()");
    if (num_seqs > 0 && (!query_start_loc || !kv_lens)) return fail(EMLX_ERR_INVALID, "attn_plan: NULL input");
    PlanLayout L = plan_layout(num_seqs, total_tokens, num_q_heads, num_kv_heads);
    attn_plan_kernel<<<1, kMetaThreads, 0, (cudaStream_t)stream>>>(query_start_loc, kv_lens, num_seqs,
                                                                    num_q_heads / num_kv_heads, sliding_window,
                                                                    (int32_t*)plan, L);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // extern "C"
