// Batch metadata on the GPU: prefix sum of query lengths, gather of the scheduled slots' page-table
// rows and lengths, per-token slot mapping.  One CTA; the batch is a few thousand integers.
#include "common.cuh"
#include "plan_device.cuh"

namespace emlx {

__global__ void __launch_bounds__(kMetaThreads) build_metadata_kernel(
    const int32_t* __restrict__ query_lens, const int32_t* __restrict__ slot_ids, int S, int T,
    const int32_t* __restrict__ bt_all, int num_slots, int MB, int32_t* kv_lens_all, int bs, int advance,
    int32_t* __restrict__ qsl, int32_t* __restrict__ bt_out, int32_t* __restrict__ kv_out,
    int64_t* __restrict__ slot_mapping, int32_t* __restrict__ token_positions, int64_t num_blocks, int32_t* status,
    int32_t* plan, PlanLayout L, int G,
    int window, int class_lo, int class_hi, bool wide, int Hkv, int num_ctas) {
    __shared__ int32_t scan_smem[kMetaThreads / 32 + 1];
    // batches of up to kSmemSeqs sequences keep their prefix sums and lengths in shared memory: every later phase
    // (work list, slot mapping) then reads them without an L2 round trip
    constexpr int kSmemSeqs = 2048, kSmemUnits = 4096;
    __shared__ int32_t s_q[kSmemSeqs + 1], s_kv[kSmemSeqs], s_off[kSmemSeqs], s_cum[kSmemUnits];
    const int tid = threadIdx.x;
    grid_dep_wait();  // a preceding attention kernel may still be reading the plan buffer and the lengths
    grid_dep_launch();
    const bool small = S <= kSmemSeqs;
    int32_t* qv = small ? s_q : qsl;
    int32_t* kvv = small ? s_kv : kv_out;

    int carry = 0;
    for (int i0 = 0; i0 < S; i0 += kMetaThreads) {
        const int i = i0 + tid;
        int q_len = 0, slot = -1, base = 0;
        if (i < S) {
            q_len = max(query_lens[i], 0);
            slot = slot_ids[i];
            if (slot >= 0 && slot < num_slots) base = kv_lens_all[slot];
            else flag_error(status, EMLX_DEV_BAD_SLOT);
        }
        int chunk_total;
        const int excl = carry + block_scan_value(q_len, scan_smem, chunk_total);
        if (i < S) {
            const bool ok = slot >= 0 && slot < num_slots;
            const int after = ok ? base + q_len : 0;
            if (ok && after > MB * bs) flag_error(status, EMLX_DEV_OVERFLOW);
            qv[i] = excl;
            kvv[i] = after;
            if (small) {
                qsl[i] = excl;
                kv_out[i] = after;
            }
            if (ok && advance) kv_lens_all[slot] = after;
        }
        carry += chunk_total;
    }
    const int total = carry;
    if (tid == 0) {
        qv[S] = total;
        if (small) qsl[S] = total;
        if (total != T) flag_error(status, EMLX_DEV_TOKEN_MISMATCH);
    }
    __syncthreads();

    // attention work list in the same launch (lengths after the write are final here)
    if (plan != nullptr)
        build_plan(qv, kvv, S, G, window, class_lo, class_hi, wide, Hkv, num_ctas, plan, L, scan_smem,
                   small ? s_off : nullptr, s_cum, kSmemUnits);

    // gathered page-table rows
    const int64_t cells = (int64_t)S * MB;
    for (int64_t c = tid; c < cells; c += kMetaThreads) {
        int row = (int)(c / MB), col = (int)(c - (int64_t)row * MB);
        int slot = slot_ids[row];
        bt_out[c] = (slot >= 0 && slot < num_slots) ? bt_all[(int64_t)slot * MB + col] : -1;
    }

    if (slot_mapping == nullptr) return;
    const int n = min(T, total);
    for (int t = tid; t < T; t += kMetaThreads) {
        int64_t dst = -1;
        int pos_out = 0;
        if (t < n) {
            int s = find_sequence(qv, S, t);
            int slot = s >= 0 ? slot_ids[s] : -1;
            if (slot >= 0 && slot < num_slots) {
                int q_len = qv[s + 1] - qv[s];
                int pos = kvv[s] - q_len + (t - qv[s]);
                pos_out = pos;
                int page_idx = pos / bs;
                if (page_idx < MB) {
                    int page = bt_all[(int64_t)slot * MB + page_idx];
                    if (page >= 0 && page < num_blocks) dst = (int64_t)page * bs + (pos - page_idx * bs);
                    else flag_error(status, EMLX_DEV_BAD_PAGE);
                }
            }
        }
        slot_mapping[t] = dst;
        if (token_positions) token_positions[t] = pos_out;
    }
}

}  // namespace emlx

extern "C" int emlx_build_metadata(const int32_t* query_lens, const int32_t* slot_ids, int32_t num_seqs,
                                   int32_t total_tokens, const int32_t* block_tables_all, int32_t num_slots,
                                   int32_t max_blocks_per_seq, int32_t* kv_lens_all, int32_t block_size,
                                   int32_t advance_kv_lens, int32_t* query_start_loc, int32_t* block_tables,
                                   int32_t* kv_lens, int64_t* slot_mapping, int32_t* token_positions,
                                   int64_t num_blocks, int32_t* status, int32_t num_q_heads, int32_t num_kv_heads, int32_t sliding_window,
                                   int32_t max_query_len, int32_t plan_flags, void* plan, size_t plan_bytes,
                                   void* stream) {
    using namespace emlx;
    if (num_seqs < 0 || total_tokens < 0) return fail(EMLX_ERR_INVALID, "num_seqs/total_tokens must be non-negative");
    if (block_size <= 0 || max_blocks_per_seq <= 0 || num_slots <= 0)
        return fail(EMLX_ERR_INVALID, "block_size, max_blocks_per_seq and num_slots must be positive");
    if (!query_start_loc || !kv_lens_all || !block_tables_all || (num_seqs > 0 && (!query_lens || !slot_ids)))
        return fail(EMLX_ERR_INVALID, "build_metadata: NULL input");
    if (num_seqs > 0 && (!block_tables || !kv_lens)) return fail(EMLX_ERR_INVALID, "build_metadata: NULL output");
    PlanLayout L{};
    int class_lo = 0, class_hi = -1, G = 1;
    if (plan) {
        if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads)
            return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
        if (block_size != kTile) return fail(EMLX_ERR_UNSUPPORTED, "the attention work list needs page size %d", kTile);
        L = plan_layout(num_seqs, total_tokens, num_q_heads, num_kv_heads);
        if (plan_bytes < (size_t)L.words * sizeof(int32_t))
            return fail(EMLX_ERR_WORKSPACE, "plan buffer smaller than emlx_attn_plan_bytes()");
        G = num_q_heads / num_kv_heads;
        class_range(G, max_query_len, (plan_flags & kPlanWideUnits) != 0, class_lo, class_hi);
    }
    EMLX_CUDA_OK(launch_pdl(build_metadata_kernel, 1, kMetaThreads, 0, (cudaStream_t)stream,
        query_lens, slot_ids, num_seqs, total_tokens, block_tables_all, num_slots, max_blocks_per_seq, kv_lens_all,
        block_size, advance_kv_lens, query_start_loc, block_tables, kv_lens, slot_mapping, token_positions, num_blocks,
        status, (int32_t*)plan, L, G, sliding_window, class_lo, class_hi, (plan_flags & kPlanWideUnits) != 0, num_kv_heads,
        min(num_sms(), kMaxGrid)));
    EMLX_LAUNCHED();
    return EMLX_OK;
}
