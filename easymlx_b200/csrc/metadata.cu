// Batch metadata on the GPU: prefix sum of query lengths, gather of the scheduled slots' page-table
// rows and lengths, per-token slot mapping.  One CTA; the batch is a few thousand integers.
#include "common.cuh"
#include "plan_device.cuh"

namespace emlx {

#ifdef EMLX_TRACE_META
#define META_STAMP(k) do { if (threadIdx.x == 0) g_meta_trace[k] = clock64(); } while (0)
#else
#define META_STAMP(k) do { } while (0)
#endif

__global__ void __launch_bounds__(kMetaThreads) build_metadata_kernel(
    const int32_t* __restrict__ query_lens, const int32_t* __restrict__ slot_ids, int S, int T,
    const int32_t* __restrict__ bt_all, int num_slots, int MB, int32_t* kv_lens_all, int bs, int advance,
    int32_t* __restrict__ qsl, int32_t* __restrict__ bt_out, int32_t* __restrict__ kv_out,
    int64_t* __restrict__ slot_mapping, int32_t* __restrict__ token_positions, int64_t num_blocks, int32_t* status,
    int32_t* plan, PlanLayout L, int G,
    int window, int class_lo, int class_hi, bool wide, int Hkv, int num_ctas, bool scatter_later, int short_ctas) {
    __shared__ int32_t scan_smem[kMetaThreads / 32 + 1];
    // batches of up to kSmemSeqs sequences keep their prefix sums and lengths in shared memory: every later phase
    // (work list, slot mapping) then reads them without an L2 round trip
    constexpr int kSmemSeqs = 2048, kSmemUnits = 4096;
    __shared__ int32_t s_q[kSmemSeqs + 1], s_kv[kSmemSeqs], s_off[kSmemSeqs], s_cum[kSmemUnits];
    const int tid = threadIdx.x;
    META_STAMP(0);
    // Nothing is read before the wait: the stored lengths were last written by the previous metadata launch, which
    // the immediate predecessor in the stream (a write or an attention kernel that started early) does not order
    // against this grid, and the query lengths / slot ids may come from a kernel that is still running.
    grid_dep_wait();
    grid_dep_launch();
    META_STAMP(1);
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
            bool ok = slot >= 0 && slot < num_slots;
            // A sequence that would outgrow its page-table row is reported and left alone: its stored length
            // stays, none of its rows is written (their slots are -1) and its gathered length is 0, so that
            // attention gives zero rows for it instead of reading past the row.
            if (ok && (int64_t)base + q_len > (int64_t)MB * bs) {
                flag_error(status, EMLX_DEV_OVERFLOW);
                ok = false;
            }
            const int after = ok ? base + q_len : 0;
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
    META_STAMP(2);

    // The page-table gather and the slot mapping do not depend on the work list: their first batch of loads is
    // issued here, before the work list is built, and stored afterwards, so that their two dependent round trips
    // run behind that computation.
    const int64_t cells = (int64_t)S * MB;
    constexpr int kBatch = 4;
    int g_val[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
        const int64_t c = tid + (int64_t)k * kMetaThreads;
        g_val[k] = -1;
        if (c < cells && !scatter_later) {
            const int row = (int)(c / MB), col = (int)(c - (int64_t)row * MB);
            const int slot = slot_ids[row];
            if (slot >= 0 && slot < num_slots) g_val[k] = bt_all[(int64_t)slot * MB + col];
        }
    }
    const int n_tok = min(T, total);
    // slot mapping of token t in two halves: everything up to the page-table load, and the address from the page
    struct TokenProbe { int pos, off, page; bool live; };
    auto probe_token = [&](int t) -> TokenProbe {
        TokenProbe r{0, 0, -1, false};
        if (t >= n_tok) return r;
        const int s = find_sequence(qv, S, t);
        const int slot = s >= 0 ? slot_ids[s] : -1;
        if (slot < 0 || slot >= num_slots) return r;
        const int q_len = qv[s + 1] - qv[s];
        if (kvv[s] < q_len) return r;  // a sequence that would overflow its row: nothing of it is written
        r.pos = kvv[s] - q_len + (t - qv[s]);
        const int page_idx = r.pos / bs;
        if (page_idx >= MB) return r;
        r.off = r.pos - page_idx * bs;
        r.page = bt_all[(int64_t)slot * MB + page_idx];  // not consumed before the work list is built
        r.live = true;
        return r;
    };
    TokenProbe probe{0, 0, -1, false};
    if (slot_mapping != nullptr && tid < T && !scatter_later) probe = probe_token(tid);

    // attention work list in the same launch (lengths after the write are final here)
    if (plan != nullptr)
        build_plan(qv, kvv, S, G, window, class_lo, class_hi, wide, Hkv, num_ctas, plan, L, scan_smem,
                   small ? s_off : nullptr, s_cum, kSmemUnits, short_ctas & 0xff, (short_ctas >> 8) != 0);

    META_STAMP(3);
    if (scatter_later) return;  // a large batch: the gather and the slot mapping run on many CTAs in a second launch
    // gathered page-table rows: the preloaded batch, then the rest
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
        const int64_t c = tid + (int64_t)k * kMetaThreads;
        if (c < cells) bt_out[c] = g_val[k];
    }
    for (int64_t c0 = tid + (int64_t)kBatch * kMetaThreads; c0 < cells; c0 += (int64_t)kBatch * kMetaThreads) {
        int v[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const int64_t c = c0 + (int64_t)k * kMetaThreads;
            v[k] = -1;
            if (c < cells) {
                const int row = (int)(c / MB), col = (int)(c - (int64_t)row * MB);
                const int slot = slot_ids[row];
                if (slot >= 0 && slot < num_slots) v[k] = bt_all[(int64_t)slot * MB + col];
            }
        }
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const int64_t c = c0 + (int64_t)k * kMetaThreads;
            if (c < cells) bt_out[c] = v[k];
        }
    }
    META_STAMP(4);
    if (slot_mapping == nullptr) return;
    for (int t = tid; t < T; t += kMetaThreads) {
        if (t >= kMetaThreads) probe = probe_token(t);
        int64_t dst = -1;
        if (probe.live) {
            if (probe.page >= 0 && probe.page < num_blocks) dst = (int64_t)probe.page * bs + probe.off;
            else flag_error(status, EMLX_DEV_BAD_PAGE);
        }
        slot_mapping[t] = dst;
        if (token_positions) token_positions[t] = probe.pos;
    }
    META_STAMP(5);
}

}  // namespace emlx

namespace emlx {

// Second launch for large batches: page-table gather and slot mapping spread over many CTAs (the first launch does
// them itself when they fit one pass of its single CTA).
__global__ void __launch_bounds__(kMetaThreads) metadata_scatter_kernel(
    const int32_t* __restrict__ slot_ids, int S, int T, const int32_t* __restrict__ bt_all, int num_slots, int MB, int bs,
    const int32_t* __restrict__ qsl, const int32_t* __restrict__ kv_out, int32_t* __restrict__ bt_out,
    int64_t* __restrict__ slot_mapping, int32_t* __restrict__ token_positions, int64_t num_blocks, int32_t* status) {
    grid_dep_wait();  // query_start_loc and the lengths come from the first launch
    grid_dep_launch();
    const int64_t cells = (int64_t)S * MB;
    const int64_t stride = (int64_t)gridDim.x * kMetaThreads;
    for (int64_t c = (int64_t)blockIdx.x * kMetaThreads + threadIdx.x; c < cells; c += stride) {
        const int row = (int)(c / MB), col = (int)(c - (int64_t)row * MB);
        const int slot = slot_ids[row];
        bt_out[c] = (slot >= 0 && slot < num_slots) ? bt_all[(int64_t)slot * MB + col] : -1;
    }
    if (slot_mapping == nullptr) return;
    const int n_tok = min(T, qsl[S]);
    for (int64_t t = (int64_t)blockIdx.x * kMetaThreads + threadIdx.x; t < T; t += stride) {
        int64_t dst = -1;
        int pos = 0;
        if (t < n_tok) {
            const int s = find_sequence(qsl, S, (int)t);
            const int slot = s >= 0 ? slot_ids[s] : -1;
            if (slot >= 0 && slot < num_slots) {
                const int q_len = qsl[s + 1] - qsl[s];
                const bool live = kv_out[s] >= q_len;  // false for a sequence that would overflow its row
                pos = live ? kv_out[s] - q_len + ((int)t - qsl[s]) : 0;
                const int page_idx = pos / bs;
                if (live && page_idx < MB) {
                    const int page = bt_all[(int64_t)slot * MB + page_idx];
                    if (page >= 0 && page < num_blocks) dst = (int64_t)page * bs + (pos - page_idx * bs);
                    else flag_error(status, EMLX_DEV_BAD_PAGE);
                }
            }
        }
        slot_mapping[t] = dst;
        if (token_positions) token_positions[t] = pos;
    }
}

}  // namespace emlx

#ifdef EMLX_TRACE_META
extern "C" __attribute__((visibility("default"))) int emlx_debug_meta_trace(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, emlx::g_meta_trace, sizeof(long long) * 32);
}
#endif

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
        if (!tiled_page_size_ok(block_size, 0)) return fail(EMLX_ERR_UNSUPPORTED, "the attention work list needs page size 16, 32, 64 or 128");
        L = plan_layout(num_seqs, total_tokens, num_q_heads, num_kv_heads);
        if (plan_bytes < (size_t)L.words * sizeof(int32_t))
            return fail(EMLX_ERR_WORKSPACE, "plan buffer smaller than emlx_attn_plan_bytes()");
        G = num_q_heads / num_kv_heads;
        class_range(G, max_query_len, (plan_flags & kPlanWideUnits) != 0, class_lo, class_hi);
    }
    // small batches: one launch does everything; large ones hand the gather and the slot mapping to a second launch
    const int64_t cells = (int64_t)num_seqs * max_blocks_per_seq;
    // (a second launch costs about as much as four passes of the single CTA)
    const bool scatter_later = cells > 16 * kMetaThreads || total_tokens > 4 * kMetaThreads;
    EMLX_CUDA_OK(launch_pdl(build_metadata_kernel, 1, kMetaThreads, 0, (cudaStream_t)stream,
        query_lens, slot_ids, num_seqs, total_tokens, block_tables_all, num_slots, max_blocks_per_seq, kv_lens_all,
        block_size, advance_kv_lens, query_start_loc, block_tables, kv_lens, slot_mapping, token_positions, num_blocks,
        status, (int32_t*)plan, L, G, sliding_window, class_lo, class_hi, (plan_flags & kPlanWideUnits) != 0, num_kv_heads,
        min(num_sms(), kMaxGrid), scatter_later,
        ((plan_flags >> kPlanShortCtasShift) & 0xff) | ((plan_flags & kPlanTwoCtas) ? 0x100 : 0)));
    if (scatter_later) {
        EMLX_LAUNCHED();
        const int64_t work = cells > total_tokens ? cells : (int64_t)total_tokens;
        const int grid = (int)min((int64_t)num_sms(), (work + kMetaThreads - 1) / kMetaThreads);
        EMLX_CUDA_OK(launch_pdl(metadata_scatter_kernel, grid, kMetaThreads, 0, (cudaStream_t)stream, slot_ids, num_seqs,
            total_tokens, block_tables_all, num_slots, max_blocks_per_seq, block_size, (const int32_t*)query_start_loc,
            (const int32_t*)kv_lens, block_tables, slot_mapping, token_positions, num_blocks, status));
    }
    EMLX_LAUNCHED();
    return EMLX_OK;
}
