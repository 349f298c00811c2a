// One step of the paged cache in one launch: batch metadata, the attention work list and the write of the step's new
// K/V rows.
//
// The two-call path (emlx_build_metadata, then emlx_kv_write, which waits for the slot mapping) is a chain of two
// launches whose second half idles until the first is done.  Nothing forces that order: where a new row goes follows
// from the stored length of its slot and the query lengths of the batch, which every CTA can work out for itself.
// One grid therefore does everything at once:
//     CTA 0        prefix sum of the query lengths, lengths after the step, the attention work list
//     CTAs 1..n    the same prefix sum (a few hundred integers), then one warp per (token, kv head): find the
//                  sequence, its slot, the position, the page; store / quantise the K and V rows (optionally rotating
//                  K, and Q in extra warps); then the gather of the scheduled slots' page-table rows
// A batch in which every sequence brings exactly one token (decode) skips the prefix sums altogether.
// The stored lengths are advanced in place, but only after every CTA has read them: each CTA takes a ticket when it is
// done reading, and the one that draws the last ticket does the advance (no CTA waits for another).
#include "kv_write_device.cuh"
#include "plan_device.cuh"

namespace emlx {

long long* trace_buffer();  // measurement aid, NULL unless the build defines EMLX_TRACE

#ifdef EMLX_TRACE_TIMELINE
#define STEP_STAMP(slot) do { if (p.trace && threadIdx.x == 0) { long long now_; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now_)); p.trace[(blockIdx.x == 0 ? 0 : 16 + 8 * (blockIdx.x - 1)) + (slot)] = now_; } } while (0)
#else
#define STEP_STAMP(slot) do { } while (0)
#endif

constexpr int kStepMaxSeqs = 2048;   // prefix sums, lengths and the work list's scans stay in shared memory
constexpr int kStepMaxUnits = 4096;

struct StepParams {
    WriteParams w;  // keys / values / pool / rotation; slot_mapping and positions are not used
    const int32_t* query_lens;  // NULL: every sequence has exactly one token
    const int32_t* slot_ids;
    const int32_t* bt_all;
    int32_t* kv_lens_all;
    int32_t* qsl;
    int32_t* bt_out;
    int32_t* kv_out;
    int32_t* plan;
    int32_t* ticket;
    long long* trace;
    PlanLayout L;
    int S, T, num_slots, MB, advance;
    int warps_per_cta;  // active warps of a write CTA (the others only help with the gather)
    int G, window, class_lo, class_hi, wide, num_ctas, two_per_sm, short_ctas;
};

template <typename TIn>
__global__ void __launch_bounds__(kMetaThreads) cache_step_kernel(const StepParams p) {
    __shared__ int32_t scan_smem[kMetaThreads / 32 + 1];
    __shared__ int32_t s_q[kStepMaxSeqs + 1], s_kv[kStepMaxSeqs], s_off[kStepMaxSeqs], s_cum[kStepMaxUnits];
    __shared__ int s_last;
    // the new rows, the stored lengths and the page table may all come from the launches right before this one
    STEP_STAMP(0);
    grid_dep_wait();
    grid_dep_launch();
    STEP_STAMP(1);
    const int tid = threadIdx.x, lane = tid & 31;
    const emlx_pool& pool = p.w.pool;
    const int S = p.S, MB = p.MB, bs = pool.block_size, Hkv = pool.num_kv_heads;
    const int64_t capacity = (int64_t)MB * bs;
    const bool ragged = p.query_lens != nullptr;

    // ---- every CTA: where the sequences' tokens start in the packed batch
    int total = S;
    if (ragged) {
        int carry = 0;
        for (int i0 = 0; i0 < S; i0 += kMetaThreads) {
            const int i = i0 + tid;
            const int q_len = i < S ? max(p.query_lens[i], 0) : 0;
            int chunk_total;
            const int excl = carry + block_scan_value(q_len, scan_smem, chunk_total);
            if (i < S) s_q[i] = excl;
            carry += chunk_total;
        }
        total = carry;
        if (tid == 0) s_q[S] = total;
        __syncthreads();
    }
    auto q_start = [&](int s) { return ragged ? s_q[s] : s; };

    if (blockIdx.x == 0) {
        // ---- lengths after the step, query_start_loc, the work list
        for (int i = tid; i < S; i += kMetaThreads) {
            const int slot = p.slot_ids[i];
            const int q_len = q_start(i + 1) - q_start(i);
            bool ok = slot >= 0 && slot < p.num_slots;
            int base = 0;
            if (ok) base = p.kv_lens_all[slot];
            else flag_error(p.w.status, EMLX_DEV_BAD_SLOT);
            // a sequence that would outgrow its row is reported and left alone (nothing written, zero rows attended)
            if (ok && (int64_t)base + q_len > capacity) {
                flag_error(p.w.status, EMLX_DEV_OVERFLOW);
                ok = false;
            }
            const int after = ok ? base + q_len : 0;
            s_kv[i] = after;
            p.qsl[i] = q_start(i);
            p.kv_out[i] = after;
        }
        if (tid == 0) {
            p.qsl[S] = total;
            if (total != p.T) flag_error(p.w.status, EMLX_DEV_TOKEN_MISMATCH);
        }
        __syncthreads();
        STEP_STAMP(2);
        if (p.plan != nullptr) {
            if (ragged)
                build_plan(s_q, s_kv, S, p.G, p.window, p.class_lo, p.class_hi, p.wide != 0, Hkv, p.num_ctas, p.plan, p.L,
                           scan_smem, s_off, s_cum, kStepMaxUnits, p.short_ctas, p.two_per_sm != 0);
            else
                build_plan_decode(s_kv, S, p.G, p.window, p.class_lo, Hkv, p.num_ctas, p.plan, p.L, scan_smem, s_cum,
                                  p.two_per_sm != 0);
        }
    } else {
        // ---- the step's rows.  A write CTA has as many threads as the work-list CTA but only its first
        // warps_per_cta warps take a row: the byte-scattered stores of a row keep one SM's store path busy for a
        // microsecond, so a small batch is spread over many SMs rather than packed into a few.
        const int n_tok = min(p.T, total);
        const int64_t kv_warps = p.w.has_pool ? (int64_t)n_tok * Hkv : 0;
        const int64_t q_warps = p.w.q_out != nullptr ? (int64_t)n_tok * p.w.Hq : 0;
        // a large batch has more rows than the grid has active warps: every warp then takes several (a CTA per handful
        // of rows would repeat the scan of the query lengths a thousand times over, in several waves)
        const int64_t all_warps = (int64_t)(gridDim.x - 1) * p.warps_per_cta;
        for (int64_t gw = (int64_t)(blockIdx.x - 1) * p.warps_per_cta + (tid >> 5);
             (tid >> 5) < p.warps_per_cta && gw < kv_warps + q_warps; gw += all_warps) {
            const bool is_kv = gw < kv_warps;
            const int t = is_kv ? (int)(gw / Hkv) : (int)((gw - kv_warps) / p.w.Hq);
            const int h = (int)(gw - (int64_t)t * Hkv);
            const bool rotate = p.w.rope_dims > 0;
            // the rows do not depend on where they go: their loads are issued ahead of the slot -> length -> page
            // chain (a rotated key needs its position first and is loaded afterwards)
            RowRegs rows;
            if (is_kv && !rotate) load_token_head<TIn>(p.w, t, h, lane, -1, rows);
            const int s = ragged ? find_sequence(s_q, S, t) : t;
            const int slot = s >= 0 ? p.slot_ids[s] : -1;
            if (slot >= 0 && slot < p.num_slots) {
                const int base = p.kv_lens_all[slot];
                const int q_len = q_start(s + 1) - q_start(s);
                const int pos = base + (t - q_start(s));  // the token's position in its sequence
                const int page_idx = pos / bs;
                if ((int64_t)base + q_len <= capacity && page_idx < MB) {
                    if (is_kv) {
                        const int page = p.bt_all[(int64_t)slot * MB + page_idx];
                        STEP_STAMP(4);
                        if (rotate) load_token_head<TIn>(p.w, t, h, lane, pos, rows);
                        if (page >= 0 && page < pool.num_blocks)
                            store_token_head<TIn>(p.w, h, lane, (int64_t)page * bs + (pos - page_idx * bs), rows);
                        else if (lane == 0)
                            flag_error(p.w.status, EMLX_DEV_BAD_PAGE);
                        STEP_STAMP(5);
                    } else {
                        rotate_query_row<TIn>(p.w, gw - kv_warps, lane, pos);
                    }
                }
            }
        }
        // rows of the scheduled slots, for the attention kernels
        const int64_t cells = (int64_t)S * MB, stride = (int64_t)(gridDim.x - 1) * kMetaThreads;
        for (int64_t c = (int64_t)(blockIdx.x - 1) * kMetaThreads + tid; c < cells; c += stride) {
            const int row = (int)(c / MB), col = (int)(c - (int64_t)row * MB);
            const int slot = p.slot_ids[row];
            p.bt_out[c] = (slot >= 0 && slot < p.num_slots) ? p.bt_all[(int64_t)slot * MB + col] : -1;
        }
    }

    STEP_STAMP(blockIdx.x == 0 ? 3 : 2);
    // A step that leaves the stored lengths alone (every layer but one of an engine step) is finished here.
    if (!p.advance) return;
    // Every load of the stored lengths in this CTA is behind us.  The CTA with the last ticket knows that this holds
    // for the whole grid and advances them.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_last = atomicAdd(p.ticket, 1) == (int)gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) {
        STEP_STAMP(blockIdx.x == 0 ? 4 : 3);
        return;
    }
    __threadfence();
    for (int i = tid; i < S; i += kMetaThreads) {
        const int slot = p.slot_ids[i];
        if (slot < 0 || slot >= p.num_slots) continue;
        const int q_len = q_start(i + 1) - q_start(i);
        const int base = p.kv_lens_all[slot];
        if ((int64_t)base + q_len <= capacity) p.kv_lens_all[slot] = base + q_len;
    }
    if (tid == 0) *p.ticket = 0;  // ready for the next launch
    STEP_STAMP(blockIdx.x == 0 ? 4 : 3);
}

template <typename TIn>
static int launch_step(const StepParams& p, unsigned grid, cudaStream_t stream) {
    // The attention kernels that follow take nearly all of an SM's shared memory.  With the same split between L1 and
    // shared memory here, their CTAs can move in beside this kernel's last ones instead of waiting for the SM to drain
    // and switch its configuration.
    static DeviceOnce configured;
    const int dev = current_device();
    if (configured.needs(dev)) {
        EMLX_CUDA_OK(cudaFuncSetAttribute(cache_step_kernel<TIn>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          (int)cudaSharedmemCarveoutMaxShared));
        configured.done(dev);
    }
    EMLX_CUDA_OK(launch_pdl(cache_step_kernel<TIn>, grid, kMetaThreads, 0, stream, p));
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // namespace emlx

extern "C" int emlx_kv_write_step(const void* queries, void* queries_out, const void* keys, const void* values,
                                  int32_t in_dtype, const int32_t* query_lens, const int32_t* slot_ids, int32_t num_seqs,
                                  int32_t total_tokens, const int32_t* block_tables_all, int32_t num_slots,
                                  int32_t max_blocks_per_seq, int32_t* kv_lens_all, int32_t advance_kv_lens,
                                  const emlx_pool* pool, const emlx_rope* rope, int32_t* query_start_loc,
                                  int32_t* block_tables, int32_t* kv_lens, int32_t num_q_heads, int32_t sliding_window,
                                  int32_t max_query_len, int32_t plan_flags, void* plan, size_t plan_bytes, int32_t* ticket,
                                  int32_t* status, void* stream) {
    using namespace emlx;
    if (int rc = validate_pool(pool)) return rc;
    if (num_seqs < 0 || total_tokens < 0) return fail(EMLX_ERR_INVALID, "num_seqs/total_tokens must be non-negative");
    if (num_seqs == 0) return EMLX_OK;
    if (num_seqs > kStepMaxSeqs)
        return fail(EMLX_ERR_UNSUPPORTED, "the single-launch step takes up to %d sequences; use emlx_build_metadata + emlx_kv_write",
                    kStepMaxSeqs);
    if (!query_lens && total_tokens != num_seqs)
        return fail(EMLX_ERR_INVALID, "without query_lens every sequence has one token: total_tokens must equal num_seqs");
    if (max_blocks_per_seq <= 0 || num_slots <= 0) return fail(EMLX_ERR_INVALID, "max_blocks_per_seq and num_slots must be positive");
    if (!slot_ids || !block_tables_all || !kv_lens_all || !query_start_loc || !block_tables || !kv_lens || !ticket)
        return fail(EMLX_ERR_INVALID, "kv_write_step: NULL argument");
    if (total_tokens > 0 && (!keys || !values)) return fail(EMLX_ERR_INVALID, "kv_write_step: NULL key/value input");
    StepParams p{};
    p.w.keys = keys; p.w.values = values; p.w.pool = *pool; p.w.T = total_tokens; p.w.status = status; p.w.has_pool = 1;
    if (rope) {
        if (!rope->inv_freq) return fail(EMLX_ERR_INVALID, "rope parameters are NULL");
        if (rope->dims <= 0 || (rope->dims & 1) || rope->dims > pool->head_dim)
            return fail(EMLX_ERR_INVALID, "rope dims must be positive, even and at most head_dim");
        p.w.inv_freq = rope->inv_freq; p.w.rope_dims = rope->dims; p.w.traditional = rope->traditional;
        p.w.pos_scale = rope->position_scale; p.w.mscale = rope->mscale;
        if (queries_out) {
            if (!queries || num_q_heads <= 0) return fail(EMLX_ERR_INVALID, "kv_write_step: queries / num_q_heads missing");
            p.w.q_in = queries; p.w.q_out = queries_out; p.w.Hq = num_q_heads;
        }
    }
    p.w.raw_ok = raw_copy_ok(p.w, in_dtype);
    p.trace = trace_buffer();
    p.query_lens = query_lens; p.slot_ids = slot_ids; p.bt_all = block_tables_all; p.kv_lens_all = kv_lens_all;
    p.qsl = query_start_loc; p.bt_out = block_tables; p.kv_out = kv_lens; p.ticket = ticket;
    p.S = num_seqs; p.T = total_tokens; p.num_slots = num_slots; p.MB = max_blocks_per_seq; p.advance = advance_kv_lens;
    p.class_lo = 0; p.class_hi = -1; p.G = 1;
    if (plan && total_tokens > 0) {
        const int Hkv = pool->num_kv_heads;
        if (num_q_heads <= 0 || num_q_heads % Hkv) return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
        if (!tiled_page_size_ok(pool->block_size, 0)) return fail(EMLX_ERR_UNSUPPORTED, "the attention work list needs page size 16, 32, 64 or 128");
        p.L = plan_layout(num_seqs, total_tokens, num_q_heads, Hkv);
        if (plan_bytes < (size_t)p.L.words * sizeof(int32_t)) return fail(EMLX_ERR_WORKSPACE, "plan buffer smaller than emlx_attn_plan_bytes()");
        p.G = num_q_heads / Hkv;
        p.wide = (plan_flags & kPlanWideUnits) != 0;
        p.two_per_sm = (plan_flags & kPlanTwoCtas) != 0;
        p.short_ctas = (plan_flags >> kPlanShortCtasShift) & 0xff;
        class_range(p.G, query_lens ? max_query_len : 1, p.wide != 0, p.class_lo, p.class_hi);
        p.plan = (int32_t*)plan; p.window = sliding_window; p.num_ctas = min(num_sms(), kMaxGrid);
    }
    const int64_t warps = (int64_t)total_tokens * pool->num_kv_heads + (p.w.q_out ? (int64_t)total_tokens * num_q_heads : 0);
    // about two write CTAs per SM at most; at least 4 and at most 32 rows per CTA
    const int64_t per_cta = (warps + 2 * num_sms() - 1) / (2 * num_sms());
    p.warps_per_cta = (int)(per_cta < 4 ? 4 : (per_cta > kMetaThreads / 32 ? kMetaThreads / 32 : per_cta));
    int64_t write_ctas = (warps + p.warps_per_cta - 1) / p.warps_per_cta;
    if (write_ctas > 2 * num_sms()) write_ctas = 2 * num_sms();  // one wave: the warps loop over the remaining rows
    const unsigned grid = 1u + (unsigned)(write_ctas > 0 ? write_ctas : 1);
    switch (in_dtype) {
        case EMLX_F16: return launch_step<__half>(p, grid, (cudaStream_t)stream);
        case EMLX_BF16: return launch_step<__nv_bfloat16>(p, grid, (cudaStream_t)stream);
        case EMLX_F32: return launch_step<float>(p, grid, (cudaStream_t)stream);
        default: return fail(EMLX_ERR_INVALID, "unknown in_dtype %d", in_dtype);
    }
}

extern "C" int emlx_kv_write_decode(const void* queries, void* queries_out, const void* keys, const void* values,
                                    int32_t in_dtype, const int32_t* slot_ids, int32_t num_seqs,
                                    const int32_t* block_tables_all, int32_t num_slots, int32_t max_blocks_per_seq,
                                    int32_t* kv_lens_all, int32_t advance_kv_lens, const emlx_pool* pool,
                                    const emlx_rope* rope, int32_t* query_start_loc, int32_t* block_tables,
                                    int32_t* kv_lens, int32_t num_q_heads, int32_t sliding_window, int32_t plan_flags,
                                    void* plan, size_t plan_bytes, int32_t* ticket, int32_t* status, void* stream) {
    return emlx_kv_write_step(queries, queries_out, keys, values, in_dtype, nullptr, slot_ids, num_seqs, num_seqs,
                              block_tables_all, num_slots, max_blocks_per_seq, kv_lens_all, advance_kv_lens, pool, rope,
                              query_start_loc, block_tables, kv_lens, num_q_heads, sliding_window, 1, plan_flags, plan,
                              plan_bytes, ticket, status, stream);
}
