// Single-token decode step in one launch: every scheduled sequence appends exactly one new token.
//
// The general path needs two dependent launches (batch metadata, then the write, which waits for the slot
// mapping).  When every sequence brings one token nothing has to be scanned: the row of sequence i goes to
// position kv_lens[slot_i] of that slot, so each write warp finds its own destination, and the attention
// work list depends only on the lengths.  One grid therefore does both at once:
//     CTA 0        lengths after the step, query_start_loc (= 0..S), the attention work list
//     CTAs 1..n    one warp per (token, kv head): locate the slot, store / quantise the K and V rows
//                  (optionally rotating K, and Q in extra warps); then the gather of the page-table rows
// The stored lengths are advanced in place, but only after every CTA has read them: each CTA takes a ticket
// when it is done reading, and the one that draws the last ticket does the advance (no CTA waits for another).
#include "kv_write_device.cuh"
#include "plan_device.cuh"

namespace emlx {

long long* trace_buffer();  // measurement aid, NULL unless the build defines EMLX_TRACE

#ifdef EMLX_TRACE_TIMELINE
#define STEP_STAMP(slot) do { if (p.trace && threadIdx.x == 0) { long long now_; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now_)); p.trace[(blockIdx.x == 0 ? 0 : 16 + 8 * (blockIdx.x - 1)) + (slot)] = now_; } } while (0)
#else
#define STEP_STAMP(slot) do { } while (0)
#endif

constexpr int kDecodeMaxSeqs = 2048;   // lengths and the work list's prefix sums stay in shared memory

struct DecodeStepParams {
    WriteParams w;  // keys / values / pool / rotation; slot_mapping and positions are not used
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
    int S, num_slots, MB, advance;
    int warps_per_cta;  // active warps of a write CTA (the others only help with the gather)
    int G, window, class_lo, class_hi, wide, num_ctas, two_per_sm;
};

template <typename TIn>
__global__ void __launch_bounds__(kMetaThreads) decode_step_kernel(const DecodeStepParams p) {
    __shared__ int32_t scan_smem[kMetaThreads / 32 + 1];
    __shared__ int32_t s_kv[kDecodeMaxSeqs], s_cum[kDecodeMaxSeqs + 1];
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

    if (blockIdx.x == 0) {
        for (int i = tid; i < S; i += kMetaThreads) {
            const int slot = p.slot_ids[i];
            bool ok = slot >= 0 && slot < p.num_slots;
            int base = 0;
            if (ok) base = p.kv_lens_all[slot];
            else flag_error(p.w.status, EMLX_DEV_BAD_SLOT);
            // a sequence whose row is full is reported and left alone (nothing written, zero rows attended)
            if (ok && (int64_t)base + 1 > capacity) {
                flag_error(p.w.status, EMLX_DEV_OVERFLOW);
                ok = false;
            }
            const int after = ok ? base + 1 : 0;
            s_kv[i] = after;
            p.qsl[i] = i;
            p.kv_out[i] = after;
        }
        if (tid == 0) p.qsl[S] = S;
        __syncthreads();
        STEP_STAMP(2);
        if (p.plan != nullptr)
            build_plan_decode(s_kv, S, p.G, p.window, p.class_lo, Hkv, p.num_ctas, p.plan, p.L, scan_smem, s_cum,
                              p.two_per_sm != 0);
    } else {
        const int64_t kv_warps = p.w.has_pool ? (int64_t)S * Hkv : 0;
        const int64_t q_warps = p.w.q_out != nullptr ? (int64_t)S * p.w.Hq : 0;
        // A write CTA has as many threads as the work-list CTA but only its first warps_per_cta warps take a row: the
        // byte-scattered stores of a row keep one SM's store path busy for a microsecond, so a small batch is spread
        // over many SMs rather than packed into a few.
        const int64_t gw = (int64_t)(blockIdx.x - 1) * p.warps_per_cta + (tid >> 5);
        if ((tid >> 5) < p.warps_per_cta && gw < kv_warps + q_warps) {
            const bool is_kv = gw < kv_warps;
            const int t = is_kv ? (int)(gw / Hkv) : (int)((gw - kv_warps) / p.w.Hq);
            const int h = (int)(gw - (int64_t)t * Hkv);
            const bool rotate = p.w.rope_dims > 0;
            // the rows do not depend on where they go: their loads are issued ahead of the slot -> length -> page
            // chain (a rotated key needs its position first and is loaded afterwards)
            RowRegs rows;
            if (is_kv && !rotate) load_token_head<TIn>(p.w, t, h, lane, -1, rows);
            const int slot = p.slot_ids[t];
            if (slot >= 0 && slot < p.num_slots) {
                const int base = p.kv_lens_all[slot];  // the new token's position in its sequence
                const int page_idx = base / bs;
                if (page_idx < MB) {
                    if (is_kv) {
                        const int page = p.bt_all[(int64_t)slot * MB + page_idx];
                        STEP_STAMP(4);
                        if (rotate) load_token_head<TIn>(p.w, t, h, lane, base, rows);
                        if (page >= 0 && page < pool.num_blocks)
                            store_token_head<TIn>(p.w, h, lane, (int64_t)page * bs + (base - page_idx * bs), rows);
                        else if (lane == 0)
                            flag_error(p.w.status, EMLX_DEV_BAD_PAGE);
                        STEP_STAMP(5);
                    } else {
                        rotate_query_row<TIn>(p.w, gw - kv_warps, lane, base);
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
    if (p.advance) {
        for (int i = tid; i < S; i += kMetaThreads) {
            const int slot = p.slot_ids[i];
            if (slot < 0 || slot >= p.num_slots) continue;
            const int base = p.kv_lens_all[slot];
            if ((int64_t)base + 1 <= capacity) p.kv_lens_all[slot] = base + 1;
        }
    }
    if (tid == 0) *p.ticket = 0;  // ready for the next launch
    STEP_STAMP(blockIdx.x == 0 ? 4 : 3);
}

template <typename TIn>
static int launch_decode_step(const DecodeStepParams& p, unsigned grid, cudaStream_t stream) {
    EMLX_CUDA_OK(launch_pdl(decode_step_kernel<TIn>, grid, kMetaThreads, 0, stream, p));
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // namespace emlx

extern "C" int emlx_kv_write_decode(const void* queries, void* queries_out, const void* keys, const void* values,
                                    int32_t in_dtype, const int32_t* slot_ids, int32_t num_seqs,
                                    const int32_t* block_tables_all, int32_t num_slots, int32_t max_blocks_per_seq,
                                    int32_t* kv_lens_all, int32_t advance_kv_lens, const emlx_pool* pool,
                                    const emlx_rope* rope, int32_t* query_start_loc, int32_t* block_tables,
                                    int32_t* kv_lens, int32_t num_q_heads, int32_t sliding_window, int32_t plan_flags,
                                    void* plan, size_t plan_bytes, int32_t* ticket, int32_t* status, void* stream) {
    using namespace emlx;
    if (int rc = validate_pool(pool)) return rc;
    if (num_seqs < 0) return fail(EMLX_ERR_INVALID, "num_seqs must be non-negative");
    if (num_seqs == 0) return EMLX_OK;
    if (num_seqs > kDecodeMaxSeqs)
        return fail(EMLX_ERR_UNSUPPORTED, "the fused decode step takes up to %d sequences; use emlx_build_metadata + emlx_kv_write",
                    kDecodeMaxSeqs);
    if (max_blocks_per_seq <= 0 || num_slots <= 0) return fail(EMLX_ERR_INVALID, "max_blocks_per_seq and num_slots must be positive");
    if (!keys || !values || !slot_ids || !block_tables_all || !kv_lens_all || !query_start_loc || !block_tables || !kv_lens || !ticket)
        return fail(EMLX_ERR_INVALID, "kv_write_decode: NULL argument");
    DecodeStepParams p{};
    p.w.keys = keys; p.w.values = values; p.w.pool = *pool; p.w.T = num_seqs; p.w.status = status; p.w.has_pool = 1;
    if (rope) {
        if (!rope->inv_freq) return fail(EMLX_ERR_INVALID, "rope parameters are NULL");
        if (rope->dims <= 0 || (rope->dims & 1) || rope->dims > pool->head_dim)
            return fail(EMLX_ERR_INVALID, "rope dims must be positive, even and at most head_dim");
        p.w.inv_freq = rope->inv_freq; p.w.rope_dims = rope->dims; p.w.traditional = rope->traditional;
        p.w.pos_scale = rope->position_scale; p.w.mscale = rope->mscale;
        if (queries_out) {
            if (!queries || num_q_heads <= 0) return fail(EMLX_ERR_INVALID, "kv_write_decode: queries / num_q_heads missing");
            p.w.q_in = queries; p.w.q_out = queries_out; p.w.Hq = num_q_heads;
        }
    }
    p.w.raw_ok = raw_copy_ok(p.w, in_dtype);
    p.trace = trace_buffer();
    p.slot_ids = slot_ids; p.bt_all = block_tables_all; p.kv_lens_all = kv_lens_all;
    p.qsl = query_start_loc; p.bt_out = block_tables; p.kv_out = kv_lens; p.ticket = ticket;
    p.S = num_seqs; p.num_slots = num_slots; p.MB = max_blocks_per_seq; p.advance = advance_kv_lens;
    p.class_lo = 0; p.class_hi = -1; p.G = 1;
    if (plan) {
        const int Hkv = pool->num_kv_heads;
        if (num_q_heads <= 0 || num_q_heads % Hkv) return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
        if (!tiled_page_size_ok(pool->block_size, 0)) return fail(EMLX_ERR_UNSUPPORTED, "the attention work list needs page size 16, 32, 64 or 128");
        p.L = plan_layout(num_seqs, num_seqs, num_q_heads, Hkv);
        if (plan_bytes < (size_t)p.L.words * sizeof(int32_t)) return fail(EMLX_ERR_WORKSPACE, "plan buffer smaller than emlx_attn_plan_bytes()");
        p.G = num_q_heads / Hkv;
        p.wide = (plan_flags & kPlanWideUnits) != 0;
        p.two_per_sm = (plan_flags & kPlanTwoCtas) != 0;
        class_range(p.G, 1, p.wide != 0, p.class_lo, p.class_hi);
        p.plan = (int32_t*)plan; p.window = sliding_window; p.num_ctas = min(num_sms(), kMaxGrid);
    }
    const int64_t warps = (int64_t)num_seqs * pool->num_kv_heads + (p.w.q_out ? (int64_t)num_seqs * num_q_heads : 0);
    // about two write CTAs per SM at most; at least 4 and at most 32 rows per CTA
    const int64_t per_cta = (warps + 2 * num_sms() - 1) / (2 * num_sms());
    p.warps_per_cta = (int)(per_cta < 4 ? 4 : (per_cta > kMetaThreads / 32 ? kMetaThreads / 32 : per_cta));
    const unsigned grid = 1u + (unsigned)((warps + p.warps_per_cta - 1) / p.warps_per_cta);
    switch (in_dtype) {
        case EMLX_F16: return launch_decode_step<__half>(p, grid, (cudaStream_t)stream);
        case EMLX_BF16: return launch_decode_step<__nv_bfloat16>(p, grid, (cudaStream_t)stream);
        case EMLX_F32: return launch_decode_step<float>(p, grid, (cudaStream_t)stream);
        default: return fail(EMLX_ERR_INVALID, "unknown in_dtype %d", in_dtype);
    }
}
