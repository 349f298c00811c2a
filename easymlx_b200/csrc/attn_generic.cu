// Reference-semantics ragged paged attention for any geometry: head_dim <= 256, any page size,
// fp16/bf16/fp32 queries and pools, affine pools.  One warp per (packed token, q head) walks the
// keys of its causal range with an fp32 online softmax; small batches (decode) put WPR warps on a row, each taking
// every WPR-th key, and fold the partial states in warp order.  This is the coverage kernel; the tiled kernels in
// attn_tiled.cu are the fast path.
#include "common.cuh"

namespace emlx {

int validate_pool(const emlx_pool* pool);

constexpr int kMaxHeadDim = 256;
constexpr int kPerLane = kMaxHeadDim / 32;

struct PoolView {
    emlx_pool p;
    __device__ __forceinline__ float key(int64_t page, int off, int h, int d) const {
        const int D = p.head_dim, Hkv = p.num_kv_heads, bs = p.block_size;
        if (p.kv_format == EMLX_KV_FLOAT) {
            const int64_t i = ((page * bs + off) * Hkv + h) * D + d;
            if (p.kv_dtype == EMLX_F16) return __half2float(((const __half*)p.key_cache)[i]);
            if (p.kv_dtype == EMLX_BF16) return __bfloat162float(((const __nv_bfloat16*)p.key_cache)[i]);
            return ((const float*)p.key_cache)[i];
        }
        const int bits = p.kv_format;
        const uint8_t* row = (const uint8_t*)p.key_cache + ((page * bs + off) * Hkv + h) * (int64_t)(D * bits / 8);
        const int code = bits == 8 ? row[d] : ((row[d >> 1] >> ((d & 1) * 4)) & 0xF);
        const int64_t sb = ((page * Hkv + h) * bs + off) * (D / kQuantGroup) + d / kQuantGroup;
        return __fadd_rn(__fmul_rn(__half2float(((const __half*)p.k_scale)[sb]), (float)code),
                         __half2float(((const __half*)p.k_bias)[sb]));
    }
    __device__ __forceinline__ float value(int64_t page, int off, int h, int d) const {
        const int D = p.head_dim, Hkv = p.num_kv_heads, bs = p.block_size;
        if (p.kv_format == EMLX_KV_FLOAT) {
            const int64_t i = ((page * bs + off) * Hkv + h) * D + d;
            if (p.kv_dtype == EMLX_F16) return __half2float(((const __half*)p.value_cache)[i]);
            if (p.kv_dtype == EMLX_BF16) return __bfloat162float(((const __nv_bfloat16*)p.value_cache)[i]);
            return ((const float*)p.value_cache)[i];
        }
        const int bits = p.kv_format;
        const uint8_t* col = (const uint8_t*)p.value_cache + ((page * Hkv + h) * D + d) * (int64_t)(bs * bits / 8);
        const int code = bits == 8 ? col[off] : ((col[off >> 1] >> ((off & 1) * 4)) & 0xF);
        const int64_t sb = ((page * Hkv + h) * bs + off) * (D / kQuantGroup) + d / kQuantGroup;
        return __fadd_rn(__fmul_rn(__half2float(((const __half*)p.v_scale)[sb]), (float)code),
                         __half2float(((const __half*)p.v_bias)[sb]));
    }
};

constexpr int kGenericThreads = 256;

template <typename TQ, int WPR>  // WPR warps share one (token, q head) row; WPR divides the warps of a CTA
__global__ void __launch_bounds__(kGenericThreads) attn_generic_kernel(emlx_attn_args a, PoolView pv) {
    constexpr int kWarps = kGenericThreads / 32, kRows = kWarps / WPR;
    __shared__ float part_acc[WPR > 1 ? kWarps : 1][WPR > 1 ? kMaxHeadDim : 1];
    __shared__ float part_ml[WPR > 1 ? kWarps : 1][2];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int sub = wid % WPR;  // this warp takes keys start_k + sub, + WPR, ...
    const int64_t row = (int64_t)blockIdx.x * kRows + wid / WPR;
    const int Hq = a.num_q_heads, D = pv.p.head_dim, Hkv = pv.p.num_kv_heads, bs = pv.p.block_size;
    const bool row_live = row < (int64_t)a.total_tokens * Hq;
    if (WPR == 1 && !row_live) return;
    const int64_t warp = row_live ? row : 0;
    const int token = (int)(warp / Hq), head = (int)(warp - (int64_t)token * Hq);
    const int kvh = head / (Hq / Hkv);
    TQ* out = (TQ*)a.out + ((int64_t)token * Hq + head) * D;

    float acc[kPerLane], q[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) acc[j] = 0.f;

    const int s = find_sequence(a.query_start_loc, a.num_seqs, token);
    int start_k = 0, max_k = -1;
    if (s >= 0) {
        const int q0 = a.query_start_loc[s], q_len = a.query_start_loc[s + 1] - q0, kv_len = a.kv_lens[s];
        if (kv_len > 0) {
            max_k = min(kv_len - 1, (kv_len - q_len) + (token - q0));
            if (a.sliding_window > 0) start_k = max(0, max_k - a.sliding_window + 1);
        }
    }
    const TQ* qrow = (const TQ*)a.queries + ((int64_t)token * Hq + head) * D;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const int d = lane + 32 * j;
        q[j] = d < D ? __fmul_rn(to_f32<TQ>(qrow[d]), a.softmax_scale) : 0.f;
    }

    float m = -INFINITY, l = 0.f;
    const int32_t* table = a.block_tables + (int64_t)max(s, 0) * a.max_blocks_per_seq;
    for (int k = start_k + sub; k <= max_k; k += WPR) {
        const int page_idx = k / bs, off = k - page_idx * bs;
        const int64_t page = page_idx < a.max_blocks_per_seq ? table[page_idx] : -1;
        const bool live = page >= 0 && page < pv.p.num_blocks;  // an unassigned page reads as zero rows
        if (!live && lane == 0) flag_error(a.status, EMLX_DEV_BAD_PAGE);
        float dot = 0.f;
        if (live) {
#pragma unroll
            for (int j = 0; j < kPerLane; ++j) {
                const int d = lane + 32 * j;
                if (d < D) dot = fmaf(q[j], pv.key(page, off, kvh, d), dot);
            }
        }
        dot = warp_sum(dot);
        const float m_new = fmaxf(m, dot);
        const float corr = expf(m - m_new), p = expf(dot - m_new);
        l = fmaf(l, corr, p);
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            const int d = lane + 32 * j;
            const float v = (live && d < D) ? pv.value(page, off, kvh, d) : 0.f;
            acc[j] = fmaf(acc[j], corr, p * v);
        }
        m = m_new;
    }
    if constexpr (WPR > 1) {
        // fold the WPR partial states of the row in warp order (the result does not depend on timing)
        part_ml[wid][0] = m;
        part_ml[wid][1] = l;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            const int d = lane + 32 * j;
            if (d < D) part_acc[wid][d] = acc[j];
        }
        __syncthreads();
        if (sub != 0 || !row_live) return;
        float M = -INFINITY;
        for (int w = 0; w < WPR; ++w)
            if (part_ml[wid + w][1] > 0.f) M = fmaxf(M, part_ml[wid + w][0]);
        l = 0.f;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) acc[j] = 0.f;
        for (int w = 0; w < WPR; ++w) {
            const float lw = part_ml[wid + w][1];
            if (lw <= 0.f) continue;
            const float f = expf(part_ml[wid + w][0] - M);
            l = fmaf(f, lw, l);
#pragma unroll
            for (int j = 0; j < kPerLane; ++j) {
                const int d = lane + 32 * j;
                if (d < D) acc[j] = fmaf(f, part_acc[wid + w][d], acc[j]);
            }
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const int d = lane + 32 * j;
        if (d < D) out[d] = from_f32<TQ>(acc[j] * inv);
    }
}

// Contiguous K/V rows of the listed sequences out of the pool, cast (float pools) or dequantised (affine pools) to TOut:
// one warp per (output token, kv head).  Pages outside the pool leave zero rows and flag EMLX_DEV_BAD_PAGE.
template <typename TOut>
__global__ void __launch_bounds__(256) gather_kv_kernel(PoolView pv, const int32_t* __restrict__ block_table, int MB,
                                                        const int32_t* __restrict__ cu_seq_lens, int S, int total,
                                                        TOut* __restrict__ k_out, TOut* __restrict__ v_out, int32_t* status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int Hkv = pv.p.num_kv_heads, D = pv.p.head_dim, bs = pv.p.block_size;
    if (warp >= (int64_t)total * Hkv) return;
    const int t = (int)(warp / Hkv), h = (int)(warp - (int64_t)t * Hkv);
    TOut* kd = k_out + ((int64_t)t * Hkv + h) * D;
    TOut* vd = v_out + ((int64_t)t * Hkv + h) * D;
    const int s = find_sequence(cu_seq_lens, S, t);
    int64_t page = -1;
    int off = 0;
    if (s >= 0) {
        const int pos = t - cu_seq_lens[s], page_idx = pos / bs;
        off = pos - page_idx * bs;
        if (page_idx < MB) page = block_table[(int64_t)s * MB + page_idx];
    }
    const bool live = page >= 0 && page < pv.p.num_blocks;
    if (!live && lane == 0) flag_error(status, EMLX_DEV_BAD_PAGE);
    for (int d = lane; d < D; d += 32) {
        kd[d] = from_f32<TOut>(live ? pv.key(page, off, h, d) : 0.f);
        vd[d] = from_f32<TOut>(live ? pv.value(page, off, h, d) : 0.f);
    }
}

int validate_attn(const emlx_attn_args* a, const emlx_pool* pool, bool need_plan) {
    if (!a) return fail(EMLX_ERR_INVALID, "attention args are NULL");
    if (int rc = validate_pool(pool)) return rc;
    if (a->total_tokens < 0 || a->num_seqs < 0) return fail(EMLX_ERR_INVALID, "total_tokens/num_seqs must be non-negative");
    if (a->num_q_heads <= 0 || a->num_q_heads % pool->num_kv_heads)
        return fail(EMLX_ERR_INVALID, "num_q_heads must be divisible by num_kv_heads (GQA)");
    if (a->q_dtype < EMLX_F16 || a->q_dtype > EMLX_F32) return fail(EMLX_ERR_INVALID, "unknown q_dtype");
    if (a->total_tokens > 0) {
        if (!a->queries || !a->out) return fail(EMLX_ERR_INVALID, "queries/out is NULL");
        if (!a->query_start_loc) return fail(EMLX_ERR_INVALID, "query_start_loc is NULL");
        if (a->num_seqs > 0 && (!a->block_tables || !a->kv_lens || a->max_blocks_per_seq <= 0))
            return fail(EMLX_ERR_INVALID, "block_tables/kv_lens missing");
    }
    if (need_plan && a->total_tokens > 0 && (!a->plan || !a->workspace))
        return fail(EMLX_ERR_WORKSPACE, "plan and workspace are required");
    return EMLX_OK;
}

}  // namespace emlx

extern "C" int emlx_attn_generic(const emlx_attn_args* args, const emlx_pool* pool, void* stream) {
    using namespace emlx;
    if (int rc = validate_attn(args, pool, false)) return rc;
    if (pool->head_dim > kMaxHeadDim) return fail(EMLX_ERR_UNSUPPORTED, "head_dim %d > %d", pool->head_dim, kMaxHeadDim);
    if (args->total_tokens == 0) return EMLX_OK;
    PoolView pv{*pool};
    // few rows (decode batches): eight warps per row, so that the GPU has enough warps in flight; many rows: one each
    const int64_t rows = (int64_t)args->total_tokens * args->num_q_heads;
    const bool split = rows * 2 <= (int64_t)num_sms() * 64;
    const int rows_per_cta = split ? 1 : kGenericThreads / 32;
    const unsigned blocks = (unsigned)((rows + rows_per_cta - 1) / rows_per_cta);
    cudaStream_t s = (cudaStream_t)stream;
    if (split) {
        switch (args->q_dtype) {
            case EMLX_F16: attn_generic_kernel<__half, 8><<<blocks, kGenericThreads, 0, s>>>(*args, pv); break;
            case EMLX_BF16: attn_generic_kernel<__nv_bfloat16, 8><<<blocks, kGenericThreads, 0, s>>>(*args, pv); break;
            default: attn_generic_kernel<float, 8><<<blocks, kGenericThreads, 0, s>>>(*args, pv); break;
        }
    } else {
        switch (args->q_dtype) {
            case EMLX_F16: attn_generic_kernel<__half, 1><<<blocks, kGenericThreads, 0, s>>>(*args, pv); break;
            case EMLX_BF16: attn_generic_kernel<__nv_bfloat16, 1><<<blocks, kGenericThreads, 0, s>>>(*args, pv); break;
            default: attn_generic_kernel<float, 1><<<blocks, kGenericThreads, 0, s>>>(*args, pv); break;
        }
    }
    EMLX_LAUNCHED();
    return EMLX_OK;
}

extern "C" int emlx_gather_kv_cache(const emlx_pool* pool, const int32_t* block_table, int32_t num_seqs,
                                    int32_t max_blocks_per_seq, const int32_t* cu_seq_lens, int32_t total_tokens,
                                    int32_t out_dtype, void* k_out, void* v_out, int32_t* status, void* stream) {
    using namespace emlx;
    if (!pool) return fail(EMLX_ERR_INVALID, "pool is NULL");
    if (int rc = validate_pool(pool)) return rc;
    if (num_seqs < 0 || total_tokens < 0 || max_blocks_per_seq <= 0) return fail(EMLX_ERR_INVALID, "gather_kv_cache: bad sizes");
    if (out_dtype < EMLX_F16 || out_dtype > EMLX_F32) return fail(EMLX_ERR_INVALID, "unknown out_dtype");
    if (total_tokens == 0) return EMLX_OK;
    if (!block_table || !cu_seq_lens || !k_out || !v_out) return fail(EMLX_ERR_INVALID, "gather_kv_cache: NULL pointer");
    PoolView pv{*pool};
    const int64_t warps = (int64_t)total_tokens * pool->num_kv_heads;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    cudaStream_t s = (cudaStream_t)stream;
    switch (out_dtype) {
        case EMLX_F16:
            gather_kv_kernel<__half><<<blocks, 256, 0, s>>>(pv, block_table, max_blocks_per_seq, cu_seq_lens, num_seqs,
                                                           total_tokens, (__half*)k_out, (__half*)v_out, status);
            break;
        case EMLX_BF16:
            gather_kv_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(pv, block_table, max_blocks_per_seq, cu_seq_lens, num_seqs,
                                                                  total_tokens, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, status);
            break;
        default:
            gather_kv_kernel<float><<<blocks, 256, 0, s>>>(pv, block_table, max_blocks_per_seq, cu_seq_lens, num_seqs,
                                                          total_tokens, (float*)k_out, (float*)v_out, status);
            break;
    }
    EMLX_LAUNCHED();
    return EMLX_OK;
}
