// Paged KV write: scatter the new K/V rows of one packed batch into the page pool, either as
// plain 16/32-bit rows or as affine group-64 codes (8 or 4 bits) with fp16 scale and bias.
// One warp per (token, kv head); HBM-bound, a few MB per batch.
#include "kv_write_device.cuh"

namespace emlx {

template <typename TIn>
__global__ void __launch_bounds__(256) kv_write_kernel(WriteParams w) {
    // Wait before the first global load: the new rows may come from the launch right before this one (a projection,
    // a copy that made them contiguous), and the slot mapping comes from the metadata kernel.
    grid_dep_wait();
    grid_dep_launch();
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int Hkv = w.pool.num_kv_heads;
    const int64_t kv_warps = w.has_pool ? (int64_t)w.T * Hkv : 0;
    if (warp >= kv_warps) {
        // rotated queries: one warp per (token, q head)
        const int64_t qw = warp - kv_warps;
        if (w.q_out == nullptr || qw >= (int64_t)w.T * w.Hq) return;
        rotate_query_row<TIn>(w, qw, lane, w.positions[(int)(qw / w.Hq)]);
        return;
    }
    const int t = (int)(warp / Hkv), h = (int)(warp - (int64_t)t * Hkv);
    // rows first, destination second: the two loads chains are independent (a rotated key needs its position)
    RowRegs rows;
    const bool rotate = w.rope_dims > 0;
    if (!rotate) load_token_head<TIn>(w, t, h, lane, -1, rows);
    const int64_t slot = w.slot_mapping[t];
    if (rotate) load_token_head<TIn>(w, t, h, lane, w.positions[t], rows);
    store_token_head<TIn>(w, h, lane, slot, rows);
}

int validate_pool(const emlx_pool* pool) {
    if (!pool) return fail(EMLX_ERR_INVALID, "pool is NULL");
    if (!pool->key_cache || !pool->value_cache) return fail(EMLX_ERR_INVALID, "key_cache/value_cache is NULL");
    if (pool->num_blocks <= 0 || pool->block_size <= 0 || pool->num_kv_heads <= 0 || pool->head_dim <= 0)
        return fail(EMLX_ERR_INVALID, "pool geometry must be positive");
    if (pool->head_dim > 256) return fail(EMLX_ERR_UNSUPPORTED, "head_dim %d > 256", pool->head_dim);
    if (pool->kv_format == EMLX_KV_FLOAT) {
        if (pool->kv_dtype < EMLX_F16 || pool->kv_dtype > EMLX_F32) return fail(EMLX_ERR_INVALID, "unknown kv_dtype");
    } else if (pool->kv_format == EMLX_KV_AFFINE8 || pool->kv_format == EMLX_KV_AFFINE4) {
        if (pool->head_dim % kQuantGroup) return fail(EMLX_ERR_INVALID, "affine KV needs head_dim %% 64 == 0");
        if (pool->block_size % 8) return fail(EMLX_ERR_INVALID, "affine KV needs block_size %% 8 == 0");
        if (!pool->k_scale || !pool->k_bias || !pool->v_scale || !pool->v_bias)
            return fail(EMLX_ERR_INVALID, "affine KV needs k/v scale and bias arrays");
    } else {
        return fail(EMLX_ERR_INVALID, "unknown kv_format %d", pool->kv_format);
    }
    return EMLX_OK;
}

}  // namespace emlx

namespace emlx {

static int launch_write(WriteParams& w, int in_dtype, cudaStream_t s) {
    const int64_t warps = (w.has_pool ? (int64_t)w.T * w.pool.num_kv_heads : 0) + (w.q_out ? (int64_t)w.T * w.Hq : 0);
    if (warps == 0) return EMLX_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
    w.raw_ok = raw_copy_ok(w, in_dtype);
    switch (in_dtype) {
        case EMLX_F16: EMLX_CUDA_OK(launch_pdl(kv_write_kernel<__half>, blocks, threads, 0, s, w)); break;
        case EMLX_BF16: EMLX_CUDA_OK(launch_pdl(kv_write_kernel<__nv_bfloat16>, blocks, threads, 0, s, w)); break;
        case EMLX_F32: EMLX_CUDA_OK(launch_pdl(kv_write_kernel<float>, blocks, threads, 0, s, w)); break;
        default: return fail(EMLX_ERR_INVALID, "unknown in_dtype %d", in_dtype);
    }
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // namespace emlx

extern "C" int emlx_kv_write(const void* keys, const void* values, int32_t in_dtype, int32_t total_tokens,
                             const int64_t* slot_mapping, const emlx_pool* pool, int32_t* status, void* stream) {
    using namespace emlx;
    if (int rc = validate_pool(pool)) return rc;
    if (total_tokens < 0) return fail(EMLX_ERR_INVALID, "total_tokens must be non-negative");
    if (total_tokens == 0) return EMLX_OK;
    if (!keys || !values || !slot_mapping) return fail(EMLX_ERR_INVALID, "kv_write: NULL input");
    WriteParams w{};
    w.keys = keys; w.values = values; w.slot_mapping = slot_mapping; w.pool = *pool; w.T = total_tokens; w.status = status;
    w.has_pool = 1;
    return launch_write(w, in_dtype, (cudaStream_t)stream);
}

extern "C" int emlx_kv_write_rope(const void* queries, void* queries_out, int32_t num_q_heads, const void* keys,
                                  const void* values, int32_t in_dtype, int32_t total_tokens,
                                  const int64_t* slot_mapping, const int32_t* token_positions, const emlx_rope* rope,
                                  const emlx_pool* pool, int32_t* status, void* stream) {
    using namespace emlx;
    if (!rope || !rope->inv_freq) return fail(EMLX_ERR_INVALID, "rope parameters are NULL");
    if (rope->dims <= 0 || (rope->dims & 1)) return fail(EMLX_ERR_INVALID, "rope dims must be positive and even");
    if (total_tokens < 0) return fail(EMLX_ERR_INVALID, "total_tokens must be non-negative");
    if (total_tokens == 0) return EMLX_OK;
    if (!token_positions) return fail(EMLX_ERR_INVALID, "token_positions is NULL");
    WriteParams w{};
    w.T = total_tokens; w.status = status;
    if (pool) {
        if (int rc = validate_pool(pool)) return rc;
        if (!keys || !values || !slot_mapping) return fail(EMLX_ERR_INVALID, "kv_write_rope: NULL key/value input");
        if (rope->dims > pool->head_dim) return fail(EMLX_ERR_INVALID, "rope dims exceed head_dim");
        w.keys = keys; w.values = values; w.slot_mapping = slot_mapping; w.pool = *pool; w.has_pool = 1;
    } else if (rope->head_dim_if_no_pool <= 0 || rope->dims > rope->head_dim_if_no_pool) {
        return fail(EMLX_ERR_INVALID, "without a pool, rope->head_dim_if_no_pool must give the row width");
    } else {
        w.pool.head_dim = rope->head_dim_if_no_pool;
        w.pool.num_kv_heads = 1;
    }
    if (queries_out) {
        if (!queries || num_q_heads <= 0) return fail(EMLX_ERR_INVALID, "kv_write_rope: queries / num_q_heads missing");
        w.q_in = queries; w.q_out = queries_out; w.Hq = num_q_heads;
    }
    w.positions = token_positions; w.inv_freq = rope->inv_freq; w.rope_dims = rope->dims;
    w.traditional = rope->traditional; w.pos_scale = rope->position_scale; w.mscale = rope->mscale;
    return launch_write(w, in_dtype, (cudaStream_t)stream);
}
