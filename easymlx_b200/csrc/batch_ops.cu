// Device-side batch and page-table maintenance around the attention path: last-token gather, token-id padding,
// page copies (copy-on-write), page zeroing, and page-table row updates.  All of it is byte and index work bound
// by HBM bandwidth or by launch latency; nothing here synchronises with the host.
#include "common.cuh"

namespace emlx {

int validate_pool(const emlx_pool* pool);

namespace {

constexpr int kThreads = 256;
constexpr int kMaxSegments = 6;

// One array of the pool as a run of equal-sized pages.
struct Segment {
    uint8_t* base;
    long long page_bytes;
    long long stage_off;  // offset of this array's page inside a staging slot
};
struct Segments {
    Segment seg[kMaxSegments];
    int count;
    long long slot_bytes;  // bytes of one staging slot (all arrays of one page, each rounded up to 16)
    long long num_blocks;
};

Segments pool_segments(const emlx_pool* pool) {
    Segments s = {};
    const long long bs = pool->block_size, h = pool->num_kv_heads, d = pool->head_dim;
    auto add = [&](void* base, long long bytes) {
        if (!base) return;
        s.seg[s.count].base = (uint8_t*)base;
        s.seg[s.count].page_bytes = bytes;
        s.seg[s.count].stage_off = s.slot_bytes;
        s.slot_bytes += (bytes + 15) & ~15LL;
        ++s.count;
    };
    if (pool->kv_format == EMLX_KV_FLOAT) {
        const long long es = pool->kv_dtype == EMLX_F32 ? 4 : 2;
        add(pool->key_cache, bs * h * d * es);
        add(pool->value_cache, bs * h * d * es);
    } else {
        const long long bits = pool->kv_format;
        add(pool->key_cache, bs * h * d * bits / 8);
        add(pool->value_cache, bs * h * d * bits / 8);
        const long long sb = h * bs * (d / kQuantGroup) * 2;
        add(pool->k_scale, sb);
        add(pool->k_bias, sb);
        add(pool->v_scale, sb);
        add(pool->v_bias, sb);
    }
    s.num_blocks = pool->num_blocks;
    return s;
}

__device__ __forceinline__ void copy_bytes(uint8_t* dst, const uint8_t* src, long long bytes, int part, int parts) {
    const bool vec = (((uintptr_t)dst | (uintptr_t)src | (uintptr_t)bytes) & 15) == 0;
    if (vec) {
        const long long n = bytes >> 4;
        for (long long i = (long long)part * kThreads + threadIdx.x; i < n; i += (long long)parts * kThreads)
            ((uint4*)dst)[i] = __ldg((const uint4*)src + i);
    } else {
        for (long long i = (long long)part * kThreads + threadIdx.x; i < bytes; i += (long long)parts * kThreads)
            dst[i] = src[i];
    }
}
__device__ __forceinline__ void zero_bytes(uint8_t* dst, long long bytes, int part, int parts) {
    const bool vec = (((uintptr_t)dst | (uintptr_t)bytes) & 15) == 0;
    if (vec) {
        const long long n = bytes >> 4;
        for (long long i = (long long)part * kThreads + threadIdx.x; i < n; i += (long long)parts * kThreads)
            ((uint4*)dst)[i] = make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (long long i = (long long)part * kThreads + threadIdx.x; i < bytes; i += (long long)parts * kThreads) dst[i] = 0;
    }
}

enum PageMode { kDirect = 0, kToStage = 1, kFromStage = 2, kZero = 3 };

// grid = (parts per page, pairs).  kDirect copies page src -> dst in place (pairs must not chain); kToStage and
// kFromStage split that into two launches through a staging slot per pair, so every read sees the pool as it
// was before the call; kZero clears page ids[i].
template <int MODE>
__global__ void __launch_bounds__(kThreads) page_kernel(const Segments s, const int32_t* __restrict__ ids, uint8_t* stage,
                                                        int32_t* status) {
    const int pair = blockIdx.y;
    long long src, dst;
    if constexpr (MODE == kZero) {
        src = 0;
        dst = ids[pair];
        if (dst < 0 || dst >= s.num_blocks) return;  // negative ids mark unused table entries; others are skipped too
    } else {
        src = ids[2 * pair];
        dst = ids[2 * pair + 1];
        if (src < 0 || src >= s.num_blocks || dst < 0 || dst >= s.num_blocks) {
            if (threadIdx.x == 0 && blockIdx.x == 0) flag_error(status, EMLX_DEV_BAD_PAGE);
            return;
        }
    }
    for (int k = 0; k < s.count; ++k) {
        const Segment g = s.seg[k];
        uint8_t* slot = stage ? stage + (long long)pair * s.slot_bytes + g.stage_off : nullptr;
        if constexpr (MODE == kDirect) copy_bytes(g.base + dst * g.page_bytes, g.base + src * g.page_bytes, g.page_bytes, blockIdx.x, gridDim.x);
        if constexpr (MODE == kToStage) copy_bytes(slot, g.base + src * g.page_bytes, g.page_bytes, blockIdx.x, gridDim.x);
        if constexpr (MODE == kFromStage) copy_bytes(g.base + dst * g.page_bytes, slot, g.page_bytes, blockIdx.x, gridDim.x);
        if constexpr (MODE == kZero) zero_bytes(g.base + dst * g.page_bytes, g.page_bytes, blockIdx.x, gridDim.x);
    }
}

int parts_for(long long slot_bytes, int pairs) {
    // enough CTAs to fill the GPU a few times over, at least 4 KiB of work each
    long long parts = (slot_bytes + 4095) / 4096;
    const long long want = (4LL * num_sms() + pairs - 1) / pairs;
    if (parts > want) parts = want;
    if (parts < 1) parts = 1;
    return (int)parts;
}

// out[s] = rows[query_start_loc[s + 1] - 1]; an index of -1 (empty batch prefix) wraps to the last row, as a take does
__global__ void __launch_bounds__(kThreads) gather_last_kernel(const uint8_t* __restrict__ rows, int T, long long row_bytes,
                                                               const int32_t* __restrict__ qsl, uint8_t* out,
                                                               int32_t* status) {
    const int s = blockIdx.x;
    int idx = qsl[s + 1] - 1;
    if (idx < 0) idx += T;
    if (idx < 0 || idx >= T) {
        if (threadIdx.x == 0) flag_error(status, EMLX_DEV_TOKEN_MISMATCH);
        return;
    }
    copy_bytes(out + (long long)s * row_bytes, rows + (long long)idx * row_bytes, row_bytes, 0, 1);
}

// out[s, i] = i < len(s) ? flat[query_start_loc[s] + i] : 0
__global__ void __launch_bounds__(kThreads) pad_ids_kernel(const int32_t* __restrict__ flat, int T,
                                                           const int32_t* __restrict__ qsl, int S, int max_q, int32_t* out) {
    const long long n = (long long)S * max_q;
    for (long long e = (long long)blockIdx.x * kThreads + threadIdx.x; e < n; e += (long long)gridDim.x * kThreads) {
        const int s = (int)(e / max_q), i = (int)(e - (long long)s * max_q);
        const int start = qsl[s], len = qsl[s + 1] - start;
        int v = 0;
        if (i < len) {
            const int src = min(start + i, max(T, 1) - 1);
            v = T > 0 ? flat[src] : 0;
        }
        out[e] = v;
    }
}

// Page-table rows.  Columns are independent of one another, so every thread walks the whole list of operations in
// order for its own columns; thread 0 of CTA 0 does the same for kv_lens.
enum RowMode { kRowMove = 0, kRowSwap = 1, kRowClear = 2 };
__global__ void __launch_bounds__(kThreads) rows_kernel(int32_t* bt, int32_t* kv_lens, int num_slots, int MB,
                                                        const int32_t* __restrict__ ops, int n, int mode, int32_t* status) {
    const int col = blockIdx.x * kThreads + threadIdx.x;
    const bool lens_thread = blockIdx.x == 0 && threadIdx.x == 0;
    for (int k = 0; k < n; ++k) {
        if (mode == kRowClear) {
            const int row = ops[k];
            if (row < 0 || row >= num_slots) { if (lens_thread) flag_error(status, EMLX_DEV_BAD_SLOT); continue; }
            if (col < MB) bt[(long long)row * MB + col] = -1;
            if (lens_thread) kv_lens[row] = 0;
            continue;
        }
        const int from = ops[2 * k], to = ops[2 * k + 1];
        if (from == to) continue;
        if (from < 0 || from >= num_slots || to < 0 || to >= num_slots) {
            if (lens_thread) flag_error(status, EMLX_DEV_BAD_SLOT);
            continue;
        }
        if (col < MB) {
            const int a = bt[(long long)from * MB + col], b = bt[(long long)to * MB + col];
            bt[(long long)to * MB + col] = a;
            bt[(long long)from * MB + col] = mode == kRowSwap ? b : -1;
        }
        if (lens_thread) {
            const int a = kv_lens[from], b = kv_lens[to];
            kv_lens[to] = a;
            kv_lens[from] = mode == kRowSwap ? b : 0;
        }
    }
}

__global__ void __launch_bounds__(kThreads) row_assign_kernel(int32_t* bt, int32_t* kv_lens, int MB, int row,
                                                              const int32_t* __restrict__ page_ids, int count, int cached) {
    const int col = blockIdx.x * kThreads + threadIdx.x;
    if (col < MB) bt[(long long)row * MB + col] = col < count ? page_ids[col] : -1;
    if (col == 0) kv_lens[row] = max(cached, 0);
}

}  // namespace
}  // namespace emlx

using namespace emlx;

extern "C" {

int emlx_gather_last_tokens(const void* rows, int32_t total_tokens, int64_t row_bytes, const int32_t* query_start_loc,
                            int32_t num_seqs, void* out, int32_t* status, void* stream) {
    if (num_seqs < 0 || total_tokens < 0 || row_bytes <= 0) return fail(EMLX_ERR_INVALID, "negative size in gather_last_tokens");
    if (num_seqs == 0) return EMLX_OK;
    if (!rows || !query_start_loc || !out) return fail(EMLX_ERR_INVALID, "gather_last_tokens: NULL pointer");
    gather_last_kernel<<<num_seqs, kThreads, 0, (cudaStream_t)stream>>>((const uint8_t*)rows, total_tokens, row_bytes,
                                                                        query_start_loc, (uint8_t*)out, status);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

int emlx_pad_token_ids(const int32_t* flat_ids, int32_t total_tokens, const int32_t* query_start_loc, int32_t num_seqs,
                       int32_t max_query_len, int32_t* out, void* stream) {
    if (num_seqs < 0 || total_tokens < 0 || max_query_len < 0) return fail(EMLX_ERR_INVALID, "negative size in pad_token_ids");
    const long long n = (long long)num_seqs * max_query_len;
    if (n == 0) return EMLX_OK;
    if (!query_start_loc || !out || (total_tokens > 0 && !flat_ids)) return fail(EMLX_ERR_INVALID, "pad_token_ids: NULL pointer");
    const long long blocks = (n + kThreads - 1) / kThreads;
    const int grid = (int)(blocks < 8LL * num_sms() ? blocks : 8LL * num_sms());
    pad_ids_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(flat_ids, total_tokens, query_start_loc, num_seqs,
                                                                max_query_len, out);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

int64_t emlx_page_staging_bytes(const emlx_pool* pool) {
    if (!pool || validate_pool(pool)) return -1;
    return pool_segments(pool).slot_bytes;
}

int emlx_copy_blocks(const emlx_pool* pool, const int32_t* block_mapping, int32_t num_pairs, void* staging,
                     int64_t staging_bytes, int32_t* status, void* stream) {
    if (!pool) return fail(EMLX_ERR_INVALID, "pool is NULL");
    if (int rc = validate_pool(pool)) return rc;
    if (num_pairs < 0) return fail(EMLX_ERR_INVALID, "num_pairs is negative");
    if (num_pairs == 0) return EMLX_OK;
    if (!block_mapping) return fail(EMLX_ERR_INVALID, "block_mapping is NULL");
    if (num_pairs > 65535) return fail(EMLX_ERR_UNSUPPORTED, "more than 65535 page pairs in one call");
    const Segments s = pool_segments(pool);
    const dim3 grid(parts_for(s.slot_bytes, num_pairs), num_pairs);
    cudaStream_t st = (cudaStream_t)stream;
    if (!staging) {
        page_kernel<kDirect><<<grid, kThreads, 0, st>>>(s, block_mapping, nullptr, status);
        EMLX_LAUNCHED();
        return EMLX_OK;
    }
    if (staging_bytes < (int64_t)num_pairs * s.slot_bytes)
        return fail(EMLX_ERR_WORKSPACE, "staging holds %lld bytes, %lld needed", (long long)staging_bytes,
                    (long long)num_pairs * s.slot_bytes);
    if ((uintptr_t)staging & 15) return fail(EMLX_ERR_INVALID, "staging must be 16-byte aligned");
    page_kernel<kToStage><<<grid, kThreads, 0, st>>>(s, block_mapping, (uint8_t*)staging, status);
    EMLX_LAUNCHED();
    page_kernel<kFromStage><<<grid, kThreads, 0, st>>>(s, block_mapping, (uint8_t*)staging, status);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

int emlx_zero_pages(const emlx_pool* pool, const int32_t* page_ids, int32_t count, void* stream) {
    if (!pool) return fail(EMLX_ERR_INVALID, "pool is NULL");
    if (int rc = validate_pool(pool)) return rc;
    if (count < 0) return fail(EMLX_ERR_INVALID, "count is negative");
    if (count == 0) return EMLX_OK;
    if (!page_ids) return fail(EMLX_ERR_INVALID, "page_ids is NULL");
    if (count > 65535) return fail(EMLX_ERR_UNSUPPORTED, "more than 65535 pages in one call");
    const Segments s = pool_segments(pool);
    const dim3 grid(parts_for(s.slot_bytes, count), count);
    page_kernel<kZero><<<grid, kThreads, 0, (cudaStream_t)stream>>>(s, page_ids, nullptr, nullptr);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

static int rows_common(int32_t* bt, int32_t* kv_lens, int32_t num_slots, int32_t MB) {
    if (!bt || !kv_lens) return fail(EMLX_ERR_INVALID, "block_tables / kv_lens is NULL");
    if (num_slots <= 0 || MB <= 0) return fail(EMLX_ERR_INVALID, "page table has no rows or no columns");
    return EMLX_OK;
}

int emlx_rows_assign(int32_t* block_tables, int32_t* kv_lens, int32_t num_slots, int32_t max_blocks_per_seq, int32_t row,
                     const int32_t* page_ids, int32_t count, int32_t cached_tokens, void* stream) {
    if (int rc = rows_common(block_tables, kv_lens, num_slots, max_blocks_per_seq)) return rc;
    if (row < 0 || row >= num_slots) return fail(EMLX_ERR_INVALID, "row %d exceeds cache capacity %d", row, num_slots);
    if (count < 0 || (count > 0 && !page_ids)) return fail(EMLX_ERR_INVALID, "bad page id list");
    if (count > max_blocks_per_seq) count = max_blocks_per_seq;
    const int grid = (max_blocks_per_seq + kThreads - 1) / kThreads;
    row_assign_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(block_tables, kv_lens, max_blocks_per_seq, row, page_ids,
                                                                   count, cached_tokens);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

int emlx_rows_update(int32_t* block_tables, int32_t* kv_lens, int32_t num_slots, int32_t max_blocks_per_seq,
                     const int32_t* ops, int32_t count, int32_t mode, int32_t* status, void* stream) {
    if (int rc = rows_common(block_tables, kv_lens, num_slots, max_blocks_per_seq)) return rc;
    if (mode < 0 || mode > 2) return fail(EMLX_ERR_INVALID, "mode must be 0 (move), 1 (swap) or 2 (clear)");
    if (count < 0) return fail(EMLX_ERR_INVALID, "count is negative");
    if (count == 0) return EMLX_OK;
    if (!ops) return fail(EMLX_ERR_INVALID, "ops is NULL");
    const int grid = (max_blocks_per_seq + kThreads - 1) / kThreads;
    rows_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(block_tables, kv_lens, num_slots, max_blocks_per_seq, ops,
                                                             count, mode, status);
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // extern "C"
