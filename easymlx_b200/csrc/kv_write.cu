// Paged KV write: scatter the new K/V rows of one packed batch into the page pool, either as
// plain 16/32-bit rows or as affine group-64 codes (8 or 4 bits) with fp16 scale and bias.
// One warp per (token, kv head); HBM-bound, a few MB per batch.
#include "common.cuh"

namespace emlx {

struct WriteParams {
    const void* keys;
    const void* values;
    const int64_t* slot_mapping;
    emlx_pool pool;
    int T;
    int32_t* status;
    // rotary embedding fused into the write (rope_dims == 0: off)
    const void* q_in;
    void* q_out;
    const int32_t* positions;
    const float* inv_freq;
    int Hq, rope_dims, traditional, has_pool;
    int raw_ok;  // rows can be copied bit for bit in 16-byte pieces
    float pos_scale, mscale;
};

// Element d of a row after the rotary embedding at position `pos`: pairs are (i, i + dims/2), or (2i, 2i + 1) in the
// "traditional" layout; angle = pos * pos_scale * inv_freq[i]; elements past rope_dims pass through.  The result is
// rounded to the input dtype, as a separate rotation step that returns an array of that dtype would.
template <typename TIn>
__device__ __forceinline__ float rope_elem(const TIn* row, int d, int pos, const WriteParams& w) {
    const float x = to_f32<TIn>(row[d]);
    if (d >= w.rope_dims) return x;
    const int half = w.rope_dims >> 1;
    const bool first = w.traditional ? ((d & 1) == 0) : (d < half);
    const int i = w.traditional ? (d >> 1) : (first ? d : d - half);
    const int partner = w.traditional ? (d ^ 1) : (first ? d + half : d - half);
    const float y = to_f32<TIn>(row[partner]);
    float sn, cs;
    sincosf((float)pos * w.pos_scale * w.inv_freq[i], &sn, &cs);
    const float a = (first ? x : y) * w.mscale, b = (first ? y : x) * w.mscale;
    const float r = first ? a * cs - b * sn : a * sn + b * cs;
    return to_f32<TIn>(from_f32<TIn>(r));
}

// Reads element d of a new row, rotated when `pos` >= 0.
template <typename TIn>
struct RowReader {
    const TIn* row;
    int pos;  // -1: no rotation
    const WriteParams* w;
    __device__ __forceinline__ float operator()(int d) const {
        return pos >= 0 ? rope_elem<TIn>(row, d, pos, *w) : to_f32<TIn>(row[d]);
    }
};

// Quantise one group of 64 elements held two per lane.  Arithmetic is spelled with the
// round-to-nearest intrinsics so that no contraction or fast-math option can change the codes.
template <int BITS>
__device__ __forceinline__ void quantize_group(float x0, float x1, int& c0, int& c1, __half& scale_h, __half& bias_h) {
    const float levels = (float)((1 << BITS) - 1);
    float lo = warp_min(fminf(x0, x1));
    float hi = warp_max(fmaxf(x0, x1));
    scale_h = __float2half_rn(__fdiv_rn(__fsub_rn(hi, lo), levels));
    if (__half2float(scale_h) == 0.0f) scale_h = __float2half_rn(1.0f);
    bias_h = __float2half_rn(lo);
    const float s = __half2float(scale_h), b = __half2float(bias_h);
    float q0 = rintf(__fdiv_rn(__fsub_rn(x0, b), s));
    float q1 = rintf(__fdiv_rn(__fsub_rn(x1, b), s));
    c0 = (int)fminf(fmaxf(q0, 0.0f), levels);
    c1 = (int)fminf(fmaxf(q1, 0.0f), levels);
}

constexpr int kMaxGroups = 4;  // head_dim <= 256

// Codes, scale and bias of one (token, head): computed before the destination is known, stored afterwards.
struct QuantRow {
    int c0[kMaxGroups], c1[kMaxGroups];
    __half s[kMaxGroups], b[kMaxGroups];
};

template <typename TIn, int BITS>
__device__ __forceinline__ void quantize_row(const RowReader<TIn>& row, int groups, int lane, QuantRow& q) {
#pragma unroll
    for (int g = 0; g < kMaxGroups; ++g) {
        if (g < groups) {
            const int d0 = g * kQuantGroup + 2 * lane;
            quantize_group<BITS>(row(d0), row(d0 + 1), q.c0[g], q.c1[g], q.s[g], q.b[g]);
        }
    }
}

template <int BITS>
__device__ __forceinline__ void store_affine_rows(const QuantRow& kq, const QuantRow& vq, const emlx_pool& p, int64_t page,
                                                  int off, int h, int lane) {
    const int D = p.head_dim, bs = p.block_size, Hkv = p.num_kv_heads, groups = D / kQuantGroup;
    const int64_t sb_base = ((page * Hkv + h) * bs + off) * groups;
    // keys: token-major codes [NB, bs, Hkv, D*BITS/8]
    uint8_t* kdst = (uint8_t*)p.key_cache + ((page * bs + off) * Hkv + h) * (int64_t)(D * BITS / 8);
    // values: [NB, Hkv, D, bs*BITS/8], the tokens of one element are contiguous
    uint8_t* vdst = (uint8_t*)p.value_cache + (page * Hkv + h) * (int64_t)D * (bs * BITS / 8);
#pragma unroll
    for (int g = 0; g < kMaxGroups; ++g) {
        if (g >= groups) break;
        const int d0 = g * kQuantGroup + 2 * lane;
        if (BITS == 8) *(uchar2*)(kdst + d0) = make_uchar2((unsigned char)kq.c0[g], (unsigned char)kq.c1[g]);
        else kdst[d0 >> 1] = (uint8_t)(kq.c0[g] | (kq.c1[g] << 4));
        if (BITS == 8) {
            vdst[(int64_t)d0 * bs + off] = (uint8_t)vq.c0[g];
            vdst[(int64_t)(d0 + 1) * bs + off] = (uint8_t)vq.c1[g];
        } else {
            // two tokens share a byte; tokens of the same batch may land in the same 32-bit word, so the
            // nibble is replaced with word atomics (each nibble has exactly one writer per batch)
            const int shift = ((off >> 1) & 3) * 8 + (off & 1) * 4;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                uint8_t* byte = vdst + (int64_t)(d0 + e) * (bs / 2) + (off >> 1);
                unsigned int* word = (unsigned int*)((uintptr_t)byte & ~(uintptr_t)3);
                atomicAnd(word, ~(0xFu << shift));
                atomicOr(word, (unsigned int)(e ? vq.c1[g] : vq.c0[g]) << shift);
            }
        }
        if (lane == 0) {
            ((__half*)p.k_scale)[sb_base + g] = kq.s[g];
            ((__half*)p.k_bias)[sb_base + g] = kq.b[g];
            ((__half*)p.v_scale)[sb_base + g] = vq.s[g];
            ((__half*)p.v_bias)[sb_base + g] = vq.b[g];
        }
    }
}

template <typename TIn>
__global__ void __launch_bounds__(256) kv_write_kernel(WriteParams w) {
    // Everything up to the stores is independent of the metadata kernel unless the rows are rotated (the rotation
    // needs the token positions that kernel writes): read and quantise the rows first, wait for the predecessor
    // only then.  The inputs themselves come from launches that precede the metadata kernel, which has already
    // waited for them by the time it lets this grid start.
    const bool early = w.rope_dims == 0;
    if (!early) grid_dep_wait();
    grid_dep_launch();
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const emlx_pool& p = w.pool;
    const int Hkv = p.num_kv_heads, D = p.head_dim;
    const int64_t kv_warps = w.has_pool ? (int64_t)w.T * Hkv : 0;
    if (warp >= kv_warps) {
        // rotated queries: one warp per (token, q head); only launched with a rotation, so the wait is behind us
        const int64_t qw = warp - kv_warps;
        if (w.q_out == nullptr || qw >= (int64_t)w.T * w.Hq) return;
        const int t = (int)(qw / w.Hq);
        const RowReader<TIn> q{(const TIn*)w.q_in + qw * D, w.positions[t], &w};
        TIn* dst = (TIn*)w.q_out + qw * D;
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<TIn>(q(d));
        return;
    }
    const int t = (int)(warp / Hkv), h = (int)(warp - (int64_t)t * Hkv);
    const RowReader<TIn> krow{(const TIn*)w.keys + ((int64_t)t * Hkv + h) * D, w.rope_dims > 0 ? w.positions[t] : -1, &w};
    const RowReader<TIn> vrow{(const TIn*)w.values + ((int64_t)t * Hkv + h) * D, -1, &w};
    const int groups = D / kQuantGroup;
    QuantRow kq, vq;
    float kf[8], vf[8];  // float pools: head_dim <= 256, element d = lane + 32 i
    // same 16-bit type on both sides, no rotation, 16-byte aligned rows: a row moves as 16-byte pieces, one per lane
    const bool raw_copy = w.raw_ok && p.kv_format == EMLX_KV_FLOAT;
    uint4 kraw = make_uint4(0u, 0u, 0u, 0u), vraw = kraw;
    if (p.kv_format == EMLX_KV_AFFINE8) {
        quantize_row<TIn, 8>(krow, groups, lane, kq);
        quantize_row<TIn, 8>(vrow, groups, lane, vq);
    } else if (p.kv_format == EMLX_KV_AFFINE4) {
        quantize_row<TIn, 4>(krow, groups, lane, kq);
        quantize_row<TIn, 4>(vrow, groups, lane, vq);
    } else if (raw_copy) {
        if (lane < D / 8) {
            kraw = *(const uint4*)((const uint16_t*)krow.row + lane * 8);
            vraw = *(const uint4*)((const uint16_t*)vrow.row + lane * 8);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            kf[i] = d < D ? krow(d) : 0.f;
            vf[i] = d < D ? vrow(d) : 0.f;
        }
    }
    if (early) grid_dep_wait();
    const int64_t slot = w.slot_mapping[t];
    if (slot < 0) return;
    if (slot >= p.num_blocks * p.block_size) {
        if (lane == 0) flag_error(w.status, EMLX_DEV_BAD_PAGE);
        return;
    }
    if (raw_copy) {
        const int64_t off = (slot * Hkv + h) * D;
        if (lane < D / 8) {
            *(uint4*)((uint16_t*)p.key_cache + off + lane * 8) = kraw;
            *(uint4*)((uint16_t*)p.value_cache + off + lane * 8) = vraw;
        }
    } else if (p.kv_format == EMLX_KV_FLOAT) {
        const int64_t off = (slot * Hkv + h) * D;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < D) {
                if (p.kv_dtype == EMLX_F16) {
                    ((__half*)p.key_cache)[off + d] = __float2half_rn(kf[i]);
                    ((__half*)p.value_cache)[off + d] = __float2half_rn(vf[i]);
                } else if (p.kv_dtype == EMLX_BF16) {
                    ((__nv_bfloat16*)p.key_cache)[off + d] = __float2bfloat16_rn(kf[i]);
                    ((__nv_bfloat16*)p.value_cache)[off + d] = __float2bfloat16_rn(vf[i]);
                } else {
                    ((float*)p.key_cache)[off + d] = kf[i];
                    ((float*)p.value_cache)[off + d] = vf[i];
                }
            }
        }
    } else {
        const int64_t page = slot / p.block_size;
        const int in_page = (int)(slot - page * p.block_size);
        if (p.kv_format == EMLX_KV_AFFINE8) store_affine_rows<8>(kq, vq, p, page, in_page, h, lane);
        else store_affine_rows<4>(kq, vq, p, page, in_page, h, lane);
    }
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
    const emlx_pool& p = w.pool;
    w.raw_ok = w.has_pool && w.rope_dims == 0 && p.kv_format == EMLX_KV_FLOAT && in_dtype == p.kv_dtype &&
               (in_dtype == EMLX_F16 || in_dtype == EMLX_BF16) && p.head_dim % 8 == 0 &&
               (((uintptr_t)w.keys | (uintptr_t)w.values | (uintptr_t)p.key_cache | (uintptr_t)p.value_cache) & 15) == 0;
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
