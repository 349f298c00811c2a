// Device side of the paged KV write, shared by the general write kernel and the fused single-token-decode
// step: one warp stores (or quantises and stores) the new K and V row of one (token, kv head) at a flat pool
// slot `page * block_size + offset`, optionally rotating the key first.
#pragma once
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

// The K and V rows of token t, head h go to flat slot `slot` (page * block_size + offset; negative: skip).  `pos` is
// the token's position in its sequence when the key is to be rotated, -1 otherwise.  Called by a whole warp.
template <typename TIn>
__device__ __forceinline__ void write_token_head(const WriteParams& w, int t, int h, int lane, int64_t slot, int pos) {
    const emlx_pool& p = w.pool;
    const int Hkv = p.num_kv_heads, D = p.head_dim;
    if (slot < 0) return;
    if (slot >= p.num_blocks * p.block_size) {
        if (lane == 0) flag_error(w.status, EMLX_DEV_BAD_PAGE);
        return;
    }
    const RowReader<TIn> krow{(const TIn*)w.keys + ((int64_t)t * Hkv + h) * D, w.rope_dims > 0 ? pos : -1, &w};
    const RowReader<TIn> vrow{(const TIn*)w.values + ((int64_t)t * Hkv + h) * D, -1, &w};
    const int groups = D / kQuantGroup;
    if (p.kv_format == EMLX_KV_AFFINE8 || p.kv_format == EMLX_KV_AFFINE4) {
        QuantRow kq, vq;
        const int64_t page = slot / p.block_size;
        const int in_page = (int)(slot - page * p.block_size);
        if (p.kv_format == EMLX_KV_AFFINE8) {
            quantize_row<TIn, 8>(krow, groups, lane, kq);
            quantize_row<TIn, 8>(vrow, groups, lane, vq);
            store_affine_rows<8>(kq, vq, p, page, in_page, h, lane);
        } else {
            quantize_row<TIn, 4>(krow, groups, lane, kq);
            quantize_row<TIn, 4>(vrow, groups, lane, vq);
            store_affine_rows<4>(kq, vq, p, page, in_page, h, lane);
        }
        return;
    }
    const int64_t off = (slot * Hkv + h) * D;
    // same 16-bit type on both sides, no rotation, 16-byte aligned rows: a row moves as 16-byte pieces, one per lane
    if (w.raw_ok) {
        if (lane < D / 8) {
            *(uint4*)((uint16_t*)p.key_cache + off + lane * 8) = *(const uint4*)((const uint16_t*)krow.row + lane * 8);
            *(uint4*)((uint16_t*)p.value_cache + off + lane * 8) = *(const uint4*)((const uint16_t*)vrow.row + lane * 8);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // head_dim <= 256, element d = lane + 32 i
        const int d = lane + 32 * i;
        if (d < D) {
            const float kf = krow(d), vf = vrow(d);
            if (p.kv_dtype == EMLX_F16) {
                ((__half*)p.key_cache)[off + d] = __float2half_rn(kf);
                ((__half*)p.value_cache)[off + d] = __float2half_rn(vf);
            } else if (p.kv_dtype == EMLX_BF16) {
                ((__nv_bfloat16*)p.key_cache)[off + d] = __float2bfloat16_rn(kf);
                ((__nv_bfloat16*)p.value_cache)[off + d] = __float2bfloat16_rn(vf);
            } else {
                ((float*)p.key_cache)[off + d] = kf;
                ((float*)p.value_cache)[off + d] = vf;
            }
        }
    }
}

// Rotated copy of query row `qw` (token * Hq + head) at position `pos`.  Called by a whole warp.
template <typename TIn>
__device__ __forceinline__ void rotate_query_row(const WriteParams& w, int64_t qw, int lane, int pos) {
    const int D = w.pool.head_dim;
    const RowReader<TIn> q{(const TIn*)w.q_in + qw * D, pos, &w};
    TIn* dst = (TIn*)w.q_out + qw * D;
    for (int d = lane; d < D; d += 32) dst[d] = from_f32<TIn>(q(d));
}

// Host side: whether rows can be copied bit for bit in 16-byte pieces.
inline bool raw_copy_ok(const WriteParams& w, int in_dtype) {
    const emlx_pool& p = w.pool;
    return w.has_pool && w.rope_dims == 0 && p.kv_format == EMLX_KV_FLOAT && in_dtype == p.kv_dtype &&
           (in_dtype == EMLX_F16 || in_dtype == EMLX_BF16) && p.head_dim % 8 == 0 &&
           (((uintptr_t)w.keys | (uintptr_t)w.values | (uintptr_t)p.key_cache | (uintptr_t)p.value_cache) & 15) == 0;
}

int validate_pool(const emlx_pool* pool);

}  // namespace emlx
