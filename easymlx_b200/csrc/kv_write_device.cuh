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

// The new K and V row of one (token, head) in registers.  The rows are loaded before the destination is known: the
// row data and the index chain that yields the slot (slot id -> stored length -> page id) are independent, and
// right after a kernel that has streamed hundreds of megabytes through L2 every one of these loads is a miss all
// the way (translation included, about 3 us) - issued together they cost one such latency instead of four.
//   affine pools : x[2g], x[2g+1] = elements 64g + 2 lane, +1 of group g
//   float pools  : x[i] = element lane + 32 i;  raw[] = 16 bytes per lane when the row is copied bit for bit
struct RowRegs {
    float k[2 * kMaxGroups], v[2 * kMaxGroups];
    uint4 kraw, vraw;
};

template <typename TIn>
__device__ __forceinline__ void load_token_head(const WriteParams& w, int t, int h, int lane, int pos, RowRegs& r) {
    const emlx_pool& p = w.pool;
    const int Hkv = p.num_kv_heads, D = p.head_dim;
    const RowReader<TIn> krow{(const TIn*)w.keys + ((int64_t)t * Hkv + h) * D, w.rope_dims > 0 ? pos : -1, &w};
    const RowReader<TIn> vrow{(const TIn*)w.values + ((int64_t)t * Hkv + h) * D, -1, &w};
    if (p.kv_format != EMLX_KV_FLOAT) {
        const int groups = D / kQuantGroup;
#pragma unroll
        for (int g = 0; g < kMaxGroups; ++g) {
            if (g < groups) {
                const int d0 = g * kQuantGroup + 2 * lane;
                r.k[2 * g] = krow(d0); r.k[2 * g + 1] = krow(d0 + 1);
                r.v[2 * g] = vrow(d0); r.v[2 * g + 1] = vrow(d0 + 1);
            }
        }
    } else if (w.raw_ok) {
        if (lane < D / 8) {
            r.kraw = *(const uint4*)((const uint16_t*)krow.row + lane * 8);
            r.vraw = *(const uint4*)((const uint16_t*)vrow.row + lane * 8);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2 * kMaxGroups; ++i) {
            const int d = lane + 32 * i;
            if (d < D) { r.k[i] = krow(d); r.v[i] = vrow(d); }
        }
    }
}

template <int BITS>
__device__ __forceinline__ void store_affine_rows(const RowRegs& r, const emlx_pool& p, int64_t page, int off, int h, int lane) {
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
        int kc0, kc1, vc0, vc1;
        __half ks, kb, vs, vb;
        quantize_group<BITS>(r.k[2 * g], r.k[2 * g + 1], kc0, kc1, ks, kb);
        quantize_group<BITS>(r.v[2 * g], r.v[2 * g + 1], vc0, vc1, vs, vb);
        if (BITS == 8) *(uchar2*)(kdst + d0) = make_uchar2((unsigned char)kc0, (unsigned char)kc1);
        else kdst[d0 >> 1] = (uint8_t)(kc0 | (kc1 << 4));
        if (BITS == 8) {
            vdst[(int64_t)d0 * bs + off] = (uint8_t)vc0;
            vdst[(int64_t)(d0 + 1) * bs + off] = (uint8_t)vc1;
        } else {
            // two tokens share a byte; tokens of the same batch may land in the same 32-bit word, so the
            // nibble is replaced with word atomics (each nibble has exactly one writer per batch)
            const int shift = ((off >> 1) & 3) * 8 + (off & 1) * 4;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                uint8_t* byte = vdst + (int64_t)(d0 + e) * (bs / 2) + (off >> 1);
                unsigned int* word = (unsigned int*)((uintptr_t)byte & ~(uintptr_t)3);
                atomicAnd(word, ~(0xFu << shift));
                atomicOr(word, (unsigned int)(e ? vc1 : vc0) << shift);
            }
        }
        if (lane == 0) {
            ((__half*)p.k_scale)[sb_base + g] = ks;
            ((__half*)p.k_bias)[sb_base + g] = kb;
            ((__half*)p.v_scale)[sb_base + g] = vs;
            ((__half*)p.v_bias)[sb_base + g] = vb;
        }
    }
}

// Store the rows loaded by load_token_head at flat slot `slot` (page * block_size + offset; negative: skip).
template <typename TIn>
__device__ __forceinline__ void store_token_head(const WriteParams& w, int h, int lane, int64_t slot, const RowRegs& r) {
    const emlx_pool& p = w.pool;
    const int Hkv = p.num_kv_heads, D = p.head_dim;
    if (slot < 0) return;
    if (slot >= p.num_blocks * p.block_size) {
        if (lane == 0) flag_error(w.status, EMLX_DEV_BAD_PAGE);
        return;
    }
    if (p.kv_format != EMLX_KV_FLOAT) {
        const int64_t page = slot / p.block_size;
        const int in_page = (int)(slot - page * p.block_size);
        if (p.kv_format == EMLX_KV_AFFINE8) store_affine_rows<8>(r, p, page, in_page, h, lane);
        else store_affine_rows<4>(r, p, page, in_page, h, lane);
        return;
    }
    const int64_t off = (slot * Hkv + h) * D;
    if (w.raw_ok) {  // same 16-bit type on both sides, no rotation, 16-byte aligned rows
        if (lane < D / 8) {
            *(uint4*)((uint16_t*)p.key_cache + off + lane * 8) = r.kraw;
            *(uint4*)((uint16_t*)p.value_cache + off + lane * 8) = r.vraw;
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2 * kMaxGroups; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
            if (p.kv_dtype == EMLX_F16) {
                ((__half*)p.key_cache)[off + d] = __float2half_rn(r.k[i]);
                ((__half*)p.value_cache)[off + d] = __float2half_rn(r.v[i]);
            } else if (p.kv_dtype == EMLX_BF16) {
                ((__nv_bfloat16*)p.key_cache)[off + d] = __float2bfloat16_rn(r.k[i]);
                ((__nv_bfloat16*)p.value_cache)[off + d] = __float2bfloat16_rn(r.v[i]);
            } else {
                ((float*)p.key_cache)[off + d] = r.k[i];
                ((float*)p.value_cache)[off + d] = r.v[i];
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
