// Prefill chunks over an affine (8/4-bit) pool on the tcgen05 kernel: the pages of the sequences that own 128-row
// units are first expanded to fp16 rows in a scratch pool laid out like a float pool ([pages, 128, Hkv, D]), and the
// 128-row kernel then reads that pool through its usual tensor maps and a scratch page table.  A chunk re-reads its
// context once per 128-row unit (hundreds of times, from L2), the expansion touches every page once: on a mixed batch
// shaped like c3 with an 8-bit pool the long rows took 6.0 ms on the 32-row mma.sync kernel.
#include "attn_tiled.cuh"
#include "tensor_maps.cuh"

namespace emlx {

constexpr int kDqThreads = 256;
constexpr int kDqPageSlots = 32;   // pages of a sequence are dealt over this many slots (times the KV heads) of CTAs

__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

struct DequantParams {
    emlx_pool pool;        // the affine pool
    void* k_out;           // scratch rows [cap, 128, Hkv, D], fp16 whatever the query type
    void* v_out;
    const int32_t* bt;     // [S, MB] pages of the scheduled sequences
    const int32_t* kv_lens;
    const int32_t* qsl;
    int32_t* sbt;          // [S, MB] scratch page of (sequence, page index), written for the pages expanded here
    int32_t* status;
    int S, MB, G, cap;     // cap: scratch pages (MB for each sequence the scratch was sized for)
    int window;            // sliding window of the call (0 = off): pages wholly before every row's window are skipped
    // bf16 queries: the rows of the sequences served here are converted to fp16 for the tensor core (which wants both
    // operands of a product in one type); nullptr for fp16 queries
    const void* q_in;
    void* q16;
    int Hq;
};

// The k-th sequence (in batch order) with more than 16 query rows, or -1; called by one warp.
__device__ __forceinline__ int kth_long_sequence(const int32_t* qsl, int S, int G, int k, int lane) {
    int seen = 0;
    for (int s0 = 0; s0 < S; s0 += 32) {
        const int s = s0 + lane;
        const bool is_long = s < S && (long long)(qsl[s + 1] - qsl[s]) * G > 16;
        const unsigned m = __ballot_sync(0xffffffffu, is_long);
        const int n = __popc(m);
        if (seen + n > k) {
            unsigned mm = m;
            for (int r = k - seen; r > 0; --r) mm &= mm - 1;  // drop the lowest set bits
            return s0 + __ffs(mm) - 1;
        }
        seen += n;
    }
    return -1;
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    const float lo = __uint_as_float(v << 16), hi = __uint_as_float(v & 0xffff0000u);
    return pack16(lo, hi);
}
__device__ __forceinline__ uint32_t f16x2_to_bf16x2(uint32_t v) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(f.y), "f"(f.x));
    return r;
}


// blockIdx.y = k: the CTA works for the k-th sequence that owns 128-row units (the host only knows an upper bound of
// their number, from the scratch size); blockIdx.x = (page slot, KV head): pages slot, slot + kDqPageSlots, ... of that
// sequence, one KV head of each.  Many small CTAs: the expansion is a chain of dependent loads per item and stands
// in front of the whole attention call.
template <int BITS>
__global__ void __launch_bounds__(kDqThreads) dequant_pages_kernel(const DequantParams p) {
    __shared__ int s_seq;
    grid_dep_wait();   // the pool's newest rows come from the step's write, the lengths from its metadata
    grid_dep_launch();
    const int tid = threadIdx.x, lane = tid & 31;
    if (tid < 32) {
        const int found = kth_long_sequence(p.qsl, p.S, p.G, (int)blockIdx.y, lane);
        if (lane == 0) s_seq = found;
        // The scratch was sized for gridDim.y sequences.  If the batch holds more with 128-row units, those cannot be
        // expanded: report it and mark their pages as absent (the 128-row kernel then reads zero rows for them).
        if (found >= 0 && blockIdx.y == gridDim.y - 1 && blockIdx.x == 0) {
            for (int s = found + 1; s < p.S; ++s) {
                if ((long long)(p.qsl[s + 1] - p.qsl[s]) * p.G <= 16) continue;
                if (lane == 0) flag_error(p.status, EMLX_DEV_OVERFLOW);
                const int pages = min(p.MB, (p.kv_lens[s] + kTile - 1) / kTile);
                for (int i = lane; i < pages; i += 32) p.sbt[(long long)s * p.MB + i] = -1;
            }
        }
    }
    __syncthreads();
    const int s = s_seq;
    if (s < 0) return;
    if (p.q16 != nullptr) {
        // this sequence's query rows, bf16 -> fp16, shared by the CTAs of the grid row
        const long long first = (long long)p.qsl[s] * p.Hq * p.pool.head_dim / 8;
        const long long count = (long long)(p.qsl[s + 1] - p.qsl[s]) * p.Hq * p.pool.head_dim / 8;
        const uint4* src = (const uint4*)p.q_in + first;
        uint4* dst = (uint4*)p.q16 + first;
        for (long long i = (long long)blockIdx.x * kDqThreads + tid; i < count; i += (long long)gridDim.x * kDqThreads) {
            const uint4 v = src[i];
            dst[i] = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
        }
    }
    const int kv_len = p.kv_lens[s];
    const emlx_pool& pool = p.pool;
    const int Hkv = pool.num_kv_heads, D = pool.head_dim, groups = D / 64;
    constexpr int bs = kTile;
    const int h = blockIdx.x % Hkv, slot = blockIdx.x / Hkv, slots = gridDim.x / Hkv;
    // with a sliding window no row of the sequence looks before the window of its first query token (the same bound
    // as the first tile of the work list's units), so the pages before it are neither expanded nor given an id
    const int q_len = p.qsl[s + 1] - p.qsl[s];
    const int first_page = p.window > 0 ? max(0, kv_len - q_len - p.window + 1) / bs : 0;
    for (int i = first_page + slot; i < p.MB && (long long)i * bs < kv_len; i += slots) {
        const int page = p.bt[(long long)s * p.MB + i];
        // the CTA of head 0 hands out the scratch page; the CTAs of the other heads of this (sequence, page) cannot
        // wait for it, so every head takes the page's id from the same rule instead: pages are numbered per sequence
        // slot k, id = k * MB + i (the scratch holds MB pages for each of its sequences)
        const int id = (page >= 0 && page < pool.num_blocks && (long long)blockIdx.y * p.MB + i < p.cap)
                           ? (int)blockIdx.y * p.MB + i : -1;
        if (h == 0 && tid == 0) {
            if (page < 0 || page >= pool.num_blocks) flag_error(p.status, EMLX_DEV_BAD_PAGE);
            else if (id < 0) flag_error(p.status, EMLX_DEV_OVERFLOW);  // the caller's scratch is smaller than the batch needs
            p.sbt[(long long)s * p.MB + i] = id;
        }
        if (id < 0) continue;
        uint16_t* kdst = (uint16_t*)p.k_out + (long long)id * bs * Hkv * D;
        uint16_t* vdst = (uint16_t*)p.v_out + (long long)id * bs * Hkv * D;
        const int chunks = D / 8, items = bs * chunks;
        // keys: codes [tok][head][D * BITS / 8]; a thread expands eight consecutive elements
        for (int it = tid; it < items; it += kDqThreads) {
            const int ch = it % chunks, tok = it / chunks;
            const int d0 = ch * 8, g = d0 / 64;
            const long long sb = (((long long)page * Hkv + h) * bs + tok) * groups + g;
            const float sc = __half2float(((const __half*)pool.k_scale)[sb]), bi = __half2float(((const __half*)pool.k_bias)[sb]);
            const uint8_t* src = (const uint8_t*)pool.key_cache + (((long long)page * bs + tok) * Hkv + h) * (D * BITS / 8);
            float x[8];
            if constexpr (BITS == 8) {
                const uint2 c = *(const uint2*)(src + d0);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    x[e] = fmaf((float)((c.x >> (8 * e)) & 0xff), sc, bi);
                    x[4 + e] = fmaf((float)((c.y >> (8 * e)) & 0xff), sc, bi);
                }
            } else {
                const uint32_t c = *(const uint32_t*)(src + d0 / 2);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = fmaf((float)((c >> (4 * e)) & 0xf), sc, bi);
            }
            uint4 o;
            o.x = pack16(x[0], x[1]); o.y = pack16(x[2], x[3]);
            o.z = pack16(x[4], x[5]); o.w = pack16(x[6], x[7]);
            *(uint4*)(kdst + ((long long)tok * Hkv + h) * D + d0) = o;
        }
        // values: codes [head][d][tok * BITS / 8] (tokens of one element contiguous); consecutive threads take
        // consecutive tokens, so that the eight byte loads of a thread are coalesced across the warp
        for (int it = tid; it < items; it += kDqThreads) {
            const int tok = it % bs, ch = it / bs;
            const int d0 = ch * 8, g = d0 / 64;
            const long long sb = (((long long)page * Hkv + h) * bs + tok) * groups + g;
            const float sc = __half2float(((const __half*)pool.v_scale)[sb]), bi = __half2float(((const __half*)pool.v_bias)[sb]);
            const uint8_t* src = (const uint8_t*)pool.value_cache + ((long long)page * Hkv + h) * D * (bs * BITS / 8);
            float x[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                int code;
                if constexpr (BITS == 8) code = src[(long long)(d0 + e) * bs + tok];
                else code = (src[(long long)(d0 + e) * (bs / 2) + (tok >> 1)] >> ((tok & 1) * 4)) & 0xf;
                x[e] = fmaf((float)code, sc, bi);
            }
            uint4 o;
            o.x = pack16(x[0], x[1]); o.y = pack16(x[2], x[3]);
            o.z = pack16(x[4], x[5]); o.w = pack16(x[6], x[7]);
            *(uint4*)(vdst + ((long long)tok * Hkv + h) * D + d0) = o;
        }
    }
}

// After the 128-row kernel, bf16 queries: the output rows of the sequences it served, fp16 -> bf16, into the caller's
// output (the other rows of that buffer belong to the short-row kernels).  Same grid rows as the expansion.
__global__ void __launch_bounds__(kDqThreads) convert_out_rows_kernel(const uint4* __restrict__ out16, uint4* __restrict__ out,
                                                                      const int32_t* __restrict__ qsl, int S, int G,
                                                                      int row_chunks /* Hq * D / 8 */) {
    __shared__ int s_seq;
    grid_dep_wait();
    grid_dep_launch();
    if (threadIdx.x < 32) {
        const int found = kth_long_sequence(qsl, S, G, (int)blockIdx.y, threadIdx.x & 31);
        if (threadIdx.x == 0) s_seq = found;
    }
    __syncthreads();
    const int s = s_seq;
    if (s < 0) return;
    const long long first = (long long)qsl[s] * row_chunks, count = (long long)(qsl[s + 1] - qsl[s]) * row_chunks;
    for (long long i = (long long)blockIdx.x * kDqThreads + threadIdx.x; i < count; i += (long long)gridDim.x * kDqThreads) {
        const uint4 v = out16[first + i];
        out[first + i] = make_uint4(f16x2_to_bf16x2(v.x), f16x2_to_bf16x2(v.y), f16x2_to_bf16x2(v.z), f16x2_to_bf16x2(v.w));
    }
}

size_t dequant_header_bytes(int S, int MB) { return ((size_t)S * MB * 4 + 255) & ~(size_t)255; }
size_t dequant_page_bytes(const emlx_pool* pool) { return (size_t)kTile * pool->num_kv_heads * pool->head_dim * 2; }
// fp16 copies of the queries and of the output when the queries are bf16
size_t dequant_rows_bytes(int T, int Hq, int D, int q_dtype) {
    return q_dtype == EMLX_BF16 ? (((size_t)T * Hq * D * 2 + 255) & ~(size_t)255) : 0;
}

// Splits the memory behind the attention workspace into the scratch page table, the fp16 copies of queries and output
// (bf16 queries only) and the two scratch pools.
bool dequant_scratch_layout(const emlx_pool* pool, const emlx_attn_args* a, uint8_t* base, size_t bytes, DequantScratch* out) {
    const size_t header = dequant_header_bytes(a->num_seqs, a->max_blocks_per_seq), page = dequant_page_bytes(pool);
    const size_t rows = dequant_rows_bytes(a->total_tokens, a->num_q_heads, pool->head_dim, a->q_dtype);
    if (bytes < header + 2 * rows + 2 * page) return false;
    const size_t cap = (bytes - header - 2 * rows) / (2 * page);
    out->sbt = (int32_t*)base;
    out->q16 = rows ? base + header : nullptr;
    out->out16 = rows ? base + header + rows : nullptr;
    out->k = base + header + 2 * rows;
    out->v = out->k + cap * page;
    out->cap = (int)(cap > (size_t)0x7fffffff / kTile ? (size_t)0x7fffffff / kTile : cap);
    return true;
}

static int dequant_grid_rows(const emlx_attn_args* a, const DequantScratch& sc) {
    const int rows = sc.cap / a->max_blocks_per_seq;
    return rows < 65535 ? rows : 65535;
}

int launch_dequant_pages(const emlx_attn_args* a, const emlx_pool* pool, const DequantScratch& sc, cudaStream_t stream) {
    DequantParams p;
    p.pool = *pool;
    p.k_out = sc.k; p.v_out = sc.v;
    p.bt = a->block_tables; p.kv_lens = a->kv_lens; p.qsl = a->query_start_loc;
    p.sbt = sc.sbt; p.status = a->status;
    p.S = a->num_seqs; p.MB = a->max_blocks_per_seq; p.G = a->num_q_heads / pool->num_kv_heads; p.cap = sc.cap;
    p.q_in = a->queries; p.q16 = sc.q16; p.Hq = a->num_q_heads;
    p.window = a->sliding_window;
    // one grid row per sequence the scratch can hold (the caller sized it for an upper bound of the sequences with
    // more than 16 rows); rows beyond the batch's own count find no sequence and leave
    const int rows = dequant_grid_rows(a, sc);
    if (rows < 1) return fail(EMLX_ERR_WORKSPACE, "the scratch behind the workspace holds less than one sequence's pages");
    const dim3 grid((unsigned)(min(kDqPageSlots, a->max_blocks_per_seq) * pool->num_kv_heads), (unsigned)rows);
    if (pool->kv_format == EMLX_KV_AFFINE4) EMLX_CUDA_OK(launch_pdl(dequant_pages_kernel<4>, grid, kDqThreads, 0, stream, p));
    else EMLX_CUDA_OK(launch_pdl(dequant_pages_kernel<8>, grid, kDqThreads, 0, stream, p));
    EMLX_LAUNCHED();
    return EMLX_OK;
}

int launch_convert_out_rows(const emlx_attn_args* a, const emlx_pool* pool, const DequantScratch& sc, cudaStream_t stream) {
    const dim3 grid(64u, (unsigned)dequant_grid_rows(a, sc));
    EMLX_CUDA_OK(launch_pdl(convert_out_rows_kernel, grid, kDqThreads, 0, stream, (const uint4*)sc.out16, (uint4*)a->out,
                            a->query_start_loc, a->num_seqs, a->num_q_heads / pool->num_kv_heads,
                            a->num_q_heads * pool->head_dim / 8));
    EMLX_LAUNCHED();
    return EMLX_OK;
}

}  // namespace emlx

extern "C" size_t emlx_attn_dequant_bytes(const emlx_pool* pool, int32_t num_seqs, int32_t max_blocks_per_seq,
                                          int32_t num_long_seqs, int32_t total_tokens, int32_t num_q_heads, int32_t q_dtype) {
    if (!pool || pool->kv_format == EMLX_KV_FLOAT || num_long_seqs <= 0 || num_seqs <= 0 || max_blocks_per_seq <= 0) return 0;
    return emlx::dequant_header_bytes(num_seqs, max_blocks_per_seq) +
           2 * emlx::dequant_rows_bytes(total_tokens, num_q_heads, pool->head_dim, q_dtype) +
           2 * emlx::dequant_page_bytes(pool) * (size_t)num_long_seqs * (size_t)max_blocks_per_seq;
}
