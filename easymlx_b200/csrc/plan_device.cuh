// Device routine that builds the tiled kernels' work list; called by the stand-alone plan kernel and, fused,
// by the batch-metadata kernel.  One CTA of kMetaThreads threads; sequences are handled 1024 at a time with
// register-resident block scans (two per class), so the whole list costs a few microseconds.
#pragma once
#include "attn_tiled.cuh"
#include "scan.cuh"

namespace emlx {

#ifdef EMLX_TRACE_META
static __device__ long long g_meta_trace[32];  // measurement aid, one copy per translation unit
#endif

constexpr int kOrderBins = 1024;  // tile-count bins of the class-3 unit order (longer units share the last bin)

// Exclusive prefix of one value per thread across the CTA; `total` receives the CTA-wide sum.
__device__ __forceinline__ int block_scan_value(int v, int32_t* smem /* [33] */, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    __syncthreads();  // smem free from the previous use
    if (lane == 31) smem[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int wsum = smem[lane];
        int wi = wsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += up;
        }
        smem[lane] = wi - wsum;
        if (lane == 31) smem[32] = wi;
    }
    __syncthreads();
    total = smem[32];
    return smem[warp] + incl - v;
}

// Tile range of the rows [row0, row1) of a sequence: first tile and number of tiles (at least one, so that a
// unit without keys still produces zero rows).
__device__ __forceinline__ void unit_tiles(int row0, int row1, int G, int q_len, int kv_len, int window, int& tile_lo,
                                           int& ntiles) {
    const int ctx = kv_len - q_len;
    const int i_min = row0 / G, i_max = (row1 - 1) / G;
    const int hi = min(kv_len, ctx + i_max + 1);
    const int lo = window > 0 ? max(0, min(kv_len - 1, ctx + i_min) - window + 1) : 0;
    tile_lo = 0;
    ntiles = 1;
    if (hi > 0 && hi > lo) {
        tile_lo = lo / kTile;
        ntiles = (hi + kTile - 1) / kTile - tile_lo;
    }
}

// Slice boundaries of class c: CTA i of num_ctas takes the flat tiles [start[i], start[i+1]), cut at equal shares of
// cost, kTileCost per tile + part_cost(c) per (unit, head) part (measured on the 8-row decode kernel: a part
// boundary costs about as much as 2.3 tiles).  `cum` is the exclusive prefix sum of tiles per unit (num_units + 1).
// Only the first `used` CTAs receive work (the others get empty slices and leave at once).
__device__ __forceinline__ void cut_slices(int c, const int32_t* cum, int num_units, int tile_base, int Hkv,
                                           int num_ctas, int32_t* plan, const PlanLayout& L, int used) {
    const int tid = threadIdx.x;
    {
        for (int i = tid; i <= num_ctas; i += kMetaThreads) {
            long long start = (long long)tile_base * Hkv;
            int first_unit = num_units;
            const long long kPartCost = part_cost(c);
            if (i < used && num_units > 0) {
                const long long total = (long long)Hkv * (kTileCost * tile_base + kPartCost * num_units);
                // 64-bit division is a long software routine; the totals of any realistic batch fit 32 bits
                const long long target = total * used < (1LL << 31) ? (long long)((unsigned)(total * i) / (unsigned)used)
                                                                    : total * i / used;
                int lo = 0, hi = num_units;  // largest u with cost_before(u) <= target
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if ((long long)Hkv * (kTileCost * cum[mid] + kPartCost * mid) <= target) lo = mid; else hi = mid;
                }
                const int u = lo, nt = cum[u + 1] - cum[u];
                const long long rem = target - (long long)Hkv * (kTileCost * cum[u] + kPartCost * u);
                const long long per_head = kTileCost * nt + kPartCost;
                const int head = (int)min((long long)Hkv - 1,
                                          rem < (1LL << 31) ? (long long)((unsigned)rem / (unsigned)per_head) : rem / per_head);
                const long long r2 = rem - head * per_head;
                const int j = r2 <= kPartCost ? 0 : (int)min((long long)nt, (r2 - kPartCost + kTileCost / 2) / kTileCost);
                start = (long long)cum[u] * Hkv + (long long)head * nt + j;
                first_unit = u;
            } else if (num_units == 0) {
                start = 0;
                first_unit = 0;
            }
            plan[L.cta_unit[c] + i] = first_unit;
            plan[L.cta_start[c] + i] = (int)start;
        }
    }
}

// How many CTAs the short-row (HBM-bound) kernel gets when the 128-row (tensor-bound) kernel runs beside it.
// Per (head, tile) both cost about the same SM time when each has the GPU to itself (measured on the Qwen3-32B-shaped
// mixed batch: 1.4 SM-us either way), but a short-row CTA that does not have to share HBM with 147 others streams
// kShortRowSpeedup times faster (measured 1.9: 85-93 GB/s per SM on 24-48 SMs against 47 GB/s on all 148; with three
// 64 KB stages in flight an SM cannot pull more).  The 128-row kernel hands its items out dynamically, so the split
// only has to keep the short-row kernel from finishing last: it gets the share that makes both end together, plus a
// margin, and never more CTAs than saturate HBM unless the short rows dominate the batch.
constexpr int kShortRowSpeedupX10 = 19;
__host__ __device__ inline int short_row_share(long long short_tiles, long long wide_tiles, int num_ctas) {
    const long long x = short_tiles * 10 / kShortRowSpeedupX10;          // short-row work at the faster rate
    long long balanced = (num_ctas * x + x + wide_tiles - 1) / (x + wide_tiles);
    balanced += (balanced + 5) / 6;                                       // margin
    const long long saturating = ((long long)num_ctas * 10 + kShortRowSpeedupX10 - 1) / kShortRowSpeedupX10;
    long long share = balanced;
    if (balanced > saturating) {
        // the short rows dominate: the 128-row kernel gets the CTAs it needs to finish within the HBM-bound time of the
        // short rows, the rest stream
        long long wide_ctas = (wide_tiles * num_ctas + short_tiles - 1) / (short_tiles > 0 ? short_tiles : 1);
        wide_ctas += (wide_ctas + 5) / 6;
        share = num_ctas - wide_ctas;
        if (share < saturating) share = saturating;
    }
    return (int)(share < 1 ? 1 : (share > num_ctas ? num_ctas : share));
}

__device__ __forceinline__ void build_plan(const int32_t* qsl, const int32_t* kv_lens, int S, int G, int window,
                                           int class_lo, int class_hi, bool wide, int Hkv, int num_ctas,
                                           int32_t* plan, const PlanLayout& L, int32_t* scan_smem,
                                           int32_t* seq_off_buf = nullptr, int32_t* cum_smem = nullptr,
                                           int cum_cap = 0, int short_ctas = 0, bool two_per_sm = false) {
    const int tid = threadIdx.x;
    const int base_ctas = num_ctas;
    // The 128-row class comes first: the short-row class that is launched right before the 128-row kernel runs
    // beside it, and how many CTAs it then gets depends on how much 128-row work there is.
    long long wide_tiles = 0;        // (unit, head, tile) triples of class 3
    bool short_class_seen = false;   // a short-row class that is launched later than the current one has work
    for (int c = kNumClasses - 1; c >= 0; --c) {
        num_ctas = class_ctas(c, base_ctas, two_per_sm);
        if (c < class_lo || c > class_hi) {
            if (tid == 0) { plan[4 * c + 0] = 0; plan[4 * c + 1] = 0; }
            for (int i = tid; i <= num_ctas; i += kMetaThreads) { plan[L.cta_start[c] + i] = 0; plan[L.cta_unit[c] + i] = 0; }
            continue;
        }
        const int rows_c = class_rows(c);
        int32_t* unit_seq = plan + L.unit_seq[c];
        int32_t* unit_row0 = plan + L.unit_row0[c];
        int32_t* unit_tile_lo = plan + L.unit_tile_lo[c];
        int32_t* unit_cum = plan + L.unit_cum[c];
        // first unit of every sequence in this class; shared memory when the caller has room for it (a global
        // store followed by a load from another thread costs an L2 round trip per phase)
        int32_t* seq_off = seq_off_buf ? seq_off_buf : plan + L.tmp;
#ifdef EMLX_TRACE_META
        if (threadIdx.x == 0 && c == class_lo) g_meta_trace[8] = clock64();
#endif
        // pass 1: units per sequence -> first-unit offsets
        int num_units = 0;
        for (int s0 = 0; s0 < S; s0 += kMetaThreads) {
            const int s = s0 + tid;
            int n = 0;
            if (s < S) {
                const int q_len = qsl[s + 1] - qsl[s], rows = q_len * G;
                if (q_len > 0 && unit_class(rows, wide) == c) n = (rows + rows_c - 1) / rows_c;
            }
            int n_total;
            const int off = num_units + block_scan_value(n, scan_smem, n_total);
            if (s < S) seq_off[s] = off;
            num_units += n_total;
        }
        __syncthreads();
#ifdef EMLX_TRACE_META
        if (threadIdx.x == 0 && c == class_lo) g_meta_trace[9] = clock64();
#endif
        // pass 2: one thread per unit: owner sequence by binary search, tile range, running tile prefix
        int tile_base = 0;
        for (int i0 = 0; i0 < num_units; i0 += kMetaThreads) {
            const int idx = i0 + tid;
            int nt = 0;
            if (idx < num_units) {
                int lo = 0, hi = S;  // largest s with seq_off[s] <= idx
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (seq_off[mid] <= idx) lo = mid; else hi = mid;
                }
                const int s = lo, u = idx - seq_off[s];
                const int q_len = qsl[s + 1] - qsl[s], rows = q_len * G;
                int tile_lo;
                unit_tiles(u * rows_c, min(rows, (u + 1) * rows_c), G, q_len, kv_lens[s], window, tile_lo, nt);
                unit_seq[idx] = s;
                unit_row0[idx] = u * rows_c;
                unit_tile_lo[idx] = tile_lo;
            }
            int t_total;
            const int t_off = tile_base + block_scan_value(nt, scan_smem, t_total);
            if (idx < num_units) {
                unit_cum[idx] = t_off;
                if (idx < cum_cap) cum_smem[idx] = t_off;
            }
            tile_base += t_total;
        }
        if (tid == 0) {
            unit_cum[num_units] = tile_base;
            if (num_units < cum_cap) cum_smem[num_units] = tile_base;
            plan[4 * c + 0] = num_units;
            plan[4 * c + 1] = tile_base;
        }
        __syncthreads();  // unit_cum is complete; seq_off is reused by the next class
        if (c == 3) {
            // the 128-row kernel hands whole (unit, head) items to its CTAs: list the units by decreasing number of
            // tiles (counting sort; the order among equals does not matter) so that dealing them out stays balanced
            __shared__ int32_t bins[kOrderBins];
            int32_t* order = plan + L.unit_order;
            for (int b = tid; b < kOrderBins; b += kMetaThreads) bins[b] = 0;
            __syncthreads();
            for (int u = tid; u < num_units; u += kMetaThreads)
                atomicAdd(&bins[kOrderBins - 1 - min(unit_cum[u + 1] - unit_cum[u], kOrderBins - 1)], 1);
            __syncthreads();
            static_assert(kOrderBins == kMetaThreads, "one bin per thread");
            int n_total;
            const int first = block_scan_value(bins[tid], scan_smem, n_total);
            __syncthreads();
            bins[tid] = first;
            __syncthreads();
            for (int u = tid; u < num_units; u += kMetaThreads)
                order[atomicAdd(&bins[kOrderBins - 1 - min(unit_cum[u + 1] - unit_cum[u], kOrderBins - 1)], 1)] = u;
            __syncthreads();
        }
#ifdef EMLX_TRACE_META
        if (threadIdx.x == 0 && c == class_lo) g_meta_trace[10] = clock64();
#endif
        int used = num_ctas;
        if (c == 3) {
            wide_tiles = (long long)tile_base * Hkv;
        } else if (tile_base > 0) {
            if (wide_tiles > 0 && !short_class_seen)
                used = short_ctas > 0 ? min(short_ctas, num_ctas) : short_row_share((long long)tile_base * Hkv, wide_tiles, num_ctas);
            short_class_seen = true;
        }
        cut_slices(c, num_units < cum_cap ? cum_smem : unit_cum, num_units, tile_base, Hkv, num_ctas, plan, L, used);
        __syncthreads();
    }
}

// Work list of a batch in which every sequence has exactly one query token (G rows): unit i is sequence i, so the
// unit counting and the owner search of build_plan fall away.  Same output as build_plan(..., max one class).
__device__ __forceinline__ void build_plan_decode(const int32_t* kv_lens /* shared memory */, int S, int G, int window,
                                                  int cls, int Hkv, int base_ctas, int32_t* plan, const PlanLayout& L,
                                                  int32_t* scan_smem, int32_t* cum_smem /* [S + 1] */, bool two_per_sm) {
    const int tid = threadIdx.x;
    for (int c = 0; c < kNumClasses; ++c) {
        if (c == cls) continue;
        if (tid == 0) { plan[4 * c + 0] = 0; plan[4 * c + 1] = 0; }
        for (int i = tid; i <= class_ctas(c, base_ctas, two_per_sm); i += kMetaThreads) { plan[L.cta_start[c] + i] = 0; plan[L.cta_unit[c] + i] = 0; }
    }
    const int num_ctas = class_ctas(cls, base_ctas, two_per_sm);
    int32_t* unit_seq = plan + L.unit_seq[cls];
    int32_t* unit_row0 = plan + L.unit_row0[cls];
    int32_t* unit_tile_lo = plan + L.unit_tile_lo[cls];
    int32_t* unit_cum = plan + L.unit_cum[cls];
    int tile_base = 0;
#pragma unroll 1
    for (int i0 = 0; i0 < S; i0 += kMetaThreads) {
        const int idx = i0 + tid;
        int nt = 0;
        if (idx < S) {
            int tile_lo;
            unit_tiles(0, G, G, 1, kv_lens[idx], window, tile_lo, nt);
            unit_seq[idx] = idx;
            unit_row0[idx] = 0;
            unit_tile_lo[idx] = tile_lo;
        }
        int t_total;
        const int t_off = tile_base + block_scan_value(nt, scan_smem, t_total);
        if (idx < S) {
            unit_cum[idx] = t_off;
            cum_smem[idx] = t_off;
        }
        tile_base += t_total;
    }
    if (tid == 0) {
        unit_cum[S] = tile_base;
        cum_smem[S] = tile_base;
        plan[4 * cls + 0] = S;
        plan[4 * cls + 1] = tile_base;
        if (cls == 3) plan[L.unit_order] = 0;
    }
    __syncthreads();
    if (cls == 3) {
        // 128-row units are dealt out by decreasing length; a decode batch reaches this class only with a GQA group
        // above 16, and its units are all alike enough for batch order
        for (int u = tid; u < S; u += kMetaThreads) plan[L.unit_order + u] = u;
    }
    cut_slices(cls, cum_smem, S, tile_base, Hkv, num_ctas, plan, L, num_ctas);
    __syncthreads();
}

// classes that can hold a sequence of 1..max_query_len tokens with G rows per token (0 = unknown: all of them)
inline void class_range(int G, int max_query_len, bool wide, int& lo, int& hi) {
    lo = unit_class(G, wide);
    const long long rows = (long long)max_query_len * G;
    hi = max_query_len > 0 ? unit_class(rows > (1 << 20) ? (1 << 20) : (int)rows, wide) : (wide ? 3 : 2);
}

}  // namespace emlx
