// Work-list ("plan") and workspace layouts shared by the plan kernel and the tiled attention kernels.
//
// A *unit* is up to 8*NT query rows of one sequence (row = query token x GQA head of one KV head,
// token-major) together with the range of 128-token KV tiles those rows may attend.  Units are sorted
// into classes by their row count so that each class runs with the smallest tile that holds it:
//     class 0: rows <= 8   (NT = 1)     decode with Hq/Hkv <= 8
//     class 1: rows <= 16  (NT = 2)
//     class 2: rows <= 32  (NT = 4)     spec-verify rows (or, without wide units, every longer row set in 32-row blocks)
//     class 3: 128-row blocks           prefill chunks, for the tcgen05 kernel (only with kPlanWideUnits)
// The work of a class is the flat sequence of (unit, kv head, tile); CTA c of P takes the contiguous
// slice [start[c], start[c+1]); the plan chooses the boundaries so that tiles + 1.5 x (unit, head) parts is equal
// across CTAs (a part boundary costs about as much as one and a half tiles).
#pragma once
#include "common.cuh"

namespace emlx {

constexpr int kTile = 128;        // tokens per KV tile = page size the tiled kernels require
constexpr int kNumClasses = 4;
constexpr int kPlanWideUnits = 1;  // plan flag: cut sequences with more than 32 rows into 128-row units (class 3)
constexpr int kPlanTwoCtas = 2;    // plan flag: the 8-row kernel runs two CTAs per SM (4-bit pools: the unpacking, not HBM, limits an SM)
constexpr int kPlanShortCtasShift = 8;  // plan flag bits 8-15: CTAs of the short-row kernel that runs beside the 128-row one (0 = automatic)
constexpr int kPlanHeaderWords = 16;
// Page sizes the tiled kernels read: a 128-token tile is one page, or 2 / 4 / 8 pages of a 16/32-bit pool (affine pools
// keep their values transposed inside a 128-token page, so they need that size).
__host__ __device__ inline bool tiled_page_size_ok(int block_size, int kv_format) {
    if (block_size == 128) return true;
    return kv_format == 0 && (block_size == 64 || block_size == 32 || block_size == 16);
}
__host__ __device__ inline int pages_per_tile_log2(int block_size) { return block_size == 128 ? 0 : block_size == 64 ? 1 : block_size == 32 ? 2 : 3; }
// relative cost of a tile and of a part boundary when slices are cut: measured 1 : 2.3 on the 8-row decode kernel;
// the 128-row kernel keeps 1 : 1.5
constexpr long long kTileCost = 4;
__host__ __device__ constexpr long long part_cost(int cls) { return cls == 3 ? 6 : 9; }
constexpr int kMaxGrid = 304;     // upper bound on CTAs per launch (two per SM on 148 SMs, rounded up), sizes the partial-result slots
constexpr int kMaxRows = 32;      // rows of the largest class

// CTAs of the launch that serves class c, given the CTA count of a one-per-SM launch
__host__ __device__ inline int class_ctas(int c, int base_ctas, bool two_per_sm) {
    const int n = (two_per_sm && c == 0) ? 2 * base_ctas : base_ctas;
    return n < kMaxGrid ? n : kMaxGrid;
}
__host__ __device__ inline int class_rows(int c) { return c < 3 ? 8 << c : 128; }
__host__ __device__ inline int unit_class(int rows, bool wide) {
    return rows <= 8 ? 0 : (rows <= 16 ? 1 : (!wide ? 2 : 3));
}

struct PlanLayout {
    int cap[kNumClasses];       // unit capacity per class
    int unit_seq[kNumClasses];  // word offsets into the plan
    int unit_row0[kNumClasses];
    int unit_tile_lo[kNumClasses];
    int unit_cum[kNumClasses];  // cap + 1 words: exclusive prefix sum of tiles per unit (per KV head)
    int cta_start[kNumClasses]; // kMaxGrid + 1 words: first flat tile of every CTA's slice (cost-balanced)
    int cta_unit[kNumClasses];  // kMaxGrid + 1 words: a unit at or before the one that holds that tile (search hint)
    int unit_order;             // class 3 only, cap words: units by decreasing number of tiles
    int tmp;                    // S words of scratch for the scans
    int words;
};

__host__ __device__ inline PlanLayout plan_layout(int S, int T, int Hq, int Hkv) {
    PlanLayout L;
    const int G = Hq / Hkv;
    int w = kPlanHeaderWords;
    for (int c = 0; c < kNumClasses; ++c) {
        L.cap[c] = c < 2 ? S : S + (int)(((long long)T * G + class_rows(c) - 1) / class_rows(c));
        if (L.cap[c] < 1) L.cap[c] = 1;
        L.unit_seq[c] = w; w += L.cap[c];
        L.unit_row0[c] = w; w += L.cap[c];
        L.unit_tile_lo[c] = w; w += L.cap[c];
        L.unit_cum[c] = w; w += L.cap[c] + 1;
        L.cta_start[c] = w; w += kMaxGrid + 1;
        L.cta_unit[c] = w; w += kMaxGrid + 1;
    }
    L.unit_order = w; w += L.cap[3];
    L.tmp = w; w += (S > 0 ? S : 1);
    L.words = w;
    return L;
}

// Workspace: [partial slots: 2 per CTA, fixed size] [arrival counters: one int per (class, unit, kv head)].
// A slot holds rows x head_dim un-normalised accumulators, then the rows' running maxima, then their
// running sums.  The counters are zero whenever no kernel is running (the merging CTA resets its counter),
// and the slot area has a fixed size, so one zero-initialised workspace serves calls of any geometry.
constexpr int kMaxHeadDimTiled = 128;
constexpr size_t kSlotFloats = (size_t)kMaxRows * (kMaxHeadDimTiled + 2);

struct WorkspaceLayout {
    size_t counter_off[kNumClasses];
    size_t slots_off;
    size_t bytes;
};

inline WorkspaceLayout workspace_layout(int S, int T, int Hq, int Hkv, int D) {
    (void)D;
    PlanLayout P = plan_layout(S, T, Hq, Hkv);
    WorkspaceLayout W;
    W.slots_off = 0;
    size_t off = (size_t)kMaxGrid * 2 * kSlotFloats * sizeof(float);
    for (int c = 0; c < kNumClasses; ++c) {
        W.counter_off[c] = off;
        off += (size_t)P.cap[c] * Hkv * sizeof(int32_t);
    }
    W.bytes = (off + 255) & ~(size_t)255;
    return W;
}

}  // namespace emlx
