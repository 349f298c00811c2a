// Tiled ragged paged attention for B200: split-KV flash-decode and short-row (spec-verify, prefill
// chunk) attention over 128-token pages, fp16/bf16 pools and affine 8/4-bit pools with fused dequant.
//
// One persistent CTA per SM walks a contiguous slice of the flat (unit, kv head, tile) work list.
// A producer warp stages K/V tiles into a shared-memory ring with TMA (tile mode, this GPU's own
// memory, no multicast) and mbarriers; eight consumer warps run
//     phase 1   S^T[128 tokens x rows] = K_tile . Q^T      (mma.sync m16n8k16; tokens on M, all GQA
//                                                           rows of the KV head on N, 16 tokens per warp)
//               online softmax (tile max through shared atomics), P^T to shared memory
//     phase 2   O^T[D x rows] += V_tile^T . P^T            (each warp owns a 16-wide slice of D)
// so that one page read serves every query row of its KV head.  A slice that ends inside a
// (unit, head) writes an un-normalised partial; the CTA that delivers the last partial merges all of
// them in CTA order (deterministic), so no CTA ever waits for another.
#include "peer.cuh"
#include "plan_device.cuh"
#include "ptx.cuh"
#include "tensor_maps.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace emlx {

int validate_attn(const emlx_attn_args* a, const emlx_pool* pool, bool need_plan);

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 64;  // + the producer warp and the split-merge warp
constexpr int kPStride = kTile * 2 + 16;  // bytes per row of a P buffer (padding keeps ldmatrix conflict-free)
constexpr int kSmemBudget = 227 * 1024 - 1024;  // dynamic shared memory minus alignment slack
constexpr int kSmemBudgetHalf = 111 * 1024;      // the same when two CTAs share an SM (228 KB per SM, 1 KB reserved per CTA)

struct TiledParams {
    const void* q;
    void* out;
    const int32_t* bt;
    const int32_t* kv_lens;
    const int32_t* qsl;
    const int32_t* hdr;  // [0] = units, [1] = tiles per head (sum over units)
    const int32_t* unit_seq;
    const int32_t* unit_row0;
    const int32_t* unit_tile_lo;
    const int32_t* unit_cum;
    const int32_t* cta_start;  // [gridDim.x + 1] first flat tile of every CTA's slice
    const int32_t* cta_unit;   // [gridDim.x + 1] a unit at or before the one holding that tile
    int32_t* counters;
    float* slots;
    int32_t* status;
    long long* trace;  // optional per-CTA records {start ns, end ns, tiles, SM id}
    const __half* k_scale;
    const __half* k_bias;
    const __half* v_scale;
    const __half* v_bias;
    long long num_blocks;
    int Hq, Hkv, G, MB, window;
    int bs, ppt_log;  // page size in tokens and log2(pages per 128-token tile)
    float scale_log2e;
    // where the rows go: `out` holds out_Hq heads per token and this call writes heads [out_head0, out_head0 + Hq).
    // A gathering call (KV heads sharded over GPUs) also stores every row into the other ranks' buffers.
    int out_Hq, out_head0;
    const PeerTable* peer;  // nullptr for an ordinary call
    int32_t* peer_flags;    // this rank's flag block
    int peer_phase;         // kPeerFirstLaunch | kPeerLastLaunch
    int few_units;          // host's guess that units span many CTAs (few sequences): selects the kernel build
};

// Element offset of (token, local head) in the output buffer.
template <int D>
__device__ __forceinline__ long long out_offset(const TiledParams& p, long long token, int head_local) {
    return (token * p.out_Hq + p.out_head0 + head_local) * D;
}

// Stores `v` at element offset `off` of this rank's output.
template <typename V>
__device__ __forceinline__ void store_out(const TiledParams& p, long long off, V v) {
    *(V*)((uint16_t*)p.out + off) = v;
}

// Gathering call: copies rows [r0, r1) of a sequence's (token, head) rows (row r = token r / G, head r % G of KV head
// `head`) from this rank's output, where they have just been stored, into every other rank's.  Kept out of line and
// out of the store loops: the kernels' hot paths are the same with and without a gather.  `t` of `nthreads` threads
// share the work; the caller makes the local rows visible to them first (a barrier or __syncwarp).
template <int D>
__device__ __noinline__ void peer_copy_rows(uint16_t* out, const PeerTable* table, int out_Hq, int out_head0, int G,
                                            int qs, int head, int r0, int r1, int t, int nthreads) {
    constexpr int CH = D / 8;  // 16-byte pieces per row
    const int n = table->num_ranks, me = table->rank;
    for (int idx = t; idx < (r1 - r0) * CH; idx += nthreads) {
        const int r = r0 + idx / CH, ch = idx % CH;
        const int i = r / G, hh = r - i * G;
        const long long off = ((long long)(qs + i) * out_Hq + out_head0 + head * G + hh) * D + ch * 8;
        const uint4 v = __ldcg((const uint4*)(out + off));
        for (int rank = 0; rank < n; ++rank)
            if (rank != me) *(uint4*)((uint16_t*)table->out[rank] + off) = v;
    }
}

// What a CTA of a gathering call keeps in shared memory (filled once after the wait on the predecessors), so that
// the end of the kernel does not chain cold loads of the table behind its last atomic.
struct PeerCache {
    int32_t* flags[kMaxPeers];  // at Cfg::OFF_PEER
};
constexpr int kMiscExit = 2;    // misc[]: warps of the CTA that have finished
constexpr int kMiscEpoch = 4;   // this call's epoch
constexpr int kMiscRanks = 5, kMiscRank = 6, kMiscPoll = 7;

// Before a warp's first remote store of a gathering call: every other rank has said that its output buffer may be
// overwritten (lane r polls rank r's flag; the flags only grow, so later calls return at once).
__device__ __forceinline__ void peer_ready(const TiledParams& p, bool& seen) {
    if (!p.peer || seen) return;
    seen = true;
    if (!(p.peer_phase & kPeerFirstLaunch)) return;  // a later kernel of the call: the first one has waited
    const int lane = threadIdx.x & 31;
    bool ok = true;
    if (lane < p.peer->num_ranks && lane != p.peer->rank)
        ok = peer_wait(p.peer_flags + kPeerReady + lane, p.peer_flags[kPeerEpoch] + 1, p.peer->poll_limit);
    if (!ok) flag_error(p.status, EMLX_DEV_WAIT_TIMEOUT);
    __syncwarp();
}

// Every warp of a gathering call passes here when it is done.  The last warp of a CTA orders the CTA's stores (remote
// ones included) before its count at GPU scope; the last CTA of the kernel then sends the done flags with
// system-scope release stores.  Fences are cumulative: everything that happened before the counts the last CTA
// has observed is ordered before its flags, so one system-scope fence per kernel is enough (one per warp, thousands
// at the end of a kernel, each waiting for the other GPUs' acknowledgements, cost tens of microseconds).
// Out of line, like everything else of the gather: an ordinary call pays one predicate here.
__device__ __noinline__ void peer_exit(int32_t* flags, int phase, int32_t* status, int* misc, const PeerCache* cache) {
    __syncwarp();
    const int lane = threadIdx.x & 31;
    int last = 0;
    if (lane == 0) {
        __threadfence_block();  // this warp's stores are ordered before the count
        if (atomicAdd_block(misc + kMiscExit, 1) == kThreads / 32 - 1) {
            __threadfence();
            last = atomicAdd(flags + kPeerTicket, 1) == (int)gridDim.x - 1 ? 1 : 0;
            if (last) __threadfence();
        }
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    __syncwarp();
    if (!last) return;
    const int n = misc[kMiscRanks], me = misc[kMiscRank], epoch = misc[kMiscEpoch];
    if (phase & kPeerLastLaunch) {
        bool ok = true;
        if (lane < n && lane != me) {
            st_release_sys(cache->flags[lane] + kPeerDone + me, epoch);
            ok = peer_wait(flags + kPeerDone + lane, epoch, misc[kMiscPoll]);
        }
        if (!ok) flag_error(status, EMLX_DEV_WAIT_TIMEOUT);
        __syncwarp();
        if (lane == 0) flags[kPeerEpoch] = epoch;
    }
    if (lane == 0) flags[kPeerTicket] = 0;  // ready for the next kernel
}
__device__ __forceinline__ void peer_warp_exit(const TiledParams& p, int* misc, const PeerCache* cache) {
    if (p.peer) peer_exit(p.peer_flags, p.peer_phase, p.status, misc, cache);
}

// Start of a gathering call's CTA, run by its merge warp (idle at that point) so that the table's cold loads stay off
// the path of the warps that start the tile loop: the call's epoch and the table of the ranks go to shared memory for
// peer_exit (whichever warp leaves last has seen this warp's count, and with it these stores), and the first CTA of
// the call's first kernel tells the other ranks that this rank's output may be overwritten (everything queued before
// the call on this rank's stream has finished).
__device__ __noinline__ void peer_enter(const PeerTable* table, int32_t* flags, int phase, int* misc, PeerCache* cache) {
    const int lane = threadIdx.x & 31;
    const int n = table->num_ranks, me = table->rank, epoch = flags[kPeerEpoch] + 1;
    if (lane < n) {
        int32_t* theirs = table->flags[lane];
        cache->flags[lane] = theirs;
        if ((phase & kPeerFirstLaunch) && blockIdx.x == 0 && lane != me) st_release_sys(theirs + kPeerReady + me, epoch);
    }
    if (lane == 0) {
        misc[kMiscEpoch] = epoch;
        misc[kMiscRanks] = n;
        misc[kMiscRank] = me;
        misc[kMiscPoll] = table->poll_limit;
    }
    __syncwarp();
}

template <int D, int NT, int FMT>
struct Cfg {
    static constexpr int ROWS = 8 * NT;
    static constexpr int KROW = FMT == 0 ? 128 : D * FMT / 8;           // bytes per smem row of the K tile
    static constexpr int KBYTES = FMT == 0 ? kTile * D * 2 : kTile * KROW;
    static constexpr int VROW = FMT == 0 ? 128 : kTile * FMT / 8;      // V: [tok][d] halves, or V^T: [d][tok bytes]
    static constexpr int VBYTES = FMT == 0 ? kTile * D * 2 : D * VROW;
    static constexpr int GROUPS = D / 64;
    static constexpr int SB1 = kTile * GROUPS * 2;                       // one scale (or bias) tile
    static constexpr int SBBYTES = FMT == 0 ? 0 : 4 * SB1;
    static constexpr int STAGE = KBYTES + VBYTES + SBBYTES;
    static constexpr int KSW = KROW == 128 ? 3 : (KROW == 64 ? 2 : 1);  // swizzle bits of the K tile
    static constexpr int VSW = VROW == 128 ? 3 : (VROW == 64 ? 2 : 1);
    static constexpr int DSL = D / 16;                                   // 16-wide slices of D
    static constexpr int TS = kConsumerWarps / DSL;                      // warps sharing a slice split the tokens
    static constexpr int NPBUF = FMT == 0 ? 1 : GROUPS;
    // Two consumer designs share the kernel: up to 16 rows every warp keeps its own softmax state and its own
    // O^T[D x rows] over its 16 tokens of each tile (no CTA barrier per tile); 32-row units split D across warps.
    static constexpr bool PRIVATE = NT <= 2;
    // 4-bit tiles are half the bytes of 8-bit ones for the same unpacking work: an SM cannot keep up with its share of
    // HBM on eight consumer warps, so the 8-row variant is built to fit twice on an SM (registers and shared memory;
    // the 16-row variant would spill a kilobyte per thread under that register limit)
    static constexpr int CTAS_PER_SM = (FMT == 4 && NT == 1) ? 2 : 1;
    static constexpr int BUDGET = CTAS_PER_SM == 2 ? kSmemBudgetHalf : kSmemBudget;
    // private design: the producer warp also stages a descriptor and the Q rows of every upcoming part
    static constexpr int QSTRIDE = D * 2;
    static constexpr int NDESC = PRIVATE ? (NT == 1 ? 4 : 2) : 0;
    static constexpr int DESC_BYTES = PRIVATE ? 64 + ROWS * QSTRIDE : 0;
    static constexpr int SMALL = 2 * 32 * 4 + 4 * kConsumerWarps * 32 * 4 + 64 + 256 + 128 + 64;  // row stats, per-warp stats, misc, barriers, requests, peer table
    static constexpr int red_bytes(int cols) { return kConsumerWarps * ROWS * (cols + 4) * 4; }
    static constexpr int stages_with(int fixed) { return (BUDGET - fixed) / STAGE > 8 ? 8 : (BUDGET - fixed) / STAGE; }
    static constexpr int PRIV_BASE = NDESC * DESC_BYTES + SMALL;
    // columns of D summed across warps per pass: the widest buffer that still leaves min(4, best) stages
    static constexpr int STAGES_BEST = stages_with(PRIV_BASE + red_bytes(16));
    static constexpr int STAGES_MIN = STAGES_BEST < 4 ? STAGES_BEST : 4;
    static constexpr int RED_COLS = stages_with(PRIV_BASE + red_bytes(D)) >= STAGES_MIN ? D
                                    : (D > 64 && stages_with(PRIV_BASE + red_bytes(64)) >= STAGES_MIN) ? 64
                                    : (stages_with(PRIV_BASE + red_bytes(32)) >= STAGES_MIN) ? 32 : 16;
    static constexpr int PBYTES = PRIVATE ? NDESC * DESC_BYTES : NPBUF * ROWS * kPStride;        // region A
    static constexpr int OREDBYTES = PRIVATE ? red_bytes(RED_COLS)                               // region B
                                             : (TS > 1 ? kConsumerWarps * 16 * ROWS * 4 : 0);
    static constexpr int OFF_SMALL = PBYTES + OREDBYTES;          // 64 floats of row statistics (tile max / merged max, sum)
    static constexpr int OFF_W = OFF_SMALL + 2 * 32 * 4;          // 4 x [warps][32] floats
    static constexpr int OFF_MISC = OFF_W + 4 * kConsumerWarps * 32 * 4;
    static constexpr int OFF_BAR = OFF_MISC + 64;                 // full[8], empty[8], dfull[4], dempty[4], mfull[2], parked, go, done
    static constexpr int OFF_MAIL = OFF_BAR + 256;                // two split-merge requests
    static constexpr int OFF_PEER = OFF_MAIL + 128;               // gathering calls: the ranks' flag blocks (8 pointers)
    static constexpr int FIXED = OFF_PEER + 64;
    static constexpr int STAGES_RAW = (BUDGET - FIXED) / STAGE;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM = STAGES * STAGE + FIXED + 1024;
    static_assert(STAGES >= 2, "shared memory holds fewer than two stages");
};

// Largest index in [lo, hi) for which the monotone predicate holds (it holds at lo), found by a whole warp: every
// round probes 32 points at once, so a table of a few hundred entries takes two dependent loads instead of nine.
template <typename Pred>
__device__ __forceinline__ int warp_last_true(int lo, int hi, int lane, Pred holds) {
    while (hi - lo > 1) {
        const int step = (hi - lo + 31) / 32;
        const int idx = lo + (lane + 1) * step;
        const bool ok = idx < hi && holds(idx);
        const int k = __popc(__ballot_sync(0xffffffffu, ok));
        hi = min(hi, lo + (k + 1) * step);
        lo = lo + k * step;
    }
    return lo;
}

// CTA whose slice holds flat tile f: the largest c with start[c] <= f (CTAs with empty slices are skipped by construction)
__device__ __forceinline__ int slice_owner(const int32_t* start, int P, long long f) {
    int lo = 0, hi = P;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (start[mid] <= f) lo = mid; else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ int slices_in_use(const int32_t* start, int c_first, int c_last) {
    int n = 0;
    for (int c = c_first; c <= c_last; ++c) n += start[c] < start[c + 1] ? 1 : 0;
    return n;
}

// ordered-int encoding so that atomicMax on ints orders floats
__device__ __forceinline__ int f2ord(float f) {
    int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

// What the consumers need to know about one (unit, head) part; written by the producer warp.
struct PartDesc {
    int seq, row0, tile_lo, qs, q_len, kv_len, head, u, j, run, ntiles, cum_u, pad[4];
};
static_assert(sizeof(PartDesc) == 64, "descriptor header is 64 bytes");

// A part that covers only some of its unit's tiles leaves its partial result in this CTA's slot and hands the rest
// (publish, count, merge when it was the last one) to the merge warp through one of these.
struct MergeRequest {
    int kind;  // 1 = a part to publish, 2 = no further request from this CTA
    int row0, rows, qs, head, unit, ntiles, cum_u;
};
static_assert(sizeof(MergeRequest) == 32, "two requests fit the mail area");

struct Walk {
    int u, head, j, ntiles;
    __device__ __forceinline__ void locate(long long f, const int32_t* cum, int num_units, int Hkv) {
        int lo = 0, hi = num_units;  // cum[lo]*Hkv <= f < cum[hi]*Hkv
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if ((long long)cum[mid] * Hkv <= f) lo = mid; else hi = mid;
        }
        u = lo;
        ntiles = cum[u + 1] - cum[u];
        long long rem = f - (long long)cum[u] * Hkv;
        head = (int)(rem / ntiles);
        j = (int)(rem - (long long)head * ntiles);
    }
    // the same result from a nearby unit: a step or two instead of a search
    __device__ __forceinline__ void locate_near(long long f, int hint, const int32_t* cum, int num_units, int Hkv) {
        u = min(max(hint, 0), num_units - 1);
        while (u > 0 && (long long)cum[u] * Hkv > f) --u;
        while (u + 1 < num_units && (long long)cum[u + 1] * Hkv <= f) ++u;
        ntiles = cum[u + 1] - cum[u];
        long long rem = f - (long long)cum[u] * Hkv;
        head = (int)(rem / ntiles);
        j = (int)(rem - (long long)head * ntiles);
    }
    __device__ __forceinline__ void next_part(const int32_t* cum, int num_units, int Hkv) {
        j = 0;
        if (++head == Hkv) {
            head = 0;
            ++u;
            if (u < num_units) ntiles = cum[u + 1] - cum[u];
        }
    }
};

// ------------------------------------------------------------------------------------------ producer
template <int D, int NT, int FMT>
__device__ __forceinline__ void producer_loop(const CUtensorMap* kmap, const CUtensorMap* vmap, const TiledParams& p,
                                              uint8_t* stages, uint8_t* fixed, uint64_t* full, uint64_t* empty,
                                              volatile int* abort_word, long long f_begin, long long f_end, int num_units) {
    using C = Cfg<D, NT, FMT>;
    const int lane = threadIdx.x & 31;
    uint64_t* dfull = full + 16;
    uint64_t* dempty = full + 20;
    uint32_t part_idx = 0;
    (void)dfull; (void)dempty; (void)part_idx; (void)fixed;
    // Units of up to 16 rows hold all rows of their sequence, so its KV tiles are read once per step: they are marked
    // evict-first.  A sequence cut into several 32-row units reads its tiles once per unit and keeps the normal policy.
    const uint64_t stream_once = C::PRIVATE ? ptx::l2_policy_evict_first() : ptx::l2_policy_evict_normal();
    Walk w;
    // Order of the slice's parts.  When the slice ends inside a unit, that unfinished part goes first: both parts
    // that need a merge with a neighbouring CTA are then done early and their merges run behind the other parts.
    long long range_lo[2] = {f_begin, f_begin}, range_hi[2] = {f_end, f_begin};
    int range_hint[2] = {p.cta_unit[blockIdx.x], p.cta_unit[blockIdx.x]};
    if constexpr (C::PRIVATE) {
        w.locate_near(f_end - 1, p.cta_unit[blockIdx.x + 1], p.unit_cum, num_units, p.Hkv);
        const long long a_last = (long long)p.unit_cum[w.u] * p.Hkv + (long long)w.head * w.ntiles;
        if (a_last + w.ntiles > f_end && a_last > f_begin) {
            range_lo[0] = a_last; range_hi[0] = f_end; range_hint[0] = w.u;
            range_lo[1] = f_begin; range_hi[1] = a_last;
        }
    }
    uint32_t it = 0;
    // Consecutive parts are usually the KV heads of one unit: same sequence, same tiles, same pages.  What the last part
    // read from global memory is kept, so that a head switch costs the producer no dependent loads (while it waits for
    // them no tile is requested, and at HBM speed the ring never makes the lost time up again).
    int c_u = -1, c_seq = 0, c_tile_lo = 0, c_kv_len = 0, c_row0 = 0, c_qs = 0, c_qlen = 0, c_cum = 0;
    int c_pages = -1, c_pages_j = -1, c_pages_run = 0;
    for (int rg = 0; rg < 2; ++rg) {
    long long f = range_lo[rg];
    const long long f_stop = range_hi[rg];
    if (f < f_stop) w.locate_near(f, range_hint[rg], p.unit_cum, num_units, p.Hkv);
    while (f < f_stop && !*abort_word) {
        if (w.u != c_u) {
            c_u = w.u;
            c_seq = p.unit_seq[w.u];
            c_tile_lo = p.unit_tile_lo[w.u];
            c_row0 = p.unit_row0[w.u];
            c_cum = p.unit_cum[w.u];
            c_kv_len = p.kv_lens[c_seq];
            c_qs = p.qsl[c_seq];
            c_qlen = p.qsl[c_seq + 1] - c_qs;
            c_pages_j = -1;
        }
        const int seq = c_seq, tile_lo = c_tile_lo, kv_len = c_kv_len;
        const int run = (int)min((long long)(w.ntiles - w.j), f_stop - f);
        // page ids of the part's first tiles: requested before the descriptor is built so that both latencies overlap.
        // A batch of 32 ids covers 32 >> ppt_log tiles: lane l holds page (l mod pages-per-tile) of tile base + l / ppt.
        const int ppt_log = p.ppt_log, ppt = 1 << ppt_log, tiles_per_batch = 32 >> ppt_log;
        auto load_ids = [&](int base) -> int {
            const int tile = base + (lane >> ppt_log);
            const long long pidx = ((long long)(tile_lo + w.j + tile) << ppt_log) + (lane & (ppt - 1));
            return (tile < run && pidx < p.MB) ? p.bt[(long long)seq * p.MB + pidx] : -1;
        };
        if (c_pages_j != w.j || run > c_pages_run) {
            c_pages = load_ids(0);
            c_pages_j = w.j;
            c_pages_run = run;
        }
        const int page_first = c_pages;
        if constexpr (C::PRIVATE) {
            // descriptor + Q rows of this part, so that the consumers start it without touching global memory
            const uint32_t slot = part_idx % C::NDESC, use = part_idx / C::NDESC;
            if (use > 0) ptx::mbar_wait(&dempty[slot], (use & 1) ^ 1, abort_word);
            if (lane == 0 && !*abort_word) {
                PartDesc* d = (PartDesc*)(fixed + (size_t)slot * C::DESC_BYTES);
                const int row0 = c_row0, qs = c_qs, q_len = c_qlen;
                const int R = q_len * p.G, rows_here = min(C::ROWS, R - row0);
                d->seq = seq; d->row0 = row0; d->tile_lo = tile_lo; d->qs = qs; d->q_len = q_len; d->kv_len = kv_len;
                d->head = w.head; d->u = w.u; d->j = w.j; d->run = run; d->ntiles = w.ntiles; d->cum_u = c_cum;
                ptx::mbar_arrive_expect_tx(&dfull[slot], (uint32_t)(rows_here * D * 2));
                uint8_t* qdst = (uint8_t*)d + 64;
                for (int r = row0; r < row0 + rows_here;) {
                    const int i = r / p.G, hh = r - i * p.G;
                    const int n = min(row0 + rows_here - r, p.G - hh);  // rows of token i inside this unit
                    const uint16_t* src = (const uint16_t*)p.q + ((long long)(qs + i) * p.Hq + w.head * p.G + hh) * D;
                    ptx::bulk_load(qdst + (size_t)(r - row0) * C::QSTRIDE, src, (uint32_t)(n * D * 2), &dfull[slot]);
                    r += n;
                }
            }
            __syncwarp();
            ++part_idx;
        }
        if (ppt_log == 0) {  // one page per tile: the common case, kept as short as it can be
            for (int base = 0; base < run; base += 32) {
                const int idx = tile_lo + w.j + base + lane;
                int page = page_first;
                if (base > 0) {
                    page = -1;
                    if (base + lane < run && idx < p.MB) page = p.bt[(long long)seq * p.MB + idx];
                }
                const int cnt = min(32, run - base);
                for (int i = 0; i < cnt; ++i) {
                    int pg = __shfl_sync(0xffffffffu, page, i);
                    const uint32_t stage = it % C::STAGES, use = it / C::STAGES;
                    if (use > 0) ptx::mbar_wait(&empty[stage], (use & 1) ^ 1, abort_word);
                    if (lane == 0 && !*abort_word) {
                        const bool bad = pg < 0 || pg >= p.num_blocks;
                        if (bad && (long long)(tile_lo + w.j + base + i) * kTile < kv_len) flag_error(p.status, EMLX_DEV_BAD_PAGE);
                        uint8_t* st = stages + (size_t)stage * C::STAGE;
                        ptx::mbar_arrive_expect_tx(&full[stage], C::STAGE);
                        if constexpr (FMT == 0) {
                            // a page id outside the pool gives out-of-range coordinates: the tile is zero-filled
                            const int tok0 = bad ? -kTile : pg * kTile;
    #pragma unroll
                            for (int h = 0; h < D / 64; ++h) {
                                ptx::tma_load_3d(st + h * (kTile * 128), kmap, &full[stage], 64 * h, w.head, tok0, stream_once);
                                ptx::tma_load_3d(st + C::KBYTES + h * (kTile * 128), vmap, &full[stage], 64 * h, w.head, tok0, stream_once);
                            }
                        } else {
                            const long long pgc = bad ? 0 : pg;  // keep every address inside the pool; such tiles are masked
                            ptx::tma_load_3d(st, kmap, &full[stage], 0, w.head, (int)(pgc * kTile), stream_once);
                            ptx::tma_load_2d(st + C::KBYTES, vmap, &full[stage], 0, (int)((pgc * p.Hkv + w.head) * D), stream_once);
                            const long long sb = (pgc * p.Hkv + w.head) * (long long)(kTile * C::GROUPS);
                            uint8_t* sbs = st + C::KBYTES + C::VBYTES;
                            ptx::bulk_load(sbs + 0 * C::SB1, p.k_scale + sb, C::SB1, &full[stage], stream_once);
                            ptx::bulk_load(sbs + 1 * C::SB1, p.k_bias + sb, C::SB1, &full[stage], stream_once);
                            ptx::bulk_load(sbs + 2 * C::SB1, p.v_scale + sb, C::SB1, &full[stage], stream_once);
                            ptx::bulk_load(sbs + 3 * C::SB1, p.v_bias + sb, C::SB1, &full[stage], stream_once);
                        }
                    }
                    __syncwarp();
                    ++it;
                }
            }
        } else {
            for (int base = 0; base < run; base += tiles_per_batch) {
                const int page = base == 0 ? page_first : load_ids(base);
                const int cnt = min(tiles_per_batch, run - base);
                for (int i = 0; i < cnt; ++i) {
                    const uint32_t stage = it % C::STAGES, use = it / C::STAGES;
                    if (use > 0) ptx::mbar_wait(&empty[stage], (use & 1) ^ 1, abort_word);
                    const bool go = lane == 0 && !*abort_word;
                    uint8_t* st = stages + (size_t)stage * C::STAGE;
                    const long long tile_tok = (long long)(tile_lo + w.j + base + i) * kTile;
                    if (go) ptx::mbar_arrive_expect_tx(&full[stage], C::STAGE);
                    if constexpr (FMT == 0) {
                        for (int sub = 0; sub < ppt; ++sub) {
                            const int pg = __shfl_sync(0xffffffffu, page, (i << ppt_log) + sub);
                            if (go) {
                                const bool bad = pg < 0 || pg >= p.num_blocks;
                                if (bad && tile_tok + (long long)sub * p.bs < kv_len) flag_error(p.status, EMLX_DEV_BAD_PAGE);
                                // a page id outside the pool gives out-of-range coordinates: its rows are zero-filled
                                const int tok0 = bad ? -p.bs : pg * p.bs;
                                uint8_t* dst = st + (size_t)sub * p.bs * 128;
    #pragma unroll
                                for (int h = 0; h < D / 64; ++h) {
                                    ptx::tma_load_3d(dst + h * (kTile * 128), kmap, &full[stage], 64 * h, w.head, tok0, stream_once);
                                    ptx::tma_load_3d(dst + C::KBYTES + h * (kTile * 128), vmap, &full[stage], 64 * h, w.head, tok0, stream_once);
                                }
                            }
                        }
                    } else {
                        const int pg = __shfl_sync(0xffffffffu, page, i);
                        if (go) {
                            const bool bad = pg < 0 || pg >= p.num_blocks;
                            if (bad && tile_tok < kv_len) flag_error(p.status, EMLX_DEV_BAD_PAGE);
                            const long long pgc = bad ? 0 : pg;  // keep every address inside the pool; such tiles are masked
                            ptx::tma_load_3d(st, kmap, &full[stage], 0, w.head, (int)(pgc * kTile), stream_once);
                            ptx::tma_load_2d(st + C::KBYTES, vmap, &full[stage], 0, (int)((pgc * p.Hkv + w.head) * D), stream_once);
                            const long long sb = (pgc * p.Hkv + w.head) * (long long)(kTile * C::GROUPS);
                            uint8_t* sbs = st + C::KBYTES + C::VBYTES;
                            ptx::bulk_load(sbs + 0 * C::SB1, p.k_scale + sb, C::SB1, &full[stage], stream_once);
                            ptx::bulk_load(sbs + 1 * C::SB1, p.k_bias + sb, C::SB1, &full[stage], stream_once);
                            ptx::bulk_load(sbs + 2 * C::SB1, p.v_scale + sb, C::SB1, &full[stage], stream_once);
                            ptx::bulk_load(sbs + 3 * C::SB1, p.v_bias + sb, C::SB1, &full[stage], stream_once);
                        }
                    }
                    __syncwarp();
                    ++it;
                }
            }
        }
        f += run;
        w.next_part(p.unit_cum, num_units, p.Hkv);
    }
    }
}

// ------------------------------------------------------------------------------------------ consumers
template <bool BF16> __device__ __forceinline__ uint16_t to_bits16(float v) {
    if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}
// two bf16 -> two fp16, round to nearest, clamped to the fp16 range: affine pools are multiplied on the fp16 tensor
// path (their codes are fp16 subnormals), so bf16 queries are converted once per part
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    const float lo = fminf(fmaxf(__uint_as_float(v << 16), -65504.f), 65504.f);
    const float hi = fminf(fmaxf(__uint_as_float(v & 0xffff0000u), -65504.f), 65504.f);
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float quad_column_max(float v) {  // over the 8 lanes that share lane%4
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
__device__ __forceinline__ float quad_column_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v + __shfl_xor_sync(0xffffffffu, v, 16);
}
__device__ __forceinline__ void consumer_sync() { ptx::named_barrier(1, kConsumerThreads); }

// 8 nibbles of x -> four half2 registers holding (n0,n2) (n4,n6) (n1,n3) (n5,n7) as fp16 bit patterns 0x000c
__device__ __forceinline__ void nibbles_to_h2(uint32_t x, uint32_t (&h)[4]) {
    const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;
    h[0] = ptx::prmt(lo, 0u, 0x4140u);
    h[1] = ptx::prmt(lo, 0u, 0x4342u);
    h[2] = ptx::prmt(hi, 0u, 0x4140u);
    h[3] = ptx::prmt(hi, 0u, 0x4342u);
}

// Softmax weights of an fp16 pool go to the tensor cores as fp16.  A weight below 2^-25 of the row's reference
// maximum would round to zero there, and in a row of 10^5 keys with one dominant key the thousands of such keys hold
// a visible share of the output.  The weights are therefore computed as 2^(s - m + kShift): the row sum and the
// accumulator carry the same factor, which cancels in O / l and in every merge of partial results (all parts use the
// same shift).  The largest weight is then 2^kShift = 256, far inside the fp16 range.  bf16 has fp32's exponent
// range and needs no shift.
template <int FMT, bool BF16> __device__ __forceinline__ constexpr float weight_shift() {
    return (FMT == 0 && !BF16) ? 8.0f : 0.0f;
}

// 8 nibbles e0..e7 of x -> four half2 registers (e0,e4) (e1,e5)*16 (e2,e6) (e3,e7)*16 as fp16 subnormal bit patterns:
// a nibble in the low four bits of a 16-bit half is the code itself, one in bits 4-7 is the code times 16 (still
// inside the ten mantissa bits, so still linear).  One shift and four masks; the factor 16 is taken out of the other
// operand (queries, or softmax weights) once per part or per tile instead of once per code.
__device__ __forceinline__ void unpack_nibbles(uint32_t x, uint32_t (&h)[4]) {
    const uint32_t y = x >> 8;
    h[0] = x & 0x000F000Fu;
    h[1] = x & 0x00F000F0u;
    h[2] = y & 0x000F000Fu;
    h[3] = y & 0x00F000F0u;
}

constexpr float kTwo24 = 16777216.0f;  // codes enter the MMA as fp16 subnormals c * 2^-24
// The value-side weights p * scale become fp16 after a multiplication by 2^8: in a long row with one dominant key the
// others have p * scale below the fp16 subnormal step (6e-8) and would be rounded away, thousands of them together
// carrying a visible share of the output.  Scales above 255.9 saturate at the largest finite fp16.
constexpr float kWeightUp = 256.0f, kHalfMax = 65504.0f, kValueDown = kTwo24 / kWeightUp;
__device__ __forceinline__ float weight_scale(float v_scale) { return fminf(v_scale * kWeightUp, kHalfMax); }

template <int D, int NT, int FMT, bool BF16, bool PEER>
__device__ __forceinline__ void consumer_loop(const TiledParams& p, uint8_t* stages, uint8_t* fixed, uint64_t* full,
                                              uint64_t* empty, volatile int* abort_word, long long f_begin,
                                              long long f_end, int num_units, long long total_flat, long long active) {
    using C = Cfg<D, NT, FMT>;
    constexpr int KS = D / 16, ROWS = C::ROWS, GROUPS = C::GROUPS;
    constexpr int NG = FMT == 0 ? 1 : GROUPS;  // accumulator sets of phase 1
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int ds = warp % C::DSL, ts = warp / C::DSL;
    const int jd = FMT == 0 ? 0 : (16 * ds) / 64;  // scale group of this warp's slice of D

    uint8_t* Ps = fixed;
    float* ored = (float*)(fixed + C::PBYTES);
    int* tmax = (int*)(fixed + C::OFF_SMALL);
    float* wl = (float*)(fixed + C::OFF_W);
    float* wb = wl + kConsumerWarps * 32;  // [2][warps][32]
    int* misc = (int*)(fixed + C::OFF_MISC);
    const int ORD_NEG_INF = f2ord(-INFINITY);
    bool peer_seen = false;

    Walk w;
    w.locate(f_begin, p.unit_cum, num_units, p.Hkv);
    long long f = f_begin;
    uint32_t it = 0;
    const uint32_t ps_base = ptx::smem_u32(Ps);

    while (f < f_end) {
        // ------------------------------------------------------------------ begin a (unit, head) part
        const int seq = p.unit_seq[w.u], row0 = p.unit_row0[w.u], tile_lo = p.unit_tile_lo[w.u];
        const int qs = p.qsl[seq], q_len = p.qsl[seq + 1] - qs, kv_len = p.kv_lens[seq];
        const int R = q_len * p.G, ctx = kv_len - q_len, head = w.head;
        const int run = (int)min((long long)(w.ntiles - w.j), f_end - f);
        const int rows_here = min(ROWS, R - row0);

        int row_hi[NT][2], row_lo[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int rr = min(row0 + 8 * nt + 2 * t + e, R - 1);  // padding rows mirror the last real row
                const int i = rr / p.G;
                int hi = min(kv_len, ctx + i + 1);
                int lo = p.window > 0 ? max(0, min(kv_len - 1, ctx + i) - p.window + 1) : 0;
                if (hi <= 0) { hi = 0; lo = 0; }
                row_hi[nt][e] = hi;
                row_lo[nt][e] = lo;
            }
        const int i_first = row0 / p.G, i_last = (row0 + rows_here - 1) / p.G;
        const int hi_min = min(kv_len, ctx + i_first + 1);
        const int lo_max = p.window > 0 ? max(0, min(kv_len - 1, ctx + i_last) - p.window + 1) : 0;

        // Q^T fragments (B operand): rows on N, head_dim on K in the order the K tile is read
        uint32_t qf[KS][NT][2];
        float qsum[NG][NT][2];
        {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int r = row0 + 8 * nt + g;
                const bool ok = r < R;
                const int i = ok ? r / p.G : 0, hh = ok ? r - i * p.G : 0;
                const uint16_t* qrow = (const uint16_t*)p.q + ((long long)(qs + i) * p.Hq + head * p.G + hh) * D;
                if constexpr (FMT == 0) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        qf[ks][nt][0] = ok ? *(const uint32_t*)(qrow + 16 * ks + 2 * t) : 0u;
                        qf[ks][nt][1] = ok ? *(const uint32_t*)(qrow + 16 * ks + 2 * t + 8) : 0u;
                    }
                } else if constexpr (FMT == 8) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        const int d0 = 64 * (ks >> 2) + 16 * t + 4 * (ks & 3);
                        const uint2 v = ok ? *(const uint2*)(qrow + d0) : make_uint2(0u, 0u);
                        qf[ks][nt][0] = v.x;
                        qf[ks][nt][1] = v.y;
                    }
                } else {
#pragma unroll
                    for (int jx = 0; jx < KS / 2; ++jx) {  // (group j, word x) -> k-steps 2*jx, 2*jx+1
                        const int db = 64 * (jx >> 1) + 16 * t + 8 * (jx & 1);
                        const uint4 v = ok ? *(const uint4*)(qrow + db) : make_uint4(0u, 0u, 0u, 0u);
                        qf[2 * jx][nt][0] = ptx::prmt(v.x, v.y, 0x5410u);      // (q0, q2)
                        qf[2 * jx][nt][1] = ptx::prmt(v.z, v.w, 0x5410u);      // (q4, q6)
                        qf[2 * jx + 1][nt][0] = ptx::prmt(v.x, v.y, 0x7632u);  // (q1, q3)
                        qf[2 * jx + 1][nt][1] = ptx::prmt(v.z, v.w, 0x7632u);  // (q5, q7)
                    }
                }
            }
            if constexpr (FMT != 0 && BF16) {
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        qf[ks][nt][0] = bf16x2_to_f16x2(qf[ks][nt][0]);
                        qf[ks][nt][1] = bf16x2_to_f16x2(qf[ks][nt][1]);
                    }
            }
            if constexpr (FMT != 0) {
                // column sums of Q per scale group through an all-ones A operand: c[e] = sum_d q[row 2t+e][d]
                const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
#pragma unroll
                for (int j = 0; j < NG; ++j)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int s = 0; s < 4; ++s) ptx::mma_16816<false>(c, ones, qf[4 * j + s][nt]);
                        qsum[j][nt][0] = c[0];
                        qsum[j][nt][1] = c[1];
                    }
            }
        }

        float m[NT][2], l[NT][2], o[NT][4], bsum[NG][NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            m[nt][0] = m[nt][1] = -INFINITY;
            l[nt][0] = l[nt][1] = 0.f;
            o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
#pragma unroll
            for (int j = 0; j < NG; ++j) bsum[j][nt][0] = bsum[j][nt][1] = 0.f;
        }

        // ------------------------------------------------------------------ tiles of this part
        for (int jj = 0; jj < run; ++jj, ++it) {
            const uint32_t stage = it % C::STAGES, buf = it & 1;
            uint8_t* st = stages + (size_t)stage * C::STAGE;
            const uint32_t ks_base = ptx::smem_u32(st), vs_base = ks_base + C::KBYTES;
            const __half* sbs = (const __half*)(st + C::KBYTES + C::VBYTES);  // [4][128][GROUPS]
            const int t0 = (tile_lo + w.j + jj) * kTile;
            const bool interior = (t0 + kTile <= hi_min) && (t0 >= lo_max);
            ptx::mbar_wait(&full[stage], (it / C::STAGES) & 1, abort_word);

            // ---- phase 1: S^T = K . Q^T for this warp's 16 tokens
            float s[NT][4];
            const int tokA = 16 * warp + g, tokB = tokA + 8;
            if constexpr (FMT == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * (kTile * 128) + (16 * warp + (lane & 15)) * 128 +
                                                    ((ks & 3) * 2 + (lane >> 4)) * 16);
                    uint32_t a[4];
                    ptx::ldmatrix_x4(a, ks_base + ptx::swz<3>(off));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<BF16>(s[nt], a, qf[ks][nt]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) s[nt][c] *= p.scale_log2e;
            } else {
                float acc[NG][NT][4];
#pragma unroll
                for (int j = 0; j < NG; ++j)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) acc[j][nt][0] = acc[j][nt][1] = acc[j][nt][2] = acc[j][nt][3] = 0.f;
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    if constexpr (FMT == 8) {
                        const uint32_t offA = (uint32_t)(tokA * C::KROW + 64 * j + 16 * t);
                        const uint32_t offB = offA + 8 * C::KROW;
                        const uint4 xa = *(const uint4*)(st + ptx::swz<C::KSW>(offA));
                        const uint4 xb = *(const uint4*)(st + ptx::swz<C::KSW>(offB));
                        const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w}, wbv[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int sidx = 0; sidx < 4; ++sidx) {
                            uint32_t a[4];
                            a[0] = ptx::prmt(wa[sidx], 0u, 0x4140u);
                            a[1] = ptx::prmt(wbv[sidx], 0u, 0x4140u);
                            a[2] = ptx::prmt(wa[sidx], 0u, 0x4342u);
                            a[3] = ptx::prmt(wbv[sidx], 0u, 0x4342u);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) ptx::mma_16816<false>(acc[j][nt], a, qf[4 * j + sidx][nt]);
                        }
                    } else {
                        const uint32_t offA = (uint32_t)(tokA * C::KROW + 32 * j + 8 * t);
                        const uint32_t offB = offA + 8 * C::KROW;
                        const uint2 xa = *(const uint2*)(st + ptx::swz<C::KSW>(offA));
                        const uint2 xb = *(const uint2*)(st + ptx::swz<C::KSW>(offB));
                        const uint32_t wa[2] = {xa.x, xa.y}, wbv[2] = {xb.x, xb.y};
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            uint32_t ha[4], hb[4];
                            nibbles_to_h2(wa[x], ha);
                            nibbles_to_h2(wbv[x], hb);
#pragma unroll
                            for (int y = 0; y < 2; ++y) {
                                const uint32_t a[4] = {ha[2 * y], hb[2 * y], ha[2 * y + 1], hb[2 * y + 1]};
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt)
                                    ptx::mma_16816<false>(acc[j][nt], a, qf[4 * j + 2 * x + y][nt]);
                            }
                        }
                    }
                }
                // S = sum_j scale_j[tok] * (2^24 * acc_j) + bias_j[tok] * qsum_j
                float ksA[NG], ksB[NG], kbA[NG], kbB[NG];
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    ksA[j] = __half2float(sbs[0 * kTile * GROUPS + tokA * GROUPS + j]) * kTwo24;
                    ksB[j] = __half2float(sbs[0 * kTile * GROUPS + tokB * GROUPS + j]) * kTwo24;
                    kbA[j] = __half2float(sbs[1 * kTile * GROUPS + tokA * GROUPS + j]);
                    kbB[j] = __half2float(sbs[1 * kTile * GROUPS + tokB * GROUPS + j]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float v = 0.f;
#pragma unroll
                        for (int j = 0; j < NG; ++j)
                            v += (c < 2 ? ksA[j] : ksB[j]) * acc[j][nt][c] + (c < 2 ? kbA[j] : kbB[j]) * qsum[j][nt][c & 1];
                        s[nt][c] = v * p.scale_log2e;
                    }
            }
            if (!interior) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int tok = t0 + (c < 2 ? tokA : tokB);
                        if (tok < row_lo[nt][c & 1] || tok >= row_hi[nt][c & 1]) s[nt][c] = -INFINITY;
                    }
            }
            // tile maximum per row: own 16 tokens, then all warps through shared atomics
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float mx = quad_column_max(fmaxf(s[nt][e], s[nt][2 + e]));
                    if (g == 0) atomicMax(&tmax[buf * 32 + 8 * nt + 2 * t + e], f2ord(mx));
                }
            if constexpr (FMT == 0) {
                // rows of V past the sequence end are stale memory: clear them so that 0 * garbage cannot be NaN
                if (t0 + kTile > kv_len) {
                    const int first = max(0, kv_len - t0);
                    for (int c = lane; c < 16 * (D / 8); c += 32) {
                        const int tok = 16 * warp + c / (D / 8), ch = c % (D / 8);
                        if (tok >= first)
                            *(uint4*)(st + C::KBYTES + (ch >> 3) * (kTile * 128) + tok * 128 + (ch & 7) * 16) =
                                make_uint4(0u, 0u, 0u, 0u);
                    }
                    ptx::fence_proxy_async();
                }
            }
            consumer_sync();
            if (warp == 0) tmax[(buf ^ 1) * 32 + lane] = ORD_NEG_INF;

            float corr[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float m_new = fmaxf(m[nt][e], ord2f(tmax[buf * 32 + 8 * nt + 2 * t + e]));
                    const float m_safe = m_new == -INFINITY ? 0.f : m_new;
                    corr[nt][e] = exp2f(m[nt][e] - m_safe);
                    m[nt][e] = m_new;
                    constexpr float kShift = weight_shift<FMT, BF16>();
                    const float pA = exp2f(s[nt][e] - m_safe + kShift), pB = exp2f(s[nt][2 + e] - m_safe + kShift);
                    l[nt][e] = l[nt][e] * corr[nt][e] + pA + pB;
                    s[nt][e] = pA;
                    s[nt][2 + e] = pB;
                }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[nt][c] *= corr[nt][c & 1];

            // P^T to shared memory, rows x tokens
            if constexpr (FMT == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int row = 8 * nt + 2 * t + (c & 1), tok = c < 2 ? tokA : tokB;
                        *(uint16_t*)(Ps + row * kPStride + tok * 2) = to_bits16<BF16>(s[nt][c]);
                    }
            } else {
                float vsA[NG], vsB[NG], vbA[NG], vbB[NG];
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    vsA[j] = weight_scale(__half2float(sbs[2 * kTile * GROUPS + tokA * GROUPS + j]));
                    vsB[j] = weight_scale(__half2float(sbs[2 * kTile * GROUPS + tokB * GROUPS + j]));
                    vbA[j] = __half2float(sbs[3 * kTile * GROUPS + tokA * GROUPS + j]);
                    vbB[j] = __half2float(sbs[3 * kTile * GROUPS + tokB * GROUPS + j]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int e = c & 1, row = 8 * nt + 2 * t + e, tok = c < 2 ? tokA : tokB;
                        const float pv = s[nt][c];
                        // 4-bit values are read eight tokens per word as (0,2)(4,6)(1,3)(5,7): store P in that order
                        const int pos = FMT == 8 ? tok : (tok & ~7) + ((tok & 1) ? 4 + ((tok & 7) >> 1) : ((tok & 7) >> 1));
#pragma unroll
                        for (int j = 0; j < NG; ++j) {
                            // stale scale/bias bytes of unwritten slots may be NaN: select, do not multiply by zero
                            const float sc = pv > 0.f ? pv * (c < 2 ? vsA[j] : vsB[j]) : 0.f;
                            const float bi = pv > 0.f ? pv * (c < 2 ? vbA[j] : vbB[j]) : 0.f;
                            *(uint16_t*)(Ps + (j * ROWS + row) * kPStride + pos * 2) = __half_as_ushort(__float2half_rn(sc));
                            if (c < 2) bsum[j][nt][e] = bsum[j][nt][e] * corr[nt][e] + bi;
                            else bsum[j][nt][e] += bi;
                        }
                    }
            }
            consumer_sync();

            // ---- phase 2: O^T[16 x rows] += V^T[16 x tokens] . P^T[tokens x rows] for this warp's slice of D
            if constexpr (FMT == 0) {
                constexpr int STEPS = kTile / C::TS / 16;
#pragma unroll
                for (int kk = 0; kk < STEPS; ++kk) {
                    const int tok0 = ts * (kTile / C::TS) + 16 * kk;
                    const int tok = tok0 + (lane & 7) + 8 * (lane >> 4);
                    const int ch = 2 * ds + ((lane >> 3) & 1);  // 16-byte chunk of the row (8 halves of D)
                    const uint32_t off = (uint32_t)((ch >> 3) * (kTile * 128) + tok * 128 + (ch & 7) * 16);
                    uint32_t a[4];
                    ptx::ldmatrix_x4_trans(a, vs_base + ptx::swz<3>(off));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        uint32_t b[2];
                        ptx::ldmatrix_x2(b, ps_base + (8 * nt + (lane & 7)) * kPStride + (tok0 + 8 * ((lane >> 3) & 1)) * 2);
                        ptx::mma_16816<BF16>(o[nt], a, b);
                    }
                }
            } else {
                const int dA = 16 * ds + g, dB = dA + 8;
#pragma unroll
                for (int Jx = 0; Jx < (kTile / 64) / C::TS; ++Jx) {
                    const int J = C::TS > 1 ? ts : Jx;  // block of 64 tokens
                    if constexpr (FMT == 8) {
                        const uint4 xa = *(const uint4*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)(dA * C::VROW + 64 * J + 16 * t)));
                        const uint4 xb = *(const uint4*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)(dB * C::VROW + 64 * J + 16 * t)));
                        const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w}, wbv[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int sidx = 0; sidx < 4; ++sidx) {
                            uint32_t a[4];
                            a[0] = ptx::prmt(wa[sidx], 0u, 0x4140u);
                            a[1] = ptx::prmt(wbv[sidx], 0u, 0x4140u);
                            a[2] = ptx::prmt(wa[sidx], 0u, 0x4342u);
                            a[3] = ptx::prmt(wbv[sidx], 0u, 0x4342u);
                            const int tok0 = 64 * J + 16 * t + 4 * sidx;
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const uint2 bv = *(const uint2*)(Ps + (jd * ROWS + 8 * nt + g) * kPStride + tok0 * 2);
                                const uint32_t b[2] = {bv.x, bv.y};
                                ptx::mma_16816<false>(o[nt], a, b);
                            }
                        }
                    } else {
                        const uint2 xa = *(const uint2*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)(dA * C::VROW + 32 * J + 8 * t)));
                        const uint2 xb = *(const uint2*)(st + C::KBYTES + ptx::swz<C::VSW>((uint32_t)(dB * C::VROW + 32 * J + 8 * t)));
                        const uint32_t wa[2] = {xa.x, xa.y}, wbv[2] = {xb.x, xb.y};
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            uint32_t ha[4], hb[4];
                            nibbles_to_h2(wa[x], ha);
                            nibbles_to_h2(wbv[x], hb);
#pragma unroll
                            for (int y = 0; y < 2; ++y) {
                                const uint32_t a[4] = {ha[2 * y], hb[2 * y], ha[2 * y + 1], hb[2 * y + 1]};
                                const int pos0 = 64 * J + 16 * t + 8 * x + 4 * y;
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) {
                                    const uint2 bv = *(const uint2*)(Ps + (jd * ROWS + 8 * nt + g) * kPStride + pos0 * 2);
                                    const uint32_t b[2] = {bv.x, bv.y};
                                    ptx::mma_16816<false>(o[nt], a, b);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[stage]);
        }

        // ------------------------------------------------------------------ end of the part
        // row sums (and the values' bias terms) across this warp's tokens, then across warps in a fixed order
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float v = quad_column_sum(l[nt][e]);
                if (g == 0) wl[warp * 32 + 8 * nt + 2 * t + e] = v;
                if constexpr (FMT != 0) {
#pragma unroll
                    for (int j = 0; j < NG; ++j) {
                        const float bv = quad_column_sum(bsum[j][nt][e]);
                        if (g == 0) wb[(j * kConsumerWarps + warp) * 32 + 8 * nt + 2 * t + e] = bv;
                    }
                }
            }
        if constexpr (C::TS > 1) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) ored[(warp * NT * 4 + nt * 4 + c) * 32 + lane] = o[nt][c];
        }
        consumer_sync();
        float lsum[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = 0.f, bv = 0.f;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) {
                    v += wl[ww * 32 + 8 * nt + 2 * t + e];
                    if constexpr (FMT != 0) bv += wb[(jd * kConsumerWarps + ww) * 32 + 8 * nt + 2 * t + e];
                }
                lsum[nt][e] = v;
                if constexpr (FMT != 0) {
                    o[nt][e] = o[nt][e] * kValueDown + bv;
                    o[nt][2 + e] = o[nt][2 + e] * kValueDown + bv;
                }
            }
        if constexpr (C::TS > 1) {
            if (ts == 0) {
#pragma unroll
                for (int k = 1; k < C::TS; ++k)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            float other = ored[((warp + k * C::DSL) * NT * 4 + nt * 4 + c) * 32 + lane];
                            if constexpr (FMT != 0) other *= kValueDown;
                            o[nt][c] += other;
                        }
            }
        }

        const long long a_flat = (long long)p.unit_cum[w.u] * p.Hkv + (long long)head * w.ntiles;
        const long long b_flat = a_flat + w.ntiles;
        const bool complete = (w.j == 0) && (run == w.ntiles);
        const uint16_t* qbase = (const uint16_t*)p.q;
        (void)qbase;
        if (complete) {
            // normalise, stage as [row][D] in the P buffer, store rows with 16-byte accesses
            if (ts == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int e = c & 1, row = 8 * nt + 2 * t + e, d = 16 * ds + g + 8 * (c >> 1);
                        const float inv = lsum[nt][e] > 0.f ? 1.0f / lsum[nt][e] : 0.f;
                        *(uint16_t*)(Ps + row * kPStride + d * 2) = to_bits16<BF16>(o[nt][c] * inv);
                    }
            }
            consumer_sync();
            constexpr int CH = D / 8;
            for (int idx = tid; idx < ROWS * CH; idx += kConsumerThreads) {
                const int row = idx / CH, ch = idx - row * CH, r = row0 + row;
                if (r < R) {
                    const int i = r / p.G, hh = r - i * p.G;
                    store_out(p, out_offset<D>(p, qs + i, head * p.G + hh) + ch * 8, *(const uint4*)(Ps + row * kPStride + ch * 16));
                }
            }
            if constexpr (PEER) {
                consumer_sync();
                peer_ready(p, peer_seen);
                peer_copy_rows<D>((uint16_t*)p.out, p.peer, p.out_Hq, p.out_head0, p.G, qs, head, row0, min(row0 + ROWS, R),
                                  tid, kConsumerThreads);
            }
        } else {
            // un-normalised partial into this CTA's slot; the CTA that delivers the last one merges
            const long long P = active;  // CTAs that hold a slice
            const int which = (max(a_flat, f_begin) != f_begin) ? 1 : 0;
            float* slot = p.slots + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;
            if (ts == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int row = 8 * nt + 2 * t + (c & 1), d = 16 * ds + g + 8 * (c >> 1);
                        slot[row * D + d] = o[nt][c];
                    }
            }
            if (warp == 0 && g == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        slot[ROWS * D + 8 * nt + 2 * t + e] = m[nt][e];
                        slot[ROWS * D + ROWS + 8 * nt + 2 * t + e] = lsum[nt][e];
                    }
            }
            __threadfence();
            consumer_sync();
            const int c_first = slice_owner(p.cta_start, (int)P, a_flat), c_last = slice_owner(p.cta_start, (int)P, b_flat - 1);
            const int nparts = slices_in_use(p.cta_start, c_first, c_last);
            int* counter = p.counters + (size_t)w.u * p.Hkv + head;
            if (tid == 0) misc[1] = atomicAdd(counter, 1);
            consumer_sync();
            if (misc[1] == nparts - 1) {
                __threadfence();
                for (int idx = tid; idx < ROWS * D; idx += kConsumerThreads) {
                    const int row = idx / D, d = idx - row * D, r = row0 + row;
                    if (r >= R) continue;
                    float M = -INFINITY;
                    for (int c = c_first; c <= c_last; ++c) {
                        const long long cb = p.cta_start[c];
                        if (cb >= p.cta_start[c + 1]) continue;
                        const float* sl = p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats;
                        if (__ldcg(sl + ROWS * D + ROWS + row) > 0.f) M = fmaxf(M, __ldcg(sl + ROWS * D + row));
                    }
                    float acc = 0.f, den = 0.f;
                    for (int c = c_first; c <= c_last; ++c) {
                        const long long cb = p.cta_start[c];
                        if (cb >= p.cta_start[c + 1]) continue;
                        const float* sl = p.slots + ((size_t)c * 2 + (max(a_flat, cb) != cb ? 1 : 0)) * kSlotFloats;
                        const float lp = __ldcg(sl + ROWS * D + ROWS + row);
                        if (lp > 0.f) {
                            const float wgt = exp2f(__ldcg(sl + ROWS * D + row) - M);
                            acc += wgt * __ldcg(sl + row * D + d);
                            den += wgt * lp;
                        }
                    }
                    const int i = r / p.G, hh = r - i * p.G;
                    store_out(p, out_offset<D>(p, qs + i, head * p.G + hh) + d, to_bits16<BF16>(den > 0.f ? acc / den : 0.f));
                }
                if (tid == 0) *counter = 0;  // ready for the next launch
                if constexpr (PEER) {  // uniform over the consumer warps (the ticket is shared)
                    consumer_sync();
                    peer_ready(p, peer_seen);
                    peer_copy_rows<D>((uint16_t*)p.out, p.peer, p.out_Hq, p.out_head0, p.G, qs, head, row0, min(row0 + ROWS, R),
                                      tid, kConsumerThreads);
                }
            }
        }
        consumer_sync();  // the P buffer and the reduction scratch are reused by the next part
        f += run;
        w.next_part(p.unit_cum, num_units, p.Hkv);
    }
}

}  // namespace emlx

#include "attn_private.cuh"

namespace emlx {

// ------------------------------------------------------------------------------------------ kernel
template <int D, int NT, int FMT, bool BF16, bool PEER, bool HELP>
// 9 warps share four 16K-register sub-partitions: three warps on one of them caps a thread at 168 registers
__global__ void __launch_bounds__(kThreads, Cfg<D, NT, FMT>::CTAS_PER_SM)
attn_tiled_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const TiledParams p) {
    using C = Cfg<D, NT, FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* fixed = smem + (size_t)C::STAGES * C::STAGE;
    uint64_t* full = (uint64_t*)(fixed + C::OFF_BAR);
    uint64_t* empty = full + 8;
    uint64_t* dfull = full + 16;
    uint64_t* dempty = full + 20;
    int* tmax = (int*)(fixed + C::OFF_SMALL);
    volatile int* abort_word = (volatile int*)(fixed + C::OFF_MISC);  // misc[0]

    if (threadIdx.x == 0) {
#ifdef EMLX_TRACE
        if (p.trace) {
            long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            p.trace[4 * blockIdx.x + 0] = now;
        }
#endif
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], kConsumerWarps);
        }
        for (int s = 0; s < C::NDESC; ++s) {
            ptx::mbar_init(&dfull[s], 1);
            ptx::mbar_init(&dempty[s], kConsumerWarps);
        }
        for (int s = 0; s < 2; ++s) ptx::mbar_init(&full[24 + s], kConsumerWarps);
        ptx::mbar_init(&full[26], kConsumerWarps);  // consumer warps that have parked
        ptx::mbar_init(&full[27], 1);               // a job (or the leave to go) from the merge warp
        ptx::mbar_init(&full[28], kConsumerWarps);  // warps that have finished the job
        ((int*)(fixed + C::OFF_MISC))[kMiscHelpExit] = 0;
        *abort_word = 0;
        ((int*)(fixed + C::OFF_MISC))[kMiscExit] = 0;  // warps of this CTA that have finished (gathering calls)
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&kmap);
        ptx::prefetch_tensormap(&vmap);
    }
    if (threadIdx.x < 64) tmax[threadIdx.x] = f2ord(-INFINITY);
    __syncthreads();
    // everything above is independent of earlier kernels; the plan, the pool and the queries are not
    grid_dep_wait();
    grid_dep_launch();
#ifdef EMLX_TRACE_TIMELINE
    if (p.trace && threadIdx.x == 0) {
        long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        p.trace[2048 + 4 * blockIdx.x + 0] = now;
    }
#endif
    int* misc_words = (int*)(fixed + C::OFF_MISC);
    const PeerCache* peer_cache = (const PeerCache*)(fixed + C::OFF_PEER);
    const int num_units = p.hdr[0];
    const long long total_flat = (long long)p.hdr[1] * p.Hkv;
    // every CTA takes the contiguous slice the plan cut for it; a CTA without tiles has nothing to do
    const long long f_begin = p.cta_start[blockIdx.x], f_end = p.cta_start[blockIdx.x + 1];
    if constexpr (PEER) {
        if (threadIdx.x >= kConsumerThreads + 32)
            peer_enter(p.peer, p.peer_flags, p.peer_phase, misc_words, (PeerCache*)(fixed + C::OFF_PEER));
    }
    if (f_begin >= f_end) {  // uniform for the CTA, and no thread waits on a barrier yet
        if constexpr (PEER) peer_warp_exit(p, misc_words, peer_cache);
        return;
    }
    const long long active = gridDim.x;

    if (threadIdx.x >= kConsumerThreads + 32) {
        if constexpr (C::PRIVATE) {
            merge_warp_loop<D, NT, FMT, BF16, PEER, HELP>(p, fixed, full, abort_word, (int)active);
            // no further job: consumer warps that are parked, or park later, may leave
            __syncwarp();
            if ((threadIdx.x & 31) == 0) {
                *(volatile int*)(misc_words + kMiscHelpExit) = 1;
                ptx::mbar_arrive(&full[27]);
            }
        }
        if constexpr (PEER) peer_warp_exit(p, misc_words, peer_cache);
        return;
    } else if (threadIdx.x >= kConsumerThreads) {
        producer_loop<D, NT, FMT>(&kmap, &vmap, p, smem, fixed, full, empty, abort_word, f_begin, f_end, num_units);
    } else {
        if constexpr (C::PRIVATE)
            consumer_loop_private<D, NT, FMT, BF16, PEER, HELP>(p, smem, fixed, full, empty, abort_word, f_begin, f_end, total_flat, active);
        else
            consumer_loop<D, NT, FMT, BF16, PEER>(p, smem, fixed, full, empty, abort_word, f_begin, f_end, num_units, total_flat, active);
    }
    if (*abort_word && threadIdx.x == 0) flag_error(p.status, EMLX_DEV_WAIT_TIMEOUT);
    if constexpr (PEER) peer_warp_exit(p, misc_words, peer_cache);
#ifdef EMLX_TRACE
    if (p.trace && threadIdx.x == 0) {
        long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        p.trace[4 * blockIdx.x + 1] = now;
        p.trace[4 * blockIdx.x + 2] = f_end - f_begin;
        unsigned smid;
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        p.trace[4 * blockIdx.x + 3] = smid;
    }
#endif
}

// ------------------------------------------------------------------------------------------ host
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    });
    return fn;
}

static CUtensorMapSwizzle swizzle_of(int row_bytes) {
    return row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// Tensor maps depend only on the pool's address and geometry; they are encoded once and cached.  The pair is
// copied out while the lock is held, so a concurrent call that evicts the cache cannot invalidate it.
int get_maps(const emlx_pool& pool, MapPair* out) {
    static std::mutex mu;
    static std::map<std::tuple<void*, void*, long long, int, int, int, int, int>, MapPair> cache;
    auto key = std::make_tuple(pool.key_cache, pool.value_cache, (long long)pool.num_blocks, pool.num_kv_heads,
                               pool.head_dim, pool.kv_format, pool.kv_dtype, pool.block_size);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return EMLX_OK;
    }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(EMLX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (((uintptr_t)pool.key_cache | (uintptr_t)pool.value_cache) & 15)
        return fail(EMLX_ERR_INVALID, "key_cache/value_cache must be 16-byte aligned");
    MapPair mp;
    const cuuint64_t NB = (cuuint64_t)pool.num_blocks, Hkv = (cuuint64_t)pool.num_kv_heads, D = (cuuint64_t)pool.head_dim;
    const cuuint32_t ones[3] = {1, 1, 1};
    CUresult r1, r2;
    if (pool.kv_format == EMLX_KV_FLOAT) {
        const CUtensorMapDataType dt = pool.kv_dtype == EMLX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const cuuint64_t bs = (cuuint64_t)pool.block_size;  // a box is one page (128 tokens, or a part of a tile)
        const cuuint64_t dims[3] = {D, Hkv, NB * bs};
        const cuuint64_t strides[2] = {D * 2, Hkv * D * 2};
        const cuuint32_t box[3] = {64, 1, (cuuint32_t)bs};
        // a tile row is D*2 contiguous bytes: do not let L2 promotion pull in the neighbouring head's row
        const CUtensorMapL2promotion promo = D * 2 >= 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
        r1 = enc(&mp.k, dt, 3, pool.key_cache, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        r2 = enc(&mp.v, dt, 3, pool.value_cache, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t bits = (cuuint64_t)pool.kv_format;
        const cuuint64_t krow = D * bits / 8, vrow = (cuuint64_t)kTile * bits / 8;
        const cuuint64_t kdims[3] = {krow, Hkv, NB * kTile};
        const cuuint64_t kstrides[2] = {krow, Hkv * krow};
        const cuuint32_t kbox[3] = {(cuuint32_t)krow, 1, kTile};
        const CUtensorMapL2promotion kpromo = krow >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                          : (krow >= 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B : CU_TENSOR_MAP_L2_PROMOTION_NONE);
        r1 = enc(&mp.k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, pool.key_cache, kdims, kstrides, kbox, ones,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of((int)krow), kpromo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        const cuuint64_t vdims[2] = {vrow, NB * Hkv * D};
        const cuuint64_t vstrides[1] = {vrow};
        const cuuint32_t vbox[2] = {(cuuint32_t)vrow, (cuuint32_t)D};
        r2 = enc(&mp.v, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, pool.value_cache, vdims, vstrides, vbox, ones,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of((int)vrow), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r1 != CUDA_SUCCESS || r2 != CUDA_SUCCESS)
        return fail(EMLX_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d, %d)", (int)r1, (int)r2);
    if (cache.size() > 256) cache.clear();
    cache[key] = mp;
    *out = mp;
    return EMLX_OK;
}

template <int D, int NT, int FMT, bool BF16>
static int launch_one(const MapPair& maps, const TiledParams& p, int grid, cudaStream_t stream) {
    using C = Cfg<D, NT, FMT>;
    // Three builds of the kernel.  Codes paths that an ordinary batch never takes still cost it a per cent or two
    // when they sit in the same kernel (measured; the tile loop is the same, its scheduling is not): the final merge
    // shared by the consumer warps is only built in for batches of few, long units, the gather only for gathering calls.
    auto go = [&](auto kernel, DeviceOnce& configured) -> int {
        EMLX_CUDA_OK(allow_dynamic_smem(kernel, C::SMEM, configured));
        EMLX_CUDA_OK(launch_pdl(kernel, grid, kThreads, C::SMEM, stream, maps.k, maps.v, p));
        return EMLX_OK;
    };
    static DeviceOnce once_plain, once_help, once_gather;
    int rc;
    if (p.peer) rc = go(attn_tiled_kernel<D, NT, FMT, BF16, true, true>, once_gather);
    else if (p.few_units) rc = go(attn_tiled_kernel<D, NT, FMT, BF16, false, true>, once_help);
    else rc = go(attn_tiled_kernel<D, NT, FMT, BF16, false, false>, once_plain);
    if (rc) return rc;
    EMLX_LAUNCHED();
    return EMLX_OK;
}

template <int D, int NT>
static int launch_fmt(int fmt, bool bf16, const MapPair& maps, const TiledParams& p, int grid, cudaStream_t stream) {
    if (fmt == EMLX_KV_AFFINE8) return bf16 ? launch_one<D, NT, 8, true>(maps, p, grid, stream) : launch_one<D, NT, 8, false>(maps, p, grid, stream);
    if (fmt == EMLX_KV_AFFINE4) return bf16 ? launch_one<D, NT, 4, true>(maps, p, grid, stream) : launch_one<D, NT, 4, false>(maps, p, grid, stream);
    return bf16 ? launch_one<D, NT, 0, true>(maps, p, grid, stream) : launch_one<D, NT, 0, false>(maps, p, grid, stream);
}

static int launch_class(int cls, int D, int fmt, bool bf16, const MapPair& maps, const TiledParams& p, int grid, cudaStream_t s) {
    if (D == 128) {
        if (cls == 0) return launch_fmt<128, 1>(fmt, bf16, maps, p, grid, s);
        if (cls == 1) return launch_fmt<128, 2>(fmt, bf16, maps, p, grid, s);
        return launch_fmt<128, 4>(fmt, bf16, maps, p, grid, s);
    }
    if (cls == 0) return launch_fmt<64, 1>(fmt, bf16, maps, p, grid, s);
    if (cls == 1) return launch_fmt<64, 2>(fmt, bf16, maps, p, grid, s);
    return launch_fmt<64, 4>(fmt, bf16, maps, p, grid, s);
}

// Measurement aid, only in builds with -DEMLX_TRACE: a device buffer of at least 4 * 256 int64 into which every CTA
// of the tiled kernel writes {start ns, end ns, tiles processed, SM id}; -DEMLX_TRACE_PARTS / -DEMLX_TRACE_PREFILL
// add per-part and per-tile records behind those (the buffer must then hold 1024 + 256 * 16 * 4 int64).
#ifdef EMLX_TRACE
static long long* g_trace = nullptr;
#ifdef EMLX_TRACE_TIMELINE
// every launch that asks gets the next of 16 regions of 8192 int64, so that the kernels of consecutive steps captured
// into one CUDA graph leave separate records
static int g_trace_launch = 0;
long long* trace_buffer() { return g_trace ? g_trace + (size_t)(g_trace_launch++ % 16) * 8192 : nullptr; }
#else
long long* trace_buffer() { return g_trace; }
#endif
#else
long long* trace_buffer() { return nullptr; }
#endif

// A gathering call: the flag block of this rank and where its heads sit in the full output.
struct GatherTarget {
    void* flag_block;
    int total_q_heads, head_offset;
};

static int run_tiled(const emlx_attn_args* a, const emlx_pool* pool, void* stream, int class_lo, int class_hi,
                     const GatherTarget* gather = nullptr) {
    if (int rc = validate_attn(a, pool, true)) return rc;
    if (a->total_tokens == 0) return EMLX_OK;
    const int D = pool->head_dim, Hq = a->num_q_heads, Hkv = pool->num_kv_heads, G = Hq / Hkv;
    if (!tiled_page_size_ok(pool->block_size, pool->kv_format))
        return fail(EMLX_ERR_UNSUPPORTED, "the tiled kernels need page size 128 (16, 32 or 64 also for fp16/bf16 pools)");
    if (D != 64 && D != 128) return fail(EMLX_ERR_UNSUPPORTED, "the tiled kernels need head_dim 64 or 128");
    if (a->q_dtype == EMLX_F32) return fail(EMLX_ERR_UNSUPPORTED, "the tiled kernels need fp16 or bf16 queries");
    const bool bf16 = a->q_dtype == EMLX_BF16;
    if (pool->kv_format == EMLX_KV_FLOAT && pool->kv_dtype != a->q_dtype)
        return fail(EMLX_ERR_UNSUPPORTED, "the tiled kernels need the pool dtype to equal the query dtype");
    const PlanLayout L = plan_layout(a->num_seqs, a->total_tokens, Hq, Hkv);
    const WorkspaceLayout W = workspace_layout(a->num_seqs, a->total_tokens, Hq, Hkv, D);
    if (a->plan_bytes < (size_t)L.words * 4 || a->workspace_bytes < W.bytes)
        return fail(EMLX_ERR_WORKSPACE, "plan/workspace smaller than emlx_attn_plan_bytes()/emlx_attn_workspace_bytes()");
    if (((uintptr_t)a->queries | (uintptr_t)a->out) & 15) return fail(EMLX_ERR_INVALID, "queries/out must be 16-byte aligned");
    MapPair maps;
    if (int rc = get_maps(*pool, &maps)) return rc;

    // the row classes a plan holds depend on the flags it was built with, not on what this pool could support
    const bool wide = (a->plan_flags & kPlanWideUnits) != 0;
    // 128-row units over an affine pool: the pages of the sequences that own them are expanded into scratch memory that
    // the caller appended to the workspace (emlx_attn_dequant_bytes), and the 128-row kernel reads that
    const bool expand = wide && pool->kv_format != EMLX_KV_FLOAT;
    DequantScratch scratch{};
    if (expand) {
        if (!prefill_geometry_ok(Hq, Hkv, D))
            return fail(EMLX_ERR_INVALID, "plan_flags ask for 128-row units, which this head geometry cannot run");
        if (!dequant_scratch_layout(pool, a, (uint8_t*)a->workspace + W.bytes, a->workspace_bytes - W.bytes, &scratch))
            return fail(EMLX_ERR_WORKSPACE, "128-row units over an affine pool need emlx_attn_dequant_bytes() of memory "
                                            "behind the workspace");
    } else if (wide && !prefill_supported(pool->kv_format, Hq, Hkv, D)) {
        return fail(EMLX_ERR_INVALID, "plan_flags ask for 128-row units, which this pool / head geometry cannot run");
    }
    int lo, hi;
    class_range(G, a->max_query_len, wide, lo, hi);
    if (max(lo, class_lo) > min(hi, class_hi))
        return fail(EMLX_ERR_UNSUPPORTED,
                    "this plan holds row classes %d..%d and the entry point serves %d..%d: nothing to launch (build "
                    "the plan with other plan_flags or call emlx_attn_unified)", lo, hi, class_lo, class_hi);
    lo = max(lo, class_lo);
    hi = min(hi, class_hi);
    const int32_t* plan = (const int32_t*)a->plan;
    bool short_rows_launched = false;
    int first_launched = -1, last_launched = -1;
    for (int c = lo; c <= hi; ++c) {
        if (a->row_class_mask != 0 && !((a->row_class_mask >> c) & 1)) continue;
        if (first_launched < 0) first_launched = c;
        last_launched = c;
    }
    if (first_launched < 0) return fail(EMLX_ERR_UNSUPPORTED, "row_class_mask names no row class that this call can launch");
    const bool class3 = hi == 3 && (a->row_class_mask == 0 || ((a->row_class_mask >> 3) & 1));
    // the expansion comes first: the short-row kernels wait for it at their start, and the 128-row kernel, which may
    // run beside them, starts only after all their CTAs have passed that wait
    if (expand && class3)
        if (int rc = launch_dequant_pages(a, pool, scratch, (cudaStream_t)stream)) return rc;
    for (int c = lo; c <= hi; ++c) {
        if (a->row_class_mask != 0 && !((a->row_class_mask >> c) & 1)) continue;  // the caller knows this class is empty
        if (c == 3) {
            // the 128-row kernel comes last; behind a short-row kernel of this call it runs beside that kernel
            emlx_attn_args a3 = *a;
            emlx_pool pool3 = *pool;
            MapPair maps3 = maps;
            if (expand) {  // the scratch pool stands in for the pool: fp16 rows (also under bf16 queries), its own page table
                pool3.key_cache = scratch.k; pool3.value_cache = scratch.v;
                pool3.k_scale = pool3.k_bias = pool3.v_scale = pool3.v_bias = nullptr;
                pool3.num_blocks = scratch.cap; pool3.block_size = kTile;
                pool3.kv_format = EMLX_KV_FLOAT; pool3.kv_dtype = EMLX_F16;
                a3.block_tables = scratch.sbt;
                if (a->q_dtype == EMLX_BF16) {
                    // the tensor core takes both operands of a product in one type: fp16 copies of these sequences'
                    // queries (made by the expansion kernel) go in, fp16 rows come out and are converted below
                    a3.queries = scratch.q16; a3.out = scratch.out16; a3.q_dtype = EMLX_F16;
                }
                if (int rc = get_maps(pool3, &maps3)) return rc;
            }
            if (int rc = launch_prefill(&a3, &pool3, plan + 4 * c, plan + L.unit_seq[c], plan + L.unit_row0[c],
                                        plan + L.unit_tile_lo[c], plan + L.unit_cum[c], plan + L.unit_order,
                                        (int32_t*)((uint8_t*)a->workspace + W.counter_off[3]), short_rows_launched, maps3,
                                        (cudaStream_t)stream))
                return rc;
            if (expand && a->q_dtype == EMLX_BF16)
                if (int rc = launch_convert_out_rows(a, pool, scratch, (cudaStream_t)stream)) return rc;
            continue;
        }
        short_rows_launched = true;
        TiledParams p;
        p.q = a->queries; p.out = a->out; p.bt = a->block_tables; p.kv_lens = a->kv_lens; p.qsl = a->query_start_loc;
        p.hdr = plan + 4 * c;
        p.unit_seq = plan + L.unit_seq[c]; p.unit_row0 = plan + L.unit_row0[c];
        p.unit_tile_lo = plan + L.unit_tile_lo[c]; p.unit_cum = plan + L.unit_cum[c];
        p.cta_start = plan + L.cta_start[c];
        p.cta_unit = plan + L.cta_unit[c];
        p.counters = (int32_t*)((uint8_t*)a->workspace + W.counter_off[c]);
        p.slots = (float*)((uint8_t*)a->workspace + W.slots_off);
        p.status = a->status;
        p.trace = trace_buffer();
        p.k_scale = (const __half*)pool->k_scale; p.k_bias = (const __half*)pool->k_bias;
        p.v_scale = (const __half*)pool->v_scale; p.v_bias = (const __half*)pool->v_bias;
        p.num_blocks = pool->num_blocks;
        p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.MB = a->max_blocks_per_seq; p.window = a->sliding_window;
        p.bs = pool->block_size; p.ppt_log = pages_per_tile_log2(pool->block_size);
        p.scale_log2e = a->softmax_scale * 1.4426950408889634f;
        p.out_Hq = gather ? gather->total_q_heads : Hq;
        p.out_head0 = gather ? gather->head_offset : 0;
        p.peer = gather ? (const PeerTable*)((const uint8_t*)gather->flag_block + kPeerTableOffset) : nullptr;
        p.peer_flags = gather ? (int32_t*)gather->flag_block : nullptr;
        p.peer_phase = (c == first_launched ? kPeerFirstLaunch : 0) | (c == last_launched ? kPeerLastLaunch : 0);
        // a (sequence, KV head) unit is shared by about grid / units CTAs
        p.few_units = (long long)a->num_seqs * Hkv * (kHelpMinParts - 1) <=
                      class_ctas(c, min(num_sms(), kMaxGrid), (a->plan_flags & kPlanTwoCtas) != 0);
        // the grid a class is launched with is the one its slices were cut for
        const int grid = class_ctas(c, min(num_sms(), kMaxGrid), (a->plan_flags & kPlanTwoCtas) != 0);
        if (int rc = launch_class(c, D, pool->kv_format, bf16, maps, p, grid, (cudaStream_t)stream)) return rc;
    }
    return EMLX_OK;
}

}  // namespace emlx

#ifdef EMLX_TRACE
extern "C" __attribute__((visibility("default"))) void emlx_set_trace_buffer(int64_t* records) {
    emlx::g_trace = (long long*)records;
#ifdef EMLX_TRACE_TIMELINE
    emlx::g_trace_launch = 0;
#endif
}
#endif
extern "C" {
int emlx_attn_unified(const emlx_attn_args* a, const emlx_pool* p, void* s) { return emlx::run_tiled(a, p, s, 0, emlx::kNumClasses - 1); }
int emlx_attn_decode(const emlx_attn_args* a, const emlx_pool* p, void* s) { return emlx::run_tiled(a, p, s, 0, 2); }
int emlx_attn_prefill(const emlx_attn_args* a, const emlx_pool* p, void* s) { return emlx::run_tiled(a, p, s, 3, 3); }
int emlx_attn_decode_gather(const emlx_attn_args* a, const emlx_pool* p, void* flag_block, int32_t total_q_heads,
                            int32_t head_offset, void* s) {
    if (!a || !flag_block) return emlx::fail(EMLX_ERR_INVALID, "gather: null argument");
    if (head_offset < 0 || total_q_heads < head_offset + a->num_q_heads)
        return emlx::fail(EMLX_ERR_INVALID, "gather: heads [%d, %d) do not fit %d output heads", head_offset,
                          head_offset + a->num_q_heads, total_q_heads);
    if (a->plan_flags & emlx::kPlanWideUnits)
        return emlx::fail(EMLX_ERR_UNSUPPORTED, "gather: build the work list without 128-row units (plan_flags bit 0)");
    const emlx::GatherTarget g{flag_block, total_q_heads, head_offset};
    return emlx::run_tiled(a, p, s, 0, 2, &g);
}
int emlx_attn_plan_flags(int32_t kv_format, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim) {
    return (emlx::prefill_supported(kv_format, num_q_heads, num_kv_heads, head_dim) ? emlx::kPlanWideUnits : 0) |
           (kv_format == EMLX_KV_AFFINE4 ? emlx::kPlanTwoCtas : 0);
}
int emlx_attn_row_class(int32_t kv_format, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, int32_t query_len) {
    if (query_len <= 0 || num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads) return -1;
    const long long rows = (long long)query_len * (num_q_heads / num_kv_heads);
    return emlx::unit_class(rows > (1 << 20) ? (1 << 20) : (int)rows,
                            emlx::prefill_supported(kv_format, num_q_heads, num_kv_heads, head_dim));
}
}
