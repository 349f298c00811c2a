// Prefill-chunk attention on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only.
//
// Work unit: 128 query rows of one sequence (row = query token x GQA head of one KV head, token-major) and
// one KV head; the plan lists the KV tiles (128-token pages) the rows may attend.  Per tile
//     S[128 rows x 128 tokens]  = Q . K^T     tcgen05.mma, both operands K-major in shared memory (TMA, 128B swizzle),
//                                             fp32 accumulator in TMEM columns [0, 128)
//     softmax                                  one TMEM lane (= one row) per thread and warpgroup, 64 keys each;
//                                             P goes back to TMEM (16-bit, two per column) as the next A operand, so the
//                                             shared-memory port only carries K and V
//     O_tile[128 rows x D]      = P . V        tcgen05.mma with A from TMEM, V read in place as an MN-major B operand
//     O = O * corr + O_tile                    in registers of the softmax threads
// Warp roles: 0-7 softmax (two warpgroups, each half of every tile's keys), 8 TMA producer, 9 MMA issuer (and TMEM
// owner).  All waits are bounded.
#include "plan_device.cuh"
#include "ptx.cuh"
#include "tensor_maps.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace emlx {

#ifdef EMLX_TRACE_PREFILL
#define PF_STAMP(cond, tile, slot) do { if (p.trace && blockIdx.x == 0 && (cond) && (tile) < 256) p.trace[(tile) * 8 + (slot)] = clock64(); } while (0)
#else
#define PF_STAMP(cond, tile, slot) do { } while (0)
#endif

constexpr int kPfWGs = 2;                       // softmax warpgroups: each takes kTile / kPfWGs keys of every tile
constexpr int kPfKeys = kTile / kPfWGs;
constexpr int kPfSoftThreads = 128 * kPfWGs;
constexpr int kPfProducerWarp = 4 * kPfWGs;     // TMA producer
constexpr int kPfMmaWarp = kPfProducerWarp + 1; // MMA issuer, owner of the TMEM allocation
constexpr int kPfThreads = kPfSoftThreads + 64;
static_assert(kPfKeys == 32 || kPfKeys == 64, "a warpgroup's keys are one or two 32-column TMEM loads");
constexpr int kPfRows = 128;

struct PrefillParams {
    void* out;
    const int32_t* bt;
    const int32_t* kv_lens;
    const int32_t* qsl;
    const int32_t* hdr;
    const int32_t* unit_seq;
    const int32_t* unit_row0;
    const int32_t* unit_tile_lo;
    const int32_t* unit_cum;
    const int32_t* unit_order;  // units by decreasing number of tiles
    int32_t* queue;             // [0] next item to hand out, [1] CTAs that have finished; both zero between launches
    int32_t* status;
    long long* trace;  // measurement aid (only with EMLX_TRACE_PREFILL): per-tile cycle stamps of CTA 0
    long long num_blocks;
    int Hq, Hkv, G, MB, window;
    int bs, ppt_log;  // page size in tokens and log2(pages per 128-token tile)
    int wait_late;    // the launch before this one is the short-row kernel of the same call: run beside it
    float scale_log2e;
};

template <int D>
struct PfCfg {
    static constexpr int HALVES = D / 64;
    static constexpr int QBYTES = kPfRows * D * 2;
    static constexpr int KBYTES = kTile * D * 2;
    static constexpr int KST = D == 128 ? 3 : 4;  // K tiles are needed one tile ahead of V (QK of tile j+1 precedes PV of tile j)
    static constexpr int VST = D == 128 ? 3 : 4;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + QBYTES;
    static constexpr int OFF_V = OFF_K + KST * KBYTES;
    static constexpr int OFF_BAR = OFF_V + VST * KBYTES;
    static constexpr int SMEM = OFF_BAR + 256 + 1024;
    static constexpr int TMEM_COLS = 512;  // S (two buffers): columns [0,128) and [128,256); O: [256, 256 + D); Q: [384, 384 + D/2); P of a tile overwrites the first 64 columns of its S
};

// ------------------------------------------------------------------ tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// A operand read from tensor memory (row = lane, two 16-bit elements of the contraction axis per 32-bit column)
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: 128-byte swizzle, 8-row groups 1024 bytes apart (stride offset); the leading
// offset is the distance between 64-element blocks along the contiguous dimension of an MN-major operand.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of sm_100
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulate, fp16 or bf16 inputs, A K-major, B K- or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool bf16, bool b_mn_major) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

struct PfBarriers {
    // q_tmem: Q copied to TMEM.  qk_done[t & 3] / pv_done[t & 3]: the QK / PV product of tile t is complete; each is
    // committed once and read by two parties (QK: the softmax warps, for S, and the producer, for the K slot; PV: the
    // softmax warps, for O, and the producer, for the V slot) because a commit costs the issuing thread as much as an
    // MMA.  Four barriers each, so that no waiter can fall two phases behind the barrier it waits on.
    // p_ready[t & 1]: P of tile t written over its S.
    uint64_t q_full, q_tmem, item_done, qk_done[4], p_ready[2], pv_done[4];
    uint64_t k_full[4], v_full[4];
    // item_full[k & 3]: the index of the CTA's k-th item is in item_ring[k & 3] (-1: no more items)
    uint64_t item_full[4];
    // x_full[t & 1]: both half-row maxima of tile t are in shared memory; l_full: both half-row sums of the item are
    uint64_t x_full[2], l_full;
    int item_ring[4];
    uint32_t tmem_base;
    int abort_word;
};

static_assert(sizeof(PfBarriers) <= 256, "the barrier block has 256 bytes of shared memory");

template <int D, bool BF16>
__global__ void __launch_bounds__(kPfThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap, const PrefillParams p) {
    using C = PfCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem + C::OFF_Q;
    uint8_t* k_smem = smem + C::OFF_K;
    uint8_t* v_smem = smem + C::OFF_V;
    PfBarriers* bars = (PfBarriers*)(smem + C::OFF_BAR);
    volatile int* abort_word = &bars->abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // The plan, the pool and the queries come from earlier kernels.  When the launch right before this one is the
    // short-row kernel of the same attention call, that kernel has already waited for all of them, and this grid
    // runs beside it (the two are bound by different resources: HBM there, tensor cores here); it then waits for that
    // kernel at its END, so that whatever follows in the stream still sees both complete.
    if (!p.wait_late) grid_dep_wait();
    grid_dep_launch();
    const int num_units = p.hdr[0];
    const int items = num_units * p.Hkv;
    // Items (unit, head), listed by decreasing length, are handed out through a counter in device memory: a CTA that
    // starts late (its SM was still busy with a short-row CTA) simply takes fewer of them.  The producer warp draws
    // the index and passes it to the other warps through a small ring in shared memory.
    auto decode_item = [&](int idx, int& u, int& head) {
        u = p.unit_order[idx / p.Hkv];
        head = idx % p.Hkv;
    };

    if (tid == 0) {
        ptx::mbar_init(&bars->q_full, 1);
        ptx::mbar_init(&bars->q_tmem, kPfSoftThreads);
        ptx::mbar_init(&bars->item_done, kPfSoftThreads);
        ptx::mbar_init(&bars->p_ready[0], kPfSoftThreads);
        ptx::mbar_init(&bars->p_ready[1], kPfSoftThreads);
        ptx::mbar_init(&bars->x_full[0], kPfSoftThreads);
        ptx::mbar_init(&bars->x_full[1], kPfSoftThreads);
        ptx::mbar_init(&bars->l_full, kPfSoftThreads);
        for (int s = 0; s < 4; ++s) {
            ptx::mbar_init(&bars->qk_done[s], 1);
            ptx::mbar_init(&bars->pv_done[s], 1);
            ptx::mbar_init(&bars->k_full[s], 1);
            ptx::mbar_init(&bars->v_full[s], 1);
            ptx::mbar_init(&bars->item_full[s], 1);
        }
        bars->abort_word = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&qmap);
        ptx::prefetch_tensormap(&kmap);
        ptx::prefetch_tensormap(&vmap);
    }
    if (warp == kPfMmaWarp) tmem_alloc(&bars->tmem_base, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 256, tmem_Q = tmem_base + 384;

    if (warp == kPfProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        uint32_t kt = 0, k = 0;
        int u, head;
        int next = lane == 0 ? atomicAdd(p.queue, 1) : 0;
        for (;; ++k) {
            int idx = __shfl_sync(0xffffffffu, next, 0);
            if (idx >= items || *abort_word) idx = -1;
            if (lane == 0) {
                bars->item_ring[k & 3] = idx;
                ptx::mbar_arrive(&bars->item_full[k & 3]);
            }
            if (idx < 0) break;
            if (lane == 0) next = atomicAdd(p.queue, 1);  // the following item, drawn while this one is loaded
            decode_item(idx, u, head);
            const int seq = p.unit_seq[u], row0 = p.unit_row0[u], tile_lo = p.unit_tile_lo[u];
            const int ntiles = p.unit_cum[u + 1] - p.unit_cum[u];
            const int qs = p.qsl[seq], kv_len = p.kv_lens[seq];
            if (k > 0) ptx::mbar_wait(&bars->item_done, (k - 1) & 1, abort_word);
            if (lane == 0 && !*abort_word) {
                ptx::mbar_arrive_expect_tx(&bars->q_full, C::QBYTES);
#pragma unroll
                for (int h = 0; h < C::HALVES; ++h)
                    ptx::tma_load_3d(q_smem + h * (kPfRows * 128), &qmap, &bars->q_full, 64 * h, head * p.G, qs + row0 / p.G);
            }
            if (p.ppt_log == 0) {  // one page per tile: the common case keeps the shortest instruction stream (this warp
                                   // shares a scheduler with a softmax warp)
                // K runs two tiles ahead of V: the K slot of tile t is free as soon as QK of tile t - 3 is done, long before
                // the V slot that PV of tile t - 3 still reads, and one warp issuing both in step would hold K back
                auto load_pages = [&](int base) -> int {
                    const int idx = tile_lo + base + lane;
                    return (base + lane < ntiles && idx < p.MB) ? p.bt[(long long)seq * p.MB + idx] : -1;
                };
                int pg_cur = load_pages(0), pg_next = load_pages(32), base = 0;
                auto page_of = [&](int i) -> int {  // tile i of the item, base <= i < base + 64; every lane takes part
                    const int a = __shfl_sync(0xffffffffu, pg_cur, (i - base) & 31), b = __shfl_sync(0xffffffffu, pg_next, (i - base) & 31);
                    return i - base < 32 ? a : b;
                };
                auto issue = [&](int i, bool is_k) {
                    const uint32_t t = kt + (uint32_t)i;
                    const int pg = page_of(i);
                    const bool bad = pg < 0 || pg >= p.num_blocks;
                    const int tok0 = bad ? -kTile : pg * kTile;  // out-of-range coordinates read as zeros
                    if (is_k) {
                        if (lane == 0 && bad && (long long)(tile_lo + i) * kTile < kv_len) flag_error(p.status, EMLX_DEV_BAD_PAGE);
                        const uint32_t ks = t % C::KST;
                        if (t >= C::KST) ptx::mbar_wait(&bars->qk_done[(t - C::KST) & 3], ((t - C::KST) >> 2) & 1, abort_word);
                        if (lane == 0 && !*abort_word) {
                            ptx::mbar_arrive_expect_tx(&bars->k_full[ks], C::KBYTES);
    #pragma unroll
                            for (int h = 0; h < C::HALVES; ++h)
                                ptx::tma_load_3d(k_smem + (size_t)ks * C::KBYTES + h * (kTile * 128), &kmap, &bars->k_full[ks], 64 * h, head, tok0);
                        }
                    } else {
                        const uint32_t vs = t % C::VST;
                        if (t >= C::VST) ptx::mbar_wait(&bars->pv_done[(t - C::VST) & 3], ((t - C::VST) >> 2) & 1, abort_word);
                        if (lane == 0 && !*abort_word) {
                            ptx::mbar_arrive_expect_tx(&bars->v_full[vs], C::KBYTES);
    #pragma unroll
                            for (int h = 0; h < C::HALVES; ++h)
                                ptx::tma_load_3d(v_smem + (size_t)vs * C::KBYTES + h * (kTile * 128), &vmap, &bars->v_full[vs], 64 * h, head, tok0);
                        }
                    }
                    __syncwarp();
                };
                issue(0, true);
                if (ntiles > 1) issue(1, true);
                for (int i = 0; i < ntiles; ++i) {
                    if (i + 2 < ntiles) issue(i + 2, true);
                    issue(i, false);
                    if (i + 1 == base + 32) {  // tiles up to base + 34 have been looked up: the older half is done with
                        base += 32;
                        pg_cur = pg_next;
                        pg_next = load_pages(base + 32);
                    }
                }
            } else {
                // K runs two tiles ahead of V: the K slot of tile t is free as soon as QK of tile t - 3 is done, long before
                // the V slot that PV of tile t - 3 still reads, and one warp issuing both in step would hold K back
                // page ids in batches of 32: lane l holds page (l mod pages-per-tile) of tile base + l / pages-per-tile, and two
                // batches (cur, next) are kept so that K can run ahead
                const int ppt_log = p.ppt_log, ppt = 1 << ppt_log, tiles_per_batch = 32 >> ppt_log;
                auto load_pages = [&](int base) -> int {
                    const int tile = base + (lane >> ppt_log);
                    const long long pidx = ((long long)(tile_lo + tile) << ppt_log) + (lane & (ppt - 1));
                    return (tile < ntiles && pidx < p.MB) ? p.bt[(long long)seq * p.MB + pidx] : -1;
                };
                int pg_cur = load_pages(0), pg_next = load_pages(tiles_per_batch), base = 0;
                auto page_of = [&](int i, int sub) -> int {  // page `sub` of tile i, base <= i < base + 2 batches; every lane takes part
                    const int idx = ((i - base) << ppt_log) + sub;
                    const int a = __shfl_sync(0xffffffffu, pg_cur, idx & 31), b = __shfl_sync(0xffffffffu, pg_next, idx & 31);
                    return idx < 32 ? a : b;
                };
                auto issue = [&](int i, bool is_k) {
                    const uint32_t t = kt + (uint32_t)i;
                    const uint32_t slot = is_k ? t % C::KST : t % C::VST;
                    if (is_k) {
                        if (t >= C::KST) ptx::mbar_wait(&bars->qk_done[(t - C::KST) & 3], ((t - C::KST) >> 2) & 1, abort_word);
                    } else {
                        if (t >= C::VST) ptx::mbar_wait(&bars->pv_done[(t - C::VST) & 3], ((t - C::VST) >> 2) & 1, abort_word);
                    }
                    const bool go = lane == 0 && !*abort_word;
                    uint64_t* bar = is_k ? &bars->k_full[slot] : &bars->v_full[slot];
                    uint8_t* tile = (is_k ? k_smem : v_smem) + (size_t)slot * C::KBYTES;
                    if (go) ptx::mbar_arrive_expect_tx(bar, C::KBYTES);
                    for (int sub = 0; sub < ppt; ++sub) {
                        const int pg = page_of(i, sub);
                        if (go) {
                            const bool bad = pg < 0 || pg >= p.num_blocks;
                            const int tok0 = bad ? -p.bs : pg * p.bs;  // out-of-range coordinates read as zeros
                            if (is_k && bad && (long long)(tile_lo + i) * kTile + (long long)sub * p.bs < kv_len)
                                flag_error(p.status, EMLX_DEV_BAD_PAGE);
    #pragma unroll
                            for (int h = 0; h < C::HALVES; ++h)
                                ptx::tma_load_3d(tile + h * (kTile * 128) + (size_t)sub * p.bs * 128, is_k ? &kmap : &vmap, bar, 64 * h, head, tok0);
                        }
                    }
                    __syncwarp();
                };
                issue(0, true);
                if (ntiles > 1) issue(1, true);
                for (int i = 0; i < ntiles; ++i) {
                    if (i + 2 < ntiles) issue(i + 2, true);
                    issue(i, false);
                    if (i + 1 == base + tiles_per_batch) {  // the tiles of the older batch are all issued (K is at most two ahead)
                        base += tiles_per_batch;
                        pg_cur = pg_next;
                        pg_next = load_pages(base + tiles_per_batch);
                    }
                }
            }
            kt += (uint32_t)ntiles;
        }
    } else if (warp == kPfMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_qk = instr_desc(128, 128, BF16, false);
        constexpr uint32_t idesc_pv = instr_desc(128, D, BF16, true);
        const uint64_t k_desc0 = smem_desc(ptx::smem_u32(k_smem), 16, 1024);
        const uint64_t v_desc0 = smem_desc(ptx::smem_u32(v_smem), kTile * 128, 1024);
        uint32_t kt = 0, k = 0;
        int u, head;
        for (;; ++k) {
            if (!ptx::mbar_wait(&bars->item_full[k & 3], (k >> 2) & 1, abort_word)) break;
            const int idx = bars->item_ring[k & 3];
            if (idx < 0) break;
            decode_item(idx, u, head);
            const int ntiles = p.unit_cum[u + 1] - p.unit_cum[u];
            ptx::mbar_wait(&bars->q_tmem, k & 1, abort_word);  // the item's Q rows are in TMEM
            tc_fence_after();
            // S is double-buffered in TMEM: QK of tile j+1 is issued before PV of tile j, so the tensor pipe
            // works while the softmax warps are busy with tile j
            // Descriptors differ from tile to tile and from k-step to k-step only in their address field (bits 0-13,
            // the shared-memory address / 16): one add per instruction instead of rebuilding them.  Q is read from
            // TMEM (the softmax warps copied it there), so the shared-memory port only serves K here.
            auto issue_qk = [&](uint32_t t) {
                const uint32_t stage = t % C::KST;
                const bool ok = ptx::mbar_wait(&bars->k_full[stage], (t / C::KST) & 1, abort_word);
                tc_fence_after();
                PF_STAMP(lane == 0, t, 4);
                if (lane == 0 && ok) {
                    const uint64_t kd = k_desc0 + (uint64_t)(stage * (C::KBYTES >> 4));
                    const uint32_t s_tmem = tmem_S + (t & 1) * 128;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        constexpr int kHalf = (kTile * 128) >> 4;
                        const uint32_t off = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 2);  // in 16-byte units
                        tc_mma_f16_ts(s_tmem, tmem_Q + ks * 8, kd + off, idesc_qk, ks > 0);
                    }
                    tc_commit(&bars->qk_done[t & 3]);
                }
                __syncwarp();
            };
            issue_qk(kt);
            for (int j = 0; j < ntiles; ++j, ++kt) {
                if (j + 1 < ntiles) issue_qk(kt + 1);
                const uint32_t stage = kt % C::VST;
                bool ok = ptx::mbar_wait(&bars->v_full[stage], (kt / C::VST) & 1, abort_word);
                PF_STAMP(lane == 0, kt, 5);
                ok = ptx::mbar_wait(&bars->p_ready[kt & 1], (kt >> 1) & 1, abort_word) && ok;
                tc_fence_after();
                PF_STAMP(lane == 0, kt, 6);
                if (lane == 0 && ok) {
                    const uint64_t vd = v_desc0 + (uint64_t)(stage * (C::KBYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk) {
                        // 16 tokens of P = 8 packed columns at the start of this tile's S buffer (the pipe runs MMAs in
                        // issue order, so QK of tile kt + 2 overwrites the buffer only after this product has read it);
                        // 16 token rows of V = 2048 bytes further on
                        tc_mma_f16_ts(tmem_O, tmem_S + (kt & 1) * 128 + kk * 8, vd + (uint64_t)(kk * ((16 * 128) >> 4)), idesc_pv, j > 0 || kk > 0);
                    }
                    tc_commit(&bars->pv_done[kt & 3]);
                }
                PF_STAMP(lane == 0, kt, 7);
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax: two warpgroups, half a tile each
        // Thread r of warpgroup g owns row r (= TMEM lane r) and the 64 keys [64 g, 64 g + 64) of every tile.  The two
        // threads of a row exchange their half-row maxima (and, at the end of an item, their sums) through the Q
        // tile's shared memory, which is idle once Q sits in TMEM; both then take the same decisions about the row's
        // reference maximum.  A tile costs 128 x 128 exponentials and the SM makes 16 per clock: with 256 threads
        // feeding that unit instead of 128 the time a tile spends between QK and PV, which is what the tensor pipe
        // waits for, drops by a sixth.
        const int wg = warp >> 2, r = tid & 127;
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        float* xmax = (float*)q_smem;                      // [tile parity][warpgroup][row]
        float* xsum = xmax + 2 * kPfWGs * kPfRows;         // [warpgroup][row]
        constexpr int OCHUNKS = D / 32;                    // 32-column chunks of O, dealt over the warpgroups
        uint32_t kt = 0;
        int u, head;
        for (uint32_t k = 0;; ++k) {
            if (!ptx::mbar_wait(&bars->item_full[k & 3], (k >> 2) & 1, abort_word)) break;
            const int idx = bars->item_ring[k & 3];
            if (idx < 0) break;
            decode_item(idx, u, head);
            const int seq = p.unit_seq[u], row0 = p.unit_row0[u], tile_lo = p.unit_tile_lo[u];
            const int ntiles = p.unit_cum[u + 1] - p.unit_cum[u];
            const int qs = p.qsl[seq], q_len = p.qsl[seq + 1] - qs, kv_len = p.kv_lens[seq];
            const int R = q_len * p.G, ctx = kv_len - q_len;
            const int rows_here = min(kPfRows, R - row0);
            // A warp whose 32 rows all lie past the unit's last row (spec-verify units hold 20 rows) keeps every
            // barrier appointment but leaves the row work out: its lanes of S, P and O hold garbage that no one
            // reads (rows of an MMA do not mix, and rows past the unit are never stored).
            const bool dead = (warp & 3) * 32 >= rows_here;
            const int rr = min(row0 + r, R - 1), ti = rr / p.G;
            int hi = min(kv_len, ctx + ti + 1);
            int lo = p.window > 0 ? max(0, min(kv_len - 1, ctx + ti) - p.window + 1) : 0;
            if (hi <= 0) { hi = 0; lo = 0; }
            const int i_first = row0 / p.G, i_last = (row0 + rows_here - 1) / p.G;
            const int hi_min = min(kv_len, ctx + i_first + 1);
            const int lo_max = p.window > 0 ? max(0, min(kv_len - 1, ctx + i_last) - p.window + 1) : 0;

            // this row of Q: shared memory (TMA, swizzled) -> TMEM, two 16-bit elements per column, as the A operand of
            // QK; warpgroup g copies the g-th 64 elements
            ptx::mbar_wait(&bars->q_full, k & 1, abort_word);
            if (wg < C::HALVES) {
                uint32_t qv[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *(const uint4*)(q_smem + wg * (kPfRows * 128) + r * 128 + ((c ^ (r & 7)) << 4));
                    qv[4 * c] = v.x; qv[4 * c + 1] = v.y; qv[4 * c + 2] = v.z; qv[4 * c + 3] = v.w;
                }
                tmem_st32(tmem_Q + lane_addr + 32 * wg, qv);
            }
            tc_fence_before();
            ptx::mbar_arrive(&bars->q_tmem);

            // m_ref is the maximum the stored probabilities and O refer to; it follows the true running maximum
            // lazily (only when that grew by more than 2^8), so O in TMEM is rarely rescaled.  Both threads of a row
            // compute it from the same numbers, so they always agree.  l is the sum over this thread's keys only.
            float m_ref = -INFINITY, l = 0.f;

            for (int j = 0; j < ntiles; ++j, ++kt) {
                const int t0 = (tile_lo + j) * kTile;
                const bool interior = (t0 + kTile <= hi_min) && (t0 >= lo_max);
                const uint32_t s_addr = tmem_S + (kt & 1) * 128 + lane_addr;
                ptx::mbar_wait(&bars->qk_done[kt & 3], (kt >> 2) & 1, abort_word);
                tc_fence_after();
                PF_STAMP(tid == 0, kt, 0);
                if (dead) {
                    ptx::mbar_arrive(&bars->x_full[kt & 1]);
                    ptx::mbar_wait(&bars->x_full[kt & 1], (kt >> 1) & 1, abort_word);
                } else {
                    uint32_t sv[kPfKeys];
#pragma unroll
                    for (int c = 0; c < kPfKeys / 32; ++c) tmem_ld32_nowait(s_addr + kPfKeys * wg + 32 * c, sv + 32 * c);
                    tmem_wait_ld();
                    if (!interior) {
#pragma unroll
                        for (int i = 0; i < kPfKeys; ++i) {
                            const int tok = t0 + kPfKeys * wg + i;
                            if (tok < lo || tok >= hi) sv[i] = 0xff800000u;  // -inf
                        }
                    }
                    float mx8[8];  // eight independent chains instead of one of 64 dependent maxima
#pragma unroll
                    for (int i = 0; i < 8; ++i) mx8[i] = __uint_as_float(sv[i]);
#pragma unroll
                    for (int i = 8; i < kPfKeys; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(sv[i]));
                    float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
                    // the other parts of the row
                    xmax[((kt & 1) * kPfWGs + wg) * kPfRows + r] = mx;
                    ptx::mbar_arrive(&bars->x_full[kt & 1]);
                    ptx::mbar_wait(&bars->x_full[kt & 1], (kt >> 1) & 1, abort_word);
#pragma unroll
                    for (int g = 0; g < kPfWGs; ++g) mx = fmaxf(mx, xmax[((kt & 1) * kPfWGs + g) * kPfRows + r]);
                    PF_STAMP(tid == 0, kt, 1);
                    const float m_new = mx * p.scale_log2e;
                    const bool grow = (j == 0) ? true : (m_new > m_ref + 8.0f);
                    float corr = 1.0f;
                    if (grow) {
                        const float m_tgt = fmaxf(m_ref, m_new);
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(corr) : "f"(m_ref - (m_tgt == -INFINITY ? 0.f : m_tgt)));
                        m_ref = m_tgt;
                    }
                    // O is only touched when the reference maximum moves (rare): every earlier PV must be complete then.
                    // P needs no such wait: it replaces this tile's own S, which nothing else uses until QK of tile kt + 2.
                    // Each warpgroup rescales its half of the row's columns.
                    if (j > 0 && __any_sync(0xffffffffu, grow)) {
                        ptx::mbar_wait(&bars->pv_done[(kt - 1) & 3], ((kt - 1) >> 2) & 1, abort_word);
                        tc_fence_after();
#pragma unroll 1
                        for (int c4 = wg; c4 < OCHUNKS; c4 += kPfWGs) {
                            uint32_t ov[32];
                            tmem_ld32_nowait(tmem_O + lane_addr + 32 * c4, ov);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                            tmem_st32(tmem_O + lane_addr + 32 * c4, ov);
                        }
                        l *= corr;
                    }
                    PF_STAMP(tid == 0, kt, 2);
                    // fp16 weights are stored as 2^(s - m_ref + 7): m_ref trails the true maximum by up to 2^8, so the
                    // largest stored weight is 2^15, and a key only rounds to zero below 2^-32 of the reference (the sum l
                    // carries the same factor, which cancels in O / l)
                    constexpr float kShift = BF16 ? 0.0f : 7.0f;
                    const float m_safe = m_ref == -INFINITY ? 0.f : m_ref;
                    const float neg_m = kShift - m_safe;
                    float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
                    uint32_t packed[kPfKeys / 2];
#pragma unroll
                    for (int e = 0; e < kPfKeys / 2; ++e) {
                        float p0, p1;
                        // (Sending a quarter of the exponentials through a cubic on the FMA pipe instead of the special-function
                        // unit was measured twice, on the tensor-bound mixed batch and on the bandwidth-bound spec-verify
                        // batch, and was 4-5 % slower on both: the issue slots it costs are as scarce as that unit.)
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(__uint_as_float(sv[2 * e]), p.scale_log2e, neg_m)));
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(__uint_as_float(sv[2 * e + 1]), p.scale_log2e, neg_m)));
                        if (e & 1) { ls2 += p0; ls3 += p1; } else { ls0 += p0; ls1 += p1; }
                        if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed[e]) : "f"(p1), "f"(p0));
                        else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(packed[e]) : "f"(p1), "f"(p0));
                    }
                    // this warpgroup's keys of the row, two per column, over the start of the tile's own S
                    if constexpr (kPfKeys == 64) tmem_st32(s_addr + 32 * wg, packed);
                    else tmem_st16(s_addr + 16 * wg, packed);
                    l += (ls0 + ls1) + (ls2 + ls3);
                }
                if (t0 + kTile > kv_len && wg < C::HALVES) {
                    // token rows of V past the sequence end are stale memory: clear them (thread r owns token r, its
                    // warpgroup the 64-element block of the row)
                    ptx::mbar_wait(&bars->v_full[kt % C::VST], (kt / C::VST) & 1, abort_word);
                    if (r >= max(0, kv_len - t0)) {
                        uint8_t* vrow = v_smem + (size_t)(kt % C::VST) * C::KBYTES + wg * (kTile * 128) + r * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) *(uint4*)(vrow + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    ptx::fence_proxy_async();  // the tensor core reads V through the async proxy
                }
                tc_fence_before();
                PF_STAMP(tid == 0, kt, 3);
                ptx::mbar_arrive(&bars->p_ready[kt & 1]);
            }
            // the last PV, then this row of O: the two sums of the row are added, each warpgroup stores half the columns
            xsum[wg * kPfRows + r] = l;
            ptx::mbar_arrive(&bars->l_full);
            ptx::mbar_wait(&bars->pv_done[(kt - 1) & 3], ((kt - 1) >> 2) & 1, abort_word);
            tc_fence_after();
            ptx::mbar_wait(&bars->l_full, k & 1, abort_word);
            l = 0.f;  // every warpgroup adds the parts in the same order and gets the same sum
#pragma unroll
            for (int g = 0; g < kPfWGs; ++g) l += xsum[g * kPfRows + r];
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const bool store = row0 + r < R;
            const int oi = (row0 + r) / p.G, ohh = (row0 + r) - oi * p.G;
            uint4* dst = (uint4*)((uint16_t*)p.out + ((long long)(qs + oi) * p.Hq + head * p.G + ohh) * D);
#pragma unroll 1
            for (int c4 = wg; c4 < OCHUNKS && !dead; c4 += kPfWGs) {
                uint32_t ov[32];
                tmem_ld32_nowait(tmem_O + lane_addr + 32 * c4, ov);
                tmem_wait_ld();
                if (store) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float x0 = __uint_as_float(ov[8 * c + 2 * e]) * inv, x1 = __uint_as_float(ov[8 * c + 2 * e + 1]) * inv;
                            if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(x1), "f"(x0));
                            else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(x1), "f"(x0));
                        }
                        dst[4 * c4 + c] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            tc_fence_before();
            ptx::fence_proxy_async();  // the next item's Q arrives by TMA over the memory the exchanges above used
            ptx::mbar_arrive(&bars->item_done);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kPfMmaWarp) tmem_dealloc(tmem_base, C::TMEM_COLS);
    if (*abort_word && tid == 0) flag_error(p.status, EMLX_DEV_WAIT_TIMEOUT);
    if (tid == 0) {
        // every draw of this CTA is behind us; the last CTA to get here puts the item counter back to zero
        __threadfence();
        if (atomicInc((unsigned int*)&p.queue[1], gridDim.x - 1) == gridDim.x - 1) p.queue[0] = 0;
    }
    if (p.wait_late) grid_dep_wait();
}

// ------------------------------------------------------------------------------------------ host
bool prefill_geometry_ok(int num_q_heads, int num_kv_heads, int head_dim) {
    if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return false;
    const int G = num_q_heads / num_kv_heads;
    return (head_dim == 64 || head_dim == 128) && G <= kPfRows && kPfRows % G == 0;
}
bool prefill_supported(int kv_format, int num_q_heads, int num_kv_heads, int head_dim) {
    return kv_format == EMLX_KV_FLOAT && prefill_geometry_ok(num_q_heads, num_kv_heads, head_dim);
}

// Q is [T, Hq, D]; a box of {64 columns, G heads, 128/G tokens} lands in shared memory as 128 rows in the
// unit's row order (token-major, then GQA head), 128 bytes per row and swizzled like the K/V tiles.
static int make_q_map(const emlx_attn_args* a, int D, int G, CUtensorMap* out) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int, int>, CUtensorMap> cache;
    auto key = std::make_tuple(a->queries, a->total_tokens, a->num_q_heads, D, G, a->q_dtype);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return EMLX_OK;
    }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(EMLX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)a->num_q_heads, (cuuint64_t)a->total_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)a->num_q_heads * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(kPfRows / G)};
    const cuuint32_t ones[3] = {1, 1, 1};
    const CUtensorMapDataType dt = a->q_dtype == EMLX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap m;
    CUresult r = enc(&m, dt, 3, const_cast<void*>(a->queries), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EMLX_ERR_CUDA, "cuTensorMapEncodeTiled failed for the query tensor (%d)", (int)r);
    if (cache.size() > 256) cache.clear();
    cache[key] = m;
    *out = m;
    return EMLX_OK;
}

template <int D, bool BF16>
static int launch_pf(const CUtensorMap& qmap, const MapPair& maps, const PrefillParams& p, cudaStream_t stream) {
    using C = PfCfg<D>;
    auto kernel = attn_prefill_kernel<D, BF16>;
    static DeviceOnce configured;
    EMLX_CUDA_OK(allow_dynamic_smem(kernel, C::SMEM, configured));
    EMLX_CUDA_OK(launch_pdl(kernel, min(num_sms(), kMaxGrid), kPfThreads, C::SMEM, stream, qmap, maps.k, maps.v, p));
    EMLX_LAUNCHED();
    return EMLX_OK;
}

int launch_prefill(const emlx_attn_args* a, const emlx_pool* pool, const int32_t* plan_class_hdr, const int32_t* unit_seq,
                   const int32_t* unit_row0, const int32_t* unit_tile_lo, const int32_t* unit_cum, const int32_t* unit_order,
                   int32_t* queue, bool wait_late, const MapPair& maps, cudaStream_t stream) {
    const int D = pool->head_dim, Hq = a->num_q_heads, Hkv = pool->num_kv_heads, G = Hq / Hkv;
    if (!prefill_supported(pool->kv_format, Hq, Hkv, D))
        return fail(EMLX_ERR_UNSUPPORTED, "the tcgen05 prefill kernel needs an fp16/bf16 pool, head_dim 64/128 and 128 %% (Hq/Hkv) == 0");
    CUtensorMap qmap;
    if (int rc = make_q_map(a, D, G, &qmap)) return rc;
    PrefillParams p;
    p.out = a->out; p.bt = a->block_tables; p.kv_lens = a->kv_lens; p.qsl = a->query_start_loc;
    p.hdr = plan_class_hdr; p.unit_seq = unit_seq; p.unit_row0 = unit_row0; p.unit_tile_lo = unit_tile_lo; p.unit_cum = unit_cum; p.unit_order = unit_order;
    p.status = a->status; p.num_blocks = pool->num_blocks; p.trace = trace_buffer();
    p.queue = queue; p.wait_late = wait_late ? 1 : 0;
    p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.MB = a->max_blocks_per_seq; p.window = a->sliding_window;
    p.bs = pool->block_size; p.ppt_log = pages_per_tile_log2(pool->block_size);
    p.scale_log2e = a->softmax_scale * 1.4426950408889634f;
    const bool bf16 = a->q_dtype == EMLX_BF16;
    if (D == 128) return bf16 ? launch_pf<128, true>(qmap, maps, p, stream) : launch_pf<128, false>(qmap, maps, p, stream);
    return bf16 ? launch_pf<64, true>(qmap, maps, p, stream) : launch_pf<64, false>(qmap, maps, p, stream);
}

}  // namespace emlx
