// Output gather over peer-mapped memory: when KV heads are sharded over GPUs every rank computes the attention of its
// own query heads and stores those rows straight into the full [T, Hq_total, D] output of every rank (plain stores
// through peer-mapped pointers; no TMA and no multicast on peer memory), instead of an all-gather afterwards.
//
// Every rank owns one flag block in memory the other ranks can write.  A call has an epoch (the rank's own counter
// + 1; all ranks make the same calls, so their epochs agree):
//   ready[src] = e   written by rank `src` when its first kernel of call e has passed the wait on its stream
//                    predecessors: everything that consumed the output of call e-1 on `src` has finished, so the
//                    other ranks may overwrite `src`'s output buffer;
//   done[src]  = e   written by rank `src` with a system-scope release store after all its CTAs have finished.
// A CTA waits for ready[r] of every rank before its first remote store, and the last CTA of the call's last kernel
// waits for done[r] of every rank before the kernel ends, so work queued behind the call on the stream sees the whole
// output.  Both waits are bounded: on expiry the kernel sets EMLX_DEV_WAIT_TIMEOUT and carries on.  No rank ever
// waits for something that itself waits: the ready flags are sent unconditionally and the done flags only wait for
// them.
#pragma once

#include "common.cuh"

namespace emlx {

constexpr int kMaxPeers = EMLX_MAX_PEERS;
// int32 slots of a flag block
constexpr int kPeerReady = 0;                 // [kMaxPeers]
constexpr int kPeerDone = kMaxPeers;          // [kMaxPeers]
constexpr int kPeerEpoch = 2 * kMaxPeers;     // calls completed by the owner
constexpr int kPeerTicket = 2 * kMaxPeers + 1;  // CTAs of the running kernel that have finished
constexpr int kPeerTableOffset = 128;         // bytes: the owner's PeerTable (only the owner reads it)

struct PeerTable {
    void* out[kMaxPeers];        // rank r's full output buffer as mapped into this process (out[rank] is local)
    int32_t* flags[kMaxPeers];   // rank r's flag block as mapped into this process
    int32_t num_ranks, rank, poll_limit, reserved;
};
static_assert(kPeerTableOffset >= (2 * kMaxPeers + 2) * 4, "flag slots overlap the table");
static_assert(kPeerTableOffset + sizeof(PeerTable) <= EMLX_PEER_FLAG_BYTES, "flag block too small");

// what a kernel of a gathering call does beside its stores
constexpr int kPeerFirstLaunch = 1;  // sends ready flags, and its CTAs wait for the others' before storing
constexpr int kPeerLastLaunch = 2;   // sends done flags, waits for the others', advances the epoch

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_relaxed_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Polls a flag in this GPU's memory until it reaches `epoch` (flags only grow; the comparison survives wrap-around).
// Gives up after `limit` polls and returns false.  The polls are relaxed loads; one acquire fence follows the one
// that succeeded (an acquire load per poll would pay a system-scope fence every time round).
__device__ __forceinline__ bool peer_wait(const int32_t* flag, int32_t epoch, int32_t limit) {
    for (int32_t i = 0; i < limit; ++i) {
        if (ld_relaxed_sys(flag) - epoch >= 0) {
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            return true;
        }
        __nanosleep(i < 256 ? 20 : 200);
    }
    return false;
}

#endif

}  // namespace emlx
