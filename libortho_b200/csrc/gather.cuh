// Output all-gather by peer stores: every rank keeps an [M, N_total] output buffer at the same offset
// of a peer-mapped allocation; a rank's kernel stores its column slice into every rank's buffer and
// the last CTA of the grid then raises a flag on every peer and waits (bounded) for the peers' flags.
// Only plain stores / loads on peer memory are used: no TMA and no multicast object ever sees it.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace ob {

constexpr int kMaxRanks = 8;

// control block at the end of every rank's allocation
struct GatherCtrl {
    int flag[kMaxRanks];     // flag[r] is written by rank r: the epoch of the last forward it finished
    int epoch;               // this rank's own count of finished gathers (device-side: survives graph replay)
    unsigned counter;        // CTAs of the running grid that have stored everything
    unsigned arrive[kMaxRanks];   // per-CTA signalling: arrive[r] grows by kArriveUnit per finished forward of rank r
};
// Per-CTA signalling: every CTA of a forward adds 1 to its counter on every peer once its own stores are out, and the
// grid's first CTA adds kArriveUnit - (CTAs of the grid) on top, so that a forward is complete on a peer exactly when
// the counter has grown by kArriveUnit.  (Grids of this library have at most a few hundred CTAs.)
constexpr unsigned kArriveUnit = 1u << 14;

// what a kernel needs to publish its slice.  world == 1 and ctrl[*] == nullptr: plain local store.
struct GatherView {
    int world, rank;
    __half *y[kMaxRanks];          // rank r's output buffer as mapped into this process ([M][ld])
    GatherCtrl *ctrl[kMaxRanks];   // rank r's control block as mapped into this process
    long long timeout_ns;          // bound of the wait for the peers' flags
    int deferred;                  // 1: a kernel waits for the PREVIOUS exchange before it reads its input and
                                   // only signals its own; 0: it signals and waits for its own exchange
    int per_cta;                   // 1: every CTA signals the peers itself (remote counters); 0: the grid's last CTA
                                   // raises one flag per peer after a device-scope count
};

__device__ __forceinline__ void st_relaxed_sys(int *p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_sys(const int *p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void red_add_relaxed_sys(unsigned *p, unsigned v) {
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// One thread: wait (bounded) until every peer's flag has reached epoch `ep`, then read the flags
// once more with acquire loads so that the peers' slices are ordered before whatever follows.
__device__ __forceinline__ bool gather_wait_flags(const GatherView &gv, int ep)
{
    const GatherCtrl *mine = gv.ctrl[gv.rank];
    bool ok = true;
    const unsigned long long t0 = global_timer_ns();
    // what a peer's word must have reached: its flag the epoch, or its counter epoch * kArriveUnit (both compared
    // as wrapped differences)
    const int want = gv.per_cta ? (int)((unsigned)ep * kArriveUnit) : ep;
    for (int r = 0; r < gv.world; r++) {
        if (r == gv.rank) continue;
        const int *f = gv.per_cta ? reinterpret_cast<const int *>(&mine->arrive[r]) : &mine->flag[r];
        unsigned spins = 0;
        while (ld_relaxed_sys(f) - want < 0) {
            if ((++spins & 63u) == 0 && (long long)(global_timer_ns() - t0) > gv.timeout_ns) { ok = false; break; }
        }
    }
    for (int r = 0; r < gv.world; r++) {
        if (r == gv.rank) continue;
        const int *f = gv.per_cta ? reinterpret_cast<const int *>(&mine->arrive[r]) : &mine->flag[r];
        if (ld_acquire_sys(f) - want < 0) ok = false;
    }
    return ok;
}

// Deferred mode, consumer side: called by every thread of a CTA after the grid dependency has been
// resolved (the previous kernel of the stream, which raised this rank's epoch, is complete) and
// before the CTA reads activations: thread 0 waits for the peers' flags of that epoch.
__device__ __forceinline__ bool gather_wait_previous(const GatherView &gv)
{
    bool ok = true;
    if (gv.world > 1 && gv.deferred) {
        if (threadIdx.x == 0) ok = gather_wait_flags(gv, ld_relaxed_sys(&gv.ctrl[gv.rank]->epoch));
        __syncthreads();
    }
    return ok;
}

// Called by every thread of every CTA once the CTA's stores to all ranks have been issued.
// `total_ctas` = CTAs of the grid.  Returns (in thread 0 of the last CTA) false when a peer's flag
// did not arrive in time; the caller records that in the device status word.  Every other thread
// returns true right after the CTA-wide barrier.
//
// Ordering: a CTA's stores -> bar.sync -> device-scope fence + counter increment by thread 0; the
// thread that takes the last count has thereby observed every CTA's stores, issues ONE
// system-scope fence (cumulative: it covers the observed stores) and then writes the flags with
// relaxed system-scope stores.  A system-scope fence waits for the NVLink round trip of the
// outstanding peer stores, so there is exactly one on the way out; on the way in the flags are
// polled with relaxed loads and read once more with an acquire load when they have arrived.
// In deferred mode the kernel returns after the flag stores: the next kernel of the stream (or
// ortho_b200_comm_wait) waits for them.
__device__ __forceinline__ bool gather_signal_and_wait(const GatherView &gv, unsigned total_ctas)
{
    if (gv.world <= 1) return true;
    __syncthreads();
    if (threadIdx.x != 0) return true;
    GatherCtrl *mine = gv.ctrl[gv.rank];
    if (gv.per_cta) {
        // this CTA's stores (ordered before this thread by the barrier) -> one system-scope fence -> one remote add
        // per peer; the device-scope count below only elects the thread that keeps the epoch and, in the
        // non-deferred mode, waits: no peer waits for it
        fence_acq_rel_sys();
        const bool first = (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
        const unsigned add = first ? kArriveUnit - total_ctas + 1u : 1u;
        for (int r = 0; r < gv.world; r++)
            if (r != gv.rank) red_add_relaxed_sys(&gv.ctrl[r]->arrive[gv.rank], add);
        if (atomicAdd(&mine->counter, 1u) != total_ctas - 1) return true;
        atomicExch(&mine->counter, 0u);
        const int ep = mine->epoch + 1;
        mine->epoch = ep;
        if (gv.deferred) return true;
        return gather_wait_flags(gv, ep);
    }
    fence_acq_rel_gpu();
    if (atomicAdd(&mine->counter, 1u) != total_ctas - 1) return true;
    fence_acq_rel_sys();
    atomicExch(&mine->counter, 0u);
    const int ep = mine->epoch + 1;
    mine->epoch = ep;
    for (int r = 0; r < gv.world; r++)
        if (r != gv.rank) st_relaxed_sys(&gv.ctrl[r]->flag[gv.rank], ep);
    if (gv.deferred) return true;
    return gather_wait_flags(gv, ep);
}

}  // namespace ob
