// Device side of the N-split tensor-parallel exchange: after a kernel has stored its slice of an
// activation into every rank's buffer (plain peer stores over NVLink), the last CTA of the grid tells
// the peers and waits until every peer has told it the same.  One flag word per (receiver, sender)
// carries the sender's launch count, so the scheme needs no reset and works unchanged inside a
// replayed CUDA graph.  The reference has no multi-GPU code; the call sites this attaches to are the
// projections of forward_layer and forward_lm_head (src/targets/qwen3_8/forward.cpp:117-125, 229-232,
// 262, 276-287, 726-732).
//
// Rules kept here: plain st.global to peer memory only (no TMA, no multicast, no multimem); every wait
// is bounded and records a status word instead of spinning forever.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace xb {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxCtas = 192;  // CTAs of a kernel that takes part in an exchange (one per SM at most)
constexpr long long kTpWaitLimitClocks = 2000000000LL;  // default limit of an exchange wait, about one second

// What a kernel needs to take part in the exchange.  world <= 1: no exchange, every field unused.
// Flags: every rank holds a matrix [sender rank][sender CTA] of launch counts.  A CTA that has finished its
// peer stores writes its launch count into its own slot on every peer (a release store at system scope, so the
// CTA's data is visible before the flag); CTA 0 of the receiving grid waits until every slot of every peer has
// reached the count.  Every rank runs the same launches on the same shapes, so grid sizes agree.
struct TpLink {
    int world;
    int rank;
    int rows_per_rank;                         // owner of activation row j (owner-mode outputs): j / rows_per_rank
    int pad;
    unsigned long long* flags_peer[kTpMaxWorld];  // rank r's flag matrix [world][kTpMaxCtas]; this rank writes row [rank]
    unsigned long long* flags_local;           // this rank's flag matrix
    unsigned long long* epoch;                 // this rank's count of completed exchanges
    int* status;                               // device status word (set when a wait gives up)
    long long wait_limit;                      // SM clocks
};

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Called by ONE WHOLE WARP of every CTA (all 32 lanes converged) after all of the CTA's peer stores are ordered
// before it (a CTA-wide barrier).  Lane 0 publishes the CTA to the peers.  In CTA 0 the warp then waits
// (bounded) until every CTA of every peer has published the same launch; when it returns there, every peer's
// slice of this exchange is visible in local memory, and the kernel boundary makes it visible to the next
// kernel of the stream.  `ctas` = gridDim.x (the same on every rank), `cta` = blockIdx.x.
__device__ __forceinline__ void tp_finish_exchange(const TpLink& tp, unsigned int ctas, unsigned int cta) {
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned long long e = *tp.epoch + 1;  // written by CTA 0 of the previous exchange, long complete
    if (lane == 0) {
        // One release fence at system scope (the CTA's data stores, ordered before this point by the CTA barrier, are
        // performed before any flag below becomes visible), then one plain store per rank: the flag writes leave
        // together instead of each waiting for the one before it.
        // (this rank's own matrix included: CTA 0 must not advance the count while a CTA of its own grid has yet to
        // read it)
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        for (int r = 0; r < tp.world; ++r) st_relaxed_sys_u64(tp.flags_peer[r] + tp.rank * kTpMaxCtas + cta, e);
    }
    if (cta != 0) return;
    const long long t0 = clock64();
    const unsigned int total = static_cast<unsigned int>(tp.world) * ctas;  // this rank's own row included
    bool all = false, timed_out = false;
    while (!all) {
        bool mine = true;
        for (unsigned int i = lane; i < total; i += 32) {
            const unsigned int r = i / ctas, c = i - r * ctas;
            if (ld_relaxed_sys_u64(tp.flags_local + r * kTpMaxCtas + c) < e) mine = false;
        }
        all = __all_sync(0xffffffffu, mine);
        if (!all && clock64() - t0 > tp.wait_limit) {
            timed_out = true;
            break;
        }
    }
    __syncwarp();
    if (lane == 0) {
        // acquire: order the peers' data (released with their flags) before everything after this point
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        if (timed_out) atomicExch(tp.status, 1);
        // The count advances even after a timeout, so that this rank stays in step with its peers' counts.
        *tp.epoch = e;
    }
}

}  // namespace xb
