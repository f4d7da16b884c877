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
constexpr long long kTpWaitLimitClocks = 2000000000LL;  // default limit of an exchange wait, about one second

// What a kernel needs to take part in the exchange.  world <= 1: no exchange, every field unused.
struct TpLink {
    int world;
    int rank;
    int rows_per_rank;                         // owner of activation row j (owner-mode outputs): j / rows_per_rank
    int pad;
    unsigned long long* flags_peer[kTpMaxWorld];  // rank r's flag array [world]; this rank writes slot [rank]
    unsigned long long* flags_local;           // this rank's flag array
    unsigned long long* epoch;                 // this rank's count of completed exchanges
    unsigned int* done;                        // CTA arrival counter, zero between launches
    int* status;                               // device status word (set when a wait gives up)
    long long wait_limit;                      // SM clocks
};

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Called by ONE thread of every CTA after all of the CTA's peer stores are ordered before it (a CTA-wide
// barrier).  The last CTA to arrive publishes this launch to the peers, then waits (bounded) for theirs.
// When it returns in the last CTA, every peer's slice of this exchange is visible in local memory; the
// kernel boundary makes it visible to the next kernel of the stream.
__device__ __forceinline__ void tp_finish_exchange(const TpLink& tp, unsigned int ctas) {
    __threadfence_system();
    const unsigned int old = atomicAdd(tp.done, 1u);
    if (old != ctas - 1) return;
    *tp.done = 0;
    __threadfence_system();
    const unsigned long long e = *tp.epoch + 1;
    for (int r = 0; r < tp.world; ++r)
        if (r != tp.rank) st_release_sys_u64(tp.flags_peer[r] + tp.rank, e);
    const long long t0 = clock64();
    bool ok = true;
    for (int r = 0; r < tp.world && ok; ++r) {
        if (r == tp.rank) continue;
        while (ld_acquire_sys_u64(tp.flags_local + r) < e) {
            if (clock64() - t0 > tp.wait_limit) {
                atomicExch(tp.status, 1);
                ok = false;
                break;
            }
        }
    }
    // The count advances even after a timeout, so that this rank stays in step with its peers' counts.
    *tp.epoch = e;
    __threadfence_system();
}

}  // namespace xb
