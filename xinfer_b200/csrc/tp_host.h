// Host side of the N-split tensor-parallel exchange (tp.cu): the per-rank exchange region and helpers
// that describe it to kernels.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "tp.cuh"
#include "w4a16.h"

struct xinfer_tp {
    int rank = 0, world = 1, device = 0;
    size_t bytes = 0;   // size of every rank's region (identical on all ranks)
    size_t bump = 0;    // next free offset
    void* peer_base[xb::kTpMaxWorld] = {};  // base of every rank's region as mapped here; [rank] is the local one
    int* status = nullptr;                  // device status word of the exchange waits
    long long wait_limit = 0;               // SM clocks
    bool connected = false;
};

namespace xb {

using TpComm = ::xinfer_tp;

// The kernel-side description of the exchange; rows_per_rank only matters for owner-mode outputs.
TpLink tp_link(const TpComm* c, int rows_per_rank);
// Copies [off, off + bytes) of the local region to every peer's region, then signals and waits.
int tp_push(const TpComm* c, cudaStream_t s, size_t off, size_t bytes);

// Points a projection's output at byte offset `off` of the exchange region on every rank.
inline void tp_fill_proj(const TpComm* c, TcProj* p, size_t off, int push) {
    p->y = static_cast<uint8_t*>(c->peer_base[c->rank]) + off;
    p->push = c->world > 1 ? push : 0;
    for (int r = 0; r < kTpMaxWorld; ++r)
        p->y_peer[r] = (r < c->world && c->peer_base[r]) ? static_cast<uint8_t*>(c->peer_base[r]) + off : nullptr;
}

// tcgen05 linear on the current device's scratch with an optional exchange; no CUDA-core fallback: returns
// XINFER_ERR_INVALID_ARGUMENT for shapes the tensor-core kernel does not take (c_api.cu).
int run_tc_linear(cudaStream_t s, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32, long long m,
                  long long k, int group_size, const TpLink* tp, int layout_flags = 0);

}  // namespace xb
