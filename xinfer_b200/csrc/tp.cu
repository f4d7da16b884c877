// N-split tensor parallelism across the GPUs of one box, one process per GPU.
//
// Every rank owns an "exchange region" (one cudaMalloc) holding the activation buffers that other ranks
// write into, the flag words of tp.cuh and a few counters.  The regions are mapped into every process
// through CUDA IPC handles that the host exchanges out of band (any all-gather of 64-byte blobs will do:
// torch.distributed, MPI, a file).  Buffers are carved out of the region in the same order on every rank,
// so an offset names the same logical buffer everywhere and a peer's address is its base plus that offset.
//
// The reference has no multi-GPU code (README.md:99 there); what this shards are the projections of
// forward_layer / forward_lm_head (src/targets/qwen3_8/forward.cpp:117-125, 229-232, 262, 276-287, 726-732):
// rank r holds the output rows [r N/g, (r+1) N/g) of every W_int4 / scales pair, computes that slice of
// Y for all activation rows and stores it into every rank's Y (plain peer stores from the GEMM epilogue,
// w4a16_tc.cu), followed by one flag per (receiver, sender).  No TMA, multicast or multimem touches peer
// memory, and every device-side wait is bounded.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "../../include/xinfer_b200.h"
#include "tp.cuh"
#include "tp_host.h"
#include "w4a16.h"

namespace xb {

namespace {

constexpr size_t kHeaderBytes = 16384;  // flag matrix | exchange count; buffers start after it

struct Header {
    unsigned long long flags[kTpMaxWorld][kTpMaxCtas];
    unsigned long long epoch;
};
static_assert(sizeof(Header) <= kHeaderBytes, "exchange header");

// Copies [off, off + bytes) of this rank's region to the same offsets of every peer (16-byte vectors),
// then runs the exchange handshake.  bytes == 0: handshake only (a barrier among the ranks).
__global__ void __launch_bounds__(256) tp_push_kernel(TpLink tp, uint8_t* local_base, uint8_t* p0, uint8_t* p1, uint8_t* p2,
                                                      uint8_t* p3, uint8_t* p4, uint8_t* p5, uint8_t* p6, uint8_t* p7,
                                                      size_t off, size_t bytes) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint8_t* peers[kTpMaxWorld] = {p0, p1, p2, p3, p4, p5, p6, p7};
    const size_t nvec = bytes / 16;
    const uint4* src = reinterpret_cast<const uint4*>(local_base + off);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint4 v = src[i];
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r)
            if (r < tp.world && r != tp.rank) reinterpret_cast<uint4*>(peers[r] + off)[i] = v;
    }
    __syncthreads();
    if (threadIdx.x < 32) tp_finish_exchange(tp, gridDim.x, blockIdx.x);
}

}  // namespace

TpLink tp_link(const TpComm* c, int rows_per_rank) {
    TpLink l;
    memset(&l, 0, sizeof(l));
    if (!c || c->world <= 1) {
        l.world = 1;
        return l;
    }
    l.world = c->world;
    l.rank = c->rank;
    l.rows_per_rank = rows_per_rank;
    for (int r = 0; r < c->world; ++r)
        l.flags_peer[r] = reinterpret_cast<unsigned long long*>(c->peer_base[r]);  // Header::flags
    Header* h = reinterpret_cast<Header*>(c->peer_base[c->rank]);
    l.flags_local = &h->flags[0][0];
    l.epoch = &h->epoch;
    l.status = c->status;
    l.wait_limit = c->wait_limit;
    return l;
}

int tp_push(const TpComm* c, cudaStream_t s, size_t off, size_t bytes) {
    if (!c || c->world <= 1) return 0;
    if (!c->connected || (off & 15) || (bytes & 15) || off + bytes > c->bytes) return -2;
    TpLink l = tp_link(c, 1);
    const size_t nvec = bytes / 16;
    unsigned ctas = static_cast<unsigned>((nvec + 255) / 256);
    ctas = ctas < 1 ? 1 : (ctas > 32 ? 32 : ctas);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    uint8_t* b[kTpMaxWorld];
    for (int r = 0; r < kTpMaxWorld; ++r) b[r] = r < c->world ? static_cast<uint8_t*>(c->peer_base[r]) : nullptr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tp_push_kernel, l, b[c->rank], b[0], b[1], b[2], b[3], b[4], b[5], b[6],
                                       b[7], off, bytes);
    return e == cudaSuccess ? 0 : -1;
}

}  // namespace xb

using xb::TpComm;

extern "C" {

int xinfer_tp_create(int rank, int world, size_t bytes, xinfer_tp** out) {
    if (!out || world < 1 || world > xb::kTpMaxWorld || rank < 0 || rank >= world) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return XINFER_ERR_NO_DEVICE;
    int rc = xinfer_b200_init(dev);
    if (rc != XINFER_OK) return rc;
    TpComm* c = new (std::nothrow) TpComm();
    if (!c) return XINFER_ERR_OUT_OF_MEMORY;
    c->rank = rank;
    c->world = world;
    c->device = dev;
    c->bytes = xb::kHeaderBytes + ((bytes + 255) & ~static_cast<size_t>(255));
    c->bump = xb::kHeaderBytes;
    c->wait_limit = xb::kTpWaitLimitClocks;
    void* p = nullptr;
    if (cudaMalloc(&p, c->bytes) != cudaSuccess || cudaMalloc(reinterpret_cast<void**>(&c->status), sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        if (p) cudaFree(p);
        delete c;
        return XINFER_ERR_OUT_OF_MEMORY;
    }
    cudaMemset(p, 0, c->bytes);
    cudaMemset(c->status, 0, sizeof(int));
    cudaDeviceSynchronize();
    c->peer_base[rank] = p;
    c->connected = (world == 1);
    *out = c;
    return XINFER_OK;
}

void xinfer_tp_destroy(xinfer_tp* c) {
    if (!c) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank || !c->peer_base[r]) continue;
        cudaIpcCloseMemHandle(c->peer_base[r]);
    }
    if (c->peer_base[c->rank]) cudaFree(c->peer_base[c->rank]);
    if (c->status) cudaFree(c->status);
    delete c;
}

size_t xinfer_tp_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int xinfer_tp_handle(xinfer_tp* c, void* out) {
    if (!c || !out) return XINFER_ERR_INVALID_ARGUMENT;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, c->peer_base[c->rank]) != cudaSuccess) {
        xb::set_last_error(cudaGetErrorString(cudaGetLastError()));
        return XINFER_ERR_CUDA;
    }
    memcpy(out, &h, sizeof(h));
    return XINFER_OK;
}

int xinfer_tp_connect(xinfer_tp* c, const void* all_handles) {
    if (!c || (!all_handles && c->world > 1)) return XINFER_ERR_INVALID_ARGUMENT;
    if (c->connected) return XINFER_OK;
    const uint8_t* hs = static_cast<const uint8_t*>(all_handles);
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, hs + static_cast<size_t>(r) * sizeof(h), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            xb::set_last_error(cudaGetErrorString(e));
            cudaGetLastError();
            return XINFER_ERR_CUDA;
        }
        c->peer_base[r] = p;
    }
    c->connected = true;
    return XINFER_OK;
}

int xinfer_tp_alloc(xinfer_tp* c, size_t bytes, size_t* offset_out) {
    if (!c || !offset_out) return XINFER_ERR_INVALID_ARGUMENT;
    const size_t b = (bytes + 255) & ~static_cast<size_t>(255);
    if (c->bump + b > c->bytes) return XINFER_ERR_OUT_OF_MEMORY;
    *offset_out = c->bump;
    c->bump += b;
    return XINFER_OK;
}

void* xinfer_tp_ptr(xinfer_tp* c, size_t offset) {
    if (!c || offset >= c->bytes) return nullptr;
    return static_cast<uint8_t*>(c->peer_base[c->rank]) + offset;
}

int xinfer_tp_rank(const xinfer_tp* c) { return c ? c->rank : -1; }
int xinfer_tp_world(const xinfer_tp* c) { return c ? c->world : 0; }

void xinfer_tp_set_wait_limit(xinfer_tp* c, int64_t limit_clocks) {
    if (c) c->wait_limit = limit_clocks > 0 ? limit_clocks : xb::kTpWaitLimitClocks;
}

int xinfer_tp_status(xinfer_tp* c) {
    if (!c) return XINFER_ERR_INVALID_ARGUMENT;
    int v = 0;
    if (cudaMemcpy(&v, c->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return XINFER_ERR_CUDA;
    if (v != 0) cudaMemset(c->status, 0, sizeof(int));
    return v == 0 ? XINFER_OK : XINFER_ERR_DEVICE_TIMEOUT;
}

int xinfer_tp_push(xinfer_tp* c, xinfer_stream_t s, size_t offset, size_t bytes) {
    const int rc = xb::tp_push(c, static_cast<cudaStream_t>(s), offset, bytes);
    return rc == 0 ? XINFER_OK : (rc == -2 ? XINFER_ERR_INVALID_ARGUMENT : XINFER_ERR_CUDA);
}

int xinfer_tp_barrier(xinfer_tp* c, xinfer_stream_t s) { return xinfer_tp_push(c, s, xb::kHeaderBytes, 0); }

int xinfer_tp_linear_int4_f16f16(xinfer_tp* c, xinfer_stream_t s, size_t y_offset, int64_t ldy, int64_t col0,
                                 const void* X, const uint8_t* W, const void* scales, const float* bias, int64_t M,
                                 int64_t N_local, int64_t K, int group_size, int rows_per_rank) {
    if (!c || !c->connected) return XINFER_ERR_INVALID_ARGUMENT;
    if (M <= 0 || N_local <= 0 || K <= 0) return XINFER_NOOP_INVALID_SHAPE;
    if (!X || !W || !scales || ldy < col0 + N_local || col0 < 0 ||
        y_offset + static_cast<size_t>(M) * ldy * 2 > c->bytes)
        return XINFER_ERR_INVALID_ARGUMENT;
    xb::TcProj p;
    p.w = W;
    p.scales = scales;
    p.bias = bias;
    p.n = N_local;
    p.ldy = ldy;
    xb::tp_fill_proj(c, &p, y_offset + static_cast<size_t>(col0) * 2, rows_per_rank > 0 ? 2 : 1);
    const xb::TpLink link = xb::tp_link(c, rows_per_rank > 0 ? rows_per_rank : 1);
    return xb::run_tc_linear(static_cast<cudaStream_t>(s), X, &p, 1, false, false, M, K, group_size, &link);
}

}  // extern "C"
