// Internal interface between the C-ABI layer and the W4A16 kernels (CUDA-core and tcgen05 paths).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "tp.cuh"

namespace xb {

// One projection of a (possibly fused) launch.  `w` is [n][k/2] packed int4 (low nibble = even k),
// `scales` is [n][k/group] fp16, `bias` is [n] fp32 or null, `y` is [m][ldy] (ldy = 0 means n).
// N-split tensor parallelism: with push != 0 the kernel stores every output element straight into the
// buffers of other ranks, `y_peer[r]` being rank r's address of the element `y` points to (y_peer[own
// rank] == y).  push 1: every rank gets every row; push 2: row j goes only to rank j / rows_per_rank
// (its sequence's owner).  push 0 (and y_peer unused): local store only.
struct TcProj {
    void* y;
    const uint8_t* w;
    const void* scales;
    const float* bias;
    long long n;
    long long ldy;
    int push = 0;
    void* y_peer[kTpMaxWorld] = {};
};

// ---- tcgen05 path (w4a16_tc.cu): fp16 activations, 1 <= m <= 32, k % 128 == 0
size_t tc_workspace_bytes(int ctas);
// Test hooks for the bounded device-side waits: their clock limit (<= 0 restores the one-second default)
// and the first activation stage that the producer never requests (-1: all are requested).
void tc_set_wait_hooks(long long limit_clocks, int withhold_x_from_stage);
// Status word of the allocation-free entry point on `device` (which must be current): read and cleared.
int tc_noalloc_take_status(int device);
long long tc_wait_limit();  // clocks after which a device-side wait gives up (tc_set_wait_hooks)
int tc_x_stage_limit();     // test hook of tc_set_wait_hooks: first activation stage that is never requested (-1: off)

// Dense GEMM for more than 32 activation rows (prefill chunks) on tcgen05, both operands from shared memory
// (w4a16_gemm.cu).  One launch per projection; gate and up of the fused MLP share one.
bool gemm_eligible(const void* x, const TcProj* proj, int num, bool swiglu, long long m, long long k, int group_size);
// `partials` / `partial_bytes`: scratch for the fp32 partial sums of a K split (null: never split).
int gemm_launch(cudaStream_t stream, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32, long long m,
                long long k, int* status, long long wait_limit, int x_stage_limit, int num_sms, float* partials, size_t partial_bytes);
// Records a message for xinfer_last_cuda_error() on the calling thread (c_api.cu).
void set_last_error(const char* msg);
// Programmatic dependent launch (on unless XINFER_PDL=0): kernels are launched with the stream-serialization
// attribute and call griddepcontrol.wait before they touch data of the previous kernel.
bool pdl_enabled();
bool tc_eligible(const void* x, const TcProj* proj, int num, bool swiglu, long long m, long long k, int group_size);
// Launch plan (a hint for L2 prefetching of the next launch's weights): record one round of the caller's
// fixed launch sequence between record_begin/record_end, then rewind at the start of every further round.
struct TcPlan;
TcPlan* tc_plan_new();
void tc_plan_delete(TcPlan* p);
// Binds a plan to the calling thread (null: the process-wide default); returns the previous binding.
TcPlan* tc_plan_bind(TcPlan* p);
void tc_plan_record_begin();
void tc_plan_record_end();
void tc_plan_rewind();
void tc_plan_clear();
// `tp` (may be null): the exchange this launch takes part in; its last CTA then signals the peers and waits
// for theirs before the kernel completes.
int tc_launch(cudaStream_t stream, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32,
              long long m, long long k, int num_sms, float* workspace, int* counters, int counter_capacity,
              int* status, const TpLink* tp = nullptr, int layout_flags = 0);
// layout_flags.  The int4 unpack yields the k of each block of eight in the order (0,4,1,5,2,6,3,7); the kernel
// normally rewrites every staged activation tile into that order itself.  A caller that owns the producer of X can
// have it written in that order once (kTcXPermuted) and skip the rewrite; kTcYPermuted makes this launch such a
// producer: its output columns are written in that order.  Permuted buffers are private to such a chain.
constexpr int kTcXPermuted = 1;
constexpr int kTcYPermuted = 2;

// ---- CUDA-core path (w4a16_simt.cu): any m, fp16 or fp32 activations, any shape the reference accepts
enum class ActType { F16, F32 };
int simt_launch(cudaStream_t stream, const void* x, ActType in, bool out_f32, const TcProj* proj, int num,
                bool swiglu, long long m, long long k, int group_size);

}  // namespace xb
