// Internal interface between the C-ABI layer and the W4A16 kernels (CUDA-core and tcgen05 paths).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace xb {

// One projection of a (possibly fused) launch.  `w` is [n][k/2] packed int4 (low nibble = even k),
// `scales` is [n][k/group] fp16, `bias` is [n] fp32 or null, `y` is [m][ldy] (ldy = 0 means n).
struct TcProj {
    void* y;
    const uint8_t* w;
    const void* scales;
    const float* bias;
    long long n;
    long long ldy;
};

// ---- tcgen05 path (w4a16_tc.cu): fp16 activations, 1 <= m <= 32, k % 128 == 0
size_t tc_workspace_bytes(int ctas);
void tc_set_trace(long long* dev_ptr);
// Programmatic dependent launch (on unless XINFER_PDL=0): kernels are launched with the stream-serialization
// attribute and call griddepcontrol.wait before they touch data of the previous kernel.
bool pdl_enabled();
bool tc_eligible(const void* x, const TcProj* proj, int num, bool swiglu, long long m, long long k, int group_size);
// Launch plan (a hint for L2 prefetching of the next launch's weights): record one round of the caller's
// fixed launch sequence between record_begin/record_end, then rewind at the start of every further round.
void tc_plan_record_begin();
void tc_plan_record_end();
void tc_plan_rewind();
void tc_plan_clear();
int tc_launch(cudaStream_t stream, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32,
              long long m, long long k, int num_sms, float* workspace, int* counters, int counter_capacity,
              int* status);

// ---- CUDA-core path (w4a16_simt.cu): any m, fp16 or fp32 activations, any shape the reference accepts
enum class ActType { F16, F32 };
int simt_launch(cudaStream_t stream, const void* x, ActType in, bool out_f32, const TcProj* proj, int num,
                bool swiglu, long long m, long long k, int group_size);

}  // namespace xb
