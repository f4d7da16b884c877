// C-ABI layer: argument checks, per-device scratch, dispatch between the tcgen05 and CUDA-core
// kernels, and the synchronous host-facing forms of argmax / speculative_accept_reject.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <new>
#include <string>

#include "../../include/xinfer_b200.h"
#include "sampling.h"
#include "tp_host.h"
#include "w4a16.h"

namespace {

constexpr int kMaxDevices = 64;
constexpr int kCounterCapacity = 8192;
constexpr size_t kSamplingScratchBytes = 4u << 20;  // rows * chunks * 16 B
constexpr size_t kGemmPartialBytes = 96u << 20;     // K-split partials of the prefill GEMM
constexpr int64_t kSliceRowsMax = 128;             // up to here M > 32 runs as 32-row slices of the decode kernel

struct DeviceCtx {
    bool ready = false;
    int num_sms = 0;
    float* workspace = nullptr;   // split-K partials
    int* counters = nullptr;      // tile arrival counters, zero between launches
    int* status = nullptr;        // device status word
    void* sampling = nullptr;     // (row, chunk) partials
    long long* small_dev = nullptr;   // staging for the synchronous sampling calls
    long long* small_host = nullptr;  // pinned
    int forced_path = 0;              // xinfer_set_linear_path, per device
    float* gemm_partials = nullptr;   // fp32 partial sums of the prefill GEMM's K splits (taken at its first use)
    bool gemm_partials_tried = false;
};

DeviceCtx g_ctx[kMaxDevices];
std::mutex g_mutex;
thread_local std::string g_last_error;
thread_local int g_last_path = 0;

constexpr size_t kSmallBytes = 64 * 1024;

int fail_cuda(cudaError_t e) {
    g_last_error = cudaGetErrorString(e);
    return XINFER_ERR_CUDA;
}

int get_ctx(DeviceCtx** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { fail_cuda(e); return XINFER_ERR_NO_DEVICE; }
    if (dev < 0 || dev >= kMaxDevices) return XINFER_ERR_INVALID_ARGUMENT;
    DeviceCtx& c = g_ctx[dev];
    if (!c.ready) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!c.ready) {
            cudaDeviceProp prop;
            if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) { fail_cuda(e); return XINFER_ERR_NO_DEVICE; }
            if (prop.major != 10) {
                g_last_error = "libxinfer_b200 carries sm_100a code only; this device is not a B200-class GPU";
                return XINFER_ERR_NO_DEVICE;
            }
            c.num_sms = prop.multiProcessorCount;
            const size_t ws = xb::tc_workspace_bytes(c.num_sms);
            if ((e = cudaMalloc(&c.workspace, ws)) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMalloc(&c.counters, kCounterCapacity * sizeof(int))) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMalloc(&c.status, sizeof(int))) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMalloc(&c.sampling, kSamplingScratchBytes)) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMalloc(&c.small_dev, kSmallBytes)) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMallocHost(&c.small_host, kSmallBytes)) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMemset(c.counters, 0, kCounterCapacity * sizeof(int))) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaMemset(c.status, 0, sizeof(int))) != cudaSuccess) return fail_cuda(e);
            if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail_cuda(e);
            c.ready = true;
        }
    }
    *out = &c;
    return XINFER_OK;
}

int run_linear(xinfer_stream_t s, const void* x, xb::ActType in, bool out_f32, const xb::TcProj* proj, int num,
               bool swiglu, int64_t m, int64_t k, int group_size) {
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(s);
    if (c->forced_path != 2 && c->forced_path != 3 && in == xb::ActType::F16 && m > 32 && m <= kSliceRowsMax &&
        xb::tc_eligible(x, proj, num, swiglu, 32, k, group_size)) {
        // 33 .. 128 rows: slices of 32 rows through the decode kernel (the reference's association, and cheaper than a
        // 256-row GEMM tile that would be mostly padding: gate-sized projection 18 us per slice against 88 us)
        const int cnt = swiglu ? 2 : num;
        const size_t ybytes = out_f32 ? 4 : 2;
        for (int64_t r0 = 0; r0 < m; r0 += 32) {
            xb::TcProj sl[4];
            for (int i = 0; i < cnt; ++i) {
                sl[i] = proj[i];
                const int64_t ld = proj[i].ldy > 0 ? proj[i].ldy : proj[i].n;
                if (sl[i].y) sl[i].y = static_cast<char*>(sl[i].y) + static_cast<size_t>(r0) * ld * ybytes;
            }
            const int64_t rows = m - r0 < 32 ? m - r0 : 32;
            const int r = xb::tc_launch(stream, static_cast<const char*>(x) + static_cast<size_t>(r0) * k * 2, sl, num, swiglu, out_f32,
                                        rows, k, c->num_sms, c->workspace, c->counters, kCounterCapacity, c->status);
            if (r == -1) return fail_cuda(cudaGetLastError());
            if (r != 0) return XINFER_ERR_INVALID_ARGUMENT;
        }
        g_last_path = 1;
        return XINFER_OK;
    }
    if (c->forced_path != 2 && in == xb::ActType::F16 && xb::gemm_eligible(x, proj, num, swiglu, m, k, group_size)) {
        // more than 32 rows (prefill chunks): the compute-bound tcgen05 GEMM
        // scratch for K splits of the GEMM: taken once per device, outside any stream capture (a failed or refused
        // allocation just means no K split)
        if (!c->gemm_partials && !c->gemm_partials_tried) {
            c->gemm_partials_tried = true;
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) {
                void* ptr = nullptr;
                if (cudaMalloc(&ptr, kGemmPartialBytes) == cudaSuccess) c->gemm_partials = static_cast<float*>(ptr);
                else cudaGetLastError();
            } else {
                c->gemm_partials_tried = false;  // try again on a call that is not being captured
            }
        }
        const int r = xb::gemm_launch(stream, x, proj, num, swiglu, out_f32, m, k, c->status, xb::tc_wait_limit(), xb::tc_x_stage_limit(), c->num_sms,
                                      c->gemm_partials, c->gemm_partials ? kGemmPartialBytes : 0);
        if (r == 0) { g_last_path = 3; return XINFER_OK; }
        if (r == -1) return fail_cuda(cudaGetLastError());
    }
    const bool want_tc = (c->forced_path != 2) && in == xb::ActType::F16 &&
                         xb::tc_eligible(x, proj, num, swiglu, m, k, group_size);
    if (want_tc) {
        int r = xb::tc_launch(stream, x, proj, num, swiglu, out_f32, m, k, c->num_sms, c->workspace, c->counters,
                              kCounterCapacity, c->status);
        if (r == 0) { g_last_path = 1; return XINFER_OK; }
        if (r == -1) return fail_cuda(cudaGetLastError());
        // r < -1: the problem could not be described to the tensor-core kernel; use CUDA cores
    }
    int r = xb::simt_launch(stream, x, in, out_f32, proj, num, swiglu, m, k, group_size);
    if (r != 0) return fail_cuda(cudaGetLastError());
    g_last_path = 2;
    return XINFER_OK;
}

int linear_one(xinfer_stream_t s, void* y, int64_t ldy, const void* x, xb::ActType in, bool out_f32, const uint8_t* w,
               const void* scales, const float* bias, int64_t m, int64_t n, int64_t k, int group_size) {
    if (m <= 0 || n <= 0 || k <= 0) return XINFER_NOOP_INVALID_SHAPE;  // src/ops/linear.cpp:176
    if (!y || !x || !w || !scales || group_size <= 0) return XINFER_ERR_INVALID_ARGUMENT;
    if (k / group_size <= 0) return XINFER_NOOP_INVALID_SHAPE;
    xb::TcProj p{y, w, scales, bias, n, ldy};
    return run_linear(s, x, in, out_f32, &p, 1, false, m, k, group_size);
}

int fused(xinfer_stream_t s, const void* x, xb::ActType in, const xinfer_fused_desc* d, int num, int64_t m, int64_t k,
          int group_size) {
    if (m <= 0 || k <= 0 || num <= 0 || !d || num > 4) return XINFER_NOOP_INVALID_SHAPE;  // src/ops/linear.cpp:359
    if (!x || group_size <= 0 || k / group_size <= 0) return XINFER_ERR_INVALID_ARGUMENT;
    xb::TcProj p[4];
    for (int i = 0; i < num; ++i) {
        if (!d[i].Y || !d[i].W_int4 || !d[i].scales || d[i].N <= 0) return XINFER_ERR_INVALID_ARGUMENT;
        p[i] = xb::TcProj{d[i].Y, d[i].W_int4, d[i].scales, d[i].bias, d[i].N, 0};
    }
    return run_linear(s, x, in, in == xb::ActType::F32, p, num, false, m, k, group_size);
}

int swiglu(xinfer_stream_t s, void* y, const void* x, xb::ActType in, const uint8_t* wg, const void* sg,
           const uint8_t* wu, const void* su, int64_t m, int64_t n, int64_t k, int group_size) {
    if (m <= 0 || n <= 0 || k <= 0) return XINFER_NOOP_INVALID_SHAPE;  // src/ops/linear.cpp:512
    if (!y || !x || !wg || !sg || !wu || !su || group_size <= 0 || k / group_size <= 0) return XINFER_ERR_INVALID_ARGUMENT;
    xb::TcProj p[2] = {xb::TcProj{y, wg, sg, nullptr, n, 0}, xb::TcProj{nullptr, wu, su, nullptr, n, 0}};
    return run_linear(s, x, in, in == xb::ActType::F32, p, 2, true, m, k, group_size);
}

const uint64_t* crc_table() {
    static uint64_t table[256];
    static bool built = [] {
        for (uint64_t b = 0; b < 256; ++b) {
            uint64_t c = b;
            for (int i = 0; i < 8; ++i) c = (c & 1) ? (c >> 1) ^ 0xC96C5795D7870F42ull : (c >> 1);
            table[b] = c;
        }
        return true;
    }();
    (void)built;
    return table;
}

uint64_t crc_update(uint64_t crc, const void* data, size_t n) {
    const uint64_t* t = crc_table();
    const uint8_t* p = static_cast<const uint8_t*>(data);
    for (size_t i = 0; i < n; ++i) crc = (crc >> 8) ^ t[static_cast<uint8_t>(crc ^ p[i])];
    return crc;
}

}  // namespace

namespace xb {
void set_last_error(const char* msg) { g_last_error = msg ? msg : ""; }

int run_tc_linear(cudaStream_t s, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32, long long m,
                  long long k, int group_size, const TpLink* tp, int layout_flags) {
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    if (!tc_eligible(x, proj, num, swiglu, m, k, group_size)) return XINFER_ERR_INVALID_ARGUMENT;
    const int r = tc_launch(s, x, proj, num, swiglu, out_f32, m, k, c->num_sms, c->workspace, c->counters,
                            kCounterCapacity, c->status, tp, layout_flags);
    if (r == 0) { g_last_path = 1; return XINFER_OK; }
    if (r == -1) return fail_cuda(cudaGetLastError());
    return XINFER_ERR_INVALID_ARGUMENT;
}
}  // namespace xb

extern "C" {

int xinfer_b200_init(int device) {
    int cur = 0;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) { fail_cuda(e); return XINFER_ERR_NO_DEVICE; }
    if ((e = cudaSetDevice(device)) != cudaSuccess) return fail_cuda(e);
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    cudaSetDevice(cur);
    return rc;
}

int xinfer_b200_init_current(void) {
    DeviceCtx* c = nullptr;
    return get_ctx(&c);
}

int xinfer_device_status(int device) {
    if (device < 0 || device >= kMaxDevices) return 0;
    int cur = 0, v = 0;
    cudaGetDevice(&cur);
    cudaSetDevice(device);
    cudaError_t e = cudaSuccess;
    if (g_ctx[device].ready) {
        e = cudaMemcpy(&v, g_ctx[device].status, sizeof(int), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess && v != 0) cudaMemset(g_ctx[device].status, 0, sizeof(int));
    }
    // the allocation-free entry point keeps its own status word (in its in-library array)
    const int v2 = xb::tc_noalloc_take_status(device);
    cudaSetDevice(cur);
    if (e != cudaSuccess) return fail_cuda(e);
    if (v2 < 0) return fail_cuda(cudaGetLastError());
    return (v == 0 && v2 == 0) ? 0 : XINFER_ERR_DEVICE_TIMEOUT;
}

const char* xinfer_last_cuda_error(void) { return g_last_error.c_str(); }
const char* xinfer_b200_version(void) { return "xinfer_b200 0.1 (sm_100a)"; }
int xinfer_last_linear_path(void) { return g_last_path; }
void xinfer_debug_set_wait_hooks(int64_t limit_clocks, int withhold_x_from_stage) {
    xb::tc_set_wait_hooks(limit_clocks, withhold_x_from_stage);
}

void xinfer_linear_plan_record_begin(void) { xb::tc_plan_record_begin(); }
void xinfer_linear_plan_record_end(void) { xb::tc_plan_record_end(); }
void xinfer_linear_plan_rewind(void) { xb::tc_plan_rewind(); }
void xinfer_linear_plan_clear(void) { xb::tc_plan_clear(); }
void xinfer_set_linear_path(int path) {
    DeviceCtx* c = nullptr;
    if (get_ctx(&c) == XINFER_OK) c->forced_path = path;
}

int xinfer_linear_int4_f16f16(xinfer_stream_t s, void* Y, const void* X, const uint8_t* W, const void* scales,
                              const float* bias, int64_t M, int64_t N, int64_t K, int group_size) {
    return linear_one(s, Y, 0, X, xb::ActType::F16, false, W, scales, bias, M, N, K, group_size);
}
int xinfer_linear_int4_f16f32(xinfer_stream_t s, float* Y, const void* X, const uint8_t* W, const void* scales,
                              const float* bias, int64_t M, int64_t N, int64_t K, int group_size) {
    return linear_one(s, Y, 0, X, xb::ActType::F16, true, W, scales, bias, M, N, K, group_size);
}
int xinfer_linear_int4_f32f32(xinfer_stream_t s, float* Y, const float* X, const uint8_t* W, const void* scales,
                              const float* bias, int64_t M, int64_t N, int64_t K, int group_size) {
    return linear_one(s, Y, 0, X, xb::ActType::F32, true, W, scales, bias, M, N, K, group_size);
}
int xinfer_linear_int4_f16f16_ld(xinfer_stream_t s, void* Y, int64_t ldy, const void* X, const uint8_t* W,
                                 const void* scales, const float* bias, int64_t M, int64_t N, int64_t K,
                                 int group_size) {
    if (ldy < N) return XINFER_ERR_INVALID_ARGUMENT;
    return linear_one(s, Y, ldy, X, xb::ActType::F16, false, W, scales, bias, M, N, K, group_size);
}
int xinfer_linear_int4_fused_f16(xinfer_stream_t s, const void* X, const xinfer_fused_desc* descs, int num_descs,
                                 int64_t M, int64_t K, int group_size) {
    return fused(s, X, xb::ActType::F16, descs, num_descs, M, K, group_size);
}
int xinfer_linear_int4_fused_f32(xinfer_stream_t s, const float* X, const xinfer_fused_desc* descs, int num_descs,
                                 int64_t M, int64_t K, int group_size) {
    return fused(s, X, xb::ActType::F32, descs, num_descs, M, K, group_size);
}
int xinfer_mlp_gate_up_swiglu_int4_f16(xinfer_stream_t s, void* Y, const void* X, const uint8_t* Wg, const void* sg,
                                       const uint8_t* Wu, const void* su, int64_t M, int64_t N, int64_t K,
                                       int group_size) {
    return swiglu(s, Y, X, xb::ActType::F16, Wg, sg, Wu, su, M, N, K, group_size);
}
int xinfer_mlp_gate_up_swiglu_int4_f32(xinfer_stream_t s, float* Y, const float* X, const uint8_t* Wg, const void* sg,
                                       const uint8_t* Wu, const void* su, int64_t M, int64_t N, int64_t K,
                                       int group_size) {
    return swiglu(s, Y, X, xb::ActType::F32, Wg, sg, Wu, su, M, N, K, group_size);
}

size_t xinfer_argmax_scratch_size(int64_t vocab_size) {
    if (vocab_size <= 0) return 0;
    return (static_cast<size_t>(vocab_size) + 255) / 256;
}

int xinfer_argmax_rows(xinfer_stream_t s, const float* logits, int64_t row_stride, int64_t rows, int64_t vocab,
                       int64_t* out_dev) {
    if (rows <= 0 || vocab <= 0) return XINFER_NOOP_INVALID_SHAPE;
    if (!logits || !out_dev) return XINFER_ERR_INVALID_ARGUMENT;
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    if (xb::sampling_scratch_bytes(rows, vocab) > kSamplingScratchBytes) return XINFER_ERR_INVALID_ARGUMENT;
    if (xb::argmax_rows(static_cast<cudaStream_t>(s), logits, row_stride, static_cast<int>(rows), vocab, c->sampling,
                        reinterpret_cast<long long*>(out_dev), nullptr, nullptr) != 0)
        return fail_cuda(cudaGetLastError());
    return XINFER_OK;
}

int64_t xinfer_argmax(xinfer_stream_t s, const float* logits, int64_t vocab, float* partial_max, int64_t* partial_idx) {
    if (vocab <= 0 || !logits) return 0;  // src/ops/sampling.cpp:17
    if (vocab == 1) return 0;             // src/ops/sampling.cpp:18
    DeviceCtx* c = nullptr;
    if (get_ctx(&c) != XINFER_OK) return -1;
    if (xb::sampling_scratch_bytes(1, vocab) > kSamplingScratchBytes) return -1;
    cudaStream_t stream = static_cast<cudaStream_t>(s);
    if (xb::argmax_rows(stream, logits, vocab, 1, vocab, c->sampling, c->small_dev, partial_max,
                        reinterpret_cast<long long*>(partial_idx)) != 0) {
        fail_cuda(cudaGetLastError());
        return -1;
    }
    cudaError_t e = cudaMemcpyAsync(c->small_host, c->small_dev, sizeof(long long), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { fail_cuda(e); return -1; }
    return c->small_host[0];
}

int xinfer_speculative_accept_reject_batched(xinfer_stream_t s, const int64_t* draft_tokens, const float* logits,
                                             int64_t row_stride, int64_t vocab, const float* draft_probs,
                                             const float* uniforms, float inv_temperature, int batch, int num_draft,
                                             int rows_per_seq, int bonus_row, xinfer_accept_record* out_dev) {
    if (batch <= 0 || num_draft <= 0 || vocab <= 0) return XINFER_NOOP_INVALID_SHAPE;
    if (!draft_tokens || !logits || !out_dev || rows_per_seq < num_draft || bonus_row < 0 || bonus_row >= rows_per_seq ||
        !(inv_temperature > 0.f) || row_stride < vocab)
        return XINFER_ERR_INVALID_ARGUMENT;
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    if (xb::sampling_scratch_bytes(static_cast<long long>(batch) * rows_per_seq, vocab) > kSamplingScratchBytes)
        return XINFER_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(xinfer_accept_record) == sizeof(xb::AcceptOut), "record layout");
    if (xb::accept_reject_batched(static_cast<cudaStream_t>(s), logits, row_stride, vocab, inv_temperature,
                                  reinterpret_cast<const long long*>(draft_tokens), draft_probs, uniforms, batch,
                                  num_draft, rows_per_seq, bonus_row, c->sampling,
                                  reinterpret_cast<xb::AcceptOut*>(out_dev)) != 0)
        return fail_cuda(cudaGetLastError());
    return XINFER_OK;
}

int xinfer_sample_tokens(xinfer_stream_t s, const float* logits, int64_t row_stride, int64_t vocab, int rows,
                         float inv_temperature, const float* uniforms, int64_t* tokens_out, float* probs_out) {
    if (rows <= 0 || vocab <= 0) return XINFER_NOOP_INVALID_SHAPE;
    if (!logits || !uniforms || !tokens_out || !probs_out || !(inv_temperature > 0.f) || row_stride < vocab)
        return XINFER_ERR_INVALID_ARGUMENT;
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    if (xb::sampling_scratch_bytes(rows, vocab) > kSamplingScratchBytes) return XINFER_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(s);
    if (xb::sampling_partials(st, logits, row_stride, rows, vocab, inv_temperature, true, 0, c->sampling) != 0 ||
        xb::sample_finish(st, c->sampling, xb::sampling_chunks(vocab), logits, row_stride, vocab, inv_temperature, uniforms, 1,
                          rows, reinterpret_cast<long long*>(tokens_out), probs_out, 1) != 0)
        return fail_cuda(cudaGetLastError());
    return XINFER_OK;
}

int xinfer_sample_tokens_top_p(xinfer_stream_t s, const float* logits, int64_t row_stride, int64_t vocab, int rows,
                               float inv_temperature, float top_p, const float* uniforms, int64_t* tokens_out,
                               float* probs_out) {
    if (rows <= 0 || vocab <= 0) return XINFER_NOOP_INVALID_SHAPE;
    if (!logits || !uniforms || !tokens_out || !probs_out || !(inv_temperature > 0.f) || row_stride < vocab ||
        !(top_p > 0.f) || top_p > 1.f)
        return XINFER_ERR_INVALID_ARGUMENT;
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    if (xb::nucleus_rows(static_cast<cudaStream_t>(s), logits, row_stride, rows, vocab, inv_temperature, top_p, uniforms, 1,
                         nullptr, reinterpret_cast<long long*>(tokens_out), probs_out, 1) != 0)
        return fail_cuda(cudaGetLastError());
    return XINFER_OK;
}

int xinfer_speculative_accept_reject(xinfer_stream_t s, const int64_t* draft_tokens, size_t n, const float* logits,
                                     int64_t vocab, const float* draft_probs, const float* rand_uniform,
                                     xinfer_accept_result* out) {
    if (!out) return XINFER_ERR_INVALID_ARGUMENT;
    memset(out, 0, sizeof(*out));
    out->bonus_or_resampled_token = -1;
    out->rejected_token = -1;
    if (n == 0 || !draft_tokens || !logits || vocab <= 0) return XINFER_OK;  // default struct, sampling.cpp:102-104
    if (n > XINFER_MAX_DRAFT_TOKENS) return XINFER_ERR_INVALID_ARGUMENT;
    DeviceCtx* c = nullptr;
    int rc = get_ctx(&c);
    if (rc != XINFER_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(s);
    // staging layout in the pinned / device small buffers (8-byte words):
    //   [0, n) tokens | [n, 2n) probs (floats, first half of the words) | [2n, 3n) uniforms | record after
    long long* h = c->small_host;
    memcpy(h, draft_tokens, n * sizeof(int64_t));
    float* h_probs = reinterpret_cast<float*>(h + n);
    float* h_unif = reinterpret_cast<float*>(h + 2 * n);
    if (draft_probs) memcpy(h_probs, draft_probs, n * sizeof(float));
    if (draft_probs) {
        if (rand_uniform) memcpy(h_unif, rand_uniform, n * sizeof(float));
        else memset(h_unif, 0, n * sizeof(float));  // missing uniforms mean r = 0, sampling.cpp:130
    }
    cudaError_t e = cudaMemcpyAsync(c->small_dev, h, 3 * n * sizeof(long long), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail_cuda(e);
    long long* d = c->small_dev;
    xinfer_accept_record* d_rec = reinterpret_cast<xinfer_accept_record*>(d + 3 * n);
    rc = xinfer_speculative_accept_reject_batched(
        s, reinterpret_cast<const int64_t*>(d), logits, vocab, vocab,
        draft_probs ? reinterpret_cast<const float*>(d + n) : nullptr,
        draft_probs ? reinterpret_cast<const float*>(d + 2 * n) : nullptr, 1.0f, 1, static_cast<int>(n),
        static_cast<int>(n), static_cast<int>(n) - 1, d_rec);
    if (rc != XINFER_OK) return rc;
    xinfer_accept_record* h_rec = reinterpret_cast<xinfer_accept_record*>(h + 3 * n);
    e = cudaMemcpyAsync(h_rec, d_rec, sizeof(*h_rec), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail_cuda(e);
    out->bonus_or_resampled_token = h_rec->bonus_or_resampled_token;
    out->rejected_token = h_rec->rejected_token;
    out->num_accepted = h_rec->num_accepted;
    out->num_rejected = h_rec->num_rejected;
    out->num_resampled = h_rec->num_resampled;
    out->num_remaining = h_rec->num_remaining;
    out->has_rejected_token = h_rec->has_rejected_token;
    for (int64_t i = 0; i < out->num_accepted; ++i) out->accepted_tokens[i] = draft_tokens[i];
    // fail-loud accounting, src/ops/sampling.cpp:174-193
    if (out->has_rejected_token) {
        if (out->num_accepted + out->num_rejected + out->num_remaining != static_cast<int64_t>(n)) return XINFER_ERR_CONTRACT;
    } else if (out->num_accepted != static_cast<int64_t>(n)) {
        return XINFER_ERR_CONTRACT;
    }
    return XINFER_OK;
}

int xinfer_philox_uniform(xinfer_stream_t s, float* out_dev, int64_t n, uint64_t seed, uint64_t subsequence) {
    if (n <= 0) return XINFER_NOOP_INVALID_SHAPE;
    if (!out_dev) return XINFER_ERR_INVALID_ARGUMENT;
    if (xb::philox_uniform(static_cast<cudaStream_t>(s), out_dev, n, seed, subsequence) != 0)
        return fail_cuda(cudaGetLastError());
    return XINFER_OK;
}

int xinfer_copy_device_to_host(void* dst_host, const void* src_dev, size_t bytes) {
    if (bytes == 0) return XINFER_OK;
    if (!dst_host || !src_dev) return XINFER_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaMemcpy(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? XINFER_OK : fail_cuda(e);
}
int xinfer_copy_host_to_device(void* dst_dev, const void* src_host, size_t bytes) {
    if (bytes == 0) return XINFER_OK;
    if (!dst_dev || !src_host) return XINFER_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaMemcpy(dst_dev, src_host, bytes, cudaMemcpyHostToDevice);
    return e == cudaSuccess ? XINFER_OK : fail_cuda(e);
}

// ------------------------------------------------------------------------------------ checksum
uint64_t xinfer_crc64(const void* data, size_t length) {
    if (!data || length == 0) return 0ull;
    return ~crc_update(~0ull, data, length);
}

uint64_t xinfer_crc64_update(uint64_t state, const void* data, size_t length) {
    if (!data || length == 0) return state;
    return crc_update(state, data, length);
}

uint64_t xinfer_crc64_file(const char* filepath, uint64_t max_bytes) {
    if (!filepath) return 0ull;
    FILE* f = fopen(filepath, "rb");
    if (!f) return 0ull;
    uint64_t crc = ~0ull;
    uint64_t left = max_bytes > 0 ? max_bytes : ~0ull;
    const size_t kBuf = 4u << 20;
    unsigned char* buf = new (std::nothrow) unsigned char[kBuf];
    if (!buf) { fclose(f); return 0ull; }
    while (left > 0) {
        const size_t want = static_cast<size_t>(left < kBuf ? left : kBuf);
        const size_t got = fread(buf, 1, want, f);
        if (got == 0) break;
        crc = crc_update(crc, buf, got);
        left -= got;
    }
    delete[] buf;
    fclose(f);
    return ~crc;
}

}  // extern "C"
