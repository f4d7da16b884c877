// Header-only C++ shim over the C-ABI of libxinfer_b200.so that restores the reference's own names,
// so that its callers (forward_layer, forward_lm_head, forward_verify, the engine's speculative loop)
// compile against this library with one change: `sycl::queue&` becomes `cudaStream_t`.
//
//   xinfer::ops::linear_int4 / linear_int4_fused / mlp_gate_up_swiglu_int4     src/ops/linear.h:30-139
//   xinfer::ops::argmax / argmax_scratch_size / speculative_accept_reject      src/ops/sampling.h:11-49
//   xinfer::core::DeviceArena                                                  src/core/arena.h:14-66
//
// Error behaviour follows the reference: invalid shapes are silent no-ops, allocation failures throw
// std::bad_alloc, bad arguments std::invalid_argument, broken accounting std::logic_error; anything
// else from the device becomes std::runtime_error.  `half` below is any 2-byte IEEE fp16 type
// (`__half`, `_Float16`); the shim only passes pointers through.
#pragma once

#include <cstddef>
#include <cstdint>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "xinfer_b200.h"

namespace xinfer {

namespace detail {
inline void check(int rc, const char* what) {
    if (rc >= 0) return;
    switch (rc) {
        case XINFER_ERR_OUT_OF_MEMORY: throw std::bad_alloc();
        case XINFER_ERR_INVALID_ARGUMENT: throw std::invalid_argument(what);
        case XINFER_ERR_CONTRACT: throw std::logic_error(std::string(what) + ": fail-loud contract violated");
        default: throw std::runtime_error(std::string(what) + ": " + xinfer_last_cuda_error());
    }
}
}  // namespace detail

namespace ops {

using stream_t = xinfer_stream_t;  // cudaStream_t

template <typename Half>
inline void linear_int4(stream_t q, Half* Y, const Half* X, const uint8_t* W_int4, const Half* scales,
                        const float* bias, int64_t M, int64_t N, int64_t K, int group_size = 128) {
    static_assert(sizeof(Half) == 2, "fp16 storage type expected");
    detail::check(xinfer_linear_int4_f16f16(q, Y, X, W_int4, scales, bias, M, N, K, group_size), "linear_int4");
}
template <typename Half>
inline void linear_int4(stream_t q, float* Y, const Half* X, const uint8_t* W_int4, const Half* scales,
                        const float* bias, int64_t M, int64_t N, int64_t K, int group_size = 128) {
    static_assert(sizeof(Half) == 2, "fp16 storage type expected");
    detail::check(xinfer_linear_int4_f16f32(q, Y, X, W_int4, scales, bias, M, N, K, group_size), "linear_int4");
}
template <typename Half>
inline void linear_int4(stream_t q, float* Y, const float* X, const uint8_t* W_int4, const Half* scales,
                        const float* bias, int64_t M, int64_t N, int64_t K, int group_size = 128) {
    detail::check(xinfer_linear_int4_f32f32(q, Y, X, W_int4, scales, bias, M, N, K, group_size), "linear_int4");
}

// FusedProjectionDesc / FusedProjectionDescFP32 (src/ops/linear.h:66-81) share one POD here.
using FusedProjectionDesc = xinfer_fused_desc;
using FusedProjectionDescFP32 = xinfer_fused_desc;

template <typename Half>
inline void linear_int4_fused(stream_t q, const Half* X, const FusedProjectionDesc* descs, int num_descs, int64_t M,
                              int64_t K, int group_size = 128) {
    static_assert(sizeof(Half) == 2, "fp16 storage type expected");
    detail::check(xinfer_linear_int4_fused_f16(q, X, descs, num_descs, M, K, group_size), "linear_int4_fused");
}
inline void linear_int4_fused(stream_t q, const float* X, const FusedProjectionDescFP32* descs, int num_descs,
                              int64_t M, int64_t K, int group_size = 128) {
    detail::check(xinfer_linear_int4_fused_f32(q, X, descs, num_descs, M, K, group_size), "linear_int4_fused");
}

template <typename Half>
inline void mlp_gate_up_swiglu_int4(stream_t q, Half* Y_swiglu, const Half* X, const uint8_t* W_gate,
                                    const Half* scales_gate, const uint8_t* W_up, const Half* scales_up, int64_t M,
                                    int64_t N, int64_t K, int group_size = 128) {
    static_assert(sizeof(Half) == 2, "fp16 storage type expected");
    detail::check(xinfer_mlp_gate_up_swiglu_int4_f16(q, Y_swiglu, X, W_gate, scales_gate, W_up, scales_up, M, N, K,
                                                     group_size), "mlp_gate_up_swiglu_int4");
}
template <typename Half>
inline void mlp_gate_up_swiglu_int4(stream_t q, float* Y_swiglu, const float* X, const uint8_t* W_gate,
                                    const Half* scales_gate, const uint8_t* W_up, const Half* scales_up, int64_t M,
                                    int64_t N, int64_t K, int group_size = 128) {
    detail::check(xinfer_mlp_gate_up_swiglu_int4_f32(q, Y_swiglu, X, W_gate, scales_gate, W_up, scales_up, M, N, K,
                                                     group_size), "mlp_gate_up_swiglu_int4");
}

inline size_t argmax_scratch_size(int64_t vocab_size) { return xinfer_argmax_scratch_size(vocab_size); }

inline int64_t argmax(stream_t q, const float* logits, int64_t vocab_size, float* partial_max = nullptr,
                      int64_t* partial_idx = nullptr) {
    const int64_t r = xinfer_argmax(q, logits, vocab_size, partial_max, partial_idx);
    if (r < 0) throw std::runtime_error(std::string("argmax: ") + xinfer_last_cuda_error());
    return r;
}

struct SpeculativeAcceptanceResult {  // src/ops/sampling.h:27-36
    std::vector<int64_t> accepted_tokens;
    int64_t bonus_or_resampled_token{-1};
    bool has_rejected_token{false};
    int64_t rejected_token{-1};
    size_t num_accepted{0};
    size_t num_rejected{0};
    size_t num_resampled{0};
    size_t num_remaining{0};
};

inline SpeculativeAcceptanceResult speculative_accept_reject(stream_t q, const int64_t* draft_tokens,
                                                             size_t num_draft_tokens, const float* target_logits,
                                                             int64_t vocab_size, const float* draft_probs = nullptr,
                                                             const float* rand_uniform = nullptr) {
    xinfer_accept_result r;
    detail::check(xinfer_speculative_accept_reject(q, draft_tokens, num_draft_tokens, target_logits, vocab_size,
                                                   draft_probs, rand_uniform, &r), "speculative_accept_reject");
    SpeculativeAcceptanceResult out;
    out.accepted_tokens.assign(r.accepted_tokens, r.accepted_tokens + r.num_accepted);
    out.bonus_or_resampled_token = r.bonus_or_resampled_token;
    out.has_rejected_token = r.has_rejected_token != 0;
    out.rejected_token = r.rejected_token;
    out.num_accepted = static_cast<size_t>(r.num_accepted);
    out.num_rejected = static_cast<size_t>(r.num_rejected);
    out.num_resampled = static_cast<size_t>(r.num_resampled);
    out.num_remaining = static_cast<size_t>(r.num_remaining);
    return out;
}

}  // namespace ops

namespace core {

class DeviceArena {  // src/core/arena.h:14-66
public:
    static constexpr size_t DEFAULT_ALIGNMENT = 64;

    explicit DeviceArena(size_t capacity_bytes, size_t default_alignment = DEFAULT_ALIGNMENT) {
        detail::check(xinfer_arena_create(capacity_bytes, default_alignment, &a_), "DeviceArena");
    }
    ~DeviceArena() { xinfer_arena_destroy(a_); }
    DeviceArena(const DeviceArena&) = delete;
    DeviceArena& operator=(const DeviceArena&) = delete;
    DeviceArena(DeviceArena&& o) noexcept : a_(o.a_) { o.a_ = nullptr; }
    DeviceArena& operator=(DeviceArena&& o) noexcept {
        if (this != &o) { xinfer_arena_destroy(a_); a_ = o.a_; o.a_ = nullptr; }
        return *this;
    }

    void* allocate(size_t bytes, size_t alignment = 0) {
        void* p = nullptr;
        detail::check(xinfer_arena_allocate(a_, bytes, alignment, &p), "DeviceArena::allocate");
        return p;
    }
    void* allocate_persistent(size_t bytes, size_t alignment = 0) {
        void* p = nullptr;
        detail::check(xinfer_arena_allocate_persistent(a_, bytes, alignment, &p), "DeviceArena::allocate_persistent");
        return p;
    }
    void* persistent_buffer(size_t bytes = 0, size_t alignment = 0) {
        void* p = nullptr;
        detail::check(xinfer_arena_persistent_buffer(a_, bytes, alignment, &p), "DeviceArena::persistent_buffer");
        return p;
    }
    void reset() noexcept { xinfer_arena_reset(a_); }
    size_t capacity() const noexcept { return xinfer_arena_capacity(a_); }
    size_t allocated_bytes() const noexcept { return xinfer_arena_allocated_bytes(a_); }
    size_t remaining_bytes() const noexcept { return xinfer_arena_remaining_bytes(a_); }
    size_t peak_allocated_bytes() const noexcept { return xinfer_arena_peak_allocated_bytes(a_); }
    void* base_ptr() noexcept { return xinfer_arena_base_ptr(a_); }

private:
    xinfer_arena* a_{nullptr};
};

}  // namespace core
}  // namespace xinfer
