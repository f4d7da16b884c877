// Header-only C++ shim over the C-ABI of libxinfer_b200.so that restores the reference's own names,
// so that its callers (forward_layer, forward_lm_head, forward_verify, the engine's speculative loop)
// compile against this library with one change: `sycl::queue&` becomes `cudaStream_t`.
//
//   xinfer::ops::linear_int4 / linear_int4_fused / mlp_gate_up_swiglu_int4     src/ops/linear.h:30-139
//   xinfer::ops::argmax / argmax_scratch_size / speculative_accept_reject      src/ops/sampling.h:11-49
//   xinfer::core::DeviceArena                                                  src/core/arena.h:14-66
//   xinfer::core::DeviceContext (allocation, copies, the queue)                src/core/device.h:26-72
//   xinfer::core::DataType / TensorShape / TensorView (what allocate_tensor needs)   src/core/types.h, tensor.h
//
// Error behaviour follows the reference: invalid shapes are silent no-ops, allocation failures throw
// std::bad_alloc, bad arguments std::invalid_argument, broken accounting std::logic_error; anything
// else from the device becomes std::runtime_error.  `half` below is any 2-byte IEEE fp16 type
// (`__half`, `_Float16`); the shim only passes pointers through.
#pragma once

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <memory>
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

enum class DataType : uint32_t {  // src/core/types.h:10-18
    Float32 = 0x0001, Float16 = 0x0002, BFloat16 = 0x0003, Int32 = 0x0004, Int8 = 0x0005, Uint8 = 0x0006, Int4 = 0x0007,
};

inline size_t compute_tensor_bytes(int64_t num_elements, DataType dtype) noexcept {  // src/core/types.h:54-60
    if (num_elements <= 0) return 0;
    switch (dtype) {
        case DataType::Int4: return static_cast<size_t>((num_elements + 1) / 2);
        case DataType::Float32: case DataType::Int32: return static_cast<size_t>(num_elements) * 4;
        case DataType::Float16: case DataType::BFloat16: return static_cast<size_t>(num_elements) * 2;
        default: return static_cast<size_t>(num_elements);
    }
}

class TensorShape {  // src/core/tensor.h:15-70 (the parts allocate_tensor and its callers use)
public:
    TensorShape() = default;
    TensorShape(std::initializer_list<int64_t> dims) : dims_(dims) {}
    explicit TensorShape(std::vector<int64_t> dims) : dims_(std::move(dims)) {}
    size_t ndim() const noexcept { return dims_.size(); }
    int64_t dim(size_t i) const {
        if (i >= dims_.size()) throw std::out_of_range("Tensor dimension index out of range");
        return dims_[i];
    }
    int64_t operator[](size_t i) const noexcept { return dims_[i]; }
    int64_t numel() const noexcept {
        if (dims_.empty()) return 0;
        int64_t n = 1;
        for (int64_t d : dims_) n *= d;
        return n;
    }
    const std::vector<int64_t>& dims() const noexcept { return dims_; }
    bool operator==(const TensorShape& o) const noexcept { return dims_ == o.dims_; }

private:
    std::vector<int64_t> dims_;
};

class TensorView {  // src/core/tensor.h:72-110: a non-owning typed view of device memory
public:
    TensorView() = default;
    TensorView(void* data, TensorShape shape, DataType dtype) : data_(data), shape_(std::move(shape)), dtype_(dtype) {}
    void* data() noexcept { return data_; }
    const void* data() const noexcept { return data_; }
    template <typename T> T* data_as() noexcept { return static_cast<T*>(data_); }
    const TensorShape& shape() const noexcept { return shape_; }
    DataType dtype() const noexcept { return dtype_; }
    int64_t numel() const noexcept { return shape_.numel(); }
    size_t byte_size() const noexcept { return compute_tensor_bytes(shape_.numel(), dtype_); }

private:
    void* data_{nullptr};
    TensorShape shape_;
    DataType dtype_{DataType::Float32};
};

// The CUDA stand-in for the reference's device context: one stream (its "queue"), device allocation and
// synchronous copies.  Device selection is the caller's (cudaSetDevice before create()).
class DeviceContext {  // src/core/device.h:26-72
public:
    static std::shared_ptr<DeviceContext> create(bool /*prefer_b60*/ = true) {
        return std::shared_ptr<DeviceContext>(new DeviceContext());
    }
    ~DeviceContext() { xinfer_stream_destroy(stream_); }
    DeviceContext(const DeviceContext&) = delete;
    DeviceContext& operator=(const DeviceContext&) = delete;

    xinfer_stream_t queue() noexcept { return stream_; }
    void* allocate_device(size_t bytes, size_t /*alignment*/ = 64) {
        void* p = nullptr;
        detail::check(xinfer_device_alloc(bytes, &p), "DeviceContext::allocate_device");
        return p;
    }
    void free_device(void* p) { xinfer_device_free(p); }
    void copy_host_to_device(void* dst, const void* src, size_t bytes, bool /*blocking*/ = true) {
        detail::check(xinfer_copy_host_to_device(dst, src, bytes), "DeviceContext::copy_host_to_device");
    }
    void copy_device_to_host(void* dst, const void* src, size_t bytes, bool /*blocking*/ = true) {
        synchronize();
        detail::check(xinfer_copy_device_to_host(dst, src, bytes), "DeviceContext::copy_device_to_host");
    }
    void synchronize() { detail::check(xinfer_stream_synchronize(stream_), "DeviceContext::synchronize"); }

private:
    DeviceContext() {
        detail::check(xinfer_b200_init_current(), "DeviceContext");
        detail::check(xinfer_stream_create(&stream_), "DeviceContext");
    }
    xinfer_stream_t stream_{nullptr};
};

class DeviceArena {  // src/core/arena.h:14-66
public:
    static constexpr size_t DEFAULT_ALIGNMENT = 64;

    DeviceArena(std::shared_ptr<DeviceContext> ctx, size_t capacity_bytes, size_t default_alignment = DEFAULT_ALIGNMENT)
        : ctx_(std::move(ctx)) {
        detail::check(xinfer_arena_create(capacity_bytes, default_alignment, &a_), "DeviceArena");
    }
    explicit DeviceArena(size_t capacity_bytes, size_t default_alignment = DEFAULT_ALIGNMENT) {
        detail::check(xinfer_arena_create(capacity_bytes, default_alignment, &a_), "DeviceArena");
    }
    ~DeviceArena() { xinfer_arena_destroy(a_); }
    DeviceArena(const DeviceArena&) = delete;
    DeviceArena& operator=(const DeviceArena&) = delete;
    DeviceArena(DeviceArena&& o) noexcept
        : ctx_(std::move(o.ctx_)), a_(o.a_), persistent_buffer_(o.persistent_buffer_),
          persistent_buffer_capacity_(o.persistent_buffer_capacity_) {
        o.a_ = nullptr;
        o.persistent_buffer_ = nullptr;
        o.persistent_buffer_capacity_ = 0;
    }
    DeviceArena& operator=(DeviceArena&& o) noexcept {
        if (this != &o) {
            xinfer_arena_destroy(a_);
            ctx_ = std::move(o.ctx_);
            a_ = o.a_;
            persistent_buffer_ = o.persistent_buffer_;
            persistent_buffer_capacity_ = o.persistent_buffer_capacity_;
            o.a_ = nullptr;
            o.persistent_buffer_ = nullptr;
            o.persistent_buffer_capacity_ = 0;
        }
        return *this;
    }

    void* allocate(size_t bytes, size_t alignment = 0) {
        void* p = nullptr;
        detail::check(xinfer_arena_allocate(a_, bytes, alignment, &p), "DeviceArena::allocate");
        return p;
    }
    TensorView allocate_tensor(TensorShape shape, DataType dtype, size_t alignment = 0) {
        void* p = allocate(compute_tensor_bytes(shape.numel(), dtype), alignment);
        return TensorView(p, std::move(shape), dtype);
    }
    void* allocate_persistent(size_t bytes, size_t alignment = 0) {
        void* p = nullptr;
        detail::check(xinfer_arena_allocate_persistent(a_, bytes, alignment, &p), "DeviceArena::allocate_persistent");
        return p;
    }
    void* persistent_buffer(size_t bytes = 0, size_t alignment = 0) {
        void* p = nullptr;
        detail::check(xinfer_arena_persistent_buffer(a_, bytes, alignment, &p), "DeviceArena::persistent_buffer");
        if (!persistent_buffer_) {
            persistent_buffer_ = p;
            persistent_buffer_capacity_ = bytes;
        }
        return p;
    }
    const void* persistent_buffer() const noexcept { return persistent_buffer_; }
    size_t persistent_buffer_capacity() const noexcept { return persistent_buffer_capacity_; }
    void reset() noexcept { xinfer_arena_reset(a_); }
    size_t capacity() const noexcept { return xinfer_arena_capacity(a_); }
    size_t allocated_bytes() const noexcept { return xinfer_arena_allocated_bytes(a_); }
    size_t remaining_bytes() const noexcept { return xinfer_arena_remaining_bytes(a_); }
    size_t peak_allocated_bytes() const noexcept { return xinfer_arena_peak_allocated_bytes(a_); }
    void* base_ptr() noexcept { return xinfer_arena_base_ptr(a_); }
    const void* base_ptr() const noexcept { return xinfer_arena_base_ptr(a_); }

private:
    std::shared_ptr<DeviceContext> ctx_;
    xinfer_arena* a_{nullptr};
    void* persistent_buffer_{nullptr};
    size_t persistent_buffer_capacity_{0};
};

}  // namespace core
}  // namespace xinfer
