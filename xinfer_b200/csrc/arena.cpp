// cudaMalloc-backed bump arena behind the C-ABI.  Semantics follow the reference's
// xinfer::core::DeviceArena (src/core/arena.h:14-66, src/core/arena.cpp:84-139): one device block
// carved by an aligned bump pointer, reset() rewinds it without freeing, persistent allocations live
// outside the block until destruction, and the single persistent buffer refuses to grow.
// Addresses handed out stay stable until reset(), which is what CUDA-graph capture relies on; the
// reference's rule "never reset during capture" (src/targets/qwen3_8/forward.cpp:334-337) carries over.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <new>
#include <vector>

#include "../../include/xinfer_b200.h"

struct xinfer_arena {
    void* base = nullptr;
    size_t capacity = 0;
    size_t offset = 0;
    size_t peak = 0;
    size_t default_alignment = 64;
    std::vector<void*> persistent;
    void* persistent_buffer = nullptr;
    size_t persistent_capacity = 0;
    int device = 0;
};

static bool pow2(size_t a) { return a != 0 && (a & (a - 1)) == 0; }

extern "C" {

int xinfer_arena_create(size_t capacity_bytes, size_t default_alignment, xinfer_arena** out) {
    if (!out) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    const size_t align = default_alignment ? default_alignment : 64;
    if (!pow2(align)) return XINFER_ERR_INVALID_ARGUMENT;
    xinfer_arena* a = new (std::nothrow) xinfer_arena();
    if (!a) return XINFER_ERR_OUT_OF_MEMORY;
    a->default_alignment = align;
    a->capacity = capacity_bytes;
    if (cudaGetDevice(&a->device) != cudaSuccess) { delete a; return XINFER_ERR_NO_DEVICE; }
    if (capacity_bytes > 0 && cudaMalloc(&a->base, capacity_bytes) != cudaSuccess) {
        cudaGetLastError();
        delete a;
        return XINFER_ERR_OUT_OF_MEMORY;
    }
    *out = a;
    return XINFER_OK;
}

void xinfer_arena_destroy(xinfer_arena* a) {
    if (!a) return;
    for (void* p : a->persistent) cudaFree(p);
    if (a->base) cudaFree(a->base);
    delete a;
}

int xinfer_arena_allocate(xinfer_arena* a, size_t bytes, size_t alignment, void** out) {
    if (!a || !out) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (bytes == 0) return XINFER_OK;  // src/core/arena.cpp:85
    if (!a->base) return XINFER_ERR_OUT_OF_MEMORY;
    const size_t align = alignment ? alignment : a->default_alignment;
    if (!pow2(align)) return XINFER_ERR_INVALID_ARGUMENT;
    const uintptr_t base = reinterpret_cast<uintptr_t>(a->base);
    const uintptr_t cur = base + a->offset;
    const uintptr_t aligned = (cur + align - 1) & ~(static_cast<uintptr_t>(align) - 1);
    const size_t new_offset = static_cast<size_t>(aligned - base) + bytes;
    if (new_offset > a->capacity || new_offset < bytes) return XINFER_ERR_OUT_OF_MEMORY;
    a->offset = new_offset;
    a->peak = std::max(a->peak, a->offset);
    *out = reinterpret_cast<void*>(aligned);
    return XINFER_OK;
}

int xinfer_arena_allocate_persistent(xinfer_arena* a, size_t bytes, size_t alignment, void** out) {
    if (!a || !out) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (bytes == 0) return XINFER_OK;
    const size_t align = alignment ? alignment : a->default_alignment;
    if (!pow2(align) || align > 256) return XINFER_ERR_INVALID_ARGUMENT;  // cudaMalloc aligns to 256 bytes
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return XINFER_ERR_OUT_OF_MEMORY;
    }
    a->persistent.push_back(p);
    *out = p;
    return XINFER_OK;
}

int xinfer_arena_persistent_buffer(xinfer_arena* a, size_t bytes, size_t alignment, void** out) {
    if (!a || !out) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (!a->persistent_buffer) {
        if (bytes == 0) return XINFER_ERR_INVALID_ARGUMENT;  // first call must size it, src/core/arena.cpp:122-126
        int rc = xinfer_arena_allocate_persistent(a, bytes, alignment, &a->persistent_buffer);
        if (rc != XINFER_OK) return rc;
        a->persistent_capacity = bytes;
    } else if (bytes > a->persistent_capacity) {
        return XINFER_ERR_INVALID_ARGUMENT;  // refuses to grow, src/core/arena.cpp:129-133
    }
    *out = a->persistent_buffer;
    return XINFER_OK;
}

void xinfer_arena_reset(xinfer_arena* a) {
    if (a) a->offset = 0;
}
size_t xinfer_arena_capacity(const xinfer_arena* a) { return a ? a->capacity : 0; }
size_t xinfer_arena_allocated_bytes(const xinfer_arena* a) { return a ? a->offset : 0; }
size_t xinfer_arena_remaining_bytes(const xinfer_arena* a) {
    return (a && a->offset < a->capacity) ? a->capacity - a->offset : 0;
}
size_t xinfer_arena_peak_allocated_bytes(const xinfer_arena* a) { return a ? a->peak : 0; }
void* xinfer_arena_base_ptr(const xinfer_arena* a) { return a ? a->base : nullptr; }

}  // extern "C"
