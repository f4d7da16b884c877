// INT4-G128 W4A16 GEMM for many activation rows (prefill chunks): Y[M,N] = X[M,K] * W^T (+ bias), M > 32.
//
// Replaces, for M = hundreds of rows, what the reference runs its prefill through: the same ops::linear_int4 /
// linear_int4_fused / mlp_gate_up_swiglu_int4 entry points (src/ops/linear.h:30-139), called with
// M = chunk length from forward_prefill_chunk (src/targets/qwen3_8/forward.cpp:402-554), where the reference
// repeats its GEMV row by row.  At M = 512 the contraction is compute-bound (2*M*N*K flops against N*K/2 bytes:
// ~2000 flop per weight byte), so this kernel is built around the tensor pipe, not around the weight stream:
//
//   * one CTA per 256 weight rows x 256 activation rows: two tcgen05.mma M = 128 x N = 256 accumulators, 2 x 256
//     columns = all of tensor memory, accumulated over the whole K (one read-out per tile);
//   * both operands from shared memory: the activations land by TMA in the canonical 128-byte-swizzled K-major
//     layout; the packed weights land raw (32 bytes per row and 64-k stage), eight warps - one thread per weight
//     row - unpack them (lop3 + one subtraction per pair, as in the decode kernel), multiply by the row's group
//     scale and write the fp16 tiles in the same swizzled layout, so every weight is unpacked once per 256
//     activation rows;
//   * three two-slot rings (raw weights, unpacked weights hi + lo, activations) and mbarriers both ways; one elected
//     thread issues the MMAs (16 per stage) and commits the stage's barriers.
//
// Numerics: the accumulators of 256 activation rows live in tensor memory for the whole K, so the group scale
// cannot be applied to a per-group dot product in registers as the decode kernels do.  Instead scale * weight
// goes into the MMA as TWO fp16 operands, hi = rn(q * s) and lo = q * s - hi, whose sum is the exact product
// (an 11-bit by 4-bit product has 15 significant bits; fp16 subnormals aside): two MMAs per k step, products and
// sums in fp32 in the tensor core.  The result differs from the reference's association only by the order of the
// fp32 sums, which the tensor core truncates over the whole K (measured against the fp64 oracle, worst element over
// rms: 3.7e-5 at K = 5120, 1.3e-4 at K = 17408), at twice the tensor work of a single rounded operand, which
// would be 3e-4 off (1.7e-3 worst element at K = 512) and outside the reference's own 1e-4 absolute test bound.
//
// Every wait is bounded (WaitState); a wait that runs out sets the device status word and the CTA leaves through
// its normal exit, releasing its tensor memory.

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "launch.cuh"
#include "ptx_sm100.cuh"
#include "w4a16.h"

namespace xb {
namespace {

constexpr int kGemmUnpackThreads = 256;             // one per weight row of the tile
constexpr int kGemmThreads = kGemmUnpackThreads + 64;  // + TMA producer warp + MMA warp
constexpr int kGemmProducerWarp = 8, kGemmMmaWarp = 9;
constexpr int kGemmTileN = 256;   // weight rows per CTA (two halves of 128)
constexpr int kGemmTileM = 256;   // activation rows per CTA (the MMA's N)
constexpr int kGemmStageK = 64;   // k per stage: one 128-byte swizzle row of fp16
constexpr int kWSlots = 2, kASlots = 2, kXSlots = 2;
constexpr int kWSlotBytes = kGemmTileN * (kGemmStageK / 2);   // 8 KB of packed weights
constexpr int kAPartBytes = kGemmTileN * kGemmStageK * 2;     // 32 KB of fp16 weights ...
constexpr int kASlotBytes = 2 * kAPartBytes;                  // ... twice: the high and the low part of scale * weight
constexpr int kXSlotBytes = kGemmTileM * kGemmStageK * 2;     // 32 KB of activations
constexpr int kGemmTmemCols = 512;

struct GemmCtrl {
    uint64_t w_full[kWSlots], w_empty[kWSlots];
    uint64_t a_ready[kASlots], a_empty[kASlots];
    uint64_t x_full[kXSlots], x_empty[kXSlots];
    uint64_t d_full;
    uint32_t tmem_base;
    WaitState ws;
};

constexpr size_t kGemmSmemBytes = 1024 /* alignment slack */ + kASlots * kASlotBytes + kXSlots * kXSlotBytes +
                                  kWSlots * kWSlotBytes + sizeof(GemmCtrl);

struct GemmParams {
    CUtensorMap w_map[2];   // packed weights of the two 128-row halves (the same tensor unless gate/up are paired)
    CUtensorMap x_map;
    const __half* scales[2];
    const float* bias;
    void* y;
    long long ldy;
    int n;          // output features
    int m;          // activation rows
    int groups;     // k / 128
    int stages;     // k / 64
    int swiglu;     // half 0 = gate rows, half 1 = up rows of the same 128 features; y = silu(gate) * up
    int out_f32;
    long long wait_limit;
    int* status;
    int x_stage_limit;  // test hook: activation stages from this index on are never requested (-1: off)
    float* partials;  // K split over gridDim.z: fp32 partial sums [split][m][n] (summed by a second kernel); else null
};

// D[tmem] (+)= A[smem descriptor] * B[smem descriptor], kind::f16, one CTA.  Issued by one thread.
__device__ __forceinline__ void umma_ss_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// scale * weight as two fp16 values whose sum is the exact product: hi = rn(q * s), lo = q * s - hi (the fused
// multiply-add rounds once, and the residual of an 11-bit by 4-bit product fits fp16 exactly, subnormals aside)
__device__ __forceinline__ void scale_split(uint32_t q2, uint32_t s2, uint32_t& hi, uint32_t& lo) {
    hi = hmul2_u32(q2, s2);
    lo = hfma2_u32(q2, s2, hi ^ 0x80008000u);
}

template <typename OutT>
__device__ __forceinline__ void store_out(void* y, long long off, float v) {
    if constexpr (sizeof(OutT) == 4) static_cast<float*>(y)[off] = v;
    else static_cast<__half*>(y)[off] = __float2half_rn(v);
}

template <typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1) w4a16_gemm_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t gemm_smem_raw[];
    // the swizzled operand tiles want 1024-byte alignment
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* a_ring = smem;
    uint8_t* x_ring = a_ring + kASlots * kASlotBytes;
    uint8_t* w_ring = x_ring + kXSlots * kXSlotBytes;
    GemmCtrl* ctrl = reinterpret_cast<GemmCtrl*>(w_ring + kWSlots * kWSlotBytes);

    const int tid = threadIdx.x;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int lane = tid & 31;
    volatile WaitState* ws = &ctrl->ws;
    griddep_launch_dependents();

    if (tid == 0) {
        for (int i = 0; i < kWSlots; ++i) { mbar_init(smem_u32(&ctrl->w_full[i]), 1); mbar_init(smem_u32(&ctrl->w_empty[i]), kGemmUnpackThreads / 32); }
        for (int i = 0; i < kASlots; ++i) { mbar_init(smem_u32(&ctrl->a_ready[i]), kGemmUnpackThreads / 32); mbar_init(smem_u32(&ctrl->a_empty[i]), 1); }
        for (int i = 0; i < kXSlots; ++i) { mbar_init(smem_u32(&ctrl->x_full[i]), 1); mbar_init(smem_u32(&ctrl->x_empty[i]), 1); }
        mbar_init(smem_u32(&ctrl->d_full), 1);
        ctrl->ws.abort_flag = 0;
        ctrl->ws.dep_ready = 0;
        ctrl->ws.limit = p.wait_limit;
        mbar_fence_init();
    }
    if (warp == kGemmMmaWarp) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), kGemmTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    // this CTA's stages: all of K, or its share when K is split over gridDim.z
    const int s_begin = static_cast<int>(static_cast<long long>(blockIdx.z) * p.stages / gridDim.z);
    const int s_end = static_cast<int>(static_cast<long long>(blockIdx.z + 1) * p.stages / gridDim.z);
    const int S = s_end - s_begin;  // ring slots and phases count from the CTA's first stage
    const int tile_n = blockIdx.x, m0 = blockIdx.y * kGemmTileM;
    // first weight row of each half
    const int row_base0 = p.swiglu ? tile_n * 128 : tile_n * kGemmTileN;
    const int row_base1 = p.swiglu ? tile_n * 128 : tile_n * kGemmTileN + 128;

    if (warp == kGemmProducerWarp) {
        // ------------------------------------------------------------------ TMA producer (whole warp waits, one lane issues)
        const bool leader = elect_one_sync();
        if (leader) {
            tma_prefetch_desc(&p.w_map[0]);
            tma_prefetch_desc(&p.w_map[1]);
            tma_prefetch_desc(&p.x_map);
        }
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        auto issue_w = [&](int s) {
            const uint32_t slot = static_cast<uint32_t>(s % kWSlots);
            const uint32_t full = smem_u32(&ctrl->w_full[slot]);
            const uint32_t dst = smem_u32(w_ring) + slot * kWSlotBytes;
            if (leader) {
                mbar_arrive_expect_tx(full, kWSlotBytes);
                tma_load_2d(dst, &p.w_map[0], full, (s_begin + s) * (kGemmStageK / 2), row_base0, pol_w);
                tma_load_2d(dst + kWSlotBytes / 2, &p.w_map[1], full, (s_begin + s) * (kGemmStageK / 2), row_base1, pol_w);
            }
        };
        auto issue_x = [&](int s) {
            const uint32_t slot = static_cast<uint32_t>(s % kXSlots);
            const uint32_t full = smem_u32(&ctrl->x_full[slot]);
            if (leader) {
                mbar_arrive_expect_tx(full, kXSlotBytes);
                tma_load_2d(smem_u32(x_ring) + slot * kXSlotBytes, &p.x_map, full, (s_begin + s) * kGemmStageK, m0, pol_x);
            }
        };
        // the weights do not depend on the kernel in front of this one, the activations do
        // (test hook: with x_stage_limit >= 0 the activation stages from that index on are never requested, so the
        // waits for them run out and the kernel leaves through its abort path)
        const int SX = (p.x_stage_limit >= 0 && p.x_stage_limit < S) ? p.x_stage_limit : S;
        int nw = 0, nx = 0;
        for (; nw < kWSlots && nw < S; ++nw) issue_w(nw);
        griddep_wait();
        if (leader) ws->dep_ready = 1;
        for (; nx < kXSlots && nx < SX; ++nx) issue_x(nx);
        bool ok = true;
        while (ok && (nw < S || nx < SX)) {
            if (nw < S) {
                ok = mbar_wait_parked(smem_u32(&ctrl->w_empty[nw % kWSlots]), ((nw / kWSlots) & 1u) ^ 1u, ws);
                if (ok) issue_w(nw++);
            }
            if (ok && nx < SX) {
                ok = mbar_wait_parked(smem_u32(&ctrl->x_empty[nx % kXSlots]), ((nx / kXSlots) & 1u) ^ 1u, ws);
                if (ok) issue_x(nx++);
            }
        }
        if (ws->abort_flag) {
            // give the copies still in flight a bounded chance to land before the CTA exits
            const long long t0 = clock64();
            for (int i = 0; i < kWSlots && i < nw; ++i) {
                const int k = nw - 1 - i;
                while (!mbar_try_wait(smem_u32(&ctrl->w_full[k % kWSlots]), (k / kWSlots) & 1u) && clock64() - t0 < p.wait_limit / 8) {
                }
            }
            for (int i = 0; i < kXSlots && i < nx; ++i) {
                const int k = nx - 1 - i;
                while (!mbar_try_wait(smem_u32(&ctrl->x_full[k % kXSlots]), (k / kXSlots) & 1u) && clock64() - t0 < p.wait_limit / 8) {
                }
            }
        }
        __syncwarp();
    } else if (warp == kGemmMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        const bool leader = elect_one_sync();
        constexpr uint32_t idesc = umma_idesc_f16_f32(128, kGemmTileM);
        // K-major, 128-byte swizzle: rows of 64 k, 8-row groups 1024 bytes apart; descriptor version 1
        constexpr uint32_t desc_hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
        constexpr uint32_t desc_lo_const = 1u << 16;
        const uint32_t a_lo0 = (smem_u32(a_ring) >> 4) & 0x3FFFu;
        const uint32_t x_lo0 = (smem_u32(x_ring) >> 4) & 0x3FFFu;
        bool ok = true;
        for (int s = 0; s < S && ok; ++s) {
            const uint32_t as = static_cast<uint32_t>(s % kASlots), xs = static_cast<uint32_t>(s % kXSlots);
            if (!mbar_wait_parked(smem_u32(&ctrl->a_ready[as]), (s / kASlots) & 1u, ws)) break;
            if (!mbar_wait_parked(smem_u32(&ctrl->x_full[xs]), (s / kXSlots) & 1u, ws)) break;
            tc_fence_after_sync();
            if (leader) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t ahi = desc_lo_const | (a_lo0 + ((as * kASlotBytes + h * (kAPartBytes / 2) + i * 32) >> 4));
                        const uint32_t alo = ahi + (kAPartBytes >> 4);
                        const uint32_t xlo = desc_lo_const | (x_lo0 + ((xs * kXSlotBytes + i * 32) >> 4));
                        const uint64_t bdesc = (static_cast<uint64_t>(desc_hi) << 32) | xlo;
                        umma_ss_f16(tmem_base + h * 256, (static_cast<uint64_t>(desc_hi) << 32) | ahi, bdesc, idesc, (s > 0 || i > 0) ? 1u : 0u);
                        umma_ss_f16(tmem_base + h * 256, (static_cast<uint64_t>(desc_hi) << 32) | alo, bdesc, idesc, 1u);
                    }
                }
                umma_commit(smem_u32(&ctrl->a_empty[as]));
                umma_commit(smem_u32(&ctrl->x_empty[xs]));
                if (s == S - 1) umma_commit(smem_u32(&ctrl->d_full));
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ unpack (then epilogue): one thread per weight row
        const int h = tid >> 7, r = tid & 127;
        const int row = (h ? row_base1 : row_base0) + r;
        const bool valid = row < p.n;
        const unsigned short* sp = reinterpret_cast<const unsigned short*>(p.scales[h]) + static_cast<long long>(valid ? row : 0) * p.groups;
        const uint32_t w_off = static_cast<uint32_t>((h * 128 + r) * (kGemmStageK / 2));
        const uint32_t a_off = static_cast<uint32_t>(h * (kAPartBytes / 2) + (r >> 3) * 1024 + (r & 7) * 128);
        const uint32_t sw = static_cast<uint32_t>(r & 7);
        bool ok = true;
        // the scale of the stage's 128-k group (two stages per group), fetched one stage ahead
        uint32_t q_next = (valid && S > 0) ? static_cast<uint32_t>(__ldg(sp + (s_begin >> 1))) : 0u;
        for (int s = 0; s < S; ++s) {
            const uint32_t sc2 = q_next | (q_next << 16);
            if (s + 1 < S) q_next = valid ? static_cast<uint32_t>(__ldg(sp + ((s_begin + s + 1) >> 1))) : 0u;
            const uint32_t wslot = static_cast<uint32_t>(s % kWSlots), aslot = static_cast<uint32_t>(s % kASlots);
            if (!mbar_wait(smem_u32(&ctrl->w_full[wslot]), (s / kWSlots) & 1u, ws)) { ok = false; break; }
            const uint32_t wsrc = smem_u32(w_ring) + wslot * kWSlotBytes + w_off;
            const uint4 v0 = lds128(wsrc), v1 = lds128(wsrc + 16);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->w_empty[wslot]));
            if (s >= kASlots) {
                if (!mbar_wait(smem_u32(&ctrl->a_empty[aslot]), ((s / kASlots) & 1u) ^ 1u, ws)) { ok = false; break; }
            }
            const uint32_t adst = smem_u32(a_ring) + aslot * kASlotBytes + a_off;
            const uint32_t words[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                uint32_t q[4];
                dequant_word(words[w], q);  // (k0,k4) (k1,k5) (k2,k6) (k3,k7)
                uint4 hi, lo;
                scale_split(prmt(q[0], q[1], 0x5410u), sc2, hi.x, lo.x);  // (k0,k1)
                scale_split(prmt(q[2], q[3], 0x5410u), sc2, hi.y, lo.y);  // (k2,k3)
                scale_split(prmt(q[0], q[1], 0x7632u), sc2, hi.z, lo.z);  // (k4,k5)
                scale_split(prmt(q[2], q[3], 0x7632u), sc2, hi.w, lo.w);  // (k6,k7)
                const uint32_t at = adst + ((static_cast<uint32_t>(w) ^ sw) << 4);
                sts128(at, hi);
                sts128(at + kAPartBytes, lo);
            }
            fence_proxy_async_smem();  // the tensor core reads this tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->a_ready[aslot]));
        }

        // ---------------------------------------------------------------- epilogue: this row's 256 sums
        if (ok) ok = mbar_wait(smem_u32(&ctrl->d_full), 0u, ws);
        // The read-out is taken by all 256 threads or by none (its gate/up exchange has barriers of its own): a wait
        // that gave up anywhere has set the abort flag before returning, and every thread arrives here.
        asm volatile("bar.sync 1, %0;" ::"n"(kGemmUnpackThreads) : "memory");
        if (!ws->abort_flag) {
            tc_fence_after_sync();
            const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
            const float bias = (valid && p.bias && !p.swiglu) ? p.bias[row] : 0.f;
            if (!p.swiglu) {
#pragma unroll 1
                for (int c = 0; c < kGemmTileM / 16; ++c) {
                    uint32_t d[16];
                    tmem_ld16(tmem_base + lane_sel + h * 256 + c * 16, d);
                    tmem_wait_ld();
                    if (valid) {
                        if (p.partials) {
                            float* ws_out = p.partials + static_cast<long long>(blockIdx.z) * p.m * p.n;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int m = m0 + c * 16 + j;
                                if (m < p.m) ws_out[static_cast<long long>(m) * p.n + row] = __uint_as_float(d[j]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int m = m0 + c * 16 + j;
                                if (m < p.m) store_out<OutT>(p.y, static_cast<long long>(m) * p.ldy + row, __uint_as_float(d[j]) + bias);
                            }
                        }
                    }
                }
            } else {
                // gate (half 0) and up (half 1) of one feature sit in different warps: the up half parks its values in
                // shared memory (the activation ring, idle by now), 16 columns at a time
                float* park = reinterpret_cast<float*>(x_ring);  // [128 rows][17]
#pragma unroll 1
                for (int c = 0; c < kGemmTileM / 16; ++c) {
                    uint32_t d[16];
                    tmem_ld16(tmem_base + lane_sel + h * 256 + c * 16, d);
                    tmem_wait_ld();
                    if (h == 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) park[r * 17 + j] = __uint_as_float(d[j]);
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(kGemmUnpackThreads) : "memory");
                    if (h == 0 && valid) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = m0 + c * 16 + j;
                            const float g = __uint_as_float(d[j]), u = park[r * 17 + j];
                            if (m < p.m) store_out<OutT>(p.y, static_cast<long long>(m) * p.ldy + row, (g / (1.0f + expf(-g))) * u);
                        }
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(kGemmUnpackThreads) : "memory");
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && ctrl->ws.abort_flag && p.status) atomicExch(p.status, kStatusWaitTimeout);
    if (warp == kGemmMmaWarp) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kGemmTmemCols);
    }
}

// Sums the K splits in split order (deterministic), adds the bias and converts.
template <typename OutT>
__global__ void __launch_bounds__(256) gemm_splitk_reduce_kernel(void* y, long long ldy, const float* partials, int splits,
                                                                 int m, int n, const float* bias) {
    griddep_prologue();
    const long long total = static_cast<long long>(m) * n;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float sum = 0.f;
        for (int z = 0; z < splits; ++z) sum += __ldcg(partials + z * total + i);
        const int row = static_cast<int>(i / n), col = static_cast<int>(i - static_cast<long long>(row) * n);
        if (bias) sum += bias[col];
        store_out<OutT>(y, static_cast<long long>(row) * ldy + col, sum);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn gemm_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// packed weights [n rows][k/2 bytes]: boxes of 128 rows x 32 bytes (64 k), dense in shared memory
bool encode_gemm_w(CUtensorMap* map, const uint8_t* w, long long n, long long k) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k / 2)};
    const cuuint32_t box[2] = {kGemmStageK / 2, 128};
    const cuuint32_t estr[2] = {1, 1};
    return gemm_encode_fn() &&
           gemm_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// activations [m rows][k] fp16: boxes of 256 rows x 64 k, 128-byte swizzled (the MMA's K-major operand layout)
bool encode_gemm_x(CUtensorMap* map, const __half* x, long long m, long long k) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {kGemmStageK, kGemmTileM};
    const cuuint32_t estr[2] = {1, 1};
    return gemm_encode_fn() &&
           gemm_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename OutT>
cudaError_t gemm_configure_and_launch(const GemmParams& p, dim3 grid, cudaStream_t stream) {
    static bool configured[64];
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev]) {
            e = cudaFuncSetAttribute(w4a16_gemm_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kGemmSmemBytes));
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
    }
    return launch_pdl(w4a16_gemm_kernel<OutT>, grid, dim3(kGemmThreads), kGemmSmemBytes, stream, p);
}

}  // namespace

bool gemm_eligible(const void* x, const TcProj* proj, int num, bool swiglu, long long m, long long k, int group_size) {
    if (m <= 32 || group_size != 128 || k < 128 || (k % 128) != 0) return false;
    if (reinterpret_cast<uintptr_t>(x) & 15) return false;
    const int cnt = swiglu ? 2 : num;
    if (cnt < 1 || cnt > 4) return false;
    for (int i = 0; i < cnt; ++i)
        if ((reinterpret_cast<uintptr_t>(proj[i].w) & 15) || proj[i].n < 1 || proj[i].push) return false;
    if (swiglu && proj[0].n != proj[1].n) return false;
    return true;
}

// One launch per projection (gate and up of the fused MLP share one).  Returns 0, -1 on a launch error, -2 when
// the problem cannot be described to the kernel.
int gemm_launch(cudaStream_t stream, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32, long long m,
                long long k, int* status, long long wait_limit, int x_stage_limit, int num_sms, float* partials, size_t partial_bytes) {
    const int launches = swiglu ? 1 : num;
    for (int i = 0; i < launches; ++i) {
        GemmParams p;
        memset(&p, 0, sizeof(p));
        const TcProj& a = proj[i];
        const TcProj& b = swiglu ? proj[1] : proj[i];
        if (!encode_gemm_w(&p.w_map[0], a.w, a.n, k) || !encode_gemm_w(&p.w_map[1], b.w, b.n, k)) return -2;
        if (!encode_gemm_x(&p.x_map, static_cast<const __half*>(x), m, k)) return -2;
        p.scales[0] = static_cast<const __half*>(a.scales);
        p.scales[1] = static_cast<const __half*>(b.scales);
        p.bias = a.bias;
        p.y = a.y;
        p.ldy = a.ldy > 0 ? a.ldy : a.n;
        p.n = static_cast<int>(a.n);
        p.m = static_cast<int>(m);
        p.groups = static_cast<int>(k / 128);
        p.stages = static_cast<int>(k / kGemmStageK);
        p.swiglu = swiglu ? 1 : 0;
        p.out_f32 = out_f32 ? 1 : 0;
        p.wait_limit = wait_limit;
        p.x_stage_limit = x_stage_limit;
        p.status = status;
        const int rows_per_cta = swiglu ? 128 : kGemmTileN;
        dim3 grid(static_cast<unsigned>((a.n + rows_per_cta - 1) / rows_per_cta), static_cast<unsigned>((m + kGemmTileM - 1) / kGemmTileM));
        // Few tiles (N = 5120 at M = 512 is 40): K is split over gridDim.z so that about two CTAs per SM's worth of
        // work exists, the fp32 partials go through a scratch buffer and a second kernel adds them in split order.
        int splits = 1;
        const long long tiles = static_cast<long long>(grid.x) * grid.y;
        if (!swiglu && partials && tiles * 2 <= num_sms) {
            splits = static_cast<int>((2LL * num_sms) / tiles);
            if (splits > 8) splits = 8;
            if (splits > p.stages / 8) splits = p.stages / 8;
            const long long per_split = static_cast<long long>(m) * a.n * 4;
            if (per_split * splits > static_cast<long long>(partial_bytes)) splits = static_cast<int>(partial_bytes / per_split);
            if (splits < 2) splits = 1;
        }
        grid.z = static_cast<unsigned>(splits);
        p.partials = splits > 1 ? partials : nullptr;
        cudaError_t e = out_f32 ? gemm_configure_and_launch<float>(p, grid, stream) : gemm_configure_and_launch<__half>(p, grid, stream);
        if (e != cudaSuccess) return -1;
        if (splits > 1) {
            const long long total = m * a.n;
            const unsigned blocks = static_cast<unsigned>(total / 1024 + 1 < 4096 ? total / 1024 + 1 : 4096);
            e = out_f32 ? launch_pdl(gemm_splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, p.y, p.ldy,
                                     static_cast<const float*>(partials), splits, p.m, p.n, p.bias)
                        : launch_pdl(gemm_splitk_reduce_kernel<__half>, dim3(blocks), dim3(256), 0, stream, p.y, p.ldy,
                                     static_cast<const float*>(partials), splits, p.m, p.n, p.bias);
            if (e != cudaSuccess) return -1;
        }
    }
    return 0;
}

}  // namespace xb
