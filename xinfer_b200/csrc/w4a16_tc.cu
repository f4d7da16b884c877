// W4A16 skinny GEMM on tcgen05 tensor cores for 1 <= M <= 32 activation rows.
//
//   Y[m, n] = sum_g scale[n, g] * ( sum_{k in group g} X[m, k] * q[n, k] )  (+ bias[n])
//
// Replaces the Xe2 sub-group kernels of the reference for fp16 activations:
//   linear_int4                 src/ops/linear.cpp:165-305   (one projection)
//   splitk_int4_impl            src/ops/linear.cpp:33-163    (small N: K is split across CTAs here)
//   linear_int4_fused           src/ops/linear.cpp:351-478   (<= 4 projections sharing X)
//   mlp_gate_up_swiglu_int4     src/ops/linear.cpp:501-602   (gate and up rows paired in one CTA)
// The weight layout is the reference's own ([N][K/2] bytes, low nibble = even k; [N][K/128] fp16
// scales), read in place, and the association is the reference's: an fp32 dot of exact integers per
// 128-k group, then one multiply by the group's scale.
//
// Mapping to the hardware.  The weights sit on the MMA's M side: a CTA owns 256 output rows as two
// 128-row halves.  Sixteen consumer warps, four per scheduler: warp (half, group, quarter) owns 32 rows
// of its half and, in every 256-k stage, one of the stage's two 128-k groups.  Its thread reads 64
// packed bytes of its row from the TMA-staged tile (128B-swizzled, conflict free), unpacks them to
// exact fp16 integers in registers, and writes them with tcgen05.st into TMEM lane t, where they are
// the A operand (128 x 16 per MMA).  The <= 32 activation rows are the MMA's N side: their K slice
// arrives as TMA boxes of 64 k per row in the 128-byte-swizzled K-major layout, in a ring of its own,
// and is the B operand from shared memory.  Each 128-k group accumulates into a fresh TMEM tile
// D[128 x NMMA]; the thread that unpacked the group reads lane t back (tcgen05.ld) one stage later and
// folds it into fp32 register accumulators with its own row's scale.  The two threads of a row add
// their partial sums in the epilogue.
//
// Helper warpgroup: a TMA producer warp, two MMA-issuing warps (one per half; the warp computes
// warp-uniformly, one elected lane issues) and a warp that rewrites the staged activations in the k
// order of the unpack, (0,4,1,5,2,6,3,7) inside each 8-k block.  The register file is re-split
// between the helper warpgroup and the consumers with setmaxnreg.
//
// Work is cut stream-K style when there is at least one tile per SM: the (tile, 256-k stage) units are
// split evenly over one CTA per SM; a tile finished by several CTAs is summed by the last one to
// arrive, in CTA order, from fp32 partials in a scratch buffer (deterministic, no float atomics).
// With fewer tiles, each tile's K range is split over a thread-block cluster that sums through
// distributed shared memory (bulk copies that count bytes on the receiver's mbarrier).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <new>
#include <vector>

#include "ptx_sm100.cuh"
#include "w4a16.h"

namespace xb {

namespace {

constexpr int kTileRows = 256;
constexpr int kHalfRows = 128;
constexpr int kStageK = 256;                                 // weights per row per stage = 2 groups
constexpr int kStageRowBytes = kStageK / 2;                  // 128 B of packed int4 per row
constexpr int kWHalfBytes = kHalfRows * kStageRowBytes;      // 16 KiB
constexpr int kWStageBytes = 2 * kWHalfBytes;                // 32 KiB
constexpr int kXBoxesPerStage = kStageK / 64;                // activation boxes of 64 k (128 bytes) per stage
constexpr int kConsumerThreads = 512;  // warps 0..15
constexpr int kProducerWarp = 16;
constexpr int kMmaWarp = 17;  // issues the MMAs of half 0 and owns the TMEM allocation; warp 18 issues half 1
// warp 19 rewrites the staged activations in the k order of the unpack
constexpr int kThreads = 640;
// Register re-split between warpgroups.  The kernel starts with kLaunchRegs per thread (what 640 threads leave
// of the 64K file); the helper warpgroup releases down to kHelperRegs and the four consumer warpgroups grow
// to kConsumerRegs.  A consumer's request blocks until the CTA's own released registers cover it, so the
// released amount must be at least the requested one.
constexpr int kLaunchRegs = 96;
constexpr int kConsumerRegs = 112;
constexpr int kHelperRegs = 32;
static_assert(kConsumerThreads * (kConsumerRegs - kLaunchRegs) <= (kThreads - kConsumerThreads) * (kLaunchRegs - kHelperRegs),
              "consumer register request exceeds what the helper warpgroup releases");
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxSegs = 4;
constexpr int kPrefetchStages = 4;  // stages of the next launch that each CTA asks L2 for

template <int NMMA>
struct Cfg {
    // Two rings.  A weight slot is free again as soon as the consumers have unpacked it; an activation slot
    // only when the MMAs that read it have completed, about a stage later.  Keeping them apart lets the
    // weight stream (the HBM traffic) run as far ahead as its own ring allows.
    static constexpr int kXStageBytes = NMMA * kStageK * 2;
    // Depth is not what limits the stream (3, 4 and 5 weight slots run at the same rate); the total is: L1 is
    // what shared memory leaves of the SM's 256 KB, and the consumers' strided 2-byte scale loads live in L1.
    // Both configurations stay under the 196 KB carve-out (about 60 KB of L1); at 224 KB the scale lines
    // thrashed (LM head 3 % slower at M <= 8, 15 % at M = 32).
    static constexpr int kStages = (NMMA == 32) ? 3 : 4;   // weight ring, 32 KiB per slot
    static constexpr int kXStages = (NMMA == 32) ? 4 : 6;  // activation ring
    static constexpr int kWRingBytes = kStages * kWStageBytes;
    static constexpr int kXRingBytes = kXStages * kXStageBytes;
    static constexpr int kXchgBytes = kTileRows * NMMA * 4;  // accumulators parked for the epilogue
    static constexpr int kCtrlBytes = 512;
    static constexpr int kSmemBytes = kWRingBytes + kXRingBytes + kXchgBytes + kCtrlBytes + 1024;  // + align slack
    static_assert(kSmemBytes <= 196 * 1024, "rings sized to leave L1 for the scale loads");
};

struct Seg {
    const __half* scales;
    const float* bias;
    void* y;
    long long ldy;  // row stride of y in elements
    int n;          // output features of this projection
    int tile_begin; // first tile index of this projection
    int push;       // 0: y only; 1: the same element in every rank's buffer; 2: in the row owner's buffer
    void* y_peer[kTpMaxWorld];
};

struct Params {
    CUtensorMap w_map[kMaxSegs];
    CUtensorMap x_map;
    Seg seg[kMaxSegs];
    int num_segs;
    int swiglu;       // 1: seg[0] = gate, seg[1] = up, one tile = 128 gate rows + the same 128 up rows
    int m;            // activation rows (<= NMMA)
    int groups;       // K / 128
    int stages;       // ceil(groups / 2), stage units per tile
    int total_tiles;
    long long total_units;
    float* workspace; // [ctas][2][32][256] fp32 partials
    int* counters;    // [total_tiles], zero between launches
    int* status;      // device status word
    int cluster;      // CTAs per thread-block cluster = K splits per tile summed through distributed shared memory (1: none)
    long long wait_limit;  // SM clocks after which a device-side wait gives up
    int x_stage_limit;     // test hook: activation stages beyond this index are never requested (-1: off)
    TpLink tp;             // N-split exchange (world <= 1: none)
    int xchg_direct;       // cluster split-K partials go by plain remote stores (1) or by bulk copies (0)
    int x_perm;            // X is stored in the unpack's k order already: no in-kernel reorder of the staged activations
    int y_perm;            // write Y with its columns in that order (it is the X of another such launch)
    // Optional: the first weight stages of the NEXT tensor-core launch in the stream, pulled into L2 while this
    // launch drains, so that launch's pipeline fills from L2 instead of HBM.  pf_ctas = 0: nothing to prefetch.
    CUtensorMap pf_map[kMaxSegs];
    int pf_tile_begin[kMaxSegs];
    int pf_num_segs;
    int pf_swiglu;
    int pf_stages;            // stage units per tile of that launch
    int pf_ctas;              // its grid size
    long long pf_total_units;
};

struct Ctrl {
    uint64_t full[8];     // weights of a stage have landed
    uint64_t empty[8];    // every consumer warp has unpacked them
    uint64_t x_full[8];   // activations of a stage have landed
    uint64_t x_ready[8];  // the reorder warp has rewritten them in the unpack's k order
    uint64_t x_empty[8];  // both halves' MMAs that read them have completed
    uint64_t a_full[2][2];
    uint64_t d_full[2][2];
    uint64_t epi;         // epilogue barrier of the consumer warps
    uint64_t red;         // counts the bytes of split-K partials that other CTAs of the cluster store here
    uint32_t tmem_base;
    int is_last;
    WaitState ws;
};
static_assert(sizeof(Ctrl) <= 512, "control block");

__device__ __forceinline__ long long unit_begin(long long cta, long long total, long long ctas) {
    return cta * total / ctas;
}
__device__ __forceinline__ int unit_owner(long long unit, long long total, long long ctas) {
    // the CTA c with unit_begin(c) <= unit < unit_begin(c + 1)
    return static_cast<int>(((unit + 1) * ctas + total - 1) / total - 1);
}

// Non-blocking L2 prefetch of [ptr, ptr + bytes), one request per 32-byte sector.
__device__ __forceinline__ void prefetch_l2_range(const void* ptr, int bytes) {
    const uintptr_t lo = reinterpret_cast<uintptr_t>(ptr) & ~uintptr_t(31);
    const uintptr_t hi = reinterpret_cast<uintptr_t>(ptr) + static_cast<uintptr_t>(bytes > 0 ? bytes : 0);
#pragma unroll 1
    for (uintptr_t a = lo; a < hi; a += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
}

template <typename OutT>
__device__ __forceinline__ void store_out(OutT* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__half>(__half* p, float v) { *p = __float2half_rn(v); }

struct TileInfo {
    int seg;
    int row0;  // first output row of the tile within its projection
};

__device__ __forceinline__ TileInfo locate_tile(const Params& p, int tile) {
    TileInfo ti;
    ti.seg = 0;
    if (!p.swiglu) {
#pragma unroll
        for (int i = 1; i < kMaxSegs; ++i)
            if (i < p.num_segs && tile >= p.seg[i].tile_begin) ti.seg = i;
    }
    ti.row0 = (tile - p.seg[ti.seg].tile_begin) * (p.swiglu ? kHalfRows : kTileRows);
    return ti;
}

// Stores output element (activation row j, element offset `off` from the projection's y) where it belongs:
// locally, or - N-split tensor parallelism - with plain peer stores into the other ranks' buffers as well.
// Position of output feature n inside its block of eight when Y is written in the unpack's k order
// (0,4,1,5,2,6,3,7): feature k < 4 of a block goes to 2k, feature k >= 4 to 2(k - 4) + 1.
__device__ __forceinline__ int perm8(int n) {
    const int k = n & 7;
    return (n & ~7) | ((k < 4) ? 2 * k : 2 * (k - 4) + 1);
}

template <typename OutT>
__device__ __forceinline__ void store_row(const Params& p, const Seg& sg, long long off, int j, float v) {
    if (sg.push == 0) {
        store_out<OutT>(static_cast<OutT*>(sg.y) + off, v);
    } else if (sg.push == 2) {
        store_out<OutT>(static_cast<OutT*>(sg.y_peer[j / p.tp.rows_per_rank]) + off, v);
    } else {
#pragma unroll 1
        for (int r = 0; r < p.tp.world; ++r) store_out<OutT>(static_cast<OutT*>(sg.y_peer[r]) + off, v);
    }
}

template <int NMMA, int NREAD, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) w4a16_tc_kernel(const __grid_constant__ Params p) {
    using C = Cfg<NMMA>;
    extern __shared__ uint8_t smem_raw[];
    // 1 KiB alignment as an offset into the shared array (not a cast through an integer), so that every pointer
    // derived from it is still known to point to shared memory and compiles to 32-bit shared loads and stores
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* xring = smem + C::kWRingBytes;
    uint8_t* xchg_raw = xring + C::kXRingBytes;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(xchg_raw + C::kXchgBytes);
    float* xchg = reinterpret_cast<float*>(xchg_raw);

    const int tid = threadIdx.x;
    // (the broadcast tells the compiler that the warp index, and every role, row block, tensor-memory address and
    // barrier address derived from it, is the same in all lanes: they then live in uniform registers instead of
    // being moved there before each tcgen05 or barrier instruction)
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int lane = tid & 31;
    volatile WaitState* abort_flag = &ctrl->ws;  // shared by every bounded wait of the CTA
    griddep_launch_dependents();

    if (tid == 0) {
        for (int i = 0; i < C::kStages; ++i) {
            mbar_init(smem_u32(&ctrl->full[i]), 1);
            mbar_init(smem_u32(&ctrl->empty[i]), kConsumerThreads / 32);
        }
        for (int i = 0; i < C::kXStages; ++i) {
            mbar_init(smem_u32(&ctrl->x_full[i]), 1);
            mbar_init(smem_u32(&ctrl->x_ready[i]), 1);
            mbar_init(smem_u32(&ctrl->x_empty[i]), 2);  // one MMA commit per half
        }
        for (int w = 0; w < 2; ++w)
            for (int b = 0; b < 2; ++b) {
                mbar_init(smem_u32(&ctrl->a_full[w][b]), kHalfRows / 32);
                mbar_init(smem_u32(&ctrl->d_full[w][b]), 1);
            }
        mbar_init(smem_u32(&ctrl->epi), kConsumerThreads / 32);
        mbar_init(smem_u32(&ctrl->red), 1);
        if (p.cluster > 1) {
            // bytes this CTA will receive: every CTA of the cluster (itself included) sends 256 floats for each
            // activation row this CTA finishes (a contiguous block of ceil(m / cluster) rows per rank)
            const int m_rows = p.m < NREAD ? p.m : NREAD;
            const int rank = static_cast<int>(cluster_ctarank());
            const int rows_cap = (m_rows + p.cluster - 1) / p.cluster;
            int owned = m_rows - rank * rows_cap;
            owned = owned < 0 ? 0 : (owned > rows_cap ? rows_cap : owned);
            mbar_arrive_expect_tx(smem_u32(&ctrl->red), static_cast<uint32_t>(p.cluster * owned * kTileRows * 4));
        }
        ctrl->ws.abort_flag = 0;
        ctrl->ws.dep_ready = 0;
        ctrl->ws.limit = p.wait_limit;
        ctrl->is_last = 0;
        mbar_fence_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    const long long ctas = gridDim.x;
    const long long u_begin = unit_begin(blockIdx.x, p.total_units, ctas);
    const long long u_end = unit_begin(blockIdx.x + 1, p.total_units, ctas);
    const int S = p.stages;

    // Every stage carries exactly two 128-k groups.  When K/128 is odd the second group of a tile's last
    // stage lies beyond the tensors' extent: TMA fills it with zeros, its products are zero, and its
    // scale is taken as zero, so the code below never branches on the group count.
    // The helper warpgroup (producer, MMA issuers) hands most of its registers to the four consumer warpgroups.
    if (warp >= kProducerWarp) {
    setmaxnreg_dec<kHelperRegs>();
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        // The whole warp runs the (warp-uniform) index arithmetic and the waits; one elected lane issues.
        const bool leader = elect_one_sync();
        if (leader) {
            for (int i = 0; i < kMaxSegs; ++i)
                if (i < (p.swiglu ? 2 : p.num_segs)) tma_prefetch_desc(&p.w_map[i]);
            tma_prefetch_desc(&p.x_map);
        }
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        const uint32_t total_mine = static_cast<uint32_t>(u_end - u_begin);
        // (tile, stage-in-tile) of the next stage to request, one cursor per ring
        int w_tile = static_cast<int>(u_begin / S);
        int w_s = static_cast<int>(u_begin - static_cast<long long>(w_tile) * S);
        int x_s = w_s;
        const uint32_t smem_w = smem_u32(smem);
        const uint32_t smem_x = smem_u32(xring);
        auto issue_w = [&](uint32_t n) {
            const uint32_t slot = n % C::kStages;
            const TileInfo ti = locate_tile(p, w_tile);
            const uint32_t full = smem_u32(&ctrl->full[slot]);
            const uint32_t dst = smem_w + slot * kWStageBytes;
            const int map_b = p.swiglu ? 1 : ti.seg;
            const int row_b = p.swiglu ? ti.row0 : ti.row0 + kHalfRows;
            if (leader) {
                mbar_arrive_expect_tx(full, kWStageBytes);
                tma_load_2d(dst, &p.w_map[ti.seg], full, w_s * kStageRowBytes, ti.row0, pol_w);
                tma_load_2d(dst + kWHalfBytes, &p.w_map[map_b], full, w_s * kStageRowBytes, row_b, pol_w);
            }
            if (++w_s == S) { w_s = 0; ++w_tile; }
        };
        auto issue_x = [&](uint32_t n) {
            // activations: four [NMMA rows][64 k] boxes, each in the 128-byte-swizzled K-major layout
            const uint32_t slot = n % C::kXStages;
            const uint32_t full = smem_u32(&ctrl->x_full[slot]);
            const uint32_t dst = smem_x + slot * C::kXStageBytes;
            if (leader) {
                mbar_arrive_expect_tx(full, C::kXStageBytes);
#pragma unroll
                for (int b = 0; b < kXBoxesPerStage; ++b)
                    tma_load_2d(dst + b * (NMMA * 128), &p.x_map, full, x_s * kStageK + b * 64, 0, pol_x);
            }
            if (++x_s == S) x_s = 0;
        };
        // The weights do not depend on the previous kernel in the stream, the activations do: the first
        // ring of weight tiles is requested before waiting for that kernel, so the weight stream is
        // already in flight while it drains (programmatic dependent launch).
        const uint32_t pre_w = total_mine < C::kStages ? total_mine : C::kStages;
        // (test hook: with x_stage_limit >= 0 the activation stages from that index on are never requested, so
        // the waits for them run out and the kernel leaves through its abort path)
        const uint32_t x_total = (p.x_stage_limit >= 0 && static_cast<uint32_t>(p.x_stage_limit) < total_mine)
                                     ? static_cast<uint32_t>(p.x_stage_limit) : total_mine;
        const uint32_t pre_x = x_total < C::kXStages ? x_total : C::kXStages;
        // All CTAs start together: were every CTA to request its whole ring at once, the first stages would
        // come back interleaved with the deeper ones and the consumers would sit idle for the whole burst.
        // Two stages go out first; the rest of the ring follows once the first stage has landed.
        const uint32_t pre_a = pre_w < 2u ? pre_w : 2u;
        for (uint32_t n = 0; n < pre_a; ++n) issue_w(n);
        griddep_wait();
        if (leader) abort_flag->dep_ready = 1;  // from here on a wait that runs out is a real timeout
        for (uint32_t n = 0; n < pre_x; ++n) issue_x(n);
        bool ok = true;
        if (pre_w > pre_a) {
            ok = mbar_wait_parked(smem_u32(&ctrl->full[0]), 0u, abort_flag);
            for (uint32_t n = pre_a; ok && n < pre_w; ++n) issue_w(n);
        }
        uint32_t nw = pre_w, nx = pre_x;
        while (ok && (nw < total_mine || nx < x_total)) {
            if (nw < total_mine) {
                ok = mbar_wait_parked(smem_u32(&ctrl->empty[nw % C::kStages]), ((nw / C::kStages) & 1u) ^ 1u, abort_flag);
                if (ok) issue_w(nw++);
            }
            if (ok && nx < x_total) {
                ok = mbar_wait_parked(smem_u32(&ctrl->x_empty[nx % C::kXStages]), ((nx / C::kXStages) & 1u) ^ 1u, abort_flag);
                if (ok) issue_x(nx++);
            }
        }
        if (leader && p.pf_ctas > 0) {
            // this CTA's own stream is fully requested: ask L2 for what CTA blockIdx.x (+ k * gridDim.x) of the
            // next launch will request first (its first two stages, same unit arithmetic as above)
            for (int c = blockIdx.x; c < p.pf_ctas; c += gridDim.x) {
                const long long pu0 = unit_begin(c, p.pf_total_units, p.pf_ctas);
                const long long pu1 = unit_begin(c + 1, p.pf_total_units, p.pf_ctas);
                for (int i = 0; i < kPrefetchStages && pu0 + i < pu1; ++i) {
                    const int ptile = static_cast<int>((pu0 + i) / p.pf_stages);
                    const int ps = static_cast<int>((pu0 + i) - static_cast<long long>(ptile) * p.pf_stages);
                    int pseg = 0;
                    if (!p.pf_swiglu)
                        for (int q = 1; q < kMaxSegs; ++q)
                            if (q < p.pf_num_segs && ptile >= p.pf_tile_begin[q]) pseg = q;
                    const int prow = (ptile - p.pf_tile_begin[pseg]) * (p.pf_swiglu ? kHalfRows : kTileRows);
                    tma_prefetch_l2_2d(&p.pf_map[pseg], ps * kStageRowBytes, prow);
                    tma_prefetch_l2_2d(&p.pf_map[p.pf_swiglu ? 1 : pseg], ps * kStageRowBytes,
                                       p.pf_swiglu ? prow : prow + kHalfRows);
                }
            }
        }
        if (abort_flag->abort_flag) {
            // give the copies still in flight a bounded chance to land before the CTA exits
            const long long t0 = clock64();
            for (int i = 0; i < C::kStages && i < static_cast<int>(nw); ++i) {
                const uint32_t k = nw - 1 - i;
                while (!mbar_try_wait(smem_u32(&ctrl->full[k % C::kStages]), (k / C::kStages) & 1u) &&
                       clock64() - t0 < p.wait_limit / 8) {
                }
            }
            for (int i = 0; i < C::kXStages && i < static_cast<int>(nx); ++i) {
                const uint32_t k = nx - 1 - i;
                while (!mbar_try_wait(smem_u32(&ctrl->x_full[k % C::kXStages]), (k / C::kXStages) & 1u) &&
                       clock64() - t0 < p.wait_limit / 8) {
                }
            }
        }
        __syncwarp();
        if (p.cluster > 1) { __syncwarp(); cluster_arrive(); cluster_wait(); cluster_arrive(); cluster_wait(); }
    } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
        // ------------------------------------------------------------------ MMA issuers, one warp per half
        // The warp waits and computes descriptors as a whole (warp-uniform values); one elected lane issues.
        {
            const bool leader = elect_one_sync();
            const int w = warp - kMmaWarp;
            constexpr uint32_t idesc = umma_idesc_f16_f32(128, NMMA);
            // Shared-memory descriptor of the activation operand: K-major, 128-byte swizzle (rows of 64 k,
            // 8-row groups 1024 bytes apart); only the 14-bit start address changes between MMAs.
            constexpr uint32_t sbo = 1024;
            constexpr uint32_t desc_hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // version 1, SWIZZLE_128B
            constexpr uint32_t desc_lo_const = 1u << 16;  // leading-dimension offset: unused for swizzled K-major
            // (in a cluster launch a shared-window address carries the CTA's rank in its upper bits: keep 14 bits)
            const uint32_t xring_lo = (smem_u32(xring) >> 4) & 0x3FFFu;
            // pre-permuted activations are usable as they land (x_full); otherwise once the reorder warp is done (x_ready)
            const uint32_t xready0 = p.x_perm ? smem_u32(&ctrl->x_full[0]) : smem_u32(&ctrl->x_ready[0]);
            const uint32_t xempty0 = smem_u32(&ctrl->x_empty[0]);
            const uint32_t afull0 = smem_u32(&ctrl->a_full[w][0]);
            const uint32_t dfull0 = smem_u32(&ctrl->d_full[w][0]);
            const uint32_t a_t0 = tmem_base + w * 128;
            const uint32_t d_t0 = tmem_base + 256 + w * 64;
            const uint32_t total_mine = static_cast<uint32_t>(u_end - u_begin);
            bool ok = true;
            for (uint32_t n = 0; n < total_mine && ok; ++n) {
                const uint32_t slot = n % C::kXStages;
                if (!mbar_wait_parked(xready0 + slot * 8, (n / C::kXStages) & 1u, abort_flag)) break;
                const uint32_t xlo = desc_lo_const | (xring_lo + slot * (C::kXStageBytes >> 4));
#pragma unroll
                for (int gi = 0; gi < 2; ++gi) {
                    if (!mbar_wait_parked(afull0 + gi * 8, n & 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    if (leader) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            // K step kk = gi * 8 + i of the stage: box kk / 4, then 32 bytes per step inside the box
                            const uint32_t kk = gi * 8 + i;
                            const uint32_t lo = xlo + (((kk >> 2) * (NMMA * 128) + (kk & 3) * 32) >> 4);
                            const uint64_t bdesc = (static_cast<uint64_t>(desc_hi) << 32) | lo;
                            umma_ts_f16(d_t0 + (n & 1u) * 128 + gi * 32, a_t0 + gi * 64 + i * 8, bdesc, idesc, i > 0 ? 1u : 0u);
                        }
                        umma_commit(dfull0 + gi * 8);
                        // the stage's activations are no longer read once both groups' MMAs have completed
                        if (gi == 1) umma_commit(xempty0 + slot * 8);
                    }
                    __syncwarp();
                }
            }
        }
        if (p.cluster > 1) { __syncwarp(); cluster_arrive(); cluster_wait(); cluster_arrive(); cluster_wait(); }
    } else {
        // ------------------------------------------------------------------ activation reorder warp
        // The unpack yields k in the order (0,4,1,5,2,6,3,7) inside each 8-k block: this warp rewrites every
        // staged activation slot to the same order, in place, before the MMAs read it.
        const uint32_t xring_base = smem_u32(xring);
        const uint32_t xfull0 = smem_u32(&ctrl->x_full[0]);
        const uint32_t xready0 = smem_u32(&ctrl->x_ready[0]);
        const uint32_t total_mine = static_cast<uint32_t>(u_end - u_begin);
        constexpr int kChunksPerLane = C::kXStageBytes / 16 / 32;
        // (nothing to do when the caller's X is in that order already)
        for (uint32_t n = 0; n < (p.x_perm ? 0u : total_mine); ++n) {
            const uint32_t xslot = n % C::kXStages;
            if (!mbar_wait_parked(xfull0 + xslot * 8, (n / C::kXStages) & 1u, abort_flag)) break;
            const uint32_t base = xring_base + xslot * C::kXStageBytes + lane * 16;
#pragma unroll 8
            for (int i = 0; i < kChunksPerLane; ++i) {
                const uint32_t addr = base + i * 512;
                const uint4 v = lds128(addr);
                uint4 o;
                o.x = prmt(v.x, v.z, 0x5410u);
                o.y = prmt(v.x, v.z, 0x7632u);
                o.z = prmt(v.y, v.w, 0x5410u);
                o.w = prmt(v.y, v.w, 0x7632u);
                sts128(addr, o);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(xready0 + xslot * 8);
        }
        if (p.cluster > 1) { __syncwarp(); cluster_arrive(); cluster_wait(); cluster_arrive(); cluster_wait(); }
    }
    } else {
        setmaxnreg_inc<kConsumerRegs>();
        // ------------------------------------------------------------------ consumers: unpack, read out, epilogue
        // Sixteen warps, four per scheduler.  Warp (half, group, quarter) owns rows quarter*32.. of its
        // 128-row half (TMEM lanes are only reachable from the warp with the same index mod 4) and, in every
        // stage, the 128 k of one group: its thread unpacks 64 bytes of its row, hands them to the MMA and
        // folds the previous stage's accumulator of the same group into its own fp32 registers.  The two
        // threads that share a row (one per group) add their partial sums in the epilogue.
        const int quarter = warp & 3;
        const int gi = (warp >> 2) & 1;
        const int wg = warp >> 3;
        const int t = quarter * 32 + lane;      // row within the half = TMEM lane
        const int rt = wg * kHalfRows + t;      // row within the tile
        const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t a_t = tmem_base + lane_sel + wg * 128 + gi * 64;
        const uint32_t d_t = tmem_base + lane_sel + 256 + wg * 64 + gi * 32;
        // byte offsets of this thread's four 16-byte chunks inside a stage (128B-swizzled rows)
        uint32_t w_off[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) w_off[c] = wg * kWHalfBytes + t * kStageRowBytes + (((gi * 4 + c) ^ (t & 7)) << 4);
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t full0 = smem_u32(&ctrl->full[0]);
        const uint32_t empty0 = smem_u32(&ctrl->empty[0]);
        const uint32_t afull = smem_u32(&ctrl->a_full[wg][gi]);
        const uint32_t dfull = smem_u32(&ctrl->d_full[wg][gi]);

        float acc[NREAD];
        uint32_t n = 0;  // stages processed by this CTA so far
        bool ok = true;
        // This thread's progress through the two cluster barriers: arrive A, wait A, arrive B, wait B.
        int cl_steps = 0;
        // Barrier among the sixteen consumer warps with a bounded wait (a plain bar.sync would hang the CTA
        // if one warp had given up on a wait and left): false when the CTA is aborting.
        const uint32_t epi_bar = smem_u32(&ctrl->epi);
        uint32_t epi_phase = 0;
        auto consumer_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_bar);
            const bool r = mbar_wait(epi_bar, epi_phase, abort_flag);
            epi_phase ^= 1u;
            if (!r) ok = false;
            return r;
        };

        // acc += scale * D: the accumulator tile of this warp's group, 16 columns at a time
        // (D alternates between two accumulator tiles, 128 columns apart, so that the tile of stage n - 1 can
        // still be read out while the MMAs of stage n run)
        auto fold = [&](const float scale, const uint32_t buf) {
            const uint32_t d_tb = d_t + buf * 128;
            if constexpr (NREAD == 8) {
                uint32_t d[8];
                tmem_ld8(d_tb, d);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(__uint_as_float(d[j]), scale, acc[j]);
            } else {
#pragma unroll
                for (int c = 0; c < NREAD / 16; ++c) {
                    uint32_t d[16];
                    tmem_ld16(d_tb + c * 16, d);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(__uint_as_float(d[j]), scale, acc[c * 16 + j]);
                }
            }
        };

        long long u = u_begin;
        while (u < u_end && ok) {
            const int tile = static_cast<int>(u / S);
            const int s0 = static_cast<int>(u - static_cast<long long>(tile) * S);
            const int s1 = static_cast<int>(min(static_cast<long long>(S), s0 + (u_end - u)));
            const TileInfo ti = locate_tile(p, tile);
            const Seg& sg = p.seg[p.swiglu ? wg : ti.seg];
            const int my_row = p.swiglu ? ti.row0 + t : ti.row0 + rt;
            const bool valid = my_row < sg.n;
            const int my_col = p.y_perm ? perm8(my_row) : my_row;  // where this feature's outputs go within a Y row
            const __half* my_scales = sg.scales + static_cast<long long>(valid ? my_row : 0) * p.groups;
            const int gmax = valid ? p.groups : 0;  // scale index limit; rows beyond N use scale 0
            // A row's scales are 2 bytes per 128 k, far apart from its neighbours': behind a saturated weight
            // stream a miss on them waits microseconds.  Pull this tile's (first tile of the CTA only) and
            // the next tile's scale bytes into L2 now, so the loads in the loop only ever see L2 latency.
            if (gi == 0) {
                if (u == u_begin && valid) prefetch_l2_range(my_scales + 2 * s0, (min(2 * s1, gmax) - 2 * s0) * 2);
                const long long u_next = u + (s1 - s0);
                if (u_next < u_end) {
                    const TileInfo tn = locate_tile(p, tile + 1);
                    const Seg& sn = p.seg[p.swiglu ? wg : tn.seg];
                    const int row_n = p.swiglu ? tn.row0 + t : tn.row0 + rt;
                    const int s1n = static_cast<int>(min(static_cast<long long>(S), u_end - u_next));
                    if (row_n < sn.n)
                        prefetch_l2_range(sn.scales + static_cast<long long>(row_n) * p.groups, min(2 * s1n, p.groups) * 2);
                }
            }

#pragma unroll
            for (int j = 0; j < NREAD; ++j) acc[j] = 0.f;

            // The scale of this warp's group is fetched two stages ahead as a raw 16-bit value and only
            // converted when its stage starts, so the load latency never sits in the loop's critical path.
            // The loop's bookkeeping is kept to running pointers and counters: the SM is issue-bound here and
            // every instruction of a consumer warp is paid sixteen-fold.
            const unsigned short* sp = reinterpret_cast<const unsigned short*>(my_scales) + 2 * s0 + gi;  // this stage's scale
            // stages [s0, s_lim) have a scale for this thread (none for rows beyond N; K/128 odd: group 1 of the last)
            const int s_lim = min(s1, (gmax - gi + 1) >> 1);
            float sc_pend = 0.f;
            uint32_t q0 = (s0 < s_lim) ? static_cast<uint32_t>(__ldg(sp)) : 0u;
            uint32_t q1 = (s0 + 1 < s_lim) ? static_cast<uint32_t>(__ldg(sp + 2)) : 0u;
            bool have_prev = false;
            uint32_t slot = n % C::kStages;                 // weight-ring slot and phase of stage n
            uint32_t full_phase = (n / C::kStages) & 1u;
            uint32_t dfull_phase = (n - 1) & 1u;            // phase of the previous stage's MMA completion
            const int s_last = (p.cluster > 1) ? s1 - 1 : -1;  // stage after which the cluster barrier is arrived at

            for (int s = s0; s < s1; ++s, ++n) {
                const float sc_cur = __half2float(__ushort_as_half(static_cast<unsigned short>(q0)));
                q0 = q1;
                q1 = 0u;
                if (s + 2 < s_lim) q1 = static_cast<uint32_t>(__ldg(sp + 4));
                sp += 2;

                if (!mbar_wait(full0 + slot * 8, full_phase, abort_flag)) { ok = false; break; }
                const uint32_t stage = smem_base + slot * kWStageBytes;
                uint4 v[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) v[c] = lds128(stage + w_off[c]);

                // The previous stage's MMAs of this group must be done before its A buffer is overwritten.
                // (Unpacking ahead of this wait was tried: the compiler re-reads and re-unpacks part of the words
                // after the wait to stay within the register budget, 20 % more instructions for no gain.)
                if (have_prev) {
                    if (!mbar_wait(dfull, dfull_phase, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                }
                dfull_phase ^= 1u;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t a[16];
                    dequant_word(v[c].x, a + 0);
                    dequant_word(v[c].y, a + 4);
                    tmem_st8(a_t + c * 16, a);
                    dequant_word(v[c].z, a + 8);
                    dequant_word(v[c].w, a + 12);
                    tmem_st8(a_t + c * 16 + 8, a + 8);
                }
                // this warp has read its weights of the stage
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + slot * 8);
                if (++slot == C::kStages) { slot = 0; full_phase ^= 1u; }
                if (s == s_last) {
                    // Last stage of this CTA's K range: its weight ring may now be overwritten by the other CTAs
                    // of the cluster.  Arriving here, not at the exchange, lets the read-out below overlap with
                    // waiting for them.
                    cluster_arrive();
                    cl_steps = 1;
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(afull);
                // previous stage's accumulator tile, read out while the MMA warp picks up this stage
                if (have_prev) fold(sc_pend, dfull_phase ^ 1u);
                sc_pend = sc_cur;
                have_prev = true;
            }
            if (!ok) break;
            // drain the tile's last stage (n already counts it)
            if (!mbar_wait(dfull, (n - 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            fold(sc_pend, (n - 1) & 1u);

            // ---------------------------------------------------------------- tile epilogue
            // Runs once per tile, so its instructions are cold in the instruction caches: the accumulators
            // are parked in shared memory and everything after that is written as rolled loops (a fully
            // unrolled epilogue cost ~10 us in instruction fetches alone).  The two threads of a row first
            // add their groups' partial sums there; afterwards they split the activation rows by parity.
            float* stage_acc = xchg;  // [NREAD][256] fp32, row rt's values at [j][rt]
            const int m_rows = p.m < NREAD ? p.m : NREAD;
            const bool whole = (s0 == 0 && s1 == S);
            const bool direct_xchg = !whole && p.cluster > 1 && p.xchg_direct;
            if (!direct_xchg) {
            if (!consumer_sync()) break;  // previous tile's readers of stage_acc are done
            if (gi == 0) {
#pragma unroll
                for (int j = 0; j < NREAD; ++j) stage_acc[j * kTileRows + rt] = acc[j];
            }
            if (!consumer_sync()) break;
            if (gi == 1) {
#pragma unroll
                for (int j = 0; j < NREAD; ++j) stage_acc[j * kTileRows + rt] += acc[j];
            }
            fence_proxy_async_smem();  // the copy engine may read the parked rows (split-K exchange)
            if (!consumer_sync()) break;
            }
            bool finish = whole;
            int j0 = gi, jstep = 2, jend = m_rows;  // activation rows this thread finishes: j0, j0 + jstep, ... < jend
            if (direct_xchg) {
                // K splits of one tile form a thread-block cluster.  CTA r of the cluster finishes a contiguous block
                // of activation rows (ceil(m / cluster) of them).  Every thread stores its fp32 partials straight from
                // its registers into the owner's shared memory (the weight ring, free once every CTA has arrived at
                // barrier A): [sender][group][row of the block][256 features].  One cluster barrier later the owner
                // adds the two groups of every sender and then the senders in rank order (deterministic).
                float* part = reinterpret_cast<float*>(smem);
                const uint32_t my_rank = cluster_ctarank();
                const uint32_t csz = static_cast<uint32_t>(p.cluster);
                const uint32_t rows_cap = (static_cast<uint32_t>(m_rows) + csz - 1) / csz;
                if (cl_steps == 0) { cluster_arrive(); cl_steps = 1; }
                cluster_wait();  // (A) every CTA of the cluster has finished reading its weight ring
                cl_steps = 2;
                {
                    const uint32_t local = smem_u32(part) + (((my_rank * 2 + gi) * rows_cap) * kTileRows + rt) * 4;
                    uint32_t owner = 0, jl = 0;
                    uint32_t dst = mapa_shared_cluster(local, 0);
#pragma unroll
                    for (int j = 0; j < NREAD; ++j) {
                        if (j < m_rows) {
                            st_shared_cluster_f32(dst, acc[j]);
                            dst += kTileRows * 4;
                            if (++jl == rows_cap) {
                                jl = 0;
                                ++owner;
                                dst = mapa_shared_cluster(local, owner < csz ? owner : 0);
                            }
                        }
                    }
                }
                cluster_arrive();  // (B) releases this thread's stores ...
                cl_steps = 3;
                cluster_wait();    // ... and acquires everyone's: this CTA's block is complete
                cl_steps = 4;
                {
                    const bool direct = !p.swiglu && valid;
                    const long long ldy = sg.ldy;
                    const float bias = (direct && sg.bias) ? sg.bias[my_row] : 0.f;
                    const uint32_t jfirst = my_rank * rows_cap;
                    uint32_t jlast = jfirst + rows_cap;
                    jlast = jlast > static_cast<uint32_t>(m_rows) ? static_cast<uint32_t>(m_rows) : jlast;
                    uint32_t j = jfirst + gi;
                    long long yoff = my_col + static_cast<long long>(j) * ldy;
                    uint32_t pa = smem_u32(part) + (gi * kTileRows + rt) * 4;  // row gi of the block, sender 0, group 0
                    const uint32_t gstep = rows_cap * (kTileRows * 4);           // group 0 -> group 1 of one sender
                    float* sa = stage_acc + j * kTileRows + rt;
#pragma unroll 1
                    for (; j < jlast; j += 2, pa += 2 * kTileRows * 4, yoff += 2 * ldy, sa += 2 * kTileRows) {
                        float sum = 0.f;
                        uint32_t a = pa;
#pragma unroll 2
                        for (uint32_t r = 0; r < csz; ++r, a += 2 * gstep) sum += lds_f32(a) + lds_f32(a + gstep);
                        if (direct) store_row<OutT>(p, sg, yoff, static_cast<int>(j), sum + bias);
                        else *sa = sum;
                    }
                    j0 = static_cast<int>(jfirst) + gi;
                    jend = static_cast<int>(jlast);
                    finish = p.swiglu != 0;  // plain projections are already written
                }
            } else if (!whole && p.cluster > 1) {
                // K splits of one tile form a thread-block cluster.  CTA r of the cluster finishes a contiguous
                // block of activation rows (ceil(m / cluster) of them): every CTA sends its fp32 partials of
                // that block, contiguous in the parked accumulators, into r's shared memory with ONE bulk copy
                // that counts its bytes on r's mbarrier, so r waits for exactly its incoming data.  It then sums
                // the `cluster` copies in rank order (deterministic).
                float* part = reinterpret_cast<float*>(smem);  // the weight ring, free once every CTA has arrived
                const uint32_t my_rank = cluster_ctarank();
                const uint32_t csz = static_cast<uint32_t>(p.cluster);
                const uint32_t rows_cap = (static_cast<uint32_t>(m_rows) + csz - 1) / csz;
                if (cl_steps == 0) { cluster_arrive(); cl_steps = 1; }
                cluster_wait();  // (A) every CTA of the cluster has finished reading its weight ring
                cl_steps = 2;
                if (warp == 0 && lane < static_cast<int>(csz)) {  // lane r sends the block owned by CTA r
                    int nr = m_rows - lane * static_cast<int>(rows_cap);
                    nr = nr > static_cast<int>(rows_cap) ? static_cast<int>(rows_cap) : nr;
                    if (nr > 0) {
                        const uint32_t dst = smem_u32(part) + (my_rank * rows_cap) * (kTileRows * 4);
                        bulk_copy_to_cluster(mapa_shared_cluster(dst, lane),
                                             smem_u32(stage_acc) + lane * rows_cap * (kTileRows * 4), nr * (kTileRows * 4),
                                             mapa_shared_cluster(smem_u32(&ctrl->red), lane));
                    }
                }
                if (!mbar_wait(smem_u32(&ctrl->red), 0u, abort_flag)) { ok = false; break; }
                // (B) this CTA has all its incoming rows, so the senders' sources may go away; waited for at exit
                cluster_arrive();
                cl_steps = 3;
                {
                    // this CTA's block of rows; the two threads of a tile row take every other one
                    const bool direct = !p.swiglu && valid;
                    const long long ldy = sg.ldy;
                    const float bias = (direct && sg.bias) ? sg.bias[my_row] : 0.f;
                    const uint32_t jfirst = my_rank * rows_cap;
                    uint32_t jlast = jfirst + rows_cap;
                    jlast = jlast > static_cast<uint32_t>(m_rows) ? static_cast<uint32_t>(m_rows) : jlast;
                    uint32_t j = jfirst + gi;
                    long long yoff = my_col + static_cast<long long>(j) * ldy;
                    uint32_t pa = smem_u32(part) + (gi * kTileRows + rt) * 4;
                    const uint32_t rstep = rows_cap * (kTileRows * 4);
                    float* sa = stage_acc + j * kTileRows + rt;
#pragma unroll 1
                    for (; j < jlast; j += 2, pa += 2 * kTileRows * 4, yoff += 2 * ldy, sa += 2 * kTileRows) {
                        float sum = 0.f;
                        uint32_t a = pa;
#pragma unroll 2
                        for (uint32_t r = 0; r < csz; ++r, a += rstep) sum += lds_f32(a);
                        if (direct) store_row<OutT>(p, sg, yoff, static_cast<int>(j), sum + bias);
                        else *sa = sum;
                    }
                    j0 = static_cast<int>(jfirst) + gi;
                    jend = static_cast<int>(jlast);
                    finish = p.swiglu != 0;  // plain projections are already written
                }
            } else if (!whole) {
                // tiles that straddle CTAs (one CTA per SM, units cut evenly): partials go through the scratch
                // buffer and the last CTA to arrive sums them in CTA order
                const int first_tile = static_cast<int>(u_begin / S);
                const int wslot = blockIdx.x * 2 + (tile == first_tile ? 0 : 1);
                float* ws = p.workspace + static_cast<long long>(wslot) * (32 * kTileRows);
#pragma unroll 4
                for (int j = gi; j < m_rows; j += 2) ws[j * kTileRows + rt] = stage_acc[j * kTileRows + rt];
                __threadfence();
                if (!consumer_sync()) break;
                const long long t_lo = static_cast<long long>(tile) * S;
                const int c_lo = unit_owner(t_lo, p.total_units, ctas);
                const int c_hi = unit_owner(t_lo + S - 1, p.total_units, ctas);
                if (tid == 0) {
                    const int old = atomicAdd(&p.counters[tile], 1);
                    ctrl->is_last = (old == c_hi - c_lo) ? 1 : 0;
                }
                if (!consumer_sync()) break;
                finish = ctrl->is_last != 0;
                if (finish) {
                    __threadfence();
                    // This thread's rows gi, gi + 2, ...: the partials of one CTA are fetched for all of them at
                    // once (independent loads in flight together), CTA after CTA in fixed order, so every sum is
                    // deterministic and the loop costs one memory latency per CTA instead of one per row.
                    float sums[NREAD / 2];
#pragma unroll
                    for (int q = 0; q < NREAD / 2; ++q) sums[q] = 0.f;
#pragma unroll 1
                    for (int c = c_lo; c <= c_hi; ++c) {
                        const int c_first_tile = static_cast<int>(unit_begin(c, p.total_units, ctas) / S);
                        const float* src = p.workspace + static_cast<long long>(c * 2 + (tile == c_first_tile ? 0 : 1)) *
                                                             (32 * kTileRows) + rt;
#pragma unroll
                        for (int q = 0; q < NREAD / 2; ++q)
                            if (gi + 2 * q < m_rows) sums[q] += __ldcg(src + (gi + 2 * q) * kTileRows);
                    }
#pragma unroll
                    for (int q = 0; q < NREAD / 2; ++q)
                        if (gi + 2 * q < m_rows) stage_acc[(gi + 2 * q) * kTileRows + rt] = sums[q];
                    if (tid == 0) p.counters[tile] = 0;
                }
            }
            if (finish) {
                if (p.swiglu) {
                    if (!consumer_sync()) break;  // the up half's values are visible to the gate half
                    if (wg == 0 && valid) {
                        const long long ldy = p.seg[0].ldy;
#pragma unroll 4
                        for (int j = j0; j < jend; j += jstep) {
                            const float g = stage_acc[j * kTileRows + t];
                            const float up = stage_acc[j * kTileRows + kHalfRows + t];
                            store_row<OutT>(p, p.seg[0], my_col + static_cast<long long>(j) * ldy, j,
                                            (g / (1.0f + expf(-g))) * up);
                        }
                    }
                } else if (valid) {
                    const long long ldy = sg.ldy;
                    const float b = sg.bias ? sg.bias[my_row] : 0.f;
#pragma unroll 4
                    for (int j = j0; j < jend; j += jstep)
                        store_row<OutT>(p, sg, my_col + static_cast<long long>(j) * ldy, j, stage_acc[j * kTileRows + rt] + b);
                }
            }
            u += (s1 - s0);
        }
        // every thread of a cluster passes both cluster barriers exactly once, also when a wait gave up
        if (p.cluster > 1) {
            __syncwarp();
            for (; cl_steps < 4; ++cl_steps) {
                if (cl_steps & 1) cluster_wait();
                else cluster_arrive();
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && ctrl->ws.abort_flag) atomicExch(p.status, kStatusWaitTimeout);
    // N-split exchange: every store of this CTA is ordered before the barrier above; warp 0 publishes the CTA to
    // the peers, and in CTA 0 waits for theirs
    if (p.tp.world > 1 && warp == 0) tp_finish_exchange(p.tp, gridDim.x, blockIdx.x);
    if (warp == kMmaWarp) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

bool encode_w_map(CUtensorMap* map, const uint8_t* w, long long n, long long k) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k / 2)};
    const cuuint32_t box[2] = {kStageRowBytes, kHalfRows};
    const cuuint32_t estr[2] = {1, 1};
    return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_x_map(CUtensorMap* map, const __half* x, long long m, long long k, int nmma) {
    // A box of [nmma rows][64 k] lands as 128-byte rows whose 16-byte chunks are XOR-swizzled by the row
    // index: the canonical 128-byte-swizzled K-major layout of the MMA's shared-memory operand.  One row of
    // the box is one 128-byte request (a 16-byte-wide box would be one request per 8 elements).
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(nmma)};
    const cuuint32_t estr[2] = {1, 1};
    return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Chooses the decomposition and launches.  With at least one tile per SM the (tile, stage) units are cut
// evenly over one CTA per SM (tiles that straddle CTAs are summed through the scratch buffer).  With fewer
// tiles every tile is split into the same whole number of K ranges and those CTAs form a thread-block
// cluster that sums its partials through distributed shared memory; the split count is the largest one
// (at most 8, the portable cluster size) whose clusters are all co-resident in one wave.
struct Decomp {
    int ctas;
    int cluster;
};

// `max_clusters[cs]`: how many clusters of cs CTAs of the kernel can be resident at once.
Decomp choose_grid(int tiles, int stages, int num_sms, const int* max_clusters) {
    Decomp d{num_sms, 1};
    if (tiles >= num_sms) return d;
    int best = tiles;  // one CTA per tile, no split
    for (int cs = 2; cs <= 8 && cs <= stages; ++cs) {
        if (max_clusters[cs] < tiles) continue;  // would need a second wave
        if (tiles * cs > best && tiles * cs <= num_sms) { best = tiles * cs; d.cluster = cs; }
    }
    d.ctas = tiles * d.cluster;
    return d;
}

// One-time set-up of a kernel instantiation on the current device; returns its cluster occupancy table.
constexpr int kMaxDevices = 64;

template <int NMMA, int NREAD, typename OutT>
cudaError_t configure(const int** table) {
    auto kern = w4a16_tc_kernel<NMMA, NREAD, OutT>;
    // per device: the function attributes live in that device's context, and so does the occupancy table
    static bool configured[kMaxDevices];
    static int clusters[kMaxDevices][9];
    static std::mutex mu;
    int dev = 0;
    cudaError_t ge = cudaGetDevice(&dev);
    if (ge != cudaSuccess) return ge;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    int* max_clusters = clusters[dev];
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NMMA>::kSmemBytes);
        if (e != cudaSuccess) return e;
        // The in-kernel register re-split is balanced for exactly kLaunchRegs per thread at launch: with any
        // other allocation the consumers' request could block forever, so such a build is refused here.
        cudaFuncAttributes fa;
        e = cudaFuncGetAttributes(&fa, kern);
        if (e != cudaSuccess) return e;
        if (fa.numRegs != kLaunchRegs) return cudaErrorInvalidDeviceFunction;
        for (int cs = 1; cs <= 8; ++cs) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(cs * 64);
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = Cfg<NMMA>::kSmemBytes;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = cs;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { n = 0; cudaGetLastError(); }
            max_clusters[cs] = n;
        }
        configured[dev] = true;
    }
    *table = max_clusters;
    return cudaSuccess;
}

// The decomposition launch() would choose for a problem of `m` activation rows (which picks the instantiation).
cudaError_t decomp_for(long long m, bool out_f32, int tiles, int stages, int num_sms, Decomp* out) {
    const int* table = nullptr;
    cudaError_t e;
    if (m <= 8) e = out_f32 ? configure<16, 8, float>(&table) : configure<16, 8, __half>(&table);
    else if (m <= 16) e = out_f32 ? configure<16, 16, float>(&table) : configure<16, 16, __half>(&table);
    else e = out_f32 ? configure<32, 32, float>(&table) : configure<32, 32, __half>(&table);
    if (e != cudaSuccess) return e;
    *out = choose_grid(tiles, stages, num_sms, table);
    return cudaSuccess;
}

template <int NMMA, int NREAD, typename OutT>
cudaError_t launch(Params& p, int tiles, int num_sms, cudaStream_t stream) {
    auto kern = w4a16_tc_kernel<NMMA, NREAD, OutT>;
    const int* table = nullptr;
    cudaError_t ce = configure<NMMA, NREAD, OutT>(&table);
    if (ce != cudaSuccess) return ce;
    const Decomp d = choose_grid(tiles, p.stages, num_sms, table);
    const int ctas = d.ctas, cluster = d.cluster;
    p.cluster = cluster;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = Cfg<NMMA>::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cluster;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

bool pdl_enabled() {
    static const bool on = [] { const char* e = getenv("XINFER_PDL"); return !(e && atoi(e) == 0); }();
    return on;
}

// Test hooks: the clock limit of the device-side waits, and an activation stage index from which on the
// producer requests nothing (the kernel then leaves through its abort path).  Defaults: one second, off.
static long long g_wait_limit = kWaitLimitClocks;
long long tc_wait_limit() { return g_wait_limit; }
static int g_x_stage_limit = -1;
int tc_x_stage_limit() { return g_x_stage_limit; }
void tc_set_wait_hooks(long long limit_clocks, int withhold_x_from_stage) {
    g_wait_limit = limit_clocks > 0 ? limit_clocks : kWaitLimitClocks;
    g_x_stage_limit = withhold_x_from_stage;
}

// ------------------------------------------------------------------------------------ launch plan
// A caller that issues the same sequence of tensor-core launches over and over (the speculative step) records
// it once; afterwards every launch of the sequence knows which weights the next one will stream and asks L2
// for that launch's first stages while it drains.  The plan is only a hint: a call that does not match the
// recorded sequence switches it off.  A plan is an object: each decoder owns one and binds it to the calling
// thread around its launches; callers of the bare entry points share the process-wide default plan.
namespace {
struct PlanEntry {
    TcProj proj[kMaxSegs];
    int num;
    bool swiglu, out_f32;
    long long m, k;
};
}  // namespace
struct TcPlan {
    std::vector<PlanEntry> entries;
    bool recording = false, active = false;
    size_t cursor = 0;
};
namespace {
TcPlan g_default_plan;
thread_local TcPlan* t_plan = nullptr;
TcPlan& cur_plan() { return t_plan ? *t_plan : g_default_plan; }

PlanEntry make_entry(const TcProj* proj, int num, bool swiglu, bool out_f32, long long m, long long k) {
    PlanEntry e;
    memset(&e, 0, sizeof(e));
    const int cnt = swiglu ? 2 : num;
    for (int i = 0; i < cnt && i < kMaxSegs; ++i) e.proj[i] = proj[i];
    e.num = num;
    e.swiglu = swiglu;
    e.out_f32 = out_f32;
    e.m = m;
    e.k = k;
    return e;
}
bool same_launch(const PlanEntry& a, const PlanEntry& b) {
    return a.proj[0].w == b.proj[0].w && a.num == b.num && a.swiglu == b.swiglu && a.m == b.m && a.k == b.k;
}
}  // namespace

TcPlan* tc_plan_new() { return new (std::nothrow) TcPlan(); }
void tc_plan_delete(TcPlan* p) {
    if (t_plan == p) t_plan = nullptr;
    delete p;
}
TcPlan* tc_plan_bind(TcPlan* p) {
    TcPlan* prev = t_plan;
    t_plan = p;
    return prev;
}
void tc_plan_record_begin() {
    TcPlan& pl = cur_plan();
    pl.entries.clear();
    pl.recording = true;
    pl.active = false;
    pl.cursor = 0;
}
void tc_plan_record_end() {
    TcPlan& pl = cur_plan();
    pl.recording = false;
    pl.active = !pl.entries.empty();
    pl.cursor = 0;
}
void tc_plan_rewind() { cur_plan().cursor = 0; }
void tc_plan_clear() {
    TcPlan& pl = cur_plan();
    pl.entries.clear();
    pl.recording = pl.active = false;
    pl.cursor = 0;
}

namespace {
// Describes the first stages of `next` to the kernel of the current launch (Params::pf_*).
void fill_prefetch(Params& p, const PlanEntry& next, int num_sms) {
    p.pf_ctas = 0;
    if (next.m < 1 || next.m > 32 || next.k < 128 || (next.k % 128) != 0) return;
    const int cnt = next.swiglu ? 2 : next.num;
    int tiles = 0;
    for (int i = 0; i < cnt; ++i) {
        if (reinterpret_cast<uintptr_t>(next.proj[i].w) & 15) return;
        if (!encode_w_map(&p.pf_map[i], next.proj[i].w, next.proj[i].n, next.k)) return;
        p.pf_tile_begin[i] = tiles;
        if (next.swiglu) {
            if (i == 0) tiles += static_cast<int>((next.proj[0].n + kHalfRows - 1) / kHalfRows);
            else p.pf_tile_begin[i] = 0;
        } else {
            tiles += static_cast<int>((next.proj[i].n + kTileRows - 1) / kTileRows);
        }
    }
    const int stages = static_cast<int>((next.k / 128 + 1) / 2);
    Decomp d;
    if (decomp_for(next.m, next.out_f32, tiles, stages, num_sms, &d) != cudaSuccess) return;
    p.pf_num_segs = next.swiglu ? 1 : next.num;
    p.pf_swiglu = next.swiglu ? 1 : 0;
    p.pf_stages = stages;
    p.pf_total_units = static_cast<long long>(tiles) * stages;
    p.pf_ctas = d.ctas;
}
}  // namespace

size_t tc_workspace_bytes(int ctas) { return static_cast<size_t>(ctas) * 2 * 32 * kTileRows * sizeof(float); }

bool tc_eligible(const void* x, const TcProj* proj, int num, bool swiglu, long long m, long long k, int group_size) {
    if (group_size != 128 || m < 1 || m > 32 || k < 128 || (k % 128) != 0) return false;
    if (k / 8 > (1ll << 31) || (reinterpret_cast<uintptr_t>(x) & 15)) return false;
    if (encode_fn() == nullptr) return false;
    const int cnt = swiglu ? 2 : num;
    for (int i = 0; i < cnt; ++i) {
        if (proj[i].n < 1 || proj[i].n > (1ll << 30)) return false;
        if (reinterpret_cast<uintptr_t>(proj[i].w) & 15) return false;
    }
    return true;
}

// Launches the tensor-core kernel.  `scratch` holds tc_workspace_bytes(ctas) bytes of partials followed by
// `counter_capacity` zeroed ints; both are owned by the caller.  Returns 0, or a negative code when the
// problem cannot be described to the kernel (the caller then uses the CUDA-core path).
int tc_launch(cudaStream_t stream, const void* x, const TcProj* proj, int num, bool swiglu, bool out_f32,
              long long m, long long k, int num_sms, float* workspace, int* counters, int counter_capacity,
              int* status, const TpLink* tp, int layout_flags) {
    Params p;
    memset(&p, 0, sizeof(p));
    const int nmma = (m <= 16) ? 16 : 32;
    p.num_segs = swiglu ? 1 : num;
    p.swiglu = swiglu ? 1 : 0;
    p.m = static_cast<int>(m);
    p.groups = static_cast<int>(k / 128);
    p.stages = (p.groups + 1) / 2;
    int tiles = 0;
    const int cnt = swiglu ? 2 : num;
    for (int i = 0; i < cnt; ++i) {
        if (!encode_w_map(&p.w_map[i], proj[i].w, proj[i].n, k)) return -2;
        p.seg[i].scales = static_cast<const __half*>(proj[i].scales);
        p.seg[i].bias = proj[i].bias;
        p.seg[i].y = proj[i].y;
        p.seg[i].ldy = proj[i].ldy > 0 ? proj[i].ldy : proj[i].n;
        p.seg[i].n = static_cast<int>(proj[i].n);
        p.seg[i].push = (tp && tp->world > 1) ? proj[i].push : 0;
        for (int r = 0; r < kTpMaxWorld; ++r) p.seg[i].y_peer[r] = proj[i].y_peer[r];
        p.seg[i].tile_begin = tiles;
        if (swiglu) {
            if (i == 0) tiles += static_cast<int>((proj[0].n + kHalfRows - 1) / kHalfRows);
            else p.seg[i].tile_begin = 0;
        } else {
            tiles += static_cast<int>((proj[i].n + kTileRows - 1) / kTileRows);
        }
    }
    if (!encode_x_map(&p.x_map, static_cast<const __half*>(x), m, k, nmma)) return -2;
    if (tiles > counter_capacity) return -3;
    p.total_tiles = tiles;
    p.total_units = static_cast<long long>(tiles) * p.stages;
    p.workspace = workspace;
    p.counters = counters;
    p.status = status;
    p.wait_limit = g_wait_limit;
    p.x_perm = (layout_flags & kTcXPermuted) ? 1 : 0;
    p.y_perm = (layout_flags & kTcYPermuted) ? 1 : 0;
    if (p.y_perm)
        for (int i = 0; i < (swiglu ? 1 : num); ++i)
            if (proj[i].n & 7) return -2;  // whole blocks of eight features only
    if (tp && tp->world > 1) {
        if (tp->world > kTpMaxWorld || tp->rows_per_rank < 1 || num_sms > kTpMaxCtas) return -2;
        p.tp = *tp;
        if (!p.tp.status) p.tp.status = status;
        if (p.tp.wait_limit <= 0) p.tp.wait_limit = g_wait_limit;
    }
    p.x_stage_limit = g_x_stage_limit;
    // few activation rows: the partials go by plain remote stores (less latency than parking them and starting a
    // bulk copy per peer); more rows: the copy engine moves them (fewer instructions per CTA)
    p.xchg_direct = m <= 8 ? 1 : 0;
    TcPlan& pl = cur_plan();
    if (pl.recording) {
        pl.entries.push_back(make_entry(proj, num, swiglu, out_f32, m, k));
    } else if (pl.active) {
        const PlanEntry cur = make_entry(proj, num, swiglu, out_f32, m, k);
        if (pl.cursor < pl.entries.size() && same_launch(pl.entries[pl.cursor], cur)) {
            // (the last launch of the sequence looks ahead to the first one of the next round)
            fill_prefetch(p, pl.entries[(pl.cursor + 1) % pl.entries.size()], num_sms);
            ++pl.cursor;
        } else {
            pl.active = false;  // not the recorded sequence: no more hints
        }
    }
    cudaError_t e;
    if (m <= 8) e = out_f32 ? launch<16, 8, float>(p, tiles, num_sms, stream) : launch<16, 8, __half>(p, tiles, num_sms, stream);
    else if (m <= 16) e = out_f32 ? launch<16, 16, float>(p, tiles, num_sms, stream) : launch<16, 16, __half>(p, tiles, num_sms, stream);
    else e = out_f32 ? launch<32, 32, float>(p, tiles, num_sms, stream) : launch<32, 32, __half>(p, tiles, num_sms, stream);
    return e == cudaSuccess ? 0 : -1;
}

// ------------------------------------------------------------------------------------ allocation-free entry point
//
// Some hosts of this library may not allocate device memory once they are up and running: an inference
// server that has handed every free byte of HBM to its KV-cache pool, a process inside a container whose
// memory quota is already committed, or a caller that is in the middle of a CUDA-graph capture, where
// cudaMalloc is forbidden.  For them the fp16 -> fp16 linear is offered once more with its scratch (split-K
// partials, tile counters) living in a fixed array inside the library image instead of in a buffer from
// cudaMalloc.  The array is sized for up to kNoAllocMaxCtas CTAs and kNoAllocMaxTiles weight tiles; every
// GPU that loads the library holds these bytes until the process exits.
namespace {

constexpr int kNoAllocMaxCtas = 160;     // B200 has 148 SMs; one CTA per SM
constexpr int kNoAllocMaxTiles = 8192;   // 256-row tiles, i.e. N up to 2,097,152 output features
constexpr size_t kNoAllocPartialFloats = static_cast<size_t>(kNoAllocMaxCtas) * 2 * 32 * kTileRows;

struct NoAllocScratch {
    float partials[kNoAllocPartialFloats];  // 10,485,760 bytes
    int counters[kNoAllocMaxTiles];
    int status;
};
// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;

struct NoAllocDevice {
    NoAllocScratch* ptr = nullptr;
    int num_sms = 0;
};
NoAllocDevice g_noalloc_dev[kMaxDevices];
std::mutex g_noalloc_mutex;

// Once per device, with that device current: resolves the array's device address and configures the three
// fp16-output instantiations, so that later calls only enqueue work.
int noalloc_setup(int dev, NoAllocDevice** out) {
    NoAllocDevice& nd = g_noalloc_dev[dev];
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!nd.ptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            set_last_error(e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned no address");
            cudaGetLastError();
            return -1;
        }
        int sms = 0;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) {
            set_last_error(cudaGetErrorString(e));
            return -1;
        }
        const int* table = nullptr;
        if ((e = configure<16, 8, __half>(&table)) != cudaSuccess || (e = configure<16, 16, __half>(&table)) != cudaSuccess ||
            (e = configure<32, 32, __half>(&table)) != cudaSuccess) {
            set_last_error(cudaGetErrorString(e));
            return -1;
        }
        nd.num_sms = sms;
        nd.ptr = static_cast<NoAllocScratch*>(p);
    }
    *out = &nd;
    return 0;
}

}  // namespace

// Reads and clears the status word of the allocation-free entry point on `device` (0 when that entry point
// has not been used there).  The caller has made `device` current.
int tc_noalloc_take_status(int device) {
    if (device < 0 || device >= kMaxDevices) return 0;
    NoAllocScratch* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        ptr = g_noalloc_dev[device].ptr;
    }
    if (!ptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, &ptr->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v != 0) cudaMemset(&ptr->status, 0, sizeof(int));
    return v;
}
}  // namespace xb

extern "C" __attribute__((visibility("default"))) int xinfer_linear_int4_f16f16_noalloc(
    void* stream, void* Y_f16, const void* X_f16, const uint8_t* W_int4, const void* scales_f16, const float* bias,
    int64_t M, int64_t N, int64_t K, int group_size) {
    using namespace xb;
    if (M <= 0 || N <= 0 || K <= 0) return 1;  // XINFER_NOOP_INVALID_SHAPE, as the allocating entry point
    if (!Y_f16 || !X_f16 || !W_int4 || !scales_f16) return -2;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -6;
    NoAllocDevice* ndp = nullptr;
    if (noalloc_setup(dev, &ndp) != 0) return -1;
    NoAllocDevice& nd = *ndp;
    TcProj proj{Y_f16, W_int4, scales_f16, bias, N, 0};
    // sizes beyond the fixed scratch, or shapes the tensor-core kernel does not take, are refused: this entry
    // point has no second code path to fall back on
    if (nd.num_sms > kNoAllocMaxCtas) return -2;
    if (!tc_eligible(X_f16, &proj, 1, false, M, K, group_size)) return -2;  // needs 1 <= M <= 32, K % 128 == 0, group 128
    const long long tiles = (N + kTileRows - 1) / kTileRows;
    if (tiles > kNoAllocMaxTiles) return -2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call left.  The tile counters must start at zero (a call that ended in
    // a timeout may have left some set); the status word is NOT cleared here: it keeps a timeout on record
    // until xinfer_device_status() has reported it.
    cudaError_t e = cudaMemsetAsync(nd.ptr->counters, 0, static_cast<size_t>(tiles) * sizeof(int), s);
    if (e != cudaSuccess) { set_last_error(cudaGetErrorString(e)); return -1; }
    const int rc = tc_launch(s, X_f16, &proj, 1, false, false, M, K, nd.num_sms, nd.ptr->partials, nd.ptr->counters,
                             kNoAllocMaxTiles, &nd.ptr->status);
    if (rc == -1) set_last_error(cudaGetErrorString(cudaGetLastError()));
    return rc == 0 ? 0 : (rc == -1 ? -1 : -2);
}
