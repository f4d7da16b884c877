// Thin inline-PTX wrappers for the sm_100a features the hot-path kernels use: mbarriers with
// bounded waits, TMA tiled loads (no multicast anywhere), tensor memory (TMEM) allocation and
// access, tcgen05.mma issue/commit and the fences between the generic, async and tensor proxies.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xb {

// Default limit of every device-side wait, in SM clocks (about one second at 1.9 GHz).  A wait that
// gives up sets the CTA's abort flag, the kernel records an error status and returns.  The limit a
// kernel actually uses is a launch parameter (WaitState::limit).
constexpr long long kWaitLimitClocks = 2000000000LL;

// Shared by all waits of one CTA (lives in shared memory).  `dep_ready` is set once the CTA has seen the
// previous kernel of the stream complete (griddepcontrol.wait returned): a wait that runs out before
// that restarts its clock instead of giving up, so a long predecessor under programmatic dependent
// launch cannot cause a false timeout.
struct WaitState {
    int abort_flag;
    int dep_ready;
    long long limit;
};

enum DeviceStatus : int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

// One lane of a fully active warp (the same lane on every call): the lane that issues TMA or MMA
// instructions while the whole warp runs the surrounding warp-uniform code.
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// Re-split of the register file between warpgroups (executed by every warp of a warpgroup).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait ran out, or another one did).
// The poll loop is kept to the try_wait and one counter: every instruction it issues competes with the
// warps that have work, so the clock and the abort flag are only looked at every 256 polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile WaitState* ws) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int spins = 0; spins < 256; ++spins)
            if (mbar_try_wait(bar, parity)) return true;
        if (ws->abort_flag) return false;
        if (clock64() - t0 > ws->limit) {
            if (!ws->dep_ready) { t0 = clock64(); continue; }
            ws->abort_flag = 1;
            return false;
        }
    }
}

// Same bounded wait for threads that poll alone (TMA producer, MMA issuers): the try_wait carries a
// suspend-time hint, so the thread is parked by the hardware until the phase completes instead of
// spinning through issue slots the unpacking warps need.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile WaitState* ws) {
    if (mbar_try_wait_parked(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_parked(bar, parity)) return true;
        if (ws->abort_flag) return false;
        if (clock64() - t0 > ws->limit) {
            if (!ws->dep_ready) { t0 = clock64(); continue; }
            ws->abort_flag = 1;
            return false;
        }
    }
}

// ----------------------------------------------------------------------------- shared memory access
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// ----------------------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ----------------------------------------------------------------------------- programmatic dependent launch
// launch_dependents: the next kernel in the stream may start being scheduled (it will block in its own
// griddep_wait until this grid has completed and its memory is visible).  wait: block until the previous
// kernel in the stream has completed.  Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ----------------------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Cluster-wide barrier; every thread of every CTA in the cluster must call it the same number of times,
// each warp with all its lanes converged (.aligned).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves of the cluster barrier, for code that has useful work between arriving and waiting.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Asynchronous 4-byte store into another CTA's shared memory that, on landing, counts 4 bytes on an mbarrier
// of that CTA (both addresses in the shared::cluster window): the receiver waits on its own barrier only.
__device__ __forceinline__ void st_async_cluster_f32(uint32_t addr, float v, uint32_t remote_bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];" ::"r"(addr),
                 "r"(__float_as_uint(v)), "r"(remote_bar)
                 : "memory");
}
// Bulk copy of `bytes` (multiple of 16, 16-byte aligned) from this CTA's shared memory into another CTA's, done
// by the copy engine; on landing it counts the bytes on an mbarrier of the receiving CTA.  `dst` and
// `remote_bar` are shared::cluster addresses (mapa), `src` a shared::cta address.  The source must stay
// allocated until the receiver has seen the bytes.
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst, uint32_t src, uint32_t bytes, uint32_t remote_bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "r"(src), "r"(bytes), "r"(remote_bar)
                 : "memory");
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared_cluster(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_shared_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t addr) {
    float v;
    // volatile keeps it between the cluster barriers; no memory clobber, so a batch can be in flight together
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// ----------------------------------------------------------------------------- TMA (tiled, no multicast)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_prefetch_desc(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// The innermost coordinate times the element size must be a multiple of 16 bytes (callers pass
// byte offsets that are multiples of 128, or element offsets of 0).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, uint32_t bar, int x, int y,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
// Pulls one box of a tiled tensor into L2 without a destination in shared memory (nothing to wait for).
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)),
                 "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* map, uint32_t bar, int x, int y, int z,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        :
        : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}

// ----------------------------------------------------------------------------- tensor memory
// Allocation and release are warp-wide (.sync.aligned): one whole warp calls each.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Lane i of the calling warp writes r[0..7] to 8 consecutive 32-bit columns of TMEM lane
// (lane base of taddr + i).  (8 columns per store measured faster than 16 or 4.)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// ----------------------------------------------------------------------------- tcgen05.mma
// D[tmem] (+)= A[tmem] * B[smem descriptor], kind::f16, one CTA.  Issued by one thread.
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives once on the mbarrier when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// Shared-memory operand descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; `lbo` is
// the byte distance between the two core matrices of one K=16 step, `sbo` between 8-row groups.
__device__ __forceinline__ uint64_t umma_smem_desc_kmajor_noswizzle(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
    return d;
}
// Instruction descriptor: fp16 A and B, fp32 accumulate, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32(int m, int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ----------------------------------------------------------------------------- small math
__device__ __forceinline__ uint32_t lop3_6a(uint32_t a, uint32_t b, uint32_t c) {
    // b ? (a ^ c) : c
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// One little-endian u32 of packed int4 (nibble i <-> k+i, two's complement) -> four half2 registers
// holding the exact integers as fp16, in the order (k0,k4) (k1,k5) (k2,k6) (k3,k7).
// Bit-exact with the reference's (word << (28-4i)) >> 28 (src/ops/linear.cpp:100-110): the sign
// bit of each nibble is flipped inside the lop3 (q+8 in 0..15) and the result is or-ed under an fp16
// exponent whose ulp equals the nibble's lowest bit: 1024 for bits 0-3 (ulp 1), 64 for bits 4-7
// (ulp 1/16); subtracting the bias 1032 (or 72) leaves the signed integer exactly.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t* out4) {
    const uint32_t hi = w >> 8;
    out4[0] = hsub2_u32(lop3_6a(w, 0x000F000Fu, 0x64086408u), 0x64086408u);
    out4[1] = hsub2_u32(lop3_6a(w, 0x00F000F0u, 0x54805480u), 0x54805480u);
    out4[2] = hsub2_u32(lop3_6a(hi, 0x000F000Fu, 0x64086408u), 0x64086408u);
    out4[3] = hsub2_u32(lop3_6a(hi, 0x00F000F0u, 0x54805480u), 0x54805480u);
}

}  // namespace xb
