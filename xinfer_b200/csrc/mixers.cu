// Per-layer glue of the speculative decode / verify step: embedding lookup, RMSNorm (+ residual add),
// the full-attention mixer (q/k head norm, partial RoPE, KV-cache write, split-KV GQA attention over an
// fp16 cache, sigmoid output gate) and the Gated-DeltaNet mixer (causal conv1d + SiLU, gated delta-rule
// recurrence with fused gated RMSNorm).
//
// Semantics follow the reference's kernels; every fp16 rounding point of the reference is kept so
// that a CPU restatement of the reference agrees to the last fp16 bit in most elements:
//   embed_tokens_lookup            src/targets/qwen3_8/forward.cpp:17-64
//   rmsnorm                        src/ops/rmsnorm.cpp:15-82
//   add_inplace (fp16)             src/ops/elementwise.cpp:213-236
//   q/gate split, sigmoid gating   src/targets/qwen3_8/forward.cpp:145-151, 217-226
//   rope                           src/ops/rope.cpp:12-62
//   attention_write_kv_cache       src/ops/attention.cpp:84-116
//   sdpa_causal_cached             src/ops/attention.cpp:151-243
//   causal_conv1d_silu             src/targets/qwen3_8/linear_attn.cpp:37-122
//   recurrent_gated_delta_net      src/targets/qwen3_8/linear_attn.cpp:144-343
//
// What is different is the batching and the speculative state handling, which the reference does not
// have: rows are (sequence b, position i) with i < R, R = 1 while drafting and k+1 while verifying;
// sequence b sees keys below ctx[b] + i + 1; and the recurrent states (DeltaNet S, conv window) are
// committed lazily: a step stores its per-token updates, and the NEXT step first replays the
// n_commit[b] accepted ones onto the stored state, bit-identically, before it processes new tokens.
// Nothing is copied or restored when draft tokens are rejected.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <mutex>

#include "launch.cuh"
#include "mixers.h"

namespace xb {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Outputs that feed a W4A16 projection can be written with every block of eight features in the order the int4
// unpack yields them, (0,4,1,5,2,6,3,7), which saves the projection kernel its in-flight rewrite of the staged
// activations.  perm8: where feature n goes;  perm8_vec: eight consecutive features (one 16-byte vector) reordered.
__device__ __forceinline__ int perm8(int n) {
    const int k = n & 7;
    return (n & ~7) | ((k < 4) ? 2 * k : 2 * (k - 4) + 1);
}
__device__ __forceinline__ uint4 perm8_vec(const uint4& v) {
    // halves (h0 h1 | h2 h3 | h4 h5 | h6 h7) -> (h0 h4 | h1 h5 | h2 h6 | h3 h7)
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    return o;
}

// block-wide sum for up to 1024 threads; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? smem[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

// ------------------------------------------------------------------------------- embedding
__global__ void embed_kernel(__half* out, const uint16_t* table_bf16, const long long* tokens, int hidden, long long vocab) {
    griddep_prologue();
    const int row = blockIdx.x;
    const long long tok = tokens[row];
    const bool ok = tok >= 0 && (vocab <= 0 || tok < vocab);
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
        float v = 0.f;
        if (ok) v = __uint_as_float(static_cast<uint32_t>(table_bf16[tok * hidden + d]) << 16);
        out[static_cast<long long>(row) * hidden + d] = __float2half_rn(v);
    }
}

// ------------------------------------------------------------------------------- RMSNorm family
// mode 0: out = rmsnorm(in) * w
// mode 1: x = half(float(x) + float(delta)); out = rmsnorm(x) * w   (residual add, then norm)
// `out` may have a wider row (ld_out) and a column offset so that two norms can fill one concatenated row.
__global__ void __launch_bounds__(256) rmsnorm_kernel(__half* out, long long ld_out, __half* x, const __half* delta,
                                                      const float* w, int hidden, float eps, int perm_out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float red[32];
    const long long row = blockIdx.x;
    __half* xr = x + row * hidden;
    const __half* dr = delta ? delta + row * hidden : nullptr;
    __half* orow = out + row * ld_out;
    const int nvec = hidden >> 3;
    const bool vec_ok = (hidden & 7) == 0 && nvec <= 4 * 256 && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(orow) & 15) == 0) &&
                        (!dr || (reinterpret_cast<uintptr_t>(dr) & 15) == 0);
    if (vec_ok) {
        // The norm weights do not depend on the previous kernel in the stream: they are fetched before waiting
        // for it, so that only the activations' latency is left on the critical path.
        float4 wv[4][2];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int i = threadIdx.x + it * 256;
            if (i < nvec) {
                wv[it][0] = __ldg(reinterpret_cast<const float4*>(w + i * 8));
                wv[it][1] = __ldg(reinterpret_cast<const float4*>(w + i * 8 + 4));
            }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // one pass: each thread keeps its (up to four) 8-element vectors in registers
        uint4 v[4];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int i = threadIdx.x + it * 256;
            if (i < nvec) {
                v[it] = *reinterpret_cast<const uint4*>(xr + i * 8);
                __half2* h = reinterpret_cast<__half2*>(&v[it]);
                if (dr) {
                    const uint4 dv = *reinterpret_cast<const uint4*>(dr + i * 8);
                    const __half2* dh = reinterpret_cast<const __half2*>(&dv);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 a = __half22float2(h[j]), b = __half22float2(dh[j]);
                        h[j] = __halves2half2(__float2half_rn(a.x + b.x), __float2half_rn(a.y + b.y));
                    }
                    *reinterpret_cast<uint4*>(xr + i * 8) = v[it];
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 a = __half22float2(h[j]);
                    ss += a.x * a.x + a.y * a.y;
                }
            }
        }
        const float total = block_sum(ss, red);
        const float r = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int i = threadIdx.x + it * 256;
            if (i < nvec) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[it]);
                const float4 w0 = wv[it][0], w1 = wv[it][1];
                const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 a = __half22float2(h[j]);
                    oh[j] = __halves2half2(__float2half_rn(a.x * r * ww[2 * j]), __float2half_rn(a.y * r * ww[2 * j + 1]));
                }
                *reinterpret_cast<uint4*>(orow + i * 8) = perm_out ? perm8_vec(o) : o;
            }
        }
        return;
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = __half2float(xr[i]);
        if (dr) {
            const __half s = __float2half_rn(v + __half2float(dr[i]));
            xr[i] = s;
            v = __half2float(s);
        }
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float r = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        orow[(perm_out && (hidden & 7) == 0) ? perm8(i) : i] = __float2half_rn(__half2float(xr[i]) * r * w[i]);
}

// ------------------------------------------------------------------------------- attention prologue
// One block per (row, head slot); head slots 0..Hq-1 are query heads, Hq..Hq+Hkv-1 key heads,
// Hq+Hkv..Hq+2Hkv-1 value heads.  256 threads = head_dim.
// Generalisations used by the stand-alone op entry points: `q_head_stride` is the distance between query
// heads in q_in (512 for the interleaved [q | gate] block, 256 for plain queries); a null norm weight skips
// that head norm; `positions` (one per row) overrides ctx[b] + i; a null ctx means context length ctx_base; a
// null cache pointer skips the write (the rotated key then goes to k_out, if given).
__global__ void __launch_bounds__(256) attn_prep_kernel(__half* q_out, __half* k_cache, __half* v_cache,
                                                        const __half* q_gate, const __half* k_in, const __half* v_in,
                                                        const float* q_norm_w, const float* k_norm_w, const int* ctx,
                                                        int rows_per_seq, int hq, int hkv, long long max_seq,
                                                        float eps, float log_theta, int rope_dim, int q_head_stride,
                                                        const long long* positions, int ctx_base, __half* k_out,
                                                        int cache_batch) {
    griddep_prologue();
    __shared__ float red[32];
    __shared__ float vals[256];
    const int row = blockIdx.x;
    const int slot = blockIdx.y;
    const int d = threadIdx.x;
    const int b = row / rows_per_seq, i = row % rows_per_seq;
    const int bc = cache_batch > 0 ? b % cache_batch : b;  // the sequence whose cache this entry writes (see attn_decode_ex)
    const long long pos = positions ? positions[row] : static_cast<long long>(ctx ? ctx[b] : ctx_base) + i;
    const bool in_cache = pos >= 0 && pos < max_seq;
    if (slot >= hq + hkv) {  // value head: plain copy into the cache
        const int h = slot - hq - hkv;
        if (in_cache && v_cache && v_in)
            v_cache[((static_cast<long long>(bc) * max_seq + pos) * hkv + h) * 256 + d] =
                v_in[(static_cast<long long>(row) * hkv + h) * 256 + d];
        return;
    }
    const bool is_q = slot < hq;
    const int h = is_q ? slot : slot - hq;
    // the reference first copies q out of the interleaved [q | gate] head block (fp16, exact)
    const float x = is_q ? __half2float(q_gate[(static_cast<long long>(row) * hq + h) * q_head_stride + d])
                         : __half2float(k_in[(static_cast<long long>(row) * hkv + h) * 256 + d]);
    const float* w = is_q ? q_norm_w : k_norm_w;
    float normed = x;
    if (w) {
        const float total = block_sum(x * x, red);
        const float r = 1.0f / sqrtf(total / 256.0f + eps);
        // rounding point: the head RMSNorm writes fp16
        normed = __half2float(__float2half_rn(x * r * w[d]));
    }
    vals[d] = normed;
    __syncthreads();
    float outv = normed;
    const int half_rot = rope_dim / 2;
    if (d < rope_dim) {
        const int pair = d < half_rot ? d : d - half_rot;
        const float freq = expf(-static_cast<float>(2 * pair) * (1.0f / static_cast<float>(rope_dim)) * log_theta);
        const float angle = static_cast<float>(pos) * freq;
        const float c = cosf(angle), s = sinf(angle);
        const float v0 = vals[pair], v1 = vals[pair + half_rot];
        outv = d < half_rot ? v0 * c - v1 * s : v1 * c + v0 * s;
    }
    const __half o = __float2half_rn(outv);
    if (is_q) {
        q_out[(static_cast<long long>(row) * hq + h) * 256 + d] = o;
    } else if (k_cache) {
        if (in_cache) k_cache[((static_cast<long long>(bc) * max_seq + pos) * hkv + h) * 256 + d] = o;
    } else if (k_out) {
        k_out[(static_cast<long long>(row) * hkv + h) * 256 + d] = o;
    }
}

// ------------------------------------------------------------------------------- split-KV GQA attention
// Grid (splits, Hkv, B), 256 threads, two CTAs per SM.  Keys stream through shared memory in chunks of 32 via
// cp.async, double buffered, and both products are computed transposed so that the G * R query rows that share
// one KV head (G = Hq / Hkv, at most 32 rows) sit on the N side of mma.sync m16n8k16, eight rows per tile, and
// nothing is padded to 16:
//   S^T = K Q^T   warp (kq, kt) owns the keys [16 kt, 16 kt + 16) of the chunk and the head dims
//                 [64 kq, 64 kq + 64); its slice of Q stays in registers as B fragments for the whole kernel,
//                 so a chunk costs one read of K from shared memory and no read of Q; the four partial sums
//                 over kq meet in shared memory, where the softmax threads add them;
//   O^T += V^T P^T  warp w owns the output dims [32 w, 32 w + 32); V is read once per chunk (ldmatrix.trans).
// The kernel is bound by shared-memory bandwidth (two CTAs per SM share it): per 32 KB chunk this layout moves
// about 100 KB through shared memory where the untransposed one moved 165 KB.
// Each CTA writes an unnormalised partial (max, sum, O) per row.
constexpr int kAttnChunk = 32;
constexpr int kAttnStages = 2;  // the loop below is written for exactly two slots
constexpr int kAttnThreads = 256;
constexpr int kAttnLd = 264;  // padded row of 256 halves (528 B): conflict-free ldmatrix
constexpr int kAttnRows = 32;
constexpr int kAttnSpLd = 36;  // row pitch (floats) of the score planes: 2 * 36 = 8 mod 32 makes the MMA threads' stores
                               // conflict-free, 144-byte rows let a softmax thread fetch its four keys with one 16-byte load

struct AttnSmem {
    __half q[kAttnRows][kAttnLd];
    __half k[kAttnStages][kAttnChunk][kAttnLd];
    __half v[kAttnStages][kAttnChunk][kAttnLd];
    float sp[4][kAttnRows][kAttnSpLd];  // score partial sums over the four dim quarters, [query row][key]
    __half p[kAttnRows][kAttnChunk + 8];
    float row_max[kAttnRows];   // running maximum of scale * log2(e) * score (the softmax runs in base 2)
    float row_sum[kAttnRows];
    float row_alpha[kAttnRows];
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t* r, const void* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t* r, const void* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// NT = number of 8-row tiles that hold query rows (1..4): arrays and loops are sized for it at compile time.
template <int NT>
__global__ void __launch_bounds__(kAttnThreads, 2) attn_split_kernel(float* part_o, float* part_ml, const __half* q,
                                                         const __half* k_cache, const __half* v_cache, const int* ctx,
                                                         int rows_per_seq, int hq, int hkv, long long max_seq,
                                                         float scale, int ctx_base, int cache_batch) {
    griddep_prologue();
    extern __shared__ __align__(16) uint8_t attn_smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(attn_smem_raw);
    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kq = warp >> 1, kt = warp & 1;  // S^T role: dim quarter, 16-key tile
    const int G = hq / hkv;
    const int nrows = G * rows_per_seq;  // valid query rows, row = g * R + i
    const int ctx_b = ctx ? ctx[b] : ctx_base;  // (null: the stand-alone entry point's host-side start position)
    const int bc = cache_batch > 0 ? b % cache_batch : b;
    const float scale2 = scale * 1.4426950408889634f;  // exp(x) = exp2(x * log2 e)
    long long total_keys = static_cast<long long>(ctx_b) + rows_per_seq;
    if (total_keys > max_seq) total_keys = max_seq;
    const int nchunks = static_cast<int>((total_keys + kAttnChunk - 1) / kAttnChunk);
    const int c_begin = static_cast<int>(static_cast<long long>(split) * nchunks / nsplit);
    const int c_end = static_cast<int>(static_cast<long long>(split + 1) * nchunks / nsplit);

    // stage the query rows (zero padded to 32)
    for (int idx = tid; idx < kAttnRows * 32; idx += kAttnThreads) {
        const int r = idx >> 5, seg = idx & 31;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) {
            const int g = r / rows_per_seq, i = r % rows_per_seq;
            const long long row = static_cast<long long>(b) * rows_per_seq + i;
            v = *reinterpret_cast<const uint4*>(q + (row * hq + kvh * G + g) * 256 + seg * 8);
        }
        *reinterpret_cast<uint4*>(&sm.q[r][seg * 8]) = v;
    }
    if (tid < kAttnRows) {
        sm.row_max[tid] = -INFINITY;
        sm.row_sum[tid] = 0.f;
    }

    // one cp.async group per chunk (an empty one past the split's end)
    auto load_chunk = [&](int c, int buf) {
        const long long key0 = static_cast<long long>(c) * kAttnChunk;
        if (c < c_end)
        for (int idx = tid; idx < kAttnChunk * 32; idx += kAttnThreads) {
            const int r = idx >> 5, seg = idx & 31;
            long long key = key0 + r;
            if (key >= total_keys) key = total_keys - 1;  // clamped rows are masked out below
            const long long off = ((static_cast<long long>(bc) * max_seq + key) * hkv + kvh) * 256 + seg * 8;
            cp_async16(&sm.k[buf][r][seg * 8], k_cache + off);
            cp_async16(&sm.v[buf][r][seg * 8], v_cache + off);
        }
        cp_async_commit();
    };

    // O^T accumulators: [16-dim tile][8-row tile]; element e of a tile is (dim g4 + 8 (e >> 1), row 2 t4 + (e & 1))
    float o_acc[2][NT][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o_acc[mi][nt][e] = 0.f;

    for (int i = 0; i < kAttnStages - 1; ++i) load_chunk(c_begin + i, i);

    // this warp's slice of Q (all rows, dims [64 kq, 64 kq + 64)) as B fragments, read once
    __syncthreads();
    uint32_t qf[4][NT][2];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            ldmatrix_x2(qf[ks][nt], &sm.q[nt * 8 + (lane & 7)][kq * 64 + ks * 16 + ((lane >> 3) & 1) * 8]);

    for (int c = c_begin; c < c_end; ++c) {
        const int buf = (c - c_begin) % kAttnStages;
        // Chunk c has landed for every thread after this barrier, and every warp has finished the previous
        // chunk's P V: the other slot may be refilled.  (Three barriers per chunk; requesting the next chunk
        // before the wait instead would need a fourth one at the end of the iteration.)
        cp_async_wait<0>();
        __syncthreads();
        load_chunk(c + 1, (c - c_begin + 1) % kAttnStages);

        // S^T = K Q^T for this warp's 16 keys, summed over its 64 dims
        {
            float s_acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s_acc[nt][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t afr[4];
                ldmatrix_x4(afr, &sm.k[buf][kt * 16 + (lane & 15)][kq * 64 + ks * 16 + (lane >> 4) * 8]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    mma16816(s_acc[nt], afr, qf[ks][nt]);
            }
            const int g4 = lane >> 2, t4 = lane & 3;
            float* sp0 = &sm.sp[kq][t4 * 2][kt * 16 + g4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                {
                    // fragment element e: key g4 + 8 (e >> 1), query row 8 nt + 2 t4 + (e & 1)
                    sp0[(nt * 8) * kAttnSpLd] = s_acc[nt][0];
                    sp0[(nt * 8 + 1) * kAttnSpLd] = s_acc[nt][1];
                    sp0[(nt * 8) * kAttnSpLd + 8] = s_acc[nt][2];
                    sp0[(nt * 8 + 1) * kAttnSpLd + 8] = s_acc[nt][3];
                }
        }
        __syncthreads();

        // online softmax: 8 threads per row, 4 keys each
        {
            const int r = tid >> 3, part = tid & 7;
            const int i = r % rows_per_seq;
            const long long limit = static_cast<long long>(ctx_b) + i + 1;  // keys visible to this row
            const long long key0 = static_cast<long long>(c) * kAttnChunk + part * 4;
            float sc[4];
            float mx = -INFINITY;
            {
                // this thread's four keys of its row, one 16-byte load per dim quarter
                const float4 q0 = *reinterpret_cast<const float4*>(&sm.sp[0][r][part * 4]);
                const float4 q1 = *reinterpret_cast<const float4*>(&sm.sp[1][r][part * 4]);
                const float4 q2 = *reinterpret_cast<const float4*>(&sm.sp[2][r][part * 4]);
                const float4 q3 = *reinterpret_cast<const float4*>(&sm.sp[3][r][part * 4]);
                sc[0] = (q0.x + q1.x) + (q2.x + q3.x);
                sc[1] = (q0.y + q1.y) + (q2.y + q3.y);
                sc[2] = (q0.z + q1.z) + (q2.z + q3.z);
                sc[3] = (q0.w + q1.w) + (q2.w + q3.w);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool vis = (r < nrows) && (key0 + j < limit) && (key0 + j < total_keys);
                sc[j] = vis ? sc[j] * scale2 : -INFINITY;
                mx = fmaxf(mx, sc[j]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float old_max = sm.row_max[r];
            const float new_max = fmaxf(old_max, mx);
            float sum = 0.f;
            float pv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                pv[j] = (sc[j] == -INFINITY) ? 0.f : exp2f(sc[j] - new_max);
                sum += pv[j];
            }
            {
                const __half2 p01 = __floats2half2_rn(pv[0], pv[1]), p23 = __floats2half2_rn(pv[2], pv[3]);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&p01);
                packed.y = *reinterpret_cast<const uint32_t*>(&p23);
                *reinterpret_cast<uint2*>(&sm.p[r][part * 4]) = packed;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            __syncwarp();
            if (part == 0) {
                const float alpha = (old_max == -INFINITY) ? 0.f : exp2f(old_max - new_max);
                sm.row_alpha[r] = alpha;
                sm.row_sum[r] = sm.row_sum[r] * alpha + sum;
                sm.row_max[r] = new_max;
            }
        }
        __syncthreads();

        // O^T = alpha * O^T + V^T P^T for this warp's 32 output dims
        {
            const int t4 = lane & 3;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float a0 = sm.row_alpha[nt * 8 + t4 * 2], a1 = sm.row_alpha[nt * 8 + t4 * 2 + 1];
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    o_acc[mi][nt][0] *= a0;
                    o_acc[mi][nt][1] *= a1;
                    o_acc[mi][nt][2] *= a0;
                    o_acc[mi][nt][3] *= a1;
                }
            }
            // P^T as B fragments: one ldmatrix.x4 per 8-row tile fetches the chunk's 32 keys (both 16-key steps)
            uint32_t pall[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) ldmatrix_x4(pall[nt], &sm.p[nt * 8 + (lane & 7)][(lane >> 3) * 8]);
#pragma unroll
            for (int ks = 0; ks < kAttnChunk / 16; ++ks) {
                uint32_t pfr[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    pfr[nt][0] = pall[nt][2 * ks];
                    pfr[nt][1] = pall[nt][2 * ks + 1];
                }
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    // A = V^T: matrix j = lane >> 3 of the four 8x8 blocks is (dims + 8 (j & 1), keys + 8 (j >> 1)),
                    // stored key-major, hence the transposing load
                    uint32_t afr[4];
                    const int j = lane >> 3;
                    ldmatrix_x4_trans(afr, &sm.v[buf][ks * 16 + (j >> 1) * 8 + (lane & 7)][warp * 32 + mi * 16 + (j & 1) * 8]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        mma16816(o_acc[mi][nt], afr, pfr[nt]);
                }
            }
        }
    }
    cp_async_wait<0>();

    // write the partial: O [rows][256] fp32, (max in base-2 units, sum) per row
    const long long pbase = (static_cast<long long>(b) * hkv + kvh) * nsplit + split;
    float* po = part_o + pbase * (kAttnRows * 256);
    const int g4 = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = nt * 8 + t4 * 2 + (e & 1);
                const int col = warp * 32 + mi * 16 + g4 + (e >> 1) * 8;
                if (r < nrows) po[r * 256 + col] = o_acc[mi][nt][e];
            }
    if (tid < nrows) {
        part_ml[pbase * (kAttnRows * 2) + tid * 2] = sm.row_max[tid];
        part_ml[pbase * (kAttnRows * 2) + tid * 2 + 1] = sm.row_sum[tid];
    }
}

// Merge the splits, normalise, apply the sigmoid output gate, write fp16 [rows][Hq * 256].
// Grid (G * R, Hkv, B), 256 threads = head_dim.
__global__ void __launch_bounds__(256) attn_combine_kernel(__half* out, const float* part_o, const float* part_ml,
                                                           const __half* q_gate, int nsplit, int rows_per_seq, int hq,
                                                           int hkv, int perm_out) {
    griddep_prologue();
    const int r = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    const int G = hq / hkv;
    const int g = r / rows_per_seq, i = r % rows_per_seq;
    const long long pbase = (static_cast<long long>(b) * hkv + kvh) * nsplit;
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(pbase + s) * (kAttnRows * 2) + r * 2]);
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = part_ml[(pbase + s) * (kAttnRows * 2) + r * 2];
        if (ms == -INFINITY) continue;
        const float w = exp2f(ms - m);  // the partial maxima are in base-2 units
        l += part_ml[(pbase + s) * (kAttnRows * 2) + r * 2 + 1] * w;
        acc += part_o[(pbase + s) * (kAttnRows * 256) + r * 256 + d] * w;
    }
    const float inv = 1.0f / (l > 0.f ? l : 1.0f);
    const long long row = static_cast<long long>(b) * rows_per_seq + i;
    const int h = kvh * G + g;
    // rounding point: the reference's SDPA writes fp16, the gate then multiplies in fp32
    const float attn = __half2float(__float2half_rn(acc * inv));
    if (!q_gate) {  // plain SDPA (the stand-alone entry point): no output gate
        out[(row * hq + h) * 256 + d] = __float2half_rn(acc * inv);
        return;
    }
    const float gate = __half2float(q_gate[(row * hq + h) * 512 + 256 + d]);
    const float sig = 1.0f / (1.0f + expf(-gate));
    out[(row * hq + h) * 256 + (perm_out ? perm8(d) : d)] = __float2half_rn(attn * sig);
}

// ------------------------------------------------------------------------------- causal conv1d + SiLU
// One thread per (sequence, channel).  state [B][3][C] holds the last three committed inputs; pending
// [B][Rmax][C] the raw inputs of the previous step, of which the first n_commit[b] were accepted.
__global__ void conv1d_spec_kernel(__half* out, const __half* in, const float* conv_w, float* state, float* pending,
                                   const int* n_commit, int rows_per_seq, int prev_rows, int channels, int nc_base,
                                   int early_state) {
    // state, pending inputs and weights do not depend on the kernel in front of this one: they are read, and the
    // committed state written, before waiting for it (only `in` comes from that kernel).  early_state = 0: the
    // caller's previous launch wrote them, so everything waits.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!early_state) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= channels) return;
    float* st = state + static_cast<long long>(b) * 3 * channels;
    float* pd = pending + static_cast<long long>(b) * 8 * channels;
    float s0 = st[c], s1 = st[channels + c], s2 = st[2 * channels + c];
    int nc = n_commit ? n_commit[b] : nc_base;
    if (nc > prev_rows) nc = prev_rows;
    for (int i = 0; i < nc; ++i) {  // replay the accepted inputs of the previous step
        s0 = s1;
        s1 = s2;
        s2 = pd[i * channels + c];
    }
    st[c] = s0;
    st[channels + c] = s1;
    st[2 * channels + c] = s2;
    const float w0 = conv_w[c * 4], w1 = conv_w[c * 4 + 1], w2 = conv_w[c * 4 + 2], w3 = conv_w[c * 4 + 3];
    if (early_state) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < rows_per_seq; ++i) {
        const long long row = static_cast<long long>(b) * rows_per_seq + i;
        const float x = __half2float(in[row * channels + c]);
        const float sum = w0 * s0 + w1 * s1 + w2 * s2 + w3 * x;
        out[row * channels + c] = __float2half_rn(sum / (1.0f + expf(-sum)));
        pd[i * channels + c] = x;
        s0 = s1;
        s1 = s2;
        s2 = x;
    }
}

// ------------------------------------------------------------------------------- Gated DeltaNet recurrence
// Grid (v heads, B), 512 threads: thread (part, j) keeps rows [32 part, 32 part + 32) of column j of the
// 128 x 128 fp32 state in registers.  Everything that does not depend on the state (q/k L2 norms, beta, the
// decay factor) is computed for all tokens at once before the recurrence, and the gated RMSNorm of the
// outputs for all tokens after it, so the sequential part is one barrier and 64 FMAs per token.
// pend_k [B][Hv][8][128] normalised keys, pend_d [B][Hv][8][128] deltas, pend_g [B][Hv][8] decay factors of
// the previous step: replaying them touches each state element with the same two operations, in the same
// order, as the step that produced them, so the committed state is bit-identical.
__global__ void __launch_bounds__(512, 2) gdn_spec_kernel(__half* out, const __half* qkv, const __half* z,
                                                          const __half* bb, const __half* aa, const float* A_log,
                                                          const float* dt_bias, const float* norm_w, float* state,
                                                          float* pend_k, float* pend_d, float* pend_g,
                                                          const int* n_commit, int rows_per_seq, int prev_rows, int hv,
                                                          int hk, int nc_base, int early_state, int perm_out) {
    // The recurrent state, the previous step's pending updates and the per-head constants were written many
    // launches ago (by this layer's kernel of the previous pass, and by the commit at the end of the previous step):
    // they are fetched BEFORE waiting for the kernel in front of this one, so that the bulk of this kernel's memory
    // traffic overlaps the projection and convolution that precede it.  Only q/k/v/z/b/a come from those.
    // (early_state = 0: the caller's previous launch wrote the state - the stand-alone op entry point chaining
    // chunks of one sequence - so everything waits.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!early_state) asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ __align__(16) float sh_q[8][128], sh_k[8][128];
    __shared__ float sh_beta[8], sh_eg[8], red[2][16];
    __shared__ float part_sum[2][4][128], attn_all[8][4][128];
    const int h = blockIdx.x, b = blockIdx.y;
    const int j = threadIdx.x & 127, part = threadIdx.x >> 7;  // part doubles as the token group in phases 0 and 2
    const int lane = threadIdx.x & 31, wig = (threadIdx.x >> 5) & 3;
    const int i0 = part * 32;
    const int h_k = h / (hv / hk);
    const int channels = 2 * hk * 128 + hv * 128;
    const int value_dim = hv * 128;
    float* S = state + (static_cast<long long>(b) * hv + h) * (128 * 128);
    const long long pbase = (static_cast<long long>(b) * hv + h) * 8;
    float col[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) col[i] = S[(i0 + i) * 128 + j];
    const float exp_a_log = expf(A_log[h]);
    const float dtb = dt_bias[h];
    int nc = n_commit ? n_commit[b] : nc_base;
    if (nc > prev_rows) nc = prev_rows;
    if (early_state) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- phase 0: per-token quantities that do not depend on the state (token tt handled by thread group tt % 4)
    for (int t0 = 0; t0 < rows_per_seq; t0 += 4) {
        const int tt = t0 + part;
        float raw_q = 0.f, raw_k = 0.f;
        if (tt < rows_per_seq) {
            const __half* cur = qkv + (static_cast<long long>(b) * rows_per_seq + tt) * channels;
            raw_q = __half2float(cur[h_k * 128 + j]);
            raw_k = __half2float(cur[hk * 128 + h_k * 128 + j]);
        }
        const float wq = warp_sum(raw_q * raw_q), wk = warp_sum(raw_k * raw_k);
        __syncthreads();
        if (lane == 0) { red[0][part * 4 + wig] = wq; red[1][part * 4 + wig] = wk; }
        __syncthreads();
        if (tt < rows_per_seq) {
            const float q_sq = ((red[0][part * 4] + red[0][part * 4 + 1]) + red[0][part * 4 + 2]) + red[0][part * 4 + 3];
            const float k_sq = ((red[1][part * 4] + red[1][part * 4 + 1]) + red[1][part * 4 + 2]) + red[1][part * 4 + 3];
            sh_q[tt][j] = (raw_q * (1.0f / sqrtf(q_sq + 1e-6f))) * 0.08838834764f;
            sh_k[tt][j] = raw_k * (1.0f / sqrtf(k_sq + 1e-6f));
            if (j == 0) {
                const long long row = static_cast<long long>(b) * rows_per_seq + tt;
                const float b_val = __half2float(bb[row * hv + h]);
                sh_beta[tt] = 1.0f / (1.0f + expf(-b_val));
                const float a_val = __half2float(aa[row * hv + h]) + dtb;
                const float softplus = (a_val > 20.0f) ? a_val : logf(1.0f + expf(a_val));
                sh_eg[tt] = expf(-exp_a_log * softplus);
            }
        }
    }

    // ---- replay of the previous step's accepted updates, then write the committed state
    if (nc > 0) {
        for (int t = 0; t < nc; ++t) {
            const float eg = pend_g[pbase + t];
            const float dj = pend_d[(pbase + t) * 128 + j];
            const float* pk = pend_k + (pbase + t) * 128 + i0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float sv = col[i] * eg;
                col[i] = sv + __ldg(pk + i) * dj;
            }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) S[(i0 + i) * 128 + j] = col[i];
    }
    __syncthreads();  // phase 0 results visible; replay reads of pend_* are done before they are overwritten

    // ---- phase 1: the recurrence
    for (int t = 0; t < rows_per_seq; ++t) {
        const long long row = static_cast<long long>(b) * rows_per_seq + t;
        const float v = __half2float(qkv[row * channels + 2 * hk * 128 + h * 128 + j]);
        const float eg = sh_eg[t];
        float kv_mem = 0.f;
        const float4* k4 = reinterpret_cast<const float4*>(&sh_k[t][i0]);  // 16-byte broadcast reads
        const float4* q4 = reinterpret_cast<const float4*>(&sh_q[t][i0]);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const float4 kk = k4[m];
            const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float sv = col[m * 4 + e] * eg;
                col[m * 4 + e] = sv;
                kv_mem += sv * kv[e];
            }
        }
        part_sum[t & 1][part][j] = kv_mem;
        __syncthreads();
        const float* ps = &part_sum[t & 1][0][j];
        const float delta = (v - (((ps[0] + ps[128]) + ps[256]) + ps[384])) * sh_beta[t];
        float attn = 0.f;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const float4 kk = k4[m], qq = q4[m];
            const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float ns = col[m * 4 + e] + kv[e] * delta;
                col[m * 4 + e] = ns;
                attn += ns * qv[e];
            }
        }
        attn_all[t][part][j] = attn;
        if (part == 0) {
            pend_k[(pbase + t) * 128 + j] = sh_k[t][j];
            pend_d[(pbase + t) * 128 + j] = delta;
            if (j == 0) pend_g[pbase + t] = eg;
        }
    }
    __syncthreads();

    // ---- phase 2: gated RMSNorm of every token's output (token tt handled by thread group tt % 4)
    for (int t0 = 0; t0 < rows_per_seq; t0 += 4) {
        const int tt = t0 + part;
        float attn = 0.f;
        if (tt < rows_per_seq) attn = ((attn_all[tt][0][j] + attn_all[tt][1][j]) + attn_all[tt][2][j]) + attn_all[tt][3][j];
        const float wsq = warp_sum(attn * attn);
        __syncthreads();
        if (lane == 0) red[0][part * 4 + wig] = wsq;
        __syncthreads();
        if (tt < rows_per_seq) {
            const float sq = ((red[0][part * 4] + red[0][part * 4 + 1]) + red[0][part * 4 + 2]) + red[0][part * 4 + 3];
            const float inv_std = 1.0f / sqrtf(sq / 128.0f + 1e-6f);
            const long long row = static_cast<long long>(b) * rows_per_seq + tt;
            const float zv = __half2float(z[row * value_dim + h * 128 + j]);
            const float silu_z = zv / (1.0f + expf(-zv));
            out[row * value_dim + h * 128 + (perm_out ? perm8(j) : j)] = __float2half_rn(attn * inv_std * norm_w[j] * silu_z);
        }
    }
}

// ------------------------------------------------------------------------------- the same two mixers over a prompt chunk
// Prefill keeps every row, so there is nothing to replay or to hold back: the delta rule walks all `rc` positions of a
// chunk in one launch with the state in registers and writes the state back once (the step kernels above would need
// rc / 4 launches, each re-reading and re-writing the state).  Rows are found through chunk_row (the chunk's group-by-group row
// order).  Per token the arithmetic is the step kernels', operation by operation, so the results are bit-identical.
// The convolution has no recurrence on its outputs (y_p needs the inputs p-3 .. p only), so every (position, channel)
// is a thread of its own; inputs in front of the chunk come from the state.  A second, tiny launch then moves the
// chunk's last three inputs into the state (it must not run while the first one still reads the old state).
__global__ void conv1d_chunk_kernel(__half* out, const __half* in, const float* conv_w, const float* state, int rc, int channels) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y, batch = gridDim.y, p = blockIdx.z;
    if (c >= channels) return;
    const float* st = state + static_cast<long long>(b) * 3 * channels;
    float x[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int q = p - 3 + t;   // input position; negative: the state's slot 3 + q
        x[t] = q >= 0 ? __half2float(in[chunk_row(q, b, batch, rc) * channels + c]) : st[(3 + q) * channels + c];
    }
    const float w0 = conv_w[c * 4], w1 = conv_w[c * 4 + 1], w2 = conv_w[c * 4 + 2], w3 = conv_w[c * 4 + 3];
    const float sum = w0 * x[0] + w1 * x[1] + w2 * x[2] + w3 * x[3];
    out[chunk_row(p, b, batch, rc) * channels + c] = __float2half_rn(sum / (1.0f + expf(-sum)));
}
__global__ void conv1d_chunk_state_kernel(const __half* in, float* state, int rc, int channels) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y, batch = gridDim.y;
    if (c >= channels) return;
    float* st = state + static_cast<long long>(b) * 3 * channels;
    float s[3];
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int q = rc - 3 + t;   // the new slot t holds the input at position rc - 3 + t
        s[t] = q >= 0 ? __half2float(in[chunk_row(q, b, batch, rc) * channels + c]) : st[(3 + q) * channels + c];
    }
#pragma unroll
    for (int t = 0; t < 3; ++t) st[t * channels + c] = s[t];
}

__global__ void __launch_bounds__(512, 2) gdn_chunk_kernel(__half* out, const __half* qkv, const __half* z,
                                                           const __half* bb, const __half* aa, const float* A_log,
                                                           const float* dt_bias, const float* norm_w, float* state, int rc,
                                                           int hv, int hk) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ __align__(16) float sh_q[8][128], sh_k[8][128];
    __shared__ float sh_v[8][128], sh_z[8][128];
    __shared__ float sh_beta[8], sh_eg[8], red[2][8][4];
    __shared__ float part_sum[2][4][128], attn_all[8][4][128];
    const int h = blockIdx.x, b = blockIdx.y, batch = gridDim.y;
    const int j = threadIdx.x & 127, part = threadIdx.x >> 7;
    const int lane = threadIdx.x & 31, wig = (threadIdx.x >> 5) & 3;
    const int i0 = part * 32;
    const int h_k = h / (hv / hk);
    const int channels = 2 * hk * 128 + hv * 128;
    const int value_dim = hv * 128;
    float* S = state + (static_cast<long long>(b) * hv + h) * (128 * 128);
    float col[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) col[i] = S[(i0 + i) * 128 + j];
    const float exp_a_log = expf(A_log[h]);
    const float dtb = dt_bias[h];
    const float nw = norm_w[j];

    // Blocks of eight positions.  With one sequence per GPU a chunk is 512 sequential tokens on 48 SMs, so what counts
    // is the latency of a token: every global load of a block (q, k, v, z of its eight tokens; thread group `part`
    // takes tokens part and part + 4) is issued at the top of the block and staged in shared memory, and the norms of
    // all eight tokens share one barrier, so that the recurrence itself touches registers and shared memory only.
    for (int p0 = 0; p0 < rc; p0 += 8) {
        const int nb = rc - p0 < 8 ? rc - p0 : 8;
        // ---- phase 0: per-token quantities that do not depend on the state
        float raw_q[2] = {0.f, 0.f}, raw_k[2] = {0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tt = part + 4 * u;
            if (tt < nb) {
                const long long row = chunk_row(p0 + tt, b, batch, rc);
                const __half* cur = qkv + row * channels;
                raw_q[u] = __half2float(cur[h_k * 128 + j]);
                raw_k[u] = __half2float(cur[hk * 128 + h_k * 128 + j]);
                sh_v[tt][j] = __half2float(cur[2 * hk * 128 + h * 128 + j]);
                sh_z[tt][j] = __half2float(z[row * value_dim + h * 128 + j]);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tt = part + 4 * u;
            const float wq = warp_sum(raw_q[u] * raw_q[u]), wk = warp_sum(raw_k[u] * raw_k[u]);
            if (lane == 0) { red[0][tt][wig] = wq; red[1][tt][wig] = wk; }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tt = part + 4 * u;
            if (tt < nb) {
                const float q_sq = ((red[0][tt][0] + red[0][tt][1]) + red[0][tt][2]) + red[0][tt][3];
                const float k_sq = ((red[1][tt][0] + red[1][tt][1]) + red[1][tt][2]) + red[1][tt][3];
                sh_q[tt][j] = (raw_q[u] * (1.0f / sqrtf(q_sq + 1e-6f))) * 0.08838834764f;
                sh_k[tt][j] = raw_k[u] * (1.0f / sqrtf(k_sq + 1e-6f));
                if (j == 0) {
                    const long long row = chunk_row(p0 + tt, b, batch, rc);
                    const float b_val = __half2float(bb[row * hv + h]);
                    sh_beta[tt] = 1.0f / (1.0f + expf(-b_val));
                    const float a_val = __half2float(aa[row * hv + h]) + dtb;
                    const float softplus = (a_val > 20.0f) ? a_val : logf(1.0f + expf(a_val));
                    sh_eg[tt] = expf(-exp_a_log * softplus);
                }
            }
        }
        __syncthreads();

        // ---- phase 1: the recurrence
        for (int t = 0; t < nb; ++t) {
            const float v = sh_v[t][j];
            const float eg = sh_eg[t];
            float kv_mem = 0.f;
            const float4* k4 = reinterpret_cast<const float4*>(&sh_k[t][i0]);
            const float4* q4 = reinterpret_cast<const float4*>(&sh_q[t][i0]);
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const float4 kk = k4[m];
                const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float sv = col[m * 4 + e] * eg;
                    col[m * 4 + e] = sv;
                    kv_mem += sv * kv[e];
                }
            }
            part_sum[t & 1][part][j] = kv_mem;
            __syncthreads();
            const float* ps = &part_sum[t & 1][0][j];
            const float delta = (v - (((ps[0] + ps[128]) + ps[256]) + ps[384])) * sh_beta[t];
            float attn = 0.f;
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const float4 kk = k4[m], qq = q4[m];
                const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float ns = col[m * 4 + e] + kv[e] * delta;
                    col[m * 4 + e] = ns;
                    attn += ns * qv[e];
                }
            }
            attn_all[t][part][j] = attn;
        }
        __syncthreads();

        // ---- phase 2: gated RMSNorm of every token's output
        float attn2[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tt = part + 4 * u;
            attn2[u] = tt < nb ? ((attn_all[tt][0][j] + attn_all[tt][1][j]) + attn_all[tt][2][j]) + attn_all[tt][3][j] : 0.f;
            const float wsq = warp_sum(attn2[u] * attn2[u]);
            if (lane == 0) red[0][tt][wig] = wsq;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tt = part + 4 * u;
            if (tt < nb) {
                const float sq = ((red[0][tt][0] + red[0][tt][1]) + red[0][tt][2]) + red[0][tt][3];
                const float inv_std = 1.0f / sqrtf(sq / 128.0f + 1e-6f);
                const long long row = chunk_row(p0 + tt, b, batch, rc);
                const float zv = sh_z[tt][j];
                const float silu_z = zv / (1.0f + expf(-zv));
                out[row * value_dim + h * 128 + j] = __float2half_rn(attn2[u] * inv_std * nw * silu_z);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) S[(i0 + i) * 128 + j] = col[i];
}

// ------------------------------------------------------------------------------- speculative bookkeeping
struct AcceptRec {
    long long bonus;
    long long rejected;
    int num_accepted, num_rejected, num_resampled, num_remaining, has_rejected, pad;
};

// After acceptance: per sequence, publish the emitted tokens (accepted drafts then the bonus token),
// advance the context, remember how many recurrent updates to replay, pick the hidden row that feeds
// the next draft, and set the next step's first token.
__global__ void spec_commit_kernel(const AcceptRec* rec, const long long* draft_tokens, int k, int rows_per_seq,
                                   int* ctx, int* n_commit, long long* cur_tok, long long* emitted, int* emitted_n,
                                   __half* h_last, const __half* hidden_rows, int hidden) {
    griddep_prologue();
    const int b = blockIdx.x;
    const int na = rec[b].num_accepted;
    if (threadIdx.x == 0) {
        for (int i = 0; i < na; ++i) emitted[b * (k + 1) + i] = draft_tokens[b * k + i];
        emitted[b * (k + 1) + na] = rec[b].bonus;
        for (int i = na + 1; i < k + 1; ++i) emitted[b * (k + 1) + i] = -1;
        emitted_n[b] = na + 1;
        ctx[b] += na + 1;
        n_commit[b] = na + 1;
        cur_tok[b] = rec[b].bonus;
    }
    const __half* src = hidden_rows + (static_cast<long long>(b) * rows_per_seq + na) * hidden;
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) h_last[static_cast<long long>(b) * hidden + d] = src[d];
}

// rows of the verify pass: row (b, 0) = current token, rows (b, 1..k) = draft tokens
__global__ void build_verify_tokens_kernel(long long* out, const long long* cur_tok, const long long* draft, int k) {
    griddep_prologue();
    const int b = blockIdx.x, i = threadIdx.x;
    if (i == 0) out[b * (k + 1)] = cur_tok[b];
    else if (i <= k) out[b * (k + 1) + i] = draft[b * k + i - 1];
}

__global__ void fill_int_kernel(int* p, int n, int v) {
    griddep_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

__global__ void copy_token_column_kernel(long long* draft, const long long* argmax_out, int k, int col) {
    griddep_prologue();
    const int b = threadIdx.x + blockIdx.x * blockDim.x;
    draft[b * k + col] = argmax_out[b];
}

}  // namespace

#define XB_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -1)

int embed_rows(cudaStream_t s, __half* out, const void* table_bf16, const long long* tokens, int rows, int hidden,
               long long vocab) {
    launch_pdl(embed_kernel, dim3(rows), dim3(256), 0, s, out, static_cast<const uint16_t*>(table_bf16), tokens, hidden, vocab);
    return XB_LAUNCH_OK();
}

int rmsnorm_rows(cudaStream_t s, __half* out, long long ld_out, const __half* in, const float* w, int rows, int hidden,
                 float eps, int perm_out) {
    launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, s, out, ld_out, const_cast<__half*>(in), nullptr, w, hidden, eps, perm_out);
    return XB_LAUNCH_OK();
}

int add_rmsnorm_rows(cudaStream_t s, __half* out, __half* x, const __half* delta, const float* w, int rows, int hidden,
                     float eps, int perm_out) {
    launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, s, out, hidden, x, delta, w, hidden, eps, perm_out);
    return XB_LAUNCH_OK();
}

int attn_prep(cudaStream_t s, __half* q_out, __half* k_cache, __half* v_cache, const __half* q_gate, const __half* k_in,
              const __half* v_in, const float* q_norm_w, const float* k_norm_w, const int* ctx, int batch,
              int rows_per_seq, int hq, int hkv, long long max_seq, float eps, float rope_theta, int rope_dim) {
    return attn_prep_ex(s, q_out, k_cache, v_cache, q_gate, k_in, v_in, q_norm_w, k_norm_w, ctx, batch, rows_per_seq, hq, hkv,
                        max_seq, eps, rope_theta, rope_dim, 512, nullptr, 0, nullptr);
}

int attn_prep_ex(cudaStream_t s, __half* q_out, __half* k_cache, __half* v_cache, const __half* q_in, const __half* k_in,
                 const __half* v_in, const float* q_norm_w, const float* k_norm_w, const int* ctx, int batch,
                 int rows_per_seq, int hq, int hkv, long long max_seq, float eps, float rope_theta, int rope_dim,
                 int q_head_stride, const long long* positions, int ctx_base, __half* k_out, int cache_batch) {
    dim3 grid(batch * rows_per_seq, hq + 2 * hkv);
    launch_pdl(attn_prep_kernel, dim3(grid), dim3(256), 0, s, q_out, k_cache, v_cache, q_in, k_in, v_in, q_norm_w, k_norm_w, ctx,
               rows_per_seq, hq, hkv, max_seq, eps, logf(rope_theta), rope_dim, q_head_stride, positions, ctx_base, k_out, cache_batch);
    return XB_LAUNCH_OK();
}

size_t attn_scratch_bytes(int batch, int hkv, int nsplit) {
    return static_cast<size_t>(batch) * hkv * nsplit * (kAttnRows * 256 + kAttnRows * 2) * sizeof(float);
}

int attn_decode(cudaStream_t s, __half* out, const __half* q, const __half* q_gate, const __half* k_cache,
                const __half* v_cache, const int* ctx, int batch, int rows_per_seq, int hq, int hkv, long long max_seq,
                int nsplit, float* scratch) {
    return attn_decode_ex(s, out, q, q_gate, k_cache, v_cache, ctx, batch, rows_per_seq, hq, hkv, max_seq, nsplit, scratch,
                          1.0f / sqrtf(256.0f), 0, 0);
}

int attn_decode_ex(cudaStream_t s, __half* out, const __half* q, const __half* q_gate, const __half* k_cache,
                   const __half* v_cache, const int* ctx, int batch, int rows_per_seq, int hq, int hkv, long long max_seq,
                   int nsplit, float* scratch, float scale, int ctx_base, int perm_out, int cache_batch) {
    if (hq % hkv != 0 || (hq / hkv) * rows_per_seq > kAttnRows) return -2;
    // the shared-memory attribute belongs to the device's context: set it once per device
    static bool configured_dev[64];
    static std::mutex configured_mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    std::lock_guard<std::mutex> lock(configured_mu);
    if (!configured_dev[dev]) {
        const int bytes = static_cast<int>(sizeof(AttnSmem));
        if (cudaFuncSetAttribute(attn_split_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_split_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_split_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_split_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
            return -1;
        configured_dev[dev] = true;
    }
    float* part_o = scratch;
    float* part_ml = scratch + static_cast<size_t>(batch) * hkv * nsplit * (kAttnRows * 256);
    dim3 grid(nsplit, hkv, batch);
    switch (((hq / hkv) * rows_per_seq + 7) / 8) {
        case 1: launch_pdl(attn_split_kernel<1>, dim3(grid), dim3(kAttnThreads), sizeof(AttnSmem), s, part_o, part_ml, q, k_cache, v_cache, ctx, rows_per_seq, hq, hkv, max_seq, scale, ctx_base, cache_batch); break;
        case 2: launch_pdl(attn_split_kernel<2>, dim3(grid), dim3(kAttnThreads), sizeof(AttnSmem), s, part_o, part_ml, q, k_cache, v_cache, ctx, rows_per_seq, hq, hkv, max_seq, scale, ctx_base, cache_batch); break;
        case 3: launch_pdl(attn_split_kernel<3>, dim3(grid), dim3(kAttnThreads), sizeof(AttnSmem), s, part_o, part_ml, q, k_cache, v_cache, ctx, rows_per_seq, hq, hkv, max_seq, scale, ctx_base, cache_batch); break;
        default: launch_pdl(attn_split_kernel<4>, dim3(grid), dim3(kAttnThreads), sizeof(AttnSmem), s, part_o, part_ml, q, k_cache, v_cache, ctx, rows_per_seq, hq, hkv, max_seq, scale, ctx_base, cache_batch); break;
    }
    dim3 grid2((hq / hkv) * rows_per_seq, hkv, batch);
    launch_pdl(attn_combine_kernel, dim3(grid2), dim3(256), 0, s, out, part_o, part_ml, q_gate, nsplit, rows_per_seq, hq, hkv,
               (q_gate && perm_out) ? 1 : 0);
    return XB_LAUNCH_OK();
}

int conv1d_spec(cudaStream_t s, __half* out, const __half* in, const float* conv_w, float* state, float* pending,
                const int* n_commit, int batch, int rows_per_seq, int prev_rows, int channels, int nc_base, int early_state) {
    dim3 grid((channels + 255) / 256, batch);
    launch_pdl(conv1d_spec_kernel, dim3(grid), dim3(256), 0, s, out, in, conv_w, state, pending, n_commit, rows_per_seq, prev_rows, channels, nc_base, early_state);
    return XB_LAUNCH_OK();
}

int gdn_spec(cudaStream_t s, __half* out, const __half* qkv, const __half* z, const __half* b, const __half* a,
             const float* A_log, const float* dt_bias, const float* norm_w, float* state, float* pend_k, float* pend_d,
             float* pend_g, const int* n_commit, int batch, int rows_per_seq, int prev_rows, int hv, int hk, int nc_base,
             int early_state, int perm_out) {
    dim3 grid(hv, batch);
    launch_pdl(gdn_spec_kernel, dim3(grid), dim3(512), 0, s, out, qkv, z, b, a, A_log, dt_bias, norm_w, state, pend_k, pend_d, pend_g,
                                         n_commit, rows_per_seq, prev_rows, hv, hk, nc_base, early_state, perm_out);
    return XB_LAUNCH_OK();
}

int conv1d_chunk(cudaStream_t s, __half* out, const __half* in, const float* conv_w, float* state, int batch, int rc,
                 int channels) {
    if (rc <= 0) return 0;
    dim3 grid((channels + 255) / 256, batch, rc);
    launch_pdl(conv1d_chunk_kernel, dim3(grid), dim3(256), 0, s, out, in, conv_w, static_cast<const float*>(state), rc, channels);
    dim3 grid2((channels + 255) / 256, batch);
    launch_pdl(conv1d_chunk_state_kernel, dim3(grid2), dim3(256), 0, s, in, state, rc, channels);
    return XB_LAUNCH_OK();
}

int gdn_chunk(cudaStream_t s, __half* out, const __half* qkv, const __half* z, const __half* b, const __half* a,
              const float* A_log, const float* dt_bias, const float* norm_w, float* state, int batch, int rc, int hv, int hk) {
    dim3 grid(hv, batch);
    launch_pdl(gdn_chunk_kernel, dim3(grid), dim3(512), 0, s, out, qkv, z, b, a, A_log, dt_bias, norm_w, state, rc, hv, hk);
    return XB_LAUNCH_OK();
}

int spec_commit(cudaStream_t s, const void* accept_records, const long long* draft_tokens, int batch, int k,
                int rows_per_seq, int* ctx, int* n_commit, long long* cur_tok, long long* emitted, int* emitted_n,
                __half* h_last, const __half* hidden_rows, int hidden) {
    launch_pdl(spec_commit_kernel, dim3(batch), dim3(256), 0, s, static_cast<const AcceptRec*>(accept_records), draft_tokens, k, rows_per_seq,
                                             ctx, n_commit, cur_tok, emitted, emitted_n, h_last, hidden_rows, hidden);
    return XB_LAUNCH_OK();
}

int build_verify_tokens(cudaStream_t s, long long* out, const long long* cur_tok, const long long* draft, int batch,
                        int k) {
    launch_pdl(build_verify_tokens_kernel, dim3(batch), dim3(32), 0, s, out, cur_tok, draft, k);
    return XB_LAUNCH_OK();
}

int fill_int(cudaStream_t s, int* p, int n, int v) {
    launch_pdl(fill_int_kernel, dim3((n + 127) / 128), dim3(128), 0, s, p, n, v);
    return XB_LAUNCH_OK();
}

int copy_token_column(cudaStream_t s, long long* draft, const long long* argmax_out, int batch, int k, int col) {
    launch_pdl(copy_token_column_kernel, dim3(1), dim3(batch), 0, s, draft, argmax_out, k, col);
    return XB_LAUNCH_OK();
}

}  // namespace xb
