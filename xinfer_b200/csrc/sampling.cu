// Greedy argmax and speculative acceptance on the device.
//
// Contracts follow the reference:
//   argmax                      src/ops/sampling.cpp:12-92   strict '>' everywhere, so the lowest index
//                               of a tie wins; vocab <= 0 or null -> 0; vocab == 1 -> 0
//   speculative_accept_reject   src/ops/sampling.cpp:94-199  greedy rule, stochastic rule
//                               r < p_target / p_draft with p_target the softmax probability of the
//                               draft token, first rejection stops the scan and the replacement is the
//                               target's argmax at that row; all accepted -> bonus = argmax of a bonus row
// The reference walks the rows on the host with one argmax launch, one synchronisation and (in the
// stochastic branch) one device-to-host copy of the whole logit row per draft token.  Here one pass
// over the logits produces, per (row, chunk), the maximum, its lowest index, and the chunk's
// sum of exp(l * inv_temperature - chunk_max); a second tiny kernel merges the chunks per row
// (online-softmax merge), evaluates p_target and runs the accept scan for every sequence of the batch.
// Nothing returns to the host until the caller asks for the result.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "sampling.h"

namespace xb {

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 4096;  // logits per block: 256 threads x 4 float4

struct Partial {
    float max_raw;   // maximum raw logit of the chunk
    int idx;         // its lowest index (global)
    float max_scaled;
    float sum_exp;   // sum over the chunk of exp(l * inv_t - max_scaled)
};

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
    // strict '>' on the value; on equal values the lower index wins; an empty candidate never wins
    if (oi < 0) return;
    if (i < 0 || ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// Top-p bookkeeping (the nucleus kernel further down and the acceptance rule): the order-preserving 32-bit key of a
// scaled logit, and a token's integer weight rn(exp(s - max) * 2^32).
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// Coarse position of a scaled logit below the row's maximum: 64 buckets per unit, reversed (higher bin = higher
// logit), everything 32 or more below the maximum in bin 0 (its weight is zero anyway).  Monotone in the logit.
constexpr int kNucBuckets = 2048;
__device__ __forceinline__ int nucleus_bucket(float scaled, float max_scaled) {
    const float d = max_scaled - scaled;
    return d >= 31.99f ? 0 : (kNucBuckets - 1) - static_cast<int>(d * 64.0f);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
__device__ __forceinline__ unsigned long long nucleus_weight(float scaled, float max_scaled) {
    return __float2ull_rn(expf(scaled - max_scaled) * 4294967296.0f);
}

// grid = (chunks, rows).  `row_stride` is the distance between logit rows in floats.
__global__ void __launch_bounds__(kThreads) logits_partials_kernel(const float* __restrict__ logits, long long row_stride,
                                                                   int vocab, float inv_t, int want_sum,
                                                                   Partial* __restrict__ out, int chunks, int idx_offset) {
    const int row = blockIdx.y;
    const int chunk = blockIdx.x;
    const float* l = logits + static_cast<long long>(row) * row_stride;
    const int base = chunk * kChunk;
    const int end = min(vocab, base + kChunk);

    float vals[16];
    float best = -INFINITY;
    int best_i = -1;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(l) & 15) == 0);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i0 = base + (r * kThreads + threadIdx.x) * 4;
        if (vec_ok && i0 + 3 < end) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(l + i0));
            vals[r * 4 + 0] = v.x; vals[r * 4 + 1] = v.y; vals[r * 4 + 2] = v.z; vals[r * 4 + 3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) vals[r * 4 + j] = (i0 + j < end) ? __ldg(l + i0 + j) : -INFINITY;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int idx = i0 + j;
            if (idx < end) {
                if (best_i < 0 || vals[r * 4 + j] > best) { best = vals[r * 4 + j]; best_i = idx; }
            }
        }
    }
    // block argmax (value, lowest index)
    __shared__ float s_v[kThreads / 32];
    __shared__ int s_i[kThreads / 32];
    __shared__ float s_f[kThreads / 32];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
        better(best, best_i, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = best; s_i[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        float v = (lane < kThreads / 32) ? s_v[lane] : -INFINITY;
        int i = (lane < kThreads / 32) ? s_i[lane] : -1;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, off);
            const int oi = __shfl_xor_sync(0xffffffffu, i, off);
            better(v, i, ov, oi);
        }
        if (lane == 0) { s_v[0] = v; s_i[0] = i; }
    }
    __syncthreads();
    Partial res;
    res.max_raw = s_v[0];
    res.idx = s_i[0] < 0 ? -1 : s_i[0] + idx_offset;  // vocabulary slice of an N-split LM head: global token id
    res.max_scaled = 0.f;
    res.sum_exp = 0.f;
    if (want_sum) {
        // maximum of the scaled logits: scaling by a positive factor is monotone but may round two
        // values together, so take the maximum of the scaled values themselves
        float ms = -INFINITY;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int idx = base + ((r >> 2) * kThreads + threadIdx.x) * 4 + (r & 3);
            if (idx < end) ms = fmaxf(ms, vals[r] * inv_t);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ms = fmaxf(ms, __shfl_xor_sync(0xffffffffu, ms, off));
        __syncthreads();
        if (lane == 0) s_f[warp] = ms;
        __syncthreads();
        ms = s_f[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) ms = fmaxf(ms, s_f[w]);
        float se = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int idx = base + ((r >> 2) * kThreads + threadIdx.x) * 4 + (r & 3);
            if (idx < end) se += expf(vals[r] * inv_t - ms);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) se += __shfl_xor_sync(0xffffffffu, se, off);
        __syncthreads();
        if (lane == 0) s_f[warp] = se;
        __syncthreads();
        se = 0.f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) se += s_f[w];
        res.max_scaled = ms;
        res.sum_exp = se;
    }
    if (threadIdx.x == 0) out[static_cast<long long>(row) * chunks + chunk] = res;
}

// Optional mirror of the reference's per-256 partial arrays (src/ops/sampling.cpp:35-73): when the
// caller passes scratch, stage 1 results are also published there, one entry per chunk.
__global__ void publish_partials_kernel(const Partial* in, int chunks, float* partial_max, long long* partial_idx) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < chunks) {
        partial_max[i] = in[i].max_raw;
        partial_idx[i] = in[i].idx;
    }
}

// `p` points at the row's chunk partials of the first vocabulary slice; slice r's are r * slice_stride entries
// further (one slice per rank of an N-split LM head; nslices = 1 otherwise).
__device__ __forceinline__ void merge_row(const Partial* p, int chunks, int nslices, long long slice_stride, int lane,
                                          float& mx, int& idx, float& ms, float& se) {
    // one warp merges the chunk partials of one row
    mx = -INFINITY; idx = -1; ms = -INFINITY; se = 0.f;
    for (int c = lane; c < chunks * nslices; c += 32) {
        const Partial q = p[static_cast<long long>(c / chunks) * slice_stride + (c % chunks)];
        better(mx, idx, q.max_raw, q.idx);
        if (q.max_scaled > ms) { se = se * expf(ms - q.max_scaled) + q.sum_exp; ms = q.max_scaled; }
        else if (q.sum_exp > 0.f) se += q.sum_exp * expf(q.max_scaled - ms);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, mx, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        better(mx, idx, ov, oi);
        const float oms = __shfl_xor_sync(0xffffffffu, ms, off);
        const float ose = __shfl_xor_sync(0xffffffffu, se, off);
        const float nm = fmaxf(ms, oms);
        float a = (ms == -INFINITY) ? 0.f : se * expf(ms - nm);
        float b = (oms == -INFINITY) ? 0.f : ose * expf(oms - nm);
        se = a + b;
        ms = nm;
    }
}

__global__ void argmax_finish_kernel(const Partial* partials, int chunks, int nslices, long long slice_stride,
                                     long long* out) {
    const int row = blockIdx.x;
    float mx, ms, se;
    int idx;
    merge_row(partials + static_cast<long long>(row) * chunks, chunks, nslices, slice_stride, threadIdx.x, mx, idx, ms, se);
    if (threadIdx.x == 0) out[row] = idx < 0 ? 0 : idx;
}

// One warp per sequence.  Rows of sequence b are b * rows_per_seq + i.
__global__ void accept_finish_kernel(const Partial* partials, int chunks, int nslices, long long slice_stride,
                                     const float* logits, long long row_stride,
                                     int vocab, float inv_t, const long long* draft_tokens, const float* draft_probs,
                                     const float* uniforms, int num_draft, int rows_per_seq, int bonus_row,
                                     const Nucleus* nucleus, AcceptOut* out) {
    const int b = blockIdx.x;
    const int lane = threadIdx.x;
    AcceptOut r;
    r.num_accepted = 0;
    r.bonus_or_resampled_token = -1;
    r.rejected_token = -1;
    r.has_rejected_token = 0;
    r.num_rejected = 0;
    r.num_resampled = 0;
    r.num_remaining = 0;
    bool rejected = false;
    for (int i = 0; i < num_draft && !rejected; ++i) {
        const long long row = static_cast<long long>(b) * rows_per_seq + i;
        float mx, ms, se;
        int t;
        merge_row(partials + row * chunks, chunks, nslices, slice_stride, lane, mx, t, ms, se);
        const long long d = draft_tokens[static_cast<long long>(b) * num_draft + i];
        bool accepted;
        if (!draft_probs) {
            accepted = (d == t);
        } else {
            const float p_draft = draft_probs[static_cast<long long>(b) * num_draft + i];
            const float rr = uniforms ? uniforms[static_cast<long long>(b) * num_draft + i] : 0.f;
            if (p_draft <= 0.f) {
                accepted = (d == t);
            } else if (d == t && rr <= 0.f) {
                accepted = true;
            } else {
                float p_target = 0.f;
                if (nucleus) {
                    // the target's distribution cut to its nucleus: zero outside, w / Z_nucleus inside
                    const Nucleus q = nucleus[row];
                    if (d >= 0 && d < vocab && q.z > 0) {
                        const float sv = logits[row * row_stride + d] * inv_t;
                        if (order_key(sv) >= q.thr_key)
                            p_target = static_cast<float>(static_cast<double>(nucleus_weight(sv, q.max_scaled)) /
                                                          static_cast<double>(q.z));
                    }
                } else if (d >= 0 && d < vocab && se > 0.f) {
                    p_target = expf(logits[row * row_stride + d] * inv_t - ms) / se;
                }
                accepted = rr < (p_target / p_draft);
            }
        }
        if (accepted) {
            r.num_accepted++;
        } else {
            rejected = true;
            r.has_rejected_token = 1;
            r.rejected_token = d;
            r.num_rejected = 1;
            r.bonus_or_resampled_token = t;
            r.num_resampled = 1;
            r.num_remaining = num_draft - (r.num_accepted + 1);
        }
    }
    if (!rejected) {
        const long long row = static_cast<long long>(b) * rows_per_seq + bonus_row;
        float mx, ms, se;
        int t;
        merge_row(partials + row * chunks, chunks, nslices, slice_stride, lane, mx, t, ms, se);
        r.bonus_or_resampled_token = t;
    }
    if (lane == 0) out[b] = r;
}

// Philox4x32-10, Salmon et al. SC'11.  Uniform i of (seed, subsequence) is word (i & 3) of the block
// with counter {lo(i>>2), hi(i>>2), lo(subsequence), hi(subsequence)} and key {lo(seed), hi(seed)},
// mapped to [0, 1) as (word >> 8) * 2^-24.
__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

__global__ void philox_uniform_kernel(float* out, long long n, unsigned long long seed, unsigned long long subseq) {
    const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk * 4 >= n) return;
    uint32_t c[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(static_cast<unsigned long long>(blk) >> 32),
                     static_cast<uint32_t>(subseq), static_cast<uint32_t>(subseq >> 32)};
    philox4x32_10(c, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (blk * 4 + j < n) out[blk * 4 + j] = static_cast<float>(c[j] >> 8) * (1.0f / 16777216.0f);
}

// The same generator with the subsequence taken from device memory (a step counter that the step's own kernels advance),
// so that a replayed CUDA graph draws fresh numbers every replay.
__global__ void philox_uniform_counter_kernel(float* out, long long n, unsigned long long seed,
                                              const unsigned long long* subseq_dev) {
    const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk * 4 >= n) return;
    const unsigned long long subseq = *subseq_dev;
    uint32_t c[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(static_cast<unsigned long long>(blk) >> 32),
                     static_cast<uint32_t>(subseq), static_cast<uint32_t>(subseq >> 32)};
    philox4x32_10(c, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (blk * 4 + j < n) out[blk * 4 + j] = static_cast<float>(c[j] >> 8) * (1.0f / 16777216.0f);
}
__global__ void add_counter_kernel(unsigned long long* counter, unsigned long long v) { *counter += v; }

// Draws one token per row from softmax(logits * inv_t) by inverting the cumulative distribution at u * Z, in two
// levels: the chunk (of 4096 logits) from the chunk sums of logits_partials_kernel, taken in chunk order; inside the
// chunk every thread owns sixteen consecutive logits, the thread is found from the thread sums taken in thread order,
// the token from the thread's own running sum.  Every sum is a fixed sequence of fp32 additions, so a (logits, u)
// pair always gives the same token.  Also returns the token's probability exp(l * inv_t - max) / Z (the p_draft of
// the acceptance rule, src/ops/sampling.cpp:129-156).  One block per row.
__global__ void __launch_bounds__(kThreads) sample_finish_kernel(const Partial* partials, int chunks, const float* logits,
                                                                 long long row_stride, int vocab, float inv_t,
                                                                 const float* uniforms, int u_stride, long long* tok_out,
                                                                 float* prob_out, int prob_stride) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const Partial* P = partials + static_cast<long long>(row) * chunks;
    const float* l = logits + static_cast<long long>(row) * row_stride;
    __shared__ float s_m, s_z, s_rest;
    __shared__ int s_chunk, s_thread;
    __shared__ float s_local[kThreads], s_prefix;
    if (tid == 0) {
        float m = -INFINITY;
        for (int c = 0; c < chunks; ++c) m = fmaxf(m, P[c].max_scaled);
        float z = 0.f;
        for (int c = 0; c < chunks; ++c) z += P[c].sum_exp * expf(P[c].max_scaled - m);
        const float target = uniforms[static_cast<long long>(row) * u_stride] * z;
        float before = 0.f;
        int pick = chunks - 1;
        for (int c = 0; c < chunks; ++c) {
            const float w = P[c].sum_exp * expf(P[c].max_scaled - m);
            if (before + w > target) { pick = c; break; }
            if (c + 1 < chunks) before += w;
        }
        s_m = m; s_z = z; s_chunk = pick; s_rest = target - before;
    }
    __syncthreads();
    const float m = s_m;
    const int base = s_chunk * kChunk + tid * 16;
    float e[16];
    float local = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        e[j] = (base + j < vocab) ? expf(l[base + j] * inv_t - m) : 0.f;
        local += e[j];
    }
    s_local[tid] = local;
    __syncthreads();
    if (tid == 0) {
        const float rest = s_rest;
        float prefix = 0.f;
        int pick = 0;
        // the last thread that holds a logit takes what rounding leaves over
        int last = (min(vocab, (s_chunk + 1) * kChunk) - 1 - s_chunk * kChunk) / 16;
        for (int t = 0; t <= last; ++t) {
            pick = t;
            if (prefix + s_local[t] > rest || t == last) break;
            prefix += s_local[t];
        }
        s_thread = pick; s_prefix = prefix;
    }
    __syncthreads();
    if (tid == s_thread) {
        const float rest = s_rest;
        float cum = s_prefix;
        int pick = -1;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (base + j < vocab) {
                pick = j;
                cum += e[j];
                if (cum > rest) break;
            }
        }
        float pe = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j == pick) pe = e[j];
        tok_out[row] = base + pick;
        prob_out[static_cast<long long>(row) * prob_stride] = pe / s_z;
    }
}


// ------------------------------------------------------------------------------------ nucleus (top-p)
// The nucleus of a row is the smallest set of highest-probability tokens of softmax(l * inv_t) whose probabilities
// add up to at least top_p; tokens whose scaled logit equals the threshold's are all in.  Sums are integers: a
// token's weight is w = rn(exp(s - max) * 2^32) with s = l * inv_t in fp32, so every sum is exact, independent of
// the order of the additions, and the same on any machine that agrees on exp's bits.  The threshold is found by a
// four-level selection, each level one pass over the row that adds the weights of the still-undecided tokens into a
// histogram in shared memory and takes the bin in which the sum over all higher bins reaches ceil(top_p * Z): first
// 2048 buckets over the distance to the row's maximum (one pass over the row), then a radix selection on the
// order-preserving 32-bit key of s among the tokens of that bucket, which are gathered into shared memory first.  With a uniform u the kernel also
// draws the row's token: the first token, in index order, at which the running sum of the nucleus weights exceeds
// floor(u * Z_nucleus); its probability is w / Z_nucleus.  A cluster of eight 1024-thread CTAs per row.
constexpr int kNucThreads = 1024;

__device__ __forceinline__ unsigned long long shfl_u64(unsigned long long v, int src) {
    return __shfl_sync(0xffffffffu, v, src);
}

// Warp 0: the bin b (scanning from the highest bin down) at which the running sum first reaches `target`, and the
// sum of all bins above it.  `hist(b)` returns bin b; `nbins` is a multiple of 32; lane l owns the l-th highest block
// of nbins / 32 bins.
template <typename G>
__device__ __forceinline__ void find_bin_desc(G hist, int nbins, unsigned long long target, int lane, int* bin_out,
                                              unsigned long long* above_out) {
    const int per = nbins / 32;
    const int top = nbins - 1 - lane * per;  // highest bin of this lane
    unsigned long long mine = 0;
    for (int i = 0; i < per; ++i) mine += hist(top - i);
    unsigned long long incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const unsigned reach = __ballot_sync(0xffffffffu, incl >= target);
    const int who = reach ? __ffs(reach) - 1 : 31;
    if (lane == who) {
        unsigned long long cum = incl - mine;
        int b = top - (per - 1);
        for (int i = 0; i < per; ++i) {
            if (cum + hist(top - i) >= target || i == per - 1) { b = top - i; break; }
            cum += hist(top - i);
        }
        *bin_out = b;
        *above_out = cum;
    }
}

// f(i, scaled logit) for every token of [i0, i1): eight coalesced loads per thread are issued before the first of them
// is used, so that a pass is not one L2 round trip per element (the histogram atomics in f would otherwise keep the
// compiler from moving any load ahead of them).
template <typename F>
__device__ __forceinline__ void nucleus_for_each(const float* l, int i0, int i1, float inv_t, int tid, F f) {
    for (int base = i0; base < i1; base += 8 * kNucThreads) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * kNucThreads + tid;
            v[j] = i < i1 ? __ldg(l + i) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * kNucThreads + tid;
            if (i < i1) f(i, v[j] * inv_t);
        }
    }
}

// A row is shared by the eight CTAs of a thread-block cluster, each with a contiguous eighth of the token ids; CTA 0
// of the cluster (the leader) holds what the others contribute through distributed shared memory: the eight partial
// maxima and sums, the merged bucket histogram, the candidate list, and the results it hands back.  Every CTA passes
// every cluster barrier.
constexpr int kNucCluster = 8;
constexpr int kNucCand = 4096;

struct NucShared {
    unsigned long long hist[4096];   // bucket limbs (24 KB) / candidate keys (16 KB) + list histogram / row histograms
    unsigned long long wsum[32];
    unsigned long long csum[kNucCluster];   // leader: per-CTA sums
    float cmax[kNucCluster];                // leader: per-CTA maxima
    float wmax[32];
    unsigned long long above, target, z_nuc;   // leader: results of a level / of the selection
    int bin, count;
    uint32_t thr;
};

__global__ void __cluster_dims__(kNucCluster, 1, 1) __launch_bounds__(kNucThreads)
nucleus_kernel(const float* logits, long long row_stride, int vocab, float inv_t, float top_p, const float* uniforms,
               int u_stride, Nucleus* nuc_out, long long* tok_out, float* prob_out, int prob_stride) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ NucShared sh;
    const int crank = static_cast<int>(cluster.block_rank());
    const int row = blockIdx.x / kNucCluster, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* l = logits + static_cast<long long>(row) * row_stride;
    NucShared* lead = cluster.map_shared_rank(&sh, 0);
    // this CTA's token ids
    const int cspan = (((vocab + kNucCluster - 1) / kNucCluster) + 31) & ~31;
    const int c0 = min(vocab, crank * cspan), c1 = min(vocab, c0 + cspan);

    // maximum of the scaled logits
    float mx = -INFINITY;
    nucleus_for_each(l, c0, c1, inv_t, tid, [&](int, float sv) { mx = fmaxf(mx, sv); });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) sh.wmax[warp] = mx;
    for (int i = tid; i < 4096; i += kNucThreads) sh.hist[i] = 0;
    if (tid == 0) sh.count = 0;
    __syncthreads();
    if (tid == 0) {
        float m = sh.wmax[0];
        for (int w = 1; w < 32; ++w) m = fmaxf(m, sh.wmax[w]);
        lead->cmax[crank] = m;
    }
    cluster.sync();
    float ms = lead->cmax[0];
#pragma unroll
    for (int r = 1; r < kNucCluster; ++r) ms = fmaxf(ms, lead->cmax[r]);

    // level 0: total weight and a histogram over the distance to the maximum, 64 buckets per unit of scaled logit
    // (the keys themselves crowd into a few exponents: their top bits would send every token of the row to a
    // handful of bins, and shared-memory atomics on one address run one after the other).  The bucket index falls
    // as the scaled logit grows, so buckets are stored in reverse: a higher bin holds higher logits.
    // (64-bit adds on shared memory are compare-and-swap loops; a weight is below 2^33, so it goes in as three 11-bit
    // limbs with native 32-bit adds - a limb's sum over a whole row stays below 2^32 - and a bin is read back as
    // l0 + (l1 << 11) + (l2 << 22))
    unsigned long long z = 0;
    uint32_t* limb = reinterpret_cast<uint32_t*>(sh.hist);
    nucleus_for_each(l, c0, c1, inv_t, tid, [&](int, float sv) {
        const unsigned long long w = nucleus_weight(sv, ms);
        z += w;
        if (w) {
            const int bk = nucleus_bucket(sv, ms);
            atomicAdd(&limb[bk], static_cast<uint32_t>(w) & 0x7FFu);
            if (w >> 11) atomicAdd(&limb[kNucBuckets + bk], static_cast<uint32_t>(w >> 11) & 0x7FFu);
            if (w >> 22) atomicAdd(&limb[2 * kNucBuckets + bk], static_cast<uint32_t>(w >> 22));
        }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += shfl_u64(z, lane ^ o);
    if (lane == 0) sh.wsum[warp] = z;
    __syncthreads();
    if (tid == 0) {
        unsigned long long tot = 0;
        for (int w = 0; w < 32; ++w) tot += sh.wsum[w];
        lead->csum[crank] = tot;
    }
    cluster.sync();
    if (crank == 0) {
        // the leader adds the other CTAs' limbs to its own, then finds the bucket in which ceil(top_p * Z) is reached
        for (int i = tid; i < 3 * kNucBuckets; i += kNucThreads) {
            uint32_t acc = limb[i];
            for (int r = 1; r < kNucCluster; ++r)
                acc += reinterpret_cast<const uint32_t*>(cluster.map_shared_rank(&sh, r)->hist)[i];
            limb[i] = acc;
        }
        __syncthreads();
        if (warp == 0) {
            unsigned long long tot = 0;
            for (int r = 0; r < kNucCluster; ++r) tot += sh.csum[r];
            double want = ceil(static_cast<double>(top_p) * static_cast<double>(tot));
            unsigned long long target = want <= 1.0 ? 1ull : static_cast<unsigned long long>(want);
            if (target > tot) target = tot;
            if (lane == 0) sh.target = target;
            find_bin_desc(
                [&](int bk) -> unsigned long long {
                    return static_cast<unsigned long long>(limb[bk]) + (static_cast<unsigned long long>(limb[kNucBuckets + bk]) << 11) +
                           (static_cast<unsigned long long>(limb[2 * kNucBuckets + bk]) << 22);
                },
                kNucBuckets, target, lane, &sh.bin, &sh.above);
        }
    }
    cluster.sync();
    const int b0 = lead->bin;
    unsigned long long above = lead->above;
    unsigned long long target = lead->target - above;
    cluster.sync();   // (every CTA has read the leader's results and the leader has read every histogram)

    // The tokens of bucket b0 (a few dozen of a 150 000-token row, unless many logits are equal) are gathered into a
    // list of keys in the leader's shared memory; the exact threshold is then a radix selection on the keys of the
    // list (four levels of 8 bits), which costs no further pass over the row.  A bucket that does not fit the list is
    // selected from the row itself (12 + 12 + 8 bits, three passes, every CTA adding into the leader's histogram).
    uint32_t* cand = reinterpret_cast<uint32_t*>(lead->hist);
    nucleus_for_each(l, c0, c1, inv_t, tid, [&](int, float sv) {
        if (nucleus_bucket(sv, ms) == b0 && nucleus_weight(sv, ms)) {
            const int pos = atomicAdd(&lead->count, 1);
            if (pos < kNucCand) cand[pos] = order_key(sv);
        }
    });
    cluster.sync();
    const int count = lead->count;
    uint32_t prefix = 0;           // the key bits decided so far
    unsigned long long last = 0;   // weight of the threshold's own bin at the last level
    if (count <= kNucCand) {
        if (crank == 0) {
            unsigned long long* hh = sh.hist + kNucCand / 2;   // behind the 4096 keys
            const uint32_t* keys = reinterpret_cast<const uint32_t*>(sh.hist);
            for (int lvl = 0; lvl < 4; ++lvl) {
                const int shift = 24 - 8 * lvl;
                const uint32_t mask = lvl == 0 ? 0u : ~0u << (shift + 8);
                for (int i = tid; i < 256; i += kNucThreads) hh[i] = 0;
                __syncthreads();
                for (int q = tid; q < count; q += kNucThreads) {
                    const uint32_t k = keys[q];
                    if ((k & mask) == prefix) {
                        const unsigned long long w = nucleus_weight(key_to_float(k), ms);
                        if (w) atomicAdd(&hh[(k >> shift) & 0xFFu], w);
                    }
                }
                __syncthreads();
                if (warp == 0) find_bin_desc([&](int bin) { return hh[bin]; }, 256, target, lane, &sh.bin, &sh.above);
                __syncthreads();
                prefix |= static_cast<uint32_t>(sh.bin) << shift;
                above += sh.above;
                target -= sh.above;
                last = hh[sh.bin];
                __syncthreads();
            }
            if (tid == 0) { sh.thr = prefix; sh.z_nuc = above + last; }
        }
        cluster.sync();
    } else {
        const int shifts[3] = {20, 8, 0}, nbs[3] = {4096, 4096, 256};
        for (int lvl = 0; lvl < 3; ++lvl) {
            const int shift = shifts[lvl], nb = nbs[lvl];
            const uint32_t mask = lvl == 0 ? 0u : (lvl == 1 ? 0xFFF00000u : 0xFFFFFF00u);
            if (crank == 0)
                for (int i = tid; i < nb; i += kNucThreads) sh.hist[i] = 0;
            cluster.sync();
            nucleus_for_each(l, c0, c1, inv_t, tid, [&](int, float sv) {
                const uint32_t k = order_key(sv);
                if ((k & mask) == prefix && nucleus_bucket(sv, ms) == b0) {
                    const unsigned long long w = nucleus_weight(sv, ms);
                    if (w) atomicAdd(&lead->hist[(k >> shift) & static_cast<uint32_t>(nb - 1)], w);
                }
            });
            cluster.sync();
            if (crank == 0 && warp == 0)
                find_bin_desc([&](int bin) { return sh.hist[bin]; }, nb, target, lane, &sh.bin, &sh.above);
            cluster.sync();
            prefix |= static_cast<uint32_t>(lead->bin) << shift;
            above += lead->above;
            target -= lead->above;
            last = lead->hist[lead->bin];
            cluster.sync();
        }
        if (crank == 0 && tid == 0) { sh.thr = prefix; sh.z_nuc = above + last; }
        cluster.sync();
    }
    const uint32_t thr = lead->thr;
    const unsigned long long z_nuc = lead->z_nuc;
    if (crank == 0 && tid == 0 && nuc_out) {
        Nucleus q;
        q.z = z_nuc;
        q.max_scaled = ms;
        q.thr_key = thr;
        nuc_out[row] = q;
    }
    if (!uniforms) {
        cluster.sync();   // nobody leaves while the leader's shared memory is still being read
        return;
    }

    // draw: inside a CTA warp w owns the contiguous span [c0 + w * span, ...) of token ids and first adds up its nucleus
    // weights (lanes interleaved, loads coalesced); the one warp of the one CTA whose range of the running sum holds
    // floor(u * Z) then walks its span 32 tokens at a time with a warp scan, which visits the tokens in index order.
    const int span = (((c1 - c0) + 31) / 32 + 31) & ~31;
    const int w0 = min(c1, c0 + warp * span), w1 = min(c1, w0 + span);
    unsigned long long mine = 0;
    for (int base = w0; base < w1; base += 8 * 32) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * 32 + lane;
            v[j] = i < w1 ? __ldg(l + i) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * 32 + lane;
            const float sv = v[j] * inv_t;
            if (i < w1 && order_key(sv) >= thr) mine += nucleus_weight(sv, ms);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += shfl_u64(mine, lane ^ o);
    __syncthreads();
    if (lane == 0) sh.wsum[warp] = mine;
    __syncthreads();
    if (tid == 0) {
        unsigned long long tot = 0;
        for (int w = 0; w < 32; ++w) tot += sh.wsum[w];
        lead->csum[crank] = tot;
    }
    cluster.sync();
    unsigned long long before = 0;
    for (int r = 0; r < crank; ++r) before += lead->csum[r];
    for (int w = 0; w < warp; ++w) before += sh.wsum[w];
    double pos = floor(static_cast<double>(uniforms[static_cast<long long>(row) * u_stride]) * static_cast<double>(z_nuc));
    unsigned long long t2 = pos <= 0.0 ? 0ull : static_cast<unsigned long long>(pos);
    if (t2 >= z_nuc) t2 = z_nuc - 1;
    if (mine > 0 && before <= t2 && t2 < before + mine) {   // warp-uniform: exactly one warp of one CTA
        unsigned long long cum = before;
        for (int base = w0; base < w1; base += 32) {
            const int i = base + lane;
            unsigned long long w = 0;
            if (i < w1) {
                const float sv = __ldg(l + i) * inv_t;
                if (order_key(sv) >= thr) w = nucleus_weight(sv, ms);
            }
            unsigned long long incl = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, w > 0 && cum + incl > t2);
            if (hit) {
                const int src = __ffs(hit) - 1;
                if (lane == src) {
                    tok_out[row] = i;
                    prob_out[static_cast<long long>(row) * prob_stride] =
                        static_cast<float>(static_cast<double>(w) / static_cast<double>(z_nuc));
                }
                break;
            }
            cum += shfl_u64(incl, 31);
        }
    }
    cluster.sync();   // nobody leaves while the leader's shared memory is still being read
}

}  // namespace

int sampling_chunks(long long vocab) { return static_cast<int>((vocab + kChunk - 1) / kChunk); }
size_t sampling_scratch_bytes(long long rows, long long vocab) {
    return static_cast<size_t>(rows) * sampling_chunks(vocab) * sizeof(Partial);
}

int sampling_partials(cudaStream_t stream, const float* logits, long long row_stride, int rows, long long vocab,
                      float inv_temperature, bool want_sum, long long idx_offset, void* partials_out) {
    const int chunks = sampling_chunks(vocab);
    logits_partials_kernel<<<dim3(chunks, rows), kThreads, 0, stream>>>(
        logits, row_stride, static_cast<int>(vocab), inv_temperature, want_sum ? 1 : 0, static_cast<Partial*>(partials_out),
        chunks, static_cast<int>(idx_offset));
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int argmax_finish(cudaStream_t stream, const void* partials, int chunks, int nslices, long long slice_stride, int rows,
                  long long* out_dev) {
    argmax_finish_kernel<<<rows, 32, 0, stream>>>(static_cast<const Partial*>(partials), chunks, nslices, slice_stride, out_dev);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int accept_finish(cudaStream_t stream, const void* partials, int chunks, int nslices, long long slice_stride,
                  const float* logits, long long row_stride, long long vocab, float inv_temperature,
                  const long long* draft_tokens, const float* draft_probs, const float* uniforms, int batch,
                  int num_draft, int rows_per_seq, int bonus_row, AcceptOut* out_dev, const Nucleus* nucleus) {
    if (nslices > 1 && draft_probs) return -2;  // the stochastic rule reads the draft token's logit: one slice only
    accept_finish_kernel<<<batch, 32, 0, stream>>>(static_cast<const Partial*>(partials), chunks, nslices, slice_stride, logits,
                                                   row_stride, static_cast<int>(vocab), inv_temperature, draft_tokens,
                                                   draft_probs, uniforms, num_draft, rows_per_seq, bonus_row, nucleus, out_dev);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int argmax_rows(cudaStream_t stream, const float* logits, long long row_stride, int rows, long long vocab,
                void* scratch, long long* out_dev, float* partial_max, long long* partial_idx) {
    const int chunks = sampling_chunks(vocab);
    Partial* part = static_cast<Partial*>(scratch);
    if (sampling_partials(stream, logits, row_stride, rows, vocab, 1.0f, false, 0, part) != 0) return -1;
    if (partial_max && partial_idx && rows == 1)
        publish_partials_kernel<<<(chunks + 127) / 128, 128, 0, stream>>>(part, chunks, partial_max, partial_idx);
    return argmax_finish(stream, part, chunks, 1, 0, rows, out_dev);
}

int accept_reject_batched(cudaStream_t stream, const float* logits, long long row_stride, long long vocab,
                          float inv_temperature, const long long* draft_tokens, const float* draft_probs,
                          const float* uniforms, int batch, int num_draft, int rows_per_seq, int bonus_row,
                          void* scratch, AcceptOut* out_dev) {
    const int chunks = sampling_chunks(vocab);
    const int rows = batch * rows_per_seq;
    if (sampling_partials(stream, logits, row_stride, rows, vocab, inv_temperature, draft_probs != nullptr, 0, scratch) != 0)
        return -1;
    return accept_finish(stream, scratch, chunks, 1, 0, logits, row_stride, vocab, inv_temperature, draft_tokens,
                         draft_probs, uniforms, batch, num_draft, rows_per_seq, bonus_row, out_dev);
}

int philox_uniform(cudaStream_t stream, float* out, long long n, unsigned long long seed, unsigned long long subseq) {
    if (n <= 0) return 0;
    const long long blocks4 = (n + 3) / 4;
    philox_uniform_kernel<<<static_cast<unsigned>((blocks4 + 127) / 128), 128, 0, stream>>>(out, n, seed, subseq);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace xb

namespace xb {
int philox_uniform_counter(cudaStream_t stream, float* out, long long n, unsigned long long seed,
                           const unsigned long long* subseq_dev) {
    const long long blocks4 = (n + 3) / 4;
    if (blocks4 <= 0) return 0;
    philox_uniform_counter_kernel<<<static_cast<unsigned>((blocks4 + 127) / 128), 128, 0, stream>>>(out, n, seed, subseq_dev);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int add_counter(cudaStream_t stream, unsigned long long* counter_dev, unsigned long long v) {
    add_counter_kernel<<<1, 1, 0, stream>>>(counter_dev, v);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int sample_finish(cudaStream_t stream, const void* partials, int chunks, const float* logits, long long row_stride,
                  long long vocab, float inv_temperature, const float* uniforms, int u_stride, int rows, long long* tok_out,
                  float* prob_out, int prob_stride) {
    sample_finish_kernel<<<rows, kThreads, 0, stream>>>(static_cast<const Partial*>(partials), chunks, logits, row_stride,
                                                        static_cast<int>(vocab), inv_temperature, uniforms, u_stride, tok_out,
                                                        prob_out, prob_stride);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int nucleus_rows(cudaStream_t stream, const float* logits, long long row_stride, int rows, long long vocab,
                 float inv_temperature, float top_p, const float* uniforms, int u_stride, Nucleus* nucleus_out,
                 long long* tok_out, float* prob_out, int prob_stride) {
    if (rows <= 0) return 0;
    nucleus_kernel<<<rows * kNucCluster, kNucThreads, 0, stream>>>(logits, row_stride, static_cast<int>(vocab), inv_temperature, top_p,
                                                     uniforms, u_stride, nucleus_out, tok_out, prob_out, prob_stride);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
}  // namespace xb
