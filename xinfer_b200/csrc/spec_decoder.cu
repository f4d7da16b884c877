// Speculative decode runtime: a random-init Qwen-hybrid target (Gated-DeltaNet and full-attention
// layers), one MTP draft head, and the step loop   k draft passes -> one batched verify pass ->
// acceptance -> commit,   for `batch` independent sequences, optionally replayed as one CUDA graph.
//
// What it stands in for in the reference:
//   forward_layer / forward_lm_head            src/targets/qwen3_8/forward.cpp:96-308
//   draft_decode_loop, forward_verify          src/targets/qwen3_8/forward.cpp:600-734
//   the speculative loop of Engine::generate   src/runtime/engine.cpp:400-525
//   DecodeGraph (capture once, replay)         src/targets/qwen3_8/decode_graph.cpp:24-176
//   KVCache advance / rollback / checkpoint    src/core/kv_cache.h:91-113
// Deliberate differences: the verify pass feeds the current token plus the k drafts (k+1 rows per
// sequence) and compares draft i with the logits of row i, the standard scheme (the reference feeds
// only the drafts and compares off by one); the drafter is a one-layer MTP head, which the reference
// does not have (it re-runs the full model); sequences are batched; rejected tokens cost no state copy
// because recurrent updates are committed lazily (mixers.cu) and KV entries are simply overwritten.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <new>
#include <string>
#include <vector>

#include "../../include/xinfer_b200.h"
#include "mixers.h"
#include "sampling.h"
#include "tp_host.h"
#include "w4a16.h"

namespace {

// ---------------------------------------------------------------------------------- random init (device)
__device__ __forceinline__ uint32_t mix32(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
    return static_cast<uint32_t>(x);
}
__device__ __forceinline__ float u01(uint64_t seed, uint64_t i) {
    return (static_cast<float>(mix32(seed * 0x9E3779B97F4A7C15ULL + i) >> 8) + 0.5f) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ float normal01(uint64_t seed, uint64_t i) {
    const float u1 = u01(seed, 2 * i), u2 = u01(seed, 2 * i + 1);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
}
// Every initialiser hashes the element's GLOBAL index (`off` + local index), so a rank that holds only a slice
// of a tensor (N-split weights, the sequences it owns) gets exactly the values of the unsharded tensor.
__global__ void init_bytes_kernel(uint8_t* p, size_t n, uint64_t seed, size_t off) {
    size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        *reinterpret_cast<uint32_t*>(p + i) = mix32(seed * 0x9E3779B97F4A7C15ULL + off + i);
    } else {
        for (; i < n; ++i) p[i] = static_cast<uint8_t>(mix32(seed * 0x9E3779B97F4A7C15ULL + off + i));
    }
}
// mode 0: |N(0, sigma)| / 7 (int4 group scales)   mode 1: mean + N(0, sigma)
__global__ void init_half_kernel(__half* p, size_t n, uint64_t seed, int mode, float mean, float sigma, size_t off) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = normal01(seed, off + i);
    p[i] = __float2half_rn(mode == 0 ? fabsf(z * sigma) / 7.0f : mean + z * sigma);
}
__global__ void init_float_kernel(float* p, size_t n, uint64_t seed, float mean, float sigma, size_t off) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = mean + normal01(seed, off + i) * sigma;
}
__global__ void init_bf16_kernel(uint16_t* p, size_t n, uint64_t seed, float sigma) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = static_cast<uint16_t>(__float_as_uint(normal01(seed, i) * sigma) >> 16);
}
__global__ void init_tokens_kernel(long long* p, int n, uint64_t seed, long long vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = static_cast<long long>(mix32(seed * 0x9E3779B97F4A7C15ULL + i)) % vocab;
}
__global__ void add_int_kernel(int* out, const int* in, int n, int v) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i] + v;
}
__global__ void last_prompt_token_kernel(long long* cur_tok, const long long* prompt, int batch, long long T) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) cur_tok[b] = prompt[static_cast<long long>(b) * T + T - 1];
}

// Prefill chunks: rows in chunk_row order (mixers.h).
__global__ void gather_prompt_chunk_kernel(long long* rows, const long long* prompt, int batch, long long T, long long c0, int Rc) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= batch * Rc) return;
    const int b = t / Rc, p = t % Rc;
    rows[xb::chunk_row(p, b, batch, Rc)] = prompt[static_cast<long long>(b) * T + c0 + p];
}
// The hidden state in front of every row of a chunk: position 0 <- h_last[b], position p <- x at position p - 1.
__global__ void shift_hidden_chunk_kernel(__half* out, const __half* h_last, const __half* x, int batch, int Rc, int H) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(batch) * Rc * H) return;
    const int col = static_cast<int>(t % H);
    const long long bp = t / H;
    const int b = static_cast<int>(bp / Rc), p = static_cast<int>(bp % Rc);
    out[xb::chunk_row(p, b, batch, Rc) * H + col] =
        p == 0 ? h_last[static_cast<long long>(b) * H + col] : x[xb::chunk_row(p - 1, b, batch, Rc) * H + col];
}
// entry e = group * batch + sequence of a chunk that starts at position c0: the keys in front of its first row
__global__ void chunk_entry_ctx_kernel(int* entry_ctx, int entries, int batch, int c0) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < entries) entry_ctx[e] = c0 + 4 * (e / batch);
}
__global__ void take_last_hidden_chunk_kernel(__half* h_last, const __half* x, int batch, int Rc, int H) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(batch) * H) return;
    const int b = static_cast<int>(t / H), col = static_cast<int>(t % H);
    h_last[t] = x[xb::chunk_row(Rc - 1, b, batch, Rc) * H + col];
}

// A projection as this rank holds it: `n` output rows starting at row `row0` of the full [n_full][k] matrix
// (n == n_full, row0 == 0 when it is not split).
struct Linear {
    uint8_t* w = nullptr;
    __half* s = nullptr;
    int64_t n = 0, k = 0, n_full = 0, row0 = 0;
};

// An activation buffer; `off` is its byte offset in the exchange region when other ranks write into it.
struct XBuf {
    __half* p = nullptr;
    size_t off = 0;
};

struct Layer {
    bool full = false;
    float *input_norm = nullptr, *post_norm = nullptr;
    Linear gate, up, down;
    // full attention
    Linear q_proj, k_proj, v_proj, o_proj;
    float *q_norm = nullptr, *k_norm = nullptr;
    __half *k_cache = nullptr, *v_cache = nullptr;
    // gated deltanet
    Linear in_qkv, in_z, in_b, in_a, out_proj;
    float *conv_w = nullptr, *A_log = nullptr, *dt_bias = nullptr, *gdn_norm = nullptr;
    float *S = nullptr, *pend_k = nullptr, *pend_d = nullptr, *pend_g = nullptr, *conv_state = nullptr, *conv_pend = nullptr;
};

}  // namespace

struct xinfer_spec_decoder {
    xinfer_model_config cfg{};
    int batch = 0, k = 0, attn_splits = 8;
    int64_t max_seq = 0;
    uint64_t seed = 0;
    int device = 0;
    // N-split tensor parallelism (world == 1: none).  This rank owns the sequences [b0, b0 + bl).
    xinfer_tp* tp = nullptr;
    int rank = 0, world = 1, bl = 0, b0 = 0;
    // one device block for weights, state and activations
    xinfer_arena* arena = nullptr;
    bool sizing = false;
    size_t need_bytes = 0;
    std::vector<Layer> layers;
    Layer mtp_layer;
    Linear mtp_fc, lm_head;
    float *mtp_enorm = nullptr, *mtp_hnorm = nullptr, *final_norm = nullptr;
    uint16_t* embed = nullptr;
    // sequence state (all sequences, replicated on every rank)
    int *ctx = nullptr, *ctx_draft = nullptr, *n_commit = nullptr, *n_commit_zero = nullptr;
    long long *cur_tok = nullptr, *draft = nullptr, *verify_tokens = nullptr, *argmax_out = nullptr, *emitted = nullptr;
    int* emitted_n = nullptr;
    __half *h_last = nullptr, *mtp_hidden = nullptr;
    xinfer_accept_record* records = nullptr;
    // activations (rows up to batch * (k + 1)); XBufs are written by other ranks under tensor parallelism
    __half *x = nullptr, *emb = nullptr, *normed = nullptr, *qbuf = nullptr, *qkv_conv = nullptr, *bbuf = nullptr,
           *abuf = nullptr, *cat = nullptr;
    XBuf x_mtp, proj_out, mlp, q_gate, kbuf, vbuf, attn_out, qkv_raw, zbuf, delta_out, partials;
    float *logits = nullptr, *attn_scratch = nullptr;
    int64_t vocab_local = 0;
    // pinned result staging
    long long* h_emitted = nullptr;
    int* h_emitted_n = nullptr;
    long long* draft_override = nullptr;  // test hook: when armed, the verify pass checks these tokens instead
    bool override_armed = false;
    // stochastic drafting and acceptance (temperature > 0): per step 2 * batch * k Philox uniforms - [0, batch * k) pick
    // the draft tokens, the rest feed the acceptance rule - from (seed, step counter), the counter in device memory
    float temperature = 0.f;
    uint64_t sample_seed = 0;
    unsigned long long* step_counter = nullptr;
    float *uniforms = nullptr, *draft_probs = nullptr;
    // activation rows of a prefill chunk (allocated by the first long prompt, freed with the decoder)
    struct ChunkBufs {
        int rows = 0;
        __half *x = nullptr, *normed = nullptr, *proj_out = nullptr, *mlp = nullptr, *wide = nullptr, *wide2 = nullptr,
               *qbuf = nullptr, *kbuf = nullptr, *vbuf = nullptr, *mix_out = nullptr, *zbuf = nullptr, *bbuf = nullptr,
               *abuf = nullptr, *cat = nullptr, *hprev = nullptr;
        long long* tokens = nullptr;
        int* entry_ctx = nullptr;        // context length in front of every (group, sequence) entry of a chunk
        float* attn_scratch = nullptr;   // split partials of one attention launch over all entries
        int attn_splits = 1;
    } chunk;
    float top_p = 1.0f;               // < 1: nucleus sampling on both sides of the stochastic rule
    xb::Nucleus* nucleus = nullptr;   // [batch * (k + 1)] nuclei of the verify rows
    int prev_rows = 0;       // rows of the previous target pass (for the lazy state commit)
    int64_t ctx_upper = 0;   // host-side upper bound of every sequence's context length
    cudaGraphExec_t graph_exec = nullptr;
    cudaGraph_t graph = nullptr;
    xb::TcPlan* plan = nullptr;  // this decoder's launch plan (next-launch prefetch hints)
    std::string error;
    size_t weight_bytes = 0, state_bytes = 0;
    long long launches_per_step = 0;
    bool linears_only = false;   // measurement mode: enqueue only the W4A16 launches of a step
    long long linear_launches = 0;
    double linear_bytes = 0;     // algorithmic bytes of those launches (this rank's share)
    long long exchanges_per_step = 0;
};

namespace {

using Dec = xinfer_spec_decoder;

constexpr size_t kAlign = 256;

// Sizing pass: only adds up.  Real pass: carves the arena.
template <typename T>
T* dalloc(Dec* d, size_t count, bool is_state = false) {
    if (count == 0) count = 1;
    const size_t bytes = (count * sizeof(T) + kAlign - 1) & ~(kAlign - 1);
    (is_state ? d->state_bytes : d->weight_bytes) += d->sizing ? 0 : count * sizeof(T);
    if (d->sizing) {
        d->need_bytes += bytes;
        return nullptr;
    }
    void* p = nullptr;
    if (xinfer_arena_allocate(d->arena, bytes, kAlign, &p) != XINFER_OK || !p) throw std::bad_alloc();
    return static_cast<T*>(p);
}

// An activation buffer that other ranks store into: from the exchange region when there are other ranks.
XBuf xalloc(Dec* d, size_t halves) {
    XBuf b;
    if (d->world <= 1) {
        b.p = dalloc<__half>(d, halves, true);
        return b;
    }
    if (d->sizing) return b;
    if (xinfer_tp_alloc(d->tp, halves * sizeof(__half), &b.off) != XINFER_OK) throw std::bad_alloc();
    b.p = static_cast<__half*>(xinfer_tp_ptr(d->tp, b.off));
    d->state_bytes += halves * sizeof(__half);
    return b;
}

unsigned blocks_for(size_t n, int per) { return static_cast<unsigned>((n + per - 1) / per); }

uint64_t next_seed(Dec* d) { return d->seed = d->seed * 6364136223846793005ULL + 1442695040888963407ULL; }

// `split`: under tensor parallelism this rank holds the output rows [rank n/world, (rank + 1) n/world).
Linear make_linear(Dec* d, int64_t n, int64_t k, bool split) {
    Linear l;
    l.n_full = n;
    l.k = k;
    const bool sp = split && d->world > 1;
    l.n = sp ? n / d->world : n;
    l.row0 = sp ? d->rank * l.n : 0;
    const size_t wb = static_cast<size_t>(l.n) * (k / 2), sc = static_cast<size_t>(l.n) * (k / 128);
    l.w = dalloc<uint8_t>(d, wb);
    l.s = dalloc<__half>(d, sc);
    const uint64_t sw = next_seed(d), ss = next_seed(d);
    if (!d->sizing) {
        init_bytes_kernel<<<blocks_for((wb + 3) / 4, 256), 256>>>(l.w, wb, sw, static_cast<size_t>(l.row0) * (k / 2));
        init_half_kernel<<<blocks_for(sc, 256), 256>>>(l.s, sc, ss, 0, 0.f, 0.02f, static_cast<size_t>(l.row0) * (k / 128));
    }
    return l;
}
float* make_floats(Dec* d, size_t n, float mean, float sigma) {
    float* p = dalloc<float>(d, n);
    const uint64_t sd = next_seed(d);
    if (!d->sizing) init_float_kernel<<<blocks_for(n, 256), 256>>>(p, n, sd, mean, sigma, 0);
    return p;
}

void make_layer(Dec* d, Layer& L, bool full) {
    const auto& c = d->cfg;
    const int64_t H = c.hidden_size, F = c.intermediate_size;
    L.full = full;
    L.input_norm = make_floats(d, H, 1.0f, 0.02f);
    L.post_norm = make_floats(d, H, 1.0f, 0.02f);
    L.gate = make_linear(d, F, H, true);
    L.up = make_linear(d, F, H, true);
    L.down = make_linear(d, H, F, true);
    if (full) {
        L.q_proj = make_linear(d, c.num_attention_heads * 512, H, true);
        L.k_proj = make_linear(d, c.num_key_value_heads * 256, H, true);
        L.v_proj = make_linear(d, c.num_key_value_heads * 256, H, true);
        L.o_proj = make_linear(d, H, c.num_attention_heads * 256, true);
        L.q_norm = make_floats(d, 256, 1.0f, 0.02f);
        L.k_norm = make_floats(d, 256, 1.0f, 0.02f);
        const size_t kv = static_cast<size_t>(d->bl) * d->max_seq * c.num_key_value_heads * 256;
        L.k_cache = dalloc<__half>(d, kv, true);
        L.v_cache = dalloc<__half>(d, kv, true);
    } else {
        const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads;
        const int64_t ch = 2 * hk * 128 + hv * 128;
        L.in_qkv = make_linear(d, ch, H, true);
        L.in_z = make_linear(d, hv * 128, H, true);
        L.in_b = make_linear(d, hv, H, false);  // tiny projections: every rank computes them whole
        L.in_a = make_linear(d, hv, H, false);
        L.out_proj = make_linear(d, H, hv * 128, true);
        L.conv_w = make_floats(d, ch * 4, 0.0f, 0.5f);
        L.A_log = make_floats(d, hv, 0.5f, 0.5f);
        L.dt_bias = make_floats(d, hv, 0.0f, 0.5f);
        L.gdn_norm = make_floats(d, 128, 1.0f, 0.02f);
        L.S = dalloc<float>(d, static_cast<size_t>(d->bl) * hv * 128 * 128, true);
        L.pend_k = dalloc<float>(d, static_cast<size_t>(d->bl) * hv * 8 * 128, true);
        L.pend_d = dalloc<float>(d, static_cast<size_t>(d->bl) * hv * 8 * 128, true);
        L.pend_g = dalloc<float>(d, static_cast<size_t>(d->bl) * hv * 8, true);
        L.conv_state = dalloc<float>(d, static_cast<size_t>(d->bl) * 3 * ch, true);
        L.conv_pend = dalloc<float>(d, static_cast<size_t>(d->bl) * 8 * ch, true);
    }
}

// Everything the decoder keeps on the device, in a fixed order (run once to size the arena, once for real).
void build_all(Dec* d) {
    const auto& c = d->cfg;
    const int64_t H = c.hidden_size, V = c.vocab_size;
    const int batch = d->batch, k = d->k;
    const int M = batch * (k + 1);
    const uint64_t seed0 = d->seed;
    d->layers.assign(static_cast<size_t>(c.num_hidden_layers), Layer());
    const int interval = c.full_attention_interval > 0 ? c.full_attention_interval : 4;
    for (int64_t l = 0; l < c.num_hidden_layers; ++l) make_layer(d, d->layers[l], (l % interval) == interval - 1);
    make_layer(d, d->mtp_layer, true);
    d->mtp_fc = make_linear(d, H, 2 * H, true);
    d->lm_head = make_linear(d, V, H, true);
    d->vocab_local = d->lm_head.n;
    d->mtp_enorm = make_floats(d, H, 1.0f, 0.02f);
    d->mtp_hnorm = make_floats(d, H, 1.0f, 0.02f);
    d->final_norm = make_floats(d, H, 1.0f, 0.02f);
    d->embed = dalloc<uint16_t>(d, static_cast<size_t>(V) * H);
    const uint64_t se = next_seed(d);
    if (!d->sizing)
        init_bf16_kernel<<<blocks_for(static_cast<size_t>(V) * H, 256), 256>>>(d->embed, static_cast<size_t>(V) * H, se, 1.0f);
    d->ctx = dalloc<int>(d, batch, true);
    d->ctx_draft = dalloc<int>(d, batch, true);
    d->n_commit = dalloc<int>(d, batch, true);
    d->n_commit_zero = dalloc<int>(d, batch, true);
    d->cur_tok = dalloc<long long>(d, batch, true);
    d->draft = dalloc<long long>(d, static_cast<size_t>(batch) * k, true);
    d->verify_tokens = dalloc<long long>(d, M, true);
    d->argmax_out = dalloc<long long>(d, M, true);
    d->emitted = dalloc<long long>(d, M, true);
    d->emitted_n = dalloc<int>(d, batch, true);
    d->h_last = dalloc<__half>(d, static_cast<size_t>(batch) * H, true);
    d->mtp_hidden = dalloc<__half>(d, static_cast<size_t>(batch) * H, true);
    d->records = dalloc<xinfer_accept_record>(d, batch, true);
    d->draft_override = dalloc<long long>(d, static_cast<size_t>(batch) * k, true);
    d->step_counter = dalloc<unsigned long long>(d, 1, true);
    d->uniforms = dalloc<float>(d, static_cast<size_t>(2) * batch * k, true);
    d->draft_probs = dalloc<float>(d, static_cast<size_t>(batch) * k, true);
    d->nucleus = dalloc<xb::Nucleus>(d, static_cast<size_t>(M), true);
    const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads, ch = 2 * hk * 128 + hv * 128;
    d->x = dalloc<__half>(d, static_cast<size_t>(M) * H, true);
    d->emb = dalloc<__half>(d, static_cast<size_t>(batch) * H, true);
    d->normed = dalloc<__half>(d, static_cast<size_t>(M) * H, true);
    d->qbuf = dalloc<__half>(d, static_cast<size_t>(M) * c.num_attention_heads * 256, true);
    d->qkv_conv = dalloc<__half>(d, static_cast<size_t>(M) * ch, true);
    d->bbuf = dalloc<__half>(d, static_cast<size_t>(M) * hv, true);
    d->abuf = dalloc<__half>(d, static_cast<size_t>(M) * hv, true);
    d->cat = dalloc<__half>(d, static_cast<size_t>(batch) * 2 * H, true);
    d->logits = dalloc<float>(d, static_cast<size_t>(M) * d->vocab_local, true);
    // buffers that other ranks store into (same order on every rank: an offset names the same buffer everywhere)
    d->x_mtp = xalloc(d, static_cast<size_t>(batch) * H);
    d->proj_out = xalloc(d, static_cast<size_t>(M) * H);
    d->mlp = xalloc(d, static_cast<size_t>(M) * c.intermediate_size);
    d->q_gate = xalloc(d, static_cast<size_t>(M) * c.num_attention_heads * 512);
    d->kbuf = xalloc(d, static_cast<size_t>(M) * c.num_key_value_heads * 256);
    d->vbuf = xalloc(d, static_cast<size_t>(M) * c.num_key_value_heads * 256);
    d->attn_out = xalloc(d, static_cast<size_t>(M) * c.num_attention_heads * 256);
    d->qkv_raw = xalloc(d, static_cast<size_t>(M) * ch);
    d->zbuf = xalloc(d, static_cast<size_t>(M) * hv * 128);
    d->delta_out = xalloc(d, static_cast<size_t>(M) * hv * 128);
    // (row, chunk) partials of the sampling kernels, one block per vocabulary slice
    d->partials = xalloc(d, static_cast<size_t>(d->world) * xb::sampling_scratch_bytes(M, d->vocab_local) / sizeof(__half));
    {
        // KV splits: with one attention CTA per SM, two waves of CTAs over (split, kv head, sequence)
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->device);
        const int units = d->bl * static_cast<int>(c.num_key_value_heads);
        int splits = (2 * sms) / (units > 0 ? units : 1);
        d->attn_splits = splits < 1 ? 1 : (splits > 16 ? 16 : splits);
    }
    d->attn_scratch = dalloc<float>(
        d, xb::attn_scratch_bytes(d->bl, static_cast<int>(c.num_key_value_heads), d->attn_splits) / sizeof(float), true);
    if (d->sizing) d->seed = seed0;  // the real pass draws the same seeds again
}

#define NL(expr)                                                        \
    do {                                                                \
        if (!d->linears_only) CK(expr);                                 \
    } while (0)

#define CK(expr)                                                        \
    do {                                                                \
        int _rc = (expr);                                               \
        if (_rc < 0) {                                                  \
            d->error = std::string(#expr) + " failed";                  \
            return _rc == XINFER_ERR_CUDA ? XINFER_ERR_CUDA : _rc;      \
        }                                                               \
    } while (0)

#define CKCUDA(expr)                                                    \
    do {                                                                \
        if ((expr) != cudaSuccess) {                                    \
            d->error = std::string(#expr) + " failed";                  \
            cudaGetLastError();                                         \
            return XINFER_ERR_CUDA;                                     \
        }                                                               \
    } while (0)

void account(Dec* d, const Linear& l, int M, int out_bytes, bool count_x) {
    d->linear_bytes += static_cast<double>(l.n) * (l.k / 2) + static_cast<double>(l.n) * (l.k / 128) * 2 +
                       (count_x ? static_cast<double>(M) * l.k * 2 : 0.0) + static_cast<double>(M) * l.n * out_bytes;
}

// How an N-split projection's output travels: to every rank, or only to the rank that owns the row's sequence.
enum Push { kLocal = 0, kAll = 1, kOwner = 2 };

// One projection of a (possibly fused) launch as this rank runs it: its slice of W writes the columns
// [row0, row0 + n) of the full-width output `y` (row stride n_full), on this rank and - push - on the others.
xb::TcProj make_proj(const Dec* d, const Linear& l, const XBuf& y, int push) {
    xb::TcProj p;
    p.w = l.w;
    p.scales = l.s;
    p.bias = nullptr;
    p.n = l.n;
    p.ldy = l.n_full;
    p.y = y.p + l.row0;
    if (d->world > 1 && push != kLocal) xb::tp_fill_proj(d->tp, &p, y.off + static_cast<size_t>(l.row0) * sizeof(__half), push);
    return p;
}
xb::TcProj make_proj_local(const Linear& l, void* y) {
    xb::TcProj p;
    p.w = l.w;
    p.scales = l.s;
    p.bias = nullptr;
    p.n = l.n;
    p.ldy = l.n;
    p.y = y;
    return p;
}

// Launches `num` projections sharing X (or a gate/up pair) on the tensor-core kernel; with other ranks around
// the launch ends with the exchange handshake, so when it completes every rank's slice has arrived here.
// Every activation buffer that feeds a projection (normed, cat, attn_out, delta_out, mlp) is written by its producer
// with each block of eight features in the order the int4 unpack yields them, so the projection kernel does not
// rewrite its staged activation tiles: all launches below pass kTcXPermuted, and the gate/up launch, whose output
// is the down projection's input, also kTcYPermuted.  Set XINFER_XPERM=0 to run everything in natural order.
bool xperm_on() {
    static const bool on = [] { const char* e = getenv("XINFER_XPERM"); return !(e && atoi(e) == 0); }();
    return on;
}

int run_lin(Dec* d, cudaStream_t s, const void* x, xb::TcProj* pr, int num, bool swiglu, bool out_f32, int M, int64_t K,
            int rows_per_rank, bool exchange) {
    ++d->launches_per_step;
    ++d->linear_launches;
    const int flags = xperm_on() ? (xb::kTcXPermuted | (swiglu ? xb::kTcYPermuted : 0)) : 0;
    if (d->world > 1 && exchange) {
        ++d->exchanges_per_step;
        const xb::TpLink link = xb::tp_link(d->tp, rows_per_rank);
        return xb::run_tc_linear(s, x, pr, num, swiglu, out_f32, M, K, 128, &link, flags);
    }
    return xb::run_tc_linear(s, x, pr, num, swiglu, out_f32, M, K, 128, nullptr, flags);
}

int lin(Dec* d, cudaStream_t s, const XBuf& y, const __half* x, const Linear& l, int M, int push) {
    account(d, l, M, 2, true);
    xb::TcProj p = make_proj(d, l, y, push);
    return run_lin(d, s, x, &p, 1, false, false, M, l.k, 1, push != kLocal);
}

// All-gather by rows of a buffer whose rows [row0, row0 + rows) this rank has just produced.
int gather_rows(Dec* d, cudaStream_t s, const XBuf& b, int row0, int rows, int64_t width) {
    if (d->world <= 1 || d->linears_only) return 0;
    ++d->launches_per_step;
    ++d->exchanges_per_step;
    const size_t rb = static_cast<size_t>(width) * sizeof(__half);
    return xb::tp_push(d->tp, s, b.off + static_cast<size_t>(row0) * rb, static_cast<size_t>(rows) * rb) == 0 ? 0 : XINFER_ERR_CUDA;
}

// y = projection(x_in);  xr = half(xr + y);  normed = rmsnorm(xr) * w.
// (Running the add + norm as a tail of the projection kernel, by the CTA that completes a block of rows last,
// was measured slower than the separate launch: under programmatic dependent launch the next projection's
// weight stream already overlaps the norm kernel.)
int lin_add_norm(Dec* d, cudaStream_t s, const XBuf& y, const __half* x_in, const Linear& l, int M, __half* xr,
                 const float* w) {
    const auto& c = d->cfg;
    CK(lin(d, s, y, x_in, l, M, kAll));
    NL(xb::add_rmsnorm_rows(s, d->normed, xr, y.p, w, M, static_cast<int>(l.n_full), c.rms_norm_eps, xperm_on()));
    ++d->launches_per_step;
    return 0;
}

// One decoder layer on M = batch * R rows.  On entry `normed` holds the layer's input norm of the residual stream
// `xr`; on exit `xr` has both residual adds applied and `normed` holds its norm under `next_norm_w` (the next
// layer's input norm, or the final norm).  Projections run on all M rows (N-split over the ranks); the mixer runs
// on the rows of this rank's own sequences.
int layer_forward(Dec* d, cudaStream_t s, Layer& L, int R, __half* xr, const float* next_norm_w, const int* ctx,
                  const int* n_commit, int prev_rows) {
    const auto& c = d->cfg;
    const int B = d->batch, M = B * R;
    const int Bl = d->bl, Ml = Bl * R, row0 = d->b0 * R;
    const int H = static_cast<int>(c.hidden_size);
    if (L.full) {
        const int hq = static_cast<int>(c.num_attention_heads), hkv = static_cast<int>(c.num_key_value_heads);
        xb::TcProj fd[3] = {make_proj(d, L.q_proj, d->q_gate, kOwner), make_proj(d, L.k_proj, d->kbuf, kOwner),
                            make_proj(d, L.v_proj, d->vbuf, kOwner)};
        account(d, L.q_proj, M, 2, true);
        account(d, L.k_proj, M, 2, false);
        account(d, L.v_proj, M, 2, false);
        CK(run_lin(d, s, d->normed, fd, 3, false, false, M, H, Ml, true));
        NL(xb::attn_prep(s, d->qbuf + static_cast<size_t>(row0) * hq * 256, L.k_cache, L.v_cache,
                         d->q_gate.p + static_cast<size_t>(row0) * hq * 512, d->kbuf.p + static_cast<size_t>(row0) * hkv * 256,
                         d->vbuf.p + static_cast<size_t>(row0) * hkv * 256, L.q_norm, L.k_norm, ctx + d->b0, Bl, R, hq, hkv,
                         d->max_seq, c.rms_norm_eps, c.rope_theta, c.rope_dim));
        NL(xb::attn_decode_ex(s, d->attn_out.p + static_cast<size_t>(row0) * hq * 256,
                              d->qbuf + static_cast<size_t>(row0) * hq * 256, d->q_gate.p + static_cast<size_t>(row0) * hq * 512,
                              L.k_cache, L.v_cache, ctx + d->b0, Bl, R, hq, hkv, d->max_seq, d->attn_splits, d->attn_scratch,
                              1.0f / sqrtf(256.0f), 0, xperm_on()));
        d->launches_per_step += 3;
        CK(gather_rows(d, s, d->attn_out, row0, Ml, static_cast<int64_t>(hq) * 256));
        // x += mixer output, post-attention RMSNorm
        CK(lin_add_norm(d, s, d->proj_out, d->attn_out.p, L.o_proj, M, xr, L.post_norm));
    } else {
        const int hv = static_cast<int>(c.linear_num_v_heads), hk = static_cast<int>(c.linear_num_k_heads);
        const int ch = 2 * hk * 128 + hv * 128;
        xb::TcProj fd[4] = {make_proj(d, L.in_qkv, d->qkv_raw, kOwner), make_proj(d, L.in_z, d->zbuf, kOwner),
                            make_proj_local(L.in_b, d->bbuf), make_proj_local(L.in_a, d->abuf)};
        account(d, L.in_qkv, M, 2, true);
        account(d, L.in_z, M, 2, false);
        account(d, L.in_b, M, 2, false);
        account(d, L.in_a, M, 2, false);
        CK(run_lin(d, s, d->normed, fd, 4, false, false, M, H, Ml, true));
        NL(xb::conv1d_spec(s, d->qkv_conv + static_cast<size_t>(row0) * ch, d->qkv_raw.p + static_cast<size_t>(row0) * ch,
                           L.conv_w, L.conv_state, L.conv_pend, n_commit + d->b0, Bl, R, prev_rows, ch, 0, 1));
        NL(xb::gdn_spec(s, d->delta_out.p + static_cast<size_t>(row0) * hv * 128, d->qkv_conv + static_cast<size_t>(row0) * ch,
                        d->zbuf.p + static_cast<size_t>(row0) * hv * 128, d->bbuf + static_cast<size_t>(row0) * hv,
                        d->abuf + static_cast<size_t>(row0) * hv, L.A_log, L.dt_bias, L.gdn_norm, L.S, L.pend_k, L.pend_d,
                        L.pend_g, n_commit + d->b0, Bl, R, prev_rows, hv, hk, 0, 1, xperm_on()));
        d->launches_per_step += 2;
        CK(gather_rows(d, s, d->delta_out, row0, Ml, static_cast<int64_t>(hv) * 128));
        CK(lin_add_norm(d, s, d->proj_out, d->delta_out.p, L.out_proj, M, xr, L.post_norm));
    }
    {
        xb::TcProj gu[2] = {make_proj(d, L.gate, d->mlp, kAll), make_proj_local(L.up, nullptr)};
        account(d, L.gate, M, 2, true);
        d->linear_bytes += static_cast<double>(L.up.n) * (L.up.k / 2) + static_cast<double>(L.up.n) * (L.up.k / 128) * 2;
        CK(run_lin(d, s, d->normed, gu, 2, true, false, M, H, 1, true));
    }
    // x += MLP output, then the norm the next consumer of the residual stream needs
    CK(lin_add_norm(d, s, d->proj_out, d->mlp.p, L.down, M, xr, next_norm_w));
    return 0;
}

// LM head on M rows -> this rank's slice of the fp32 logits, then the (row, chunk) partials of the sampling
// kernels over that slice; under tensor parallelism the partial blocks are exchanged so that every rank can
// finish argmax / acceptance over the whole vocabulary.
int lm_head_and_partials(Dec* d, cudaStream_t s, int M) {
    const bool stochastic = d->temperature > 0.f;
    const float inv_t = stochastic ? 1.0f / d->temperature : 1.0f;
    xb::TcProj p = make_proj_local(d->lm_head, d->logits);
    account(d, d->lm_head, M, 4, true);
    CK(run_lin(d, s, d->normed, &p, 1, false, true, M, d->lm_head.k, 1, false));
    if (d->linears_only) return 0;
    const size_t block = xb::sampling_scratch_bytes(M, d->vocab_local);
    uint8_t* mine = reinterpret_cast<uint8_t*>(d->partials.p) + static_cast<size_t>(d->rank) * block;
    CK(xb::sampling_partials(s, d->logits, d->vocab_local, M, d->vocab_local, inv_t, stochastic, d->lm_head.row0, mine));
    ++d->launches_per_step;
    if (d->world > 1) {
        ++d->launches_per_step;
        ++d->exchanges_per_step;
        if (xb::tp_push(d->tp, s, d->partials.off + static_cast<size_t>(d->rank) * block, block) != 0) return XINFER_ERR_CUDA;
    }
    return 0;
}
long long partial_slice_stride(const Dec* d, int M) {
    return static_cast<long long>(xb::sampling_scratch_bytes(M, d->vocab_local) / 16);  // in (row, chunk) entries
}

// The MTP head up to (and including) its attention layer's KV write for the token at position ctx + i.
// `full`: the whole head (attention, MLP, final norm, LM head, argmax -> draft token i).  Otherwise only the
// part that fills the head's KV slot: after k accepted drafts the next step's first draft pass attends to
// position ctx + k, which no draft pass of this step has written.
int draft_pass(Dec* d, cudaStream_t s, int i, bool full) {
    const auto& c = d->cfg;
    const int B = d->batch, H = static_cast<int>(c.hidden_size);
    const long long* tok = (i == 0) ? d->cur_tok : d->argmax_out;
    const __half* hprev = (i == 0) ? d->h_last : d->mtp_hidden;
    // cat = [rmsnorm(embed(tok)) ; rmsnorm(h_prev)]  ->  fc  ->  x
    NL(xb::embed_rows(s, d->emb, d->embed, tok, B, H, c.vocab_size));
    NL(xb::rmsnorm_rows(s, d->cat, 2 * H, d->emb, d->mtp_enorm, B, H, c.rms_norm_eps, xperm_on()));
    NL(xb::rmsnorm_rows(s, d->cat + H, 2 * H, hprev, d->mtp_hnorm, B, H, c.rms_norm_eps, xperm_on()));
    CK(lin(d, s, d->x_mtp, d->cat, d->mtp_fc, B, kAll));
    if (!d->linears_only) add_int_kernel<<<1, 64, 0, s>>>(d->ctx_draft, d->ctx, B, i);
    d->launches_per_step += 4;
    if (!full) {
        // input norm -> k, v projections of the head's layer -> head norm, RoPE, cache write
        Layer& L = d->mtp_layer;
        const int hq = static_cast<int>(c.num_attention_heads), hkv = static_cast<int>(c.num_key_value_heads);
        const int Bl = d->bl, row0 = d->b0;
        NL(xb::rmsnorm_rows(s, d->normed, H, d->x_mtp.p, L.input_norm, B, H, c.rms_norm_eps, xperm_on()));
        // (the query projection is not needed: the prologue kernel is told there are no query heads)
        xb::TcProj fd[2] = {make_proj(d, L.k_proj, d->kbuf, kOwner), make_proj(d, L.v_proj, d->vbuf, kOwner)};
        account(d, L.k_proj, B, 2, true);
        account(d, L.v_proj, B, 2, false);
        CK(run_lin(d, s, d->normed, fd, 2, false, false, B, H, Bl, true));
        (void)hq;
        NL(xb::attn_prep(s, d->qbuf, L.k_cache, L.v_cache, d->q_gate.p, d->kbuf.p + static_cast<size_t>(row0) * hkv * 256,
                         d->vbuf.p + static_cast<size_t>(row0) * hkv * 256, L.q_norm, L.k_norm, d->ctx_draft + d->b0, Bl, 1, 0,
                         hkv, d->max_seq, c.rms_norm_eps, c.rope_theta, c.rope_dim));
        d->launches_per_step += 2;
        return 0;
    }
    NL(xb::rmsnorm_rows(s, d->normed, H, d->x_mtp.p, d->mtp_layer.input_norm, B, H, c.rms_norm_eps, xperm_on()));
    ++d->launches_per_step;
    CK(layer_forward(d, s, d->mtp_layer, 1, d->x_mtp.p, d->final_norm, d->ctx_draft, d->n_commit_zero, 0));
    // keep the head's output hidden (pre final norm) for the next draft pass
    if (!d->linears_only)
        CKCUDA(cudaMemcpyAsync(d->mtp_hidden, d->x_mtp.p, static_cast<size_t>(B) * H * sizeof(__half), cudaMemcpyDeviceToDevice, s));
    CK(lm_head_and_partials(d, s, B));
    if (d->temperature > 0.f) {
        // draft token i of every sequence from softmax(logits / T) at its uniform; its probability is the rule's p_draft
        if (d->top_p < 1.0f)
            NL(xb::nucleus_rows(s, d->logits, d->vocab_local, B, d->vocab_local, 1.0f / d->temperature, d->top_p, d->uniforms + i,
                                d->k, nullptr, d->argmax_out, d->draft_probs + i, d->k));
        else
        NL(xb::sample_finish(s, d->partials.p, xb::sampling_chunks(d->vocab_local), d->logits, d->vocab_local, d->vocab_local,
                             1.0f / d->temperature, d->uniforms + i, d->k, B, d->argmax_out, d->draft_probs + i, d->k));
    } else {
        NL(xb::argmax_finish(s, d->partials.p, xb::sampling_chunks(d->vocab_local), d->world, partial_slice_stride(d, B), B,
                             d->argmax_out));
    }
    NL(xb::copy_token_column(s, d->draft, d->argmax_out, B, d->k, i));
    d->launches_per_step += 4;
    return 0;
}

int target_pass(Dec* d, cudaStream_t s, int R, const long long* tokens) {
    const auto& c = d->cfg;
    const int M = d->batch * R, H = static_cast<int>(c.hidden_size);
    NL(xb::embed_rows(s, d->x, d->embed, tokens, M, H, c.vocab_size));
    NL(xb::rmsnorm_rows(s, d->normed, H, d->x, d->layers[0].input_norm, M, H, c.rms_norm_eps, xperm_on()));
    d->launches_per_step += 2;
    const size_t nl = d->layers.size();
    for (size_t l = 0; l < nl; ++l)
        CK(layer_forward(d, s, d->layers[l], R, d->x, l + 1 < nl ? d->layers[l + 1].input_norm : d->final_norm, d->ctx,
                         d->n_commit, d->prev_rows));
    // `normed` now holds the final norm of the residual stream: LM head -> fp32 logits
    CK(lm_head_and_partials(d, s, M));
    if (!d->linears_only) d->prev_rows = R;
    return 0;
}

// ---------------------------------------------------------------------------------------------- prefill chunks
// A prompt goes through the model in chunks of up to 512 rows (all sequences together), so that the projections see
// M = hundreds of rows and run on the prefill GEMM.  Between them the attention kernels take the chunk four positions
// at a time (their own row limit; the row order of a chunk, chunk_row, makes every such group a contiguous block, and
// one launch takes all groups of all sequences as separate entries); the convolution
// and the gated delta rule walk the whole chunk in one launch each (conv1d_chunk, gdn_chunk).  Natural feature
// order everywhere (the permuted order of the decode step is a property of its 32-row kernel).

int ensure_chunk_bufs(Dec* d, int rows) {
    auto& cb = d->chunk;
    if (cb.rows >= rows) return 0;
    const auto& c = d->cfg;
    const size_t H = static_cast<size_t>(c.hidden_size), F = static_cast<size_t>(c.intermediate_size);
    const size_t hq = static_cast<size_t>(c.num_attention_heads), hkv = static_cast<size_t>(c.num_key_value_heads);
    const size_t hv = static_cast<size_t>(c.linear_num_v_heads), hk = static_cast<size_t>(c.linear_num_k_heads);
    const size_t ch = 2 * hk * 128 + hv * 128;
    auto mx = [](size_t a, size_t b2) { return a > b2 ? a : b2; };
    const size_t wide = mx(hq * 512, ch), mix = mx(mx(hq * 256, hv * 128), H);
    const size_t per_row = 3 * H + F + wide + ch + hq * 256 + 2 * hkv * 256 + mix + hv * 128 + 2 * hv + 2 * H + H;
    const size_t halves = (per_row + 64) * static_cast<size_t>(rows);
    if (cb.x) { cudaFree(cb.x); cudaFree(cb.attn_scratch); cb = Dec::ChunkBufs(); }
    __half* base = nullptr;
    if (cudaMalloc(&base, halves * sizeof(__half) + static_cast<size_t>(rows) * (sizeof(long long) + sizeof(int)) + 256) != cudaSuccess) {
        cudaGetLastError();
        return XINFER_ERR_OUT_OF_MEMORY;
    }
    size_t off = 0;
    auto take = [&](size_t per) {
        __half* ptr = base + off;
        off += (per * static_cast<size_t>(rows) + 63) & ~static_cast<size_t>(63);   // 128-byte aligned (TMA, vector loads)
        return ptr;
    };
    cb.x = take(H); cb.normed = take(H); cb.proj_out = take(H); cb.mlp = take(F); cb.wide = take(wide); cb.wide2 = take(ch);
    cb.qbuf = take(hq * 256); cb.kbuf = take(hkv * 256); cb.vbuf = take(hkv * 256); cb.mix_out = take(mix);
    cb.zbuf = take(hv * 128); cb.bbuf = take(hv); cb.abuf = take(hv); cb.cat = take(2 * H); cb.hprev = take(H);
    cb.tokens = reinterpret_cast<long long*>(base + ((off + 63) & ~static_cast<size_t>(63)));
    cb.entry_ctx = reinterpret_cast<int*>(cb.tokens + rows);
    // one attention launch takes every full group of four positions of every sequence as an entry of its own: enough
    // entries fill the GPU without splitting the keys, few entries are split as in the step
    const int entries = (rows + 3) / 4;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->device);
    int ns = (2 * sms + entries * static_cast<int>(hkv) - 1) / (entries * static_cast<int>(hkv));
    ns = ns < 1 ? 1 : (ns > d->attn_splits ? d->attn_splits : ns);
    cb.attn_splits = ns;
    if (cudaMalloc(&cb.attn_scratch, xb::attn_scratch_bytes(entries, static_cast<int>(hkv), ns)) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(base);
        cb = Dec::ChunkBufs();
        return XINFER_ERR_OUT_OF_MEMORY;
    }
    cb.rows = rows;
    return 0;
}

#define LIN(expr)                                                        \
    do {                                                                 \
        const int lrc_ = (expr);                                         \
        if (lrc_ < 0) { d->error = "prefill: a projection failed"; return lrc_; } \
    } while (0)

// One chunk: positions c0 .. c0 + Rc - 1 of every sequence through the target model and into the MTP head's cache.
// `prev_r` comes back as the number of recurrent updates left pending for the next pass (none).
int prefill_chunk(Dec* d, cudaStream_t s, const long long* prompt, int64_t T, int64_t c0, int Rc, int* prev_r) {
    const auto& c = d->cfg;
    auto& cb = d->chunk;
    const int B = d->batch, M = B * Rc, H = static_cast<int>(c.hidden_size), F = static_cast<int>(c.intermediate_size);
    const int hq = static_cast<int>(c.num_attention_heads), hkv = static_cast<int>(c.num_key_value_heads);
    const int hv = static_cast<int>(c.linear_num_v_heads), hk = static_cast<int>(c.linear_num_k_heads);
    const int ch = 2 * hk * 128 + hv * 128, groups = (Rc + 3) / 4;
    const float eps = c.rms_norm_eps;
    void* st = s;
    auto desc = [](void* y, const Linear& l) {
        xinfer_fused_desc f;
        f.Y = y; f.W_int4 = l.w; f.scales = l.s; f.bias = nullptr; f.N = l.n;
        return f;
    };
    const int full_groups = Rc / 4;
    gather_prompt_chunk_kernel<<<blocks_for(static_cast<size_t>(M), 128), 128, 0, s>>>(cb.tokens, prompt, B, T, c0, Rc);
    if (full_groups > 0)
        chunk_entry_ctx_kernel<<<blocks_for(static_cast<size_t>(full_groups) * B, 128), 128, 0, s>>>(cb.entry_ctx, full_groups * B, B,
                                                                                                 static_cast<int>(c0));
    NL(xb::embed_rows(s, cb.x, d->embed, cb.tokens, M, H, c.vocab_size));
    NL(xb::rmsnorm_rows(s, cb.normed, H, cb.x, d->layers[0].input_norm, M, H, eps, 0));
    const size_t nl = d->layers.size();
    for (size_t l = 0; l < nl; ++l) {
        Layer& L = d->layers[l];
        if (L.full) {
            const xinfer_fused_desc fd[3] = {desc(cb.wide, L.q_proj), desc(cb.kbuf, L.k_proj), desc(cb.vbuf, L.v_proj)};
            LIN(xinfer_linear_int4_fused_f16(st, cb.normed, fd, 3, M, H, 128));
            // every full group of four positions of every sequence is one entry (rows [entry][4], its own context length,
            // the cache of sequence entry % B): one launch each for the prologue, the split attention and the combine;
            // a last short group goes through the same kernels on its own
            if (full_groups > 0) {
                NL(xb::attn_prep_ex(s, cb.qbuf, L.k_cache, L.v_cache, cb.wide, cb.kbuf, cb.vbuf, L.q_norm, L.k_norm, cb.entry_ctx,
                                    full_groups * B, 4, hq, hkv, d->max_seq, eps, c.rope_theta, c.rope_dim, 512, nullptr, 0, nullptr, B));
                NL(xb::attn_decode_ex(s, cb.mix_out, cb.qbuf, cb.wide, L.k_cache, L.v_cache, cb.entry_ctx, full_groups * B, 4, hq, hkv,
                                      d->max_seq, cb.attn_splits, cb.attn_scratch, 1.0f / sqrtf(256.0f), 0, 0, B));
            }
            if (full_groups < groups) {
                const int rj = Rc - 4 * full_groups;
                const size_t r0 = static_cast<size_t>(full_groups) * B * 4;
                const int pos0 = static_cast<int>(c0) + 4 * full_groups;
                NL(xb::attn_prep_ex(s, cb.qbuf + r0 * hq * 256, L.k_cache, L.v_cache, cb.wide + r0 * hq * 512, cb.kbuf + r0 * hkv * 256,
                                    cb.vbuf + r0 * hkv * 256, L.q_norm, L.k_norm, nullptr, B, rj, hq, hkv, d->max_seq, eps,
                                    c.rope_theta, c.rope_dim, 512, nullptr, pos0, nullptr));
                NL(xb::attn_decode_ex(s, cb.mix_out + r0 * hq * 256, cb.qbuf + r0 * hq * 256, cb.wide + r0 * hq * 512, L.k_cache,
                                      L.v_cache, nullptr, B, rj, hq, hkv, d->max_seq, d->attn_splits, d->attn_scratch,
                                      1.0f / sqrtf(256.0f), pos0, 0));
            }
            LIN(xinfer_linear_int4_f16f16(st, cb.proj_out, cb.mix_out, L.o_proj.w, L.o_proj.s, nullptr, M, L.o_proj.n, L.o_proj.k, 128));
        } else {
            const xinfer_fused_desc fd[4] = {desc(cb.wide, L.in_qkv), desc(cb.zbuf, L.in_z), desc(cb.bbuf, L.in_b), desc(cb.abuf, L.in_a)};
            LIN(xinfer_linear_int4_fused_f16(st, cb.normed, fd, 4, M, H, 128));
            NL(xb::conv1d_chunk(s, cb.wide2, cb.wide, L.conv_w, L.conv_state, B, Rc, ch));
            NL(xb::gdn_chunk(s, cb.mix_out, cb.wide2, cb.zbuf, cb.bbuf, cb.abuf, L.A_log, L.dt_bias, L.gdn_norm, L.S, B, Rc, hv, hk));
            LIN(xinfer_linear_int4_f16f16(st, cb.proj_out, cb.mix_out, L.out_proj.w, L.out_proj.s, nullptr, M, L.out_proj.n,
                                          L.out_proj.k, 128));
        }
        NL(xb::add_rmsnorm_rows(s, cb.normed, cb.x, cb.proj_out, L.post_norm, M, H, eps, 0));
        LIN(xinfer_mlp_gate_up_swiglu_int4_f16(st, cb.mlp, cb.normed, L.gate.w, L.gate.s, L.up.w, L.up.s, M, L.gate.n, H, 128));
        LIN(xinfer_linear_int4_f16f16(st, cb.proj_out, cb.mlp, L.down.w, L.down.s, nullptr, M, L.down.n, F, 128));
        NL(xb::add_rmsnorm_rows(s, cb.normed, cb.x, cb.proj_out, l + 1 < nl ? d->layers[l + 1].input_norm : d->final_norm, M, H, eps, 0));
    }
    *prev_r = 0;   // the chunk kernels leave nothing pending
    // the MTP head's KV slots of the same positions: (token of the row, hidden state in front of the row) -> fc ->
    // input norm -> k, v projections -> head norm, RoPE, cache write
    Layer& ML = d->mtp_layer;
    const size_t nH = static_cast<size_t>(M) * H;
    shift_hidden_chunk_kernel<<<blocks_for(nH, 256), 256, 0, s>>>(cb.hprev, d->h_last, cb.x, B, Rc, H);
    NL(xb::embed_rows(s, cb.proj_out, d->embed, cb.tokens, M, H, c.vocab_size));
    NL(xb::rmsnorm_rows(s, cb.cat, 2 * H, cb.proj_out, d->mtp_enorm, M, H, eps, 0));
    NL(xb::rmsnorm_rows(s, cb.cat + H, 2 * H, cb.hprev, d->mtp_hnorm, M, H, eps, 0));
    LIN(xinfer_linear_int4_f16f16(st, cb.mix_out, cb.cat, d->mtp_fc.w, d->mtp_fc.s, nullptr, M, d->mtp_fc.n, d->mtp_fc.k, 128));
    NL(xb::rmsnorm_rows(s, cb.normed, H, cb.mix_out, ML.input_norm, M, H, eps, 0));
    const xinfer_fused_desc kv[2] = {desc(cb.kbuf, ML.k_proj), desc(cb.vbuf, ML.v_proj)};
    LIN(xinfer_linear_int4_fused_f16(st, cb.normed, kv, 2, M, H, 128));
    if (full_groups > 0)
        NL(xb::attn_prep_ex(s, cb.qbuf, ML.k_cache, ML.v_cache, cb.wide, cb.kbuf, cb.vbuf, ML.q_norm, ML.k_norm, cb.entry_ctx,
                            full_groups * B, 4, 0, hkv, d->max_seq, eps, c.rope_theta, c.rope_dim, 512, nullptr, 0, nullptr, B));
    if (full_groups < groups) {
        const size_t r0 = static_cast<size_t>(full_groups) * B * 4;
        NL(xb::attn_prep_ex(s, cb.qbuf, ML.k_cache, ML.v_cache, cb.wide, cb.kbuf + r0 * hkv * 256, cb.vbuf + r0 * hkv * 256, ML.q_norm,
                            ML.k_norm, nullptr, B, Rc - 4 * full_groups, 0, hkv, d->max_seq, eps, c.rope_theta, c.rope_dim, 512,
                            nullptr, static_cast<int>(c0) + 4 * full_groups, nullptr));
    }
    take_last_hidden_chunk_kernel<<<blocks_for(static_cast<size_t>(B) * H, 256), 256, 0, s>>>(d->h_last, cb.x, B, Rc, H);
    CKCUDA(cudaGetLastError());
    return 0;
}
#undef LIN

int enqueue_step(Dec* d, cudaStream_t s) {
    const auto& c = d->cfg;
    const int B = d->batch, k = d->k, R = k + 1;
    d->launches_per_step = 0;
    d->linear_launches = 0;
    d->linear_bytes = 0;
    d->exchanges_per_step = 0;
    xb::TcPlan* prev_plan = xb::tc_plan_bind(d->plan);
    xb::tc_plan_rewind();  // the step's linears come in the recorded order (if a plan was recorded at capture)
    const bool stochastic = d->temperature > 0.f && !d->override_armed;
    int rc = [&]() -> int {
        if (stochastic) {
            NL(xb::philox_uniform_counter(s, d->uniforms, 2LL * B * k, d->sample_seed, d->step_counter));
            ++d->launches_per_step;
        }
        for (int i = 0; i < k; ++i) CK(draft_pass(d, s, i, true));
        CK(draft_pass(d, s, k, false));  // the head's KV slot at ctx + k
        if (d->override_armed && !d->linears_only)
            CKCUDA(cudaMemcpyAsync(d->draft, d->draft_override, static_cast<size_t>(B) * k * sizeof(long long),
                                   cudaMemcpyDeviceToDevice, s));
        NL(xb::build_verify_tokens(s, d->verify_tokens, d->cur_tok, d->draft, B, k));
        CK(target_pass(d, s, R, d->verify_tokens));
        // greedy: draft i is kept iff it is the target's argmax of row i.  Stochastic: the reference's rule with the draft
        // token's probability under the head and this step's acceptance uniforms, logits scaled by 1 / T on both sides
        // (src/ops/sampling.cpp:129-171; with forced drafts there is no draft probability, so the greedy rule applies)
        const bool nucleus_on = stochastic && d->top_p < 1.0f;
        if (nucleus_on) {
            // the nucleus of every verify row's own distribution: the rule takes the target's probability inside it
            NL(xb::nucleus_rows(s, d->logits, d->vocab_local, B * R, d->vocab_local, 1.0f / d->temperature, d->top_p, nullptr, 0,
                                d->nucleus, nullptr, nullptr, 0));
            ++d->launches_per_step;
        }
        NL(xb::accept_finish(s, d->partials.p, xb::sampling_chunks(d->vocab_local), d->world,
                             partial_slice_stride(d, B * R), d->logits, d->vocab_local, d->vocab_local,
                             d->temperature > 0.f ? 1.0f / d->temperature : 1.0f, d->draft, stochastic ? d->draft_probs : nullptr,
                             stochastic ? d->uniforms + static_cast<size_t>(B) * k : nullptr, B, k, R, k,
                             reinterpret_cast<xb::AcceptOut*>(d->records), nucleus_on ? d->nucleus : nullptr));
        if (d->temperature > 0.f) {
            NL(xb::add_counter(s, d->step_counter, 1));
            ++d->launches_per_step;
        }
        // x still holds the pre-norm hidden rows of the verify pass (the final norm added the last MLP output)
        NL(xb::spec_commit(s, d->records, d->draft, B, k, R, d->ctx, d->n_commit, d->cur_tok, d->emitted, d->emitted_n,
                           d->h_last, d->x, static_cast<int>(c.hidden_size)));
        d->launches_per_step += 4;
        return 0;
    }();
    xb::tc_plan_bind(prev_plan);
    return rc;
}

}  // namespace

extern "C" {

size_t xinfer_spec_decoder_exchange_bytes(const xinfer_model_config* cfg, int batch, int k, int world) {
    if (!cfg || batch < 1 || k < 1 || world < 1) return 0;
    const auto& c = *cfg;
    const size_t M = static_cast<size_t>(batch) * (k + 1);
    const size_t ch = static_cast<size_t>(2 * c.linear_num_k_heads * 128 + c.linear_num_v_heads * 128);
    size_t halves = static_cast<size_t>(batch) * c.hidden_size + M * c.hidden_size + M * c.intermediate_size +
                    M * c.num_attention_heads * 512 + 2 * M * c.num_key_value_heads * 256 + M * c.num_attention_heads * 256 +
                    M * ch + 2 * M * c.linear_num_v_heads * 128;
    const size_t vl = static_cast<size_t>(c.vocab_size) / world + 1;
    const size_t part = static_cast<size_t>(world) * xb::sampling_scratch_bytes(static_cast<long long>(M), static_cast<long long>(vl));
    return halves * 2 + part + 16 * 256;  // + alignment slack of the eleven buffers
}

int xinfer_spec_decoder_create_tp(const xinfer_model_config* cfg, int batch, int k, int64_t max_seq, uint64_t seed,
                                  xinfer_tp* tp, xinfer_spec_decoder** out) {
    if (!cfg || !out || batch < 1 || k < 1 || k > 7 || max_seq < 8) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    const auto& c = *cfg;
    if (c.num_hidden_layers < 1 || c.hidden_size % 128 || c.intermediate_size % 128 || c.num_key_value_heads < 1 ||
        c.num_attention_heads % c.num_key_value_heads || (c.num_attention_heads / c.num_key_value_heads) * (k + 1) > 32 ||
        c.linear_num_k_heads < 1 || c.linear_num_v_heads % c.linear_num_k_heads || batch * (k + 1) > 32 ||
        c.rope_dim > 256 || c.rope_dim % 2)
        return XINFER_ERR_INVALID_ARGUMENT;
    const int world = tp ? xinfer_tp_world(tp) : 1;
    const int rank = tp ? xinfer_tp_rank(tp) : 0;
    if (world > 1) {
        // every split extent must divide evenly, and keep whole row pairs (and the 16-byte row alignment of TMA)
        const int64_t ch = 2 * c.linear_num_k_heads * 128 + c.linear_num_v_heads * 128;
        const int64_t split[] = {c.intermediate_size, c.hidden_size, c.num_attention_heads * 512, c.num_key_value_heads * 256,
                                 ch, c.linear_num_v_heads * 128, c.vocab_size};
        for (int64_t n : split)
            if (n % world || (n / world) % 8) return XINFER_ERR_INVALID_ARGUMENT;
        if (batch % world || !tp->connected) return XINFER_ERR_INVALID_ARGUMENT;
    }
    {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return XINFER_ERR_NO_DEVICE;
        int rc = xinfer_b200_init(dev);
        if (rc != XINFER_OK) return rc;
    }
    Dec* d = new (std::nothrow) Dec();
    if (!d) return XINFER_ERR_OUT_OF_MEMORY;
    d->cfg = c;
    d->batch = batch;
    d->k = k;
    d->max_seq = max_seq;
    d->seed = seed * 2654435761ULL + 12345;
    d->tp = world > 1 ? tp : nullptr;
    d->world = world;
    d->rank = rank;
    d->bl = batch / world;
    d->b0 = rank * d->bl;
    cudaGetDevice(&d->device);
    d->plan = xb::tc_plan_new();
    try {
        if (!d->plan) throw std::bad_alloc();
        const int M = batch * (k + 1);
        // first pass adds up what the decoder needs, the arena is created with exactly that, second pass carves it
        d->sizing = true;
        build_all(d);
        d->sizing = false;
        if (xinfer_arena_create(d->need_bytes + kAlign, kAlign, &d->arena) != XINFER_OK) throw std::bad_alloc();
        build_all(d);
        if (cudaMallocHost(&d->h_emitted, static_cast<size_t>(M) * sizeof(long long)) != cudaSuccess ||
            cudaMallocHost(&d->h_emitted_n, static_cast<size_t>(batch) * sizeof(int)) != cudaSuccess)
            throw std::bad_alloc();
    } catch (const std::bad_alloc&) {
        cudaGetLastError();
        xinfer_spec_decoder_destroy(d);
        return XINFER_ERR_OUT_OF_MEMORY;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) {
        xinfer_spec_decoder_destroy(d);
        return XINFER_ERR_CUDA;
    }
    *out = d;
    return xinfer_spec_decoder_reset(d, 0, seed);
}

int xinfer_spec_decoder_create(const xinfer_model_config* cfg, int batch, int k, int64_t max_seq, uint64_t seed,
                               xinfer_spec_decoder** out) {
    return xinfer_spec_decoder_create_tp(cfg, batch, k, max_seq, seed, nullptr, out);
}

void xinfer_spec_decoder_destroy(xinfer_spec_decoder* d) {
    if (!d) return;
    cudaDeviceSynchronize();
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    if (d->plan) xb::tc_plan_delete(d->plan);  // the recorded plan points into this decoder's weights
    if (d->arena) xinfer_arena_destroy(d->arena);
    if (d->chunk.x) { cudaFree(d->chunk.x); cudaFree(d->chunk.attn_scratch); }
    if (d->h_emitted) cudaFreeHost(d->h_emitted);
    if (d->h_emitted_n) cudaFreeHost(d->h_emitted_n);
    delete d;
}

int xinfer_spec_decoder_reset(xinfer_spec_decoder* d, int64_t context_len, uint64_t seed) {
    if (!d || context_len < 0 || context_len + 2 * (d->k + 1) > d->max_seq) return XINFER_ERR_INVALID_ARGUMENT;
    const auto& c = d->cfg;
    const int B = d->batch, Bl = d->bl, b0 = d->b0;
    uint64_t sd = seed * 0x9E3779B97F4A7C15ULL + 777;
    auto nxt = [&]() { return sd = sd * 6364136223846793005ULL + 1442695040888963407ULL; };
    // state tensors are [sequence][...]: this rank fills the slices of its own sequences with the values the
    // unsharded decoder would hold there
    auto fill_layer = [&](Layer& L) {
        if (L.full) {
            const size_t per = static_cast<size_t>(d->max_seq) * c.num_key_value_heads * 256;
            init_half_kernel<<<blocks_for(Bl * per, 256), 256>>>(L.k_cache, Bl * per, nxt(), 1, 0.f, 1.0f, b0 * per);
            init_half_kernel<<<blocks_for(Bl * per, 256), 256>>>(L.v_cache, Bl * per, nxt(), 1, 0.f, 1.0f, b0 * per);
        } else {
            const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads, ch = 2 * hk * 128 + hv * 128;
            const size_t per = static_cast<size_t>(hv) * 128 * 128;
            const float sig = context_len > 0 ? 0.05f : 0.0f;  // an empty context starts from zero state
            init_float_kernel<<<blocks_for(Bl * per, 256), 256>>>(L.S, Bl * per, nxt(), 0.f, sig, b0 * per);
            const size_t cper = static_cast<size_t>(3) * ch;
            init_float_kernel<<<blocks_for(Bl * cper, 256), 256>>>(L.conv_state, Bl * cper, nxt(), 0.f,
                                                                    context_len > 0 ? 1.0f : 0.0f, b0 * cper);
            cudaMemset(L.pend_k, 0, static_cast<size_t>(Bl) * hv * 8 * 128 * sizeof(float));
            cudaMemset(L.pend_d, 0, static_cast<size_t>(Bl) * hv * 8 * 128 * sizeof(float));
            cudaMemset(L.pend_g, 0, static_cast<size_t>(Bl) * hv * 8 * sizeof(float));
            cudaMemset(L.conv_pend, 0, static_cast<size_t>(Bl) * 8 * ch * sizeof(float));
        }
    };
    for (auto& L : d->layers) fill_layer(L);
    fill_layer(d->mtp_layer);
    xb::fill_int(nullptr, d->ctx, B, static_cast<int>(context_len));
    xb::fill_int(nullptr, d->n_commit, B, 0);
    xb::fill_int(nullptr, d->n_commit_zero, B, 0);
    init_tokens_kernel<<<1, 64>>>(d->cur_tok, B, nxt(), c.vocab_size);
    init_half_kernel<<<blocks_for(static_cast<size_t>(B) * c.hidden_size, 256), 256>>>(
        d->h_last, static_cast<size_t>(B) * c.hidden_size, nxt(), 1, 0.f, 1.0f, 0);
    cudaMemset(d->step_counter, 0, sizeof(unsigned long long));
    d->prev_rows = 0;
    d->ctx_upper = context_len;
    return cudaDeviceSynchronize() == cudaSuccess ? XINFER_OK : XINFER_ERR_CUDA;
}

int xinfer_spec_decoder_step(xinfer_spec_decoder* d, xinfer_stream_t stream) {
    if (!d) return XINFER_ERR_INVALID_ARGUMENT;
    // A step writes cache positions up to ctx + k.  The context lengths advance on the device; the host keeps an
    // upper bound (every step adds at most k + 1) and refuses a step that could run past the caches, where the
    // kernels would drop the newest keys silently (the reference's KVCache throws when it is full,
    // src/core/kv_cache.cpp advance()).
    if (d->ctx_upper + (d->k + 1) > d->max_seq) {
        d->error = "context would exceed max_seq";
        return XINFER_ERR_INVALID_ARGUMENT;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc;
    // The graph holds the previous pass's row count as a constant (k + 1): right after a prefill whose last chunk was
    // shorter, one step runs eagerly.
    if (d->graph_exec && d->prev_rows == d->k + 1) rc = cudaGraphLaunch(d->graph_exec, s) == cudaSuccess ? XINFER_OK : XINFER_ERR_CUDA;
    else rc = enqueue_step(d, s);
    if (rc >= 0) d->ctx_upper += d->k + 1;
    return rc;
}

int xinfer_spec_decoder_capture(xinfer_spec_decoder* d, xinfer_stream_t stream) {
    if (!d || !stream) return XINFER_ERR_INVALID_ARGUMENT;  // capture needs a non-default stream
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d->graph_exec) return XINFER_OK;
    // The lazy state commit reads the previous pass's row count, a host constant baked into the graph:
    // run one eager step first so that every replay sees prev_rows = k + 1.
    // The same eager step records the order of the tensor-core launches, so that in the captured step
    // every linear can ask L2 for the first weight stages of the one after it.
    if (d->prev_rows != d->k + 1) {
        if (d->ctx_upper + (d->k + 1) > d->max_seq) return XINFER_ERR_INVALID_ARGUMENT;
        xb::TcPlan* prev_plan = xb::tc_plan_bind(d->plan);
        xb::tc_plan_record_begin();
        int rc = enqueue_step(d, s);
        xb::tc_plan_bind(d->plan);  // (enqueue_step restored the previous binding)
        xb::tc_plan_record_end();
        xb::tc_plan_bind(prev_plan);
        if (rc < 0) return rc;
        d->ctx_upper += d->k + 1;
        if (cudaStreamSynchronize(s) != cudaSuccess) return XINFER_ERR_CUDA;
    }
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return XINFER_ERR_CUDA;
    int rc = enqueue_step(d, s);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(s, &g);
    if (rc < 0 || e != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        return rc < 0 ? rc : XINFER_ERR_CUDA;
    }
    if (cudaGraphInstantiate(&d->graph_exec, g, 0) != cudaSuccess) {
        cudaGraphDestroy(g);
        return XINFER_ERR_CUDA;
    }
    d->graph = g;
    return XINFER_OK;
}

int xinfer_spec_decoder_results(xinfer_spec_decoder* d, xinfer_stream_t stream, int64_t* emitted_host, int* counts_host) {
    if (!d || !emitted_host || !counts_host) return XINFER_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int M = d->batch * (d->k + 1);
    if (cudaMemcpyAsync(d->h_emitted, d->emitted, static_cast<size_t>(M) * sizeof(long long), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(d->h_emitted_n, d->emitted_n, static_cast<size_t>(d->batch) * sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        cudaGetLastError();
        return XINFER_ERR_CUDA;
    }
    memcpy(emitted_host, d->h_emitted, static_cast<size_t>(M) * sizeof(long long));
    memcpy(counts_host, d->h_emitted_n, static_cast<size_t>(d->batch) * sizeof(int));
    return XINFER_OK;
}

int xinfer_spec_decoder_set_tokens(xinfer_spec_decoder* d, const int64_t* cur_tokens_host) {
    if (!d || !cur_tokens_host) return XINFER_ERR_INVALID_ARGUMENT;
    memcpy(d->h_emitted, cur_tokens_host, static_cast<size_t>(d->batch) * sizeof(long long));  // pinned staging
    return cudaMemcpy(d->cur_tok, d->h_emitted, static_cast<size_t>(d->batch) * sizeof(long long),
                      cudaMemcpyHostToDevice) == cudaSuccess ? XINFER_OK : XINFER_ERR_CUDA;
}

// Measurement entry: enqueue only the W4A16 launches of one step, in the step's order and on the step's
// weights, so that their device time can be taken with events apart from the mixers.
int xinfer_spec_decoder_enqueue_linears(xinfer_spec_decoder* d, xinfer_stream_t stream) {
    if (!d) return XINFER_ERR_INVALID_ARGUMENT;
    d->linears_only = true;
    int rc = enqueue_step(d, static_cast<cudaStream_t>(stream));
    d->linears_only = false;
    return rc;
}

int xinfer_spec_decoder_override_drafts(xinfer_spec_decoder* d, const int64_t* drafts_host) {
    if (!d || d->graph_exec) return XINFER_ERR_INVALID_ARGUMENT;
    d->override_armed = drafts_host != nullptr;
    if (!drafts_host) return XINFER_OK;
    return cudaMemcpy(d->draft_override, drafts_host, static_cast<size_t>(d->batch) * d->k * sizeof(long long),
                      cudaMemcpyHostToDevice) == cudaSuccess ? XINFER_OK : XINFER_ERR_CUDA;
}

int64_t xinfer_spec_decoder_info(const xinfer_spec_decoder* d, int what) {
    if (!d) return -1;
    switch (what) {
        case 0: return static_cast<int64_t>(d->weight_bytes);
        case 1: return static_cast<int64_t>(d->state_bytes);
        case 2: return d->launches_per_step;
        case 3: return d->graph_exec ? 1 : 0;
        case 4: return static_cast<int64_t>(d->linear_bytes);
        case 5: return d->linear_launches;
        case 6: return d->exchanges_per_step;
        case 7: return d->arena ? static_cast<int64_t>(xinfer_arena_capacity(d->arena)) : 0;
        default: return -1;
    }
}

// temperature <= 0: greedy drafting and acceptance (the default, what the reference's engine runs).  temperature > 0:
// every draft token is drawn from softmax(head logits / T) and the verify pass applies the reference's stochastic rule
// (src/ops/sampling.cpp:129-171) to the target's logits / T with the draft's probability; both consume Philox4x32-10
// uniforms of (seed, step index): element b * k + i picks draft i of sequence b, element batch * k + b * k + i is its
// acceptance uniform.  The step index lives in device memory (reset sets it to 0), so a captured step draws fresh
// numbers on every replay.  Call before xinfer_spec_decoder_capture.  One GPU only (the rule reads the draft token's
// logit, which an N-split LM head holds on one rank).
int xinfer_spec_decoder_set_sampling(xinfer_spec_decoder* d, float temperature, uint64_t seed) {
    if (!d) return XINFER_ERR_INVALID_ARGUMENT;
    if (temperature > 0.f && d->world > 1) { d->error = "stochastic acceptance runs on one GPU"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (d->graph_exec) { d->error = "set the sampling mode before capture"; return XINFER_ERR_INVALID_ARGUMENT; }
    d->temperature = temperature > 0.f ? temperature : 0.f;
    d->sample_seed = seed;
    return XINFER_OK;
}

int xinfer_spec_decoder_set_top_p(xinfer_spec_decoder* d, float top_p) {
    if (!d || !(top_p > 0.f) || top_p > 1.f) return XINFER_ERR_INVALID_ARGUMENT;
    if (d->graph_exec) { d->error = "set the sampling mode before capture"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (top_p < 1.f && d->world > 1) { d->error = "stochastic acceptance runs on one GPU"; return XINFER_ERR_INVALID_ARGUMENT; }
    d->top_p = top_p;
    return XINFER_OK;
}

// Builds the context from a prompt: tokens [batch][T] (host), all sequences the same length, starting from the empty
// context of reset(0, seed).  Positions 0 .. T-2 go through the target model in chunks of up to 512 rows over all
// sequences (prefill_chunk: projections on the prefill GEMM, mixers four positions at a time with every row kept,
// so KV caches, Gated-DeltaNet and convolution state advance as in steps whose drafts were all accepted), the MTP
// head's KV slots of the same positions are written from (token, hidden state in front of it; zeros in front of
// position 0), and the last prompt token becomes the current token.  Afterwards ctx = T - 1 and
// xinfer_spec_decoder_step continues from there.  Stands where the reference's chunked prefill does
// (forward_prefill_chunk, src/targets/qwen3_8/forward.cpp:402-554, called from engine.cpp:330-398).  One GPU only.
int xinfer_spec_decoder_prefill(xinfer_spec_decoder* d, xinfer_stream_t stream, const int64_t* prompt_host, int64_t T) {
    if (!d || !prompt_host || T < 1) return XINFER_ERR_INVALID_ARGUMENT;
    const int B = d->batch, R = d->k + 1, H = static_cast<int>(d->cfg.hidden_size);
    if (d->world > 1) { d->error = "prefill runs on one GPU"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (d->ctx_upper != 0) { d->error = "prefill starts from the empty context (reset(0, seed))"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (T - 1 + 2 * R > d->max_seq) { d->error = "prompt does not fit the cache"; return XINFER_ERR_INVALID_ARGUMENT; }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // positions per sequence and chunk: 512 rows over all sequences, a multiple of the mixers' four
    int Cp = (512 / B) & ~3;
    if (Cp < 4) Cp = 4;
    if (T - 1 < Cp) Cp = static_cast<int>(((T - 1) + 3) & ~3LL);
    if (Cp > 0) {
        int rc0 = ensure_chunk_bufs(d, B * Cp);
        if (rc0 < 0) return rc0;
    }
    long long* prompt = nullptr;
    const size_t pbytes = static_cast<size_t>(B) * T * sizeof(long long);
    if (cudaMalloc(&prompt, pbytes) != cudaSuccess) { cudaGetLastError(); return XINFER_ERR_OUT_OF_MEMORY; }
    int prev_r = 0;
    int rc = [&]() -> int {
        CKCUDA(cudaMemcpyAsync(prompt, prompt_host, pbytes, cudaMemcpyHostToDevice, s));
        CKCUDA(cudaMemsetAsync(d->h_last, 0, static_cast<size_t>(B) * H * sizeof(__half), s));
        for (long long c0 = 0; c0 < T - 1; c0 += Cp) {
            const int Rc = static_cast<int>((T - 1 - c0) < Cp ? (T - 1 - c0) : Cp);
            CK(prefill_chunk(d, s, prompt, T, c0, Rc, &prev_r));
        }
        // as after a step whose rows were all kept: the last mixer launch's rows are replayed by the next pass
        CK(xb::fill_int(s, d->ctx, B, static_cast<int>(T - 1)));
        CK(xb::fill_int(s, d->n_commit, B, prev_r));
        last_prompt_token_kernel<<<1, 64, 0, s>>>(d->cur_tok, prompt, B, T);
        CKCUDA(cudaGetLastError());
        CKCUDA(cudaStreamSynchronize(s));
        return XINFER_OK;
    }();
    cudaFree(prompt);
    if (rc == XINFER_OK) {
        d->prev_rows = prev_r;
        d->ctx_upper = T - 1;
    }
    return rc;
}

// The device side of Engine::generate's speculative loop (src/runtime/engine.cpp:262-560) for a batch of prompts of one
// length: argument checks in the reference's order and words, reset to the empty context, prefill, then steps until
// every sequence has stopped.  A sequence stops on eos_token_id / im_end_token_id (the stop token is not returned,
// finish reason 0 = "stop", engine.cpp:452-468) or when it holds max_new_tokens tokens (1 = "length"); tokens a step
// emits beyond that are dropped, where the reference shortens its last draft instead (engine.cpp:420).  The sequences
// run in lockstep: one that has stopped keeps its lane, its context length is put back after every step so that it
// cannot run into the end of the cache while the others finish.  Uses the captured graph when there is one.
int xinfer_spec_decoder_generate(xinfer_spec_decoder* d, xinfer_stream_t stream, const int64_t* prompt_host, int64_t T,
                                 const xinfer_generation_config* g, int64_t* token_ids_out, int32_t* generated_out,
                                 int32_t* finish_out, xinfer_generation_stats* stats) {
    if (!d || !g || !token_ids_out || !generated_out || !finish_out) return XINFER_ERR_INVALID_ARGUMENT;
    const int B = d->batch, R = d->k + 1;
    if (g->max_new_tokens <= 0) { d->error = "Invalid max_new_tokens: must be greater than 0"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (g->temperature < 0.f) { d->error = "Invalid temperature: must be >= 0.0"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (!(g->top_p > 0.f) || g->top_p > 1.0f) { d->error = "Invalid top_p: must be in (0, 1]"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (g->top_p < 1.0f && !(g->temperature > 0.f)) {
        d->error = "top_p < 1 needs temperature > 0 (greedy decoding takes the arg-max of the whole distribution)";
        return XINFER_ERR_INVALID_ARGUMENT;
    }
    if (!prompt_host || T < 1) { d->error = "empty prompt"; return XINFER_ERR_INVALID_ARGUMENT; }
    if (T + g->max_new_tokens + d->k > d->max_seq) {
        d->error = "This model's maximum context length is " + std::to_string(d->max_seq - d->k) + " tokens. However, you requested " +
                   std::to_string(T + g->max_new_tokens) + " tokens (" + std::to_string(T) + " in the messages, " +
                   std::to_string(g->max_new_tokens) + " in the completion).";
        return XINFER_ERR_INVALID_ARGUMENT;
    }
    if (g->temperature != d->temperature || (g->temperature > 0.f && g->seed != d->sample_seed)) {
        int rc = xinfer_spec_decoder_set_sampling(d, g->temperature, g->seed);
        if (rc < 0) return rc;
    }
    if (g->top_p != d->top_p) {
        int rc = xinfer_spec_decoder_set_top_p(d, g->top_p);
        if (rc < 0) return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto t0 = std::chrono::steady_clock::now();
    int rc = xinfer_spec_decoder_reset(d, 0, g->seed);
    if (rc < 0) return rc;
    rc = xinfer_spec_decoder_prefill(d, stream, prompt_host, T);
    if (rc < 0) return rc;
    const int64_t cap = g->max_new_tokens;
    std::vector<int64_t> emitted(static_cast<size_t>(B) * R);
    std::vector<int> counts(B), ctx(B, static_cast<int>(T - 1));
    std::vector<char> running(B, 1);
    for (int b = 0; b < B; ++b) { generated_out[b] = 0; finish_out[b] = 1; }
    int n_running = B;
    int64_t steps = 0, first_step_tokens = 0;
    auto t_first = t0;
    while (n_running > 0) {
        int64_t top = 0;
        for (int b = 0; b < B; ++b) top = ctx[b] > top ? ctx[b] : top;
        d->ctx_upper = top;                       // exact: the host has read every step's counts
        if (top + R > d->max_seq) break;          // the reference's "Context length limit reached": the rest end on "length"
        rc = xinfer_spec_decoder_step(d, stream);
        if (rc < 0) return rc;
        rc = xinfer_spec_decoder_results(d, stream, emitted.data(), counts.data());
        if (rc < 0) return rc;
        ++steps;
        for (int b = 0; b < B; ++b) {
            if (!running[b]) {                    // a parked lane: put its context length back
                if (cudaMemcpyAsync(d->ctx + b, &ctx[b], sizeof(int), cudaMemcpyHostToDevice, s) != cudaSuccess) return XINFER_ERR_CUDA;
                continue;
            }
            ctx[b] += counts[b];
            for (int j = 0; j < counts[b] && running[b]; ++j) {
                const int64_t tok = emitted[static_cast<size_t>(b) * R + j];
                if ((g->eos_token_id >= 0 && tok == g->eos_token_id) || (g->im_end_token_id >= 0 && tok == g->im_end_token_id)) {
                    finish_out[b] = 0;
                    running[b] = 0;
                } else {
                    token_ids_out[static_cast<size_t>(b) * cap + generated_out[b]++] = tok;
                    if (steps == 1) ++first_step_tokens;
                    if (generated_out[b] == cap) running[b] = 0;   // finish reason stays "length"
                }
            }
            if (!running[b]) --n_running;
        }
        if (steps == 1) t_first = std::chrono::steady_clock::now();
    }
    if (cudaStreamSynchronize(s) != cudaSuccess) return XINFER_ERR_CUDA;
    if (stats) {
        const auto t1 = std::chrono::steady_clock::now();
        int64_t total = 0;
        for (int b = 0; b < B; ++b) total += generated_out[b];
        stats->prompt_tokens = T;
        stats->steps = steps;
        stats->generated_tokens = total;
        stats->time_to_first_token_sec = std::chrono::duration<double>(t_first - t0).count();
        stats->total_time_sec = std::chrono::duration<double>(t1 - t0).count();
        const double dt = std::chrono::duration<double>(t1 - t_first).count();
        stats->decode_tokens_per_sec = steps > 1 && dt > 0 ? static_cast<double>(total - first_step_tokens) / dt : 0.0;
    }
    return XINFER_OK;
}

// Replaces the decoder's synthetic weights by the tensors of a `.xinfer` artifact, under the section names the
// reference's loader uses (src/targets/qwen3_8_27b/weights.cpp:358-640): `model.language_model.embed_tokens.weight`
// (BF16 table, kept as BF16), `model.language_model.norm.weight`, `lm_head.weight` (+ `.scales`), and per layer
// `model.language_model.layers.<l>.{input_layernorm,post_attention_layernorm}.weight`, `.mlp.{gate,up,down}_proj.weight`,
// `.self_attn.{q,k,v,o}_proj.weight`, `.self_attn.{q,k}_norm.weight` or `.linear_attn.{in_proj_qkv,in_proj_z,in_proj_b,
// in_proj_a,out_proj}.weight`, `.linear_attn.{conv1d.weight,A_log,dt_bias,norm.weight}`.  RMSNorm vectors follow the
// checkpoint's "1 + w" convention except the gated norm of the linear-attention block (weights.cpp:306-318).  Under
// tensor parallelism every rank loads its own row range of every split projection.  The layer kind found in the file
// must be the one this decoder was built with.  The MTP head is not part of the reference's artifacts: its tensors
// (`mtp.fc.weight`, `mtp.pre_fc_norm_embedding.weight`, `mtp.pre_fc_norm_hidden.weight`, `mtp.layers.0.*` named like a
// full-attention layer) are loaded when present and left as they are otherwise.
int xinfer_spec_decoder_load_artifact(xinfer_spec_decoder* d, xinfer_artifact* a, int verify) {
    if (!d || !a) return XINFER_ERR_INVALID_ARGUMENT;
    const auto& c = d->cfg;
    int rc = XINFER_OK;  // (the caller's current device is the decoder's, as for every other call on it)
    auto lin = [&](const std::string& name, Linear& l) {
        if (rc != XINFER_OK) return;
        rc = xinfer_artifact_load_linear(a, name.c_str(), l.n_full, l.k, 128, l.row0, l.n, l.w, l.s, verify);
        if (rc != XINFER_OK) xb::set_last_error((name + ": " + xinfer_artifact_error(a)).c_str());
    };
    auto vec = [&](const std::string& name, float* dst, int64_t count, int unit_offset) {
        if (rc != XINFER_OK) return;
        rc = xinfer_artifact_load_bf16_as_f32(a, name.c_str(), count, unit_offset, dst);
        if (rc != XINFER_OK) xb::set_last_error((name + ": " + xinfer_artifact_error(a)).c_str());
    };
    auto has = [&](const std::string& name) { return xinfer_artifact_find(a, name.c_str()) >= 0; };
    auto layer = [&](const std::string& prefix, Layer& L) {
        const bool file_full = has(prefix + ".self_attn.q_proj.weight");
        const bool file_lin = has(prefix + ".linear_attn.in_proj_qkv.weight");
        if (rc == XINFER_OK && (file_full == file_lin || file_full != L.full)) {
            xb::set_last_error((prefix + ": the artifact's layer kind is not the one this decoder was built with").c_str());
            rc = XINFER_ERR_CONTRACT;
            return;
        }
        vec(prefix + ".input_layernorm.weight", L.input_norm, c.hidden_size, 1);
        vec(prefix + ".post_attention_layernorm.weight", L.post_norm, c.hidden_size, 1);
        lin(prefix + ".mlp.gate_proj.weight", L.gate);
        lin(prefix + ".mlp.up_proj.weight", L.up);
        lin(prefix + ".mlp.down_proj.weight", L.down);
        if (L.full) {
            lin(prefix + ".self_attn.q_proj.weight", L.q_proj);
            lin(prefix + ".self_attn.k_proj.weight", L.k_proj);
            lin(prefix + ".self_attn.v_proj.weight", L.v_proj);
            lin(prefix + ".self_attn.o_proj.weight", L.o_proj);
            vec(prefix + ".self_attn.q_norm.weight", L.q_norm, 256, 1);
            vec(prefix + ".self_attn.k_norm.weight", L.k_norm, 256, 1);
        } else {
            const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads, ch = 2 * hk * 128 + hv * 128;
            lin(prefix + ".linear_attn.in_proj_qkv.weight", L.in_qkv);
            lin(prefix + ".linear_attn.in_proj_z.weight", L.in_z);
            lin(prefix + ".linear_attn.in_proj_b.weight", L.in_b);
            lin(prefix + ".linear_attn.in_proj_a.weight", L.in_a);
            lin(prefix + ".linear_attn.out_proj.weight", L.out_proj);
            vec(prefix + ".linear_attn.conv1d.weight", L.conv_w, ch * 4, 0);
            vec(prefix + ".linear_attn.A_log", L.A_log, hv, 0);
            vec(prefix + ".linear_attn.dt_bias", L.dt_bias, hv, 0);
            vec(prefix + ".linear_attn.norm.weight", L.gdn_norm, 128, 0);
        }
    };
    const std::string embed_name = "model.language_model.embed_tokens.weight";
    rc = xinfer_artifact_load_section(a, embed_name.c_str(), 0, static_cast<uint64_t>(c.vocab_size) * c.hidden_size * 2, d->embed, verify);
    if (rc != XINFER_OK) xb::set_last_error((embed_name + ": " + xinfer_artifact_error(a)).c_str());
    vec("model.language_model.norm.weight", d->final_norm, c.hidden_size, 1);
    lin("lm_head.weight", d->lm_head);
    for (size_t l = 0; l < d->layers.size() && rc == XINFER_OK; ++l)
        layer("model.language_model.layers." + std::to_string(l), d->layers[l]);
    if (rc == XINFER_OK && has("mtp.fc.weight")) {
        lin("mtp.fc.weight", d->mtp_fc);
        vec("mtp.pre_fc_norm_embedding.weight", d->mtp_enorm, c.hidden_size, 1);
        vec("mtp.pre_fc_norm_hidden.weight", d->mtp_hnorm, c.hidden_size, 1);
        layer("mtp.layers.0", d->mtp_layer);
    }
    if (cudaDeviceSynchronize() != cudaSuccess && rc == XINFER_OK) rc = XINFER_ERR_CUDA;
    return rc;
}

// Device pointer of a named tensor, for tests that mirror weights and state on the host.
// layer = -1 addresses the model-level tensors, layer = num_hidden_layers the MTP head's layer.
void* xinfer_spec_decoder_tensor(xinfer_spec_decoder* d, int layer, const char* name, int64_t* bytes) {
    if (!d || !name) return nullptr;
    const auto& c = d->cfg;
    const std::string n(name);
    int64_t dummy = 0;
    int64_t& nb = bytes ? *bytes : dummy;
    auto lin_w = [&](const Linear& l) { nb = l.n * (l.k / 2); return static_cast<void*>(l.w); };
    auto lin_s = [&](const Linear& l) { nb = l.n * (l.k / 128) * 2; return static_cast<void*>(l.s); };
    const int64_t H = c.hidden_size, B = d->batch, M = B * (d->k + 1);
    const int64_t Bl = d->bl;  // state tensors hold this rank's own sequences only
    if (layer < 0) {
        if (n == "embed") { nb = c.vocab_size * H * 2; return d->embed; }
        if (n == "final_norm") { nb = H * 4; return d->final_norm; }
        if (n == "mtp_enorm") { nb = H * 4; return d->mtp_enorm; }
        if (n == "mtp_hnorm") { nb = H * 4; return d->mtp_hnorm; }
        if (n == "lm_head.w") return lin_w(d->lm_head);
        if (n == "lm_head.s") return lin_s(d->lm_head);
        if (n == "mtp_fc.w") return lin_w(d->mtp_fc);
        if (n == "mtp_fc.s") return lin_s(d->mtp_fc);
        if (n == "ctx") { nb = B * 4; return d->ctx; }
        if (n == "n_commit") { nb = B * 4; return d->n_commit; }
        if (n == "cur_tok") { nb = B * 8; return d->cur_tok; }
        if (n == "draft") { nb = B * d->k * 8; return d->draft; }
        if (n == "h_last") { nb = B * H * 2; return d->h_last; }
        if (n == "logits") { nb = M * d->vocab_local * 4; return d->logits; }
        if (n == "x") { nb = M * H * 2; return d->x; }
        if (n == "records") { nb = B * static_cast<int64_t>(sizeof(xinfer_accept_record)); return d->records; }
        return nullptr;
    }
    Layer* L = nullptr;
    if (layer < static_cast<int>(d->layers.size())) L = &d->layers[layer];
    else if (layer == static_cast<int>(d->layers.size())) L = &d->mtp_layer;
    if (!L) return nullptr;
    if (n == "is_full") { nb = 0; return L->full ? reinterpret_cast<void*>(1) : nullptr; }
    if (n == "input_norm") { nb = H * 4; return L->input_norm; }
    if (n == "post_norm") { nb = H * 4; return L->post_norm; }
    if (n == "gate.w") return lin_w(L->gate);
    if (n == "gate.s") return lin_s(L->gate);
    if (n == "up.w") return lin_w(L->up);
    if (n == "up.s") return lin_s(L->up);
    if (n == "down.w") return lin_w(L->down);
    if (n == "down.s") return lin_s(L->down);
    if (L->full) {
        const int64_t kv = Bl * d->max_seq * c.num_key_value_heads * 256 * 2;
        if (n == "q_proj.w") return lin_w(L->q_proj);
        if (n == "q_proj.s") return lin_s(L->q_proj);
        if (n == "k_proj.w") return lin_w(L->k_proj);
        if (n == "k_proj.s") return lin_s(L->k_proj);
        if (n == "v_proj.w") return lin_w(L->v_proj);
        if (n == "v_proj.s") return lin_s(L->v_proj);
        if (n == "o_proj.w") return lin_w(L->o_proj);
        if (n == "o_proj.s") return lin_s(L->o_proj);
        if (n == "q_norm") { nb = 256 * 4; return L->q_norm; }
        if (n == "k_norm") { nb = 256 * 4; return L->k_norm; }
        if (n == "k_cache") { nb = kv; return L->k_cache; }
        if (n == "v_cache") { nb = kv; return L->v_cache; }
    } else {
        const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads, ch = 2 * hk * 128 + hv * 128;
        if (n == "in_qkv.w") return lin_w(L->in_qkv);
        if (n == "in_qkv.s") return lin_s(L->in_qkv);
        if (n == "in_z.w") return lin_w(L->in_z);
        if (n == "in_z.s") return lin_s(L->in_z);
        if (n == "in_b.w") return lin_w(L->in_b);
        if (n == "in_b.s") return lin_s(L->in_b);
        if (n == "in_a.w") return lin_w(L->in_a);
        if (n == "in_a.s") return lin_s(L->in_a);
        if (n == "out_proj.w") return lin_w(L->out_proj);
        if (n == "out_proj.s") return lin_s(L->out_proj);
        if (n == "conv_w") { nb = ch * 4 * 4; return L->conv_w; }
        if (n == "A_log") { nb = hv * 4; return L->A_log; }
        if (n == "dt_bias") { nb = hv * 4; return L->dt_bias; }
        if (n == "gdn_norm") { nb = 128 * 4; return L->gdn_norm; }
        if (n == "S") { nb = Bl * hv * 128 * 128 * 4; return L->S; }
        if (n == "conv_state") { nb = Bl * 3 * ch * 4; return L->conv_state; }
    }
    return nullptr;
}

const char* xinfer_spec_decoder_error(const xinfer_spec_decoder* d) { return d ? d->error.c_str() : ""; }

}  // extern "C"
