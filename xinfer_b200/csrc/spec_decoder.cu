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
#include <string.h>

#include <new>
#include <string>
#include <vector>

#include "../../include/xinfer_b200.h"
#include "mixers.h"
#include "w4a16.h"
#include "sampling.h"

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
__global__ void init_bytes_kernel(uint8_t* p, size_t n, uint64_t seed) {
    size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        *reinterpret_cast<uint32_t*>(p + i) = mix32(seed * 0x9E3779B97F4A7C15ULL + i);
    } else {
        for (; i < n; ++i) p[i] = static_cast<uint8_t>(mix32(seed * 0x9E3779B97F4A7C15ULL + i));
    }
}
// mode 0: |N(0, sigma)| / 7 (int4 group scales)   mode 1: mean + N(0, sigma)
__global__ void init_half_kernel(__half* p, size_t n, uint64_t seed, int mode, float mean, float sigma) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = normal01(seed, i);
    p[i] = __float2half_rn(mode == 0 ? fabsf(z * sigma) / 7.0f : mean + z * sigma);
}
__global__ void init_float_kernel(float* p, size_t n, uint64_t seed, float mean, float sigma) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = mean + normal01(seed, i) * sigma;
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

struct Linear {
    uint8_t* w = nullptr;
    __half* s = nullptr;
    int64_t n = 0, k = 0;
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
    std::vector<void*> allocs;
    std::vector<Layer> layers;
    Layer mtp_layer;
    Linear mtp_fc, lm_head;
    float *mtp_enorm = nullptr, *mtp_hnorm = nullptr, *final_norm = nullptr;
    uint16_t* embed = nullptr;
    // sequence state
    int *ctx = nullptr, *ctx_draft = nullptr, *n_commit = nullptr, *n_commit_zero = nullptr;
    long long *cur_tok = nullptr, *draft = nullptr, *verify_tokens = nullptr, *argmax_out = nullptr, *emitted = nullptr;
    int* emitted_n = nullptr;
    __half *h_last = nullptr, *mtp_hidden = nullptr;
    xinfer_accept_record* records = nullptr;
    // activations (rows up to batch * (k + 1))
    __half *x = nullptr, *normed = nullptr, *proj_out = nullptr, *mlp = nullptr, *q_gate = nullptr, *qbuf = nullptr,
           *kbuf = nullptr, *vbuf = nullptr, *attn_out = nullptr, *qkv_raw = nullptr, *qkv_conv = nullptr, *zbuf = nullptr,
           *bbuf = nullptr, *abuf = nullptr, *delta_out = nullptr, *cat = nullptr;
    float *logits = nullptr, *attn_scratch = nullptr;
    // pinned result staging
    long long* h_emitted = nullptr;
    int* h_emitted_n = nullptr;
    long long* draft_override = nullptr;  // test hook: when armed, the verify pass checks these tokens instead
    bool override_armed = false;
    int prev_rows = 0;       // rows of the previous target pass (for the lazy state commit)
    cudaGraphExec_t graph_exec = nullptr;
    cudaGraph_t graph = nullptr;
    std::string error;
    size_t weight_bytes = 0, state_bytes = 0;
    long long launches_per_step = 0;
    bool linears_only = false;   // measurement mode: enqueue only the W4A16 launches of a step
    long long linear_launches = 0;
    double linear_bytes = 0;     // algorithmic bytes of those launches
};

namespace {

using Dec = xinfer_spec_decoder;

template <typename T>
T* dalloc(Dec* d, size_t count, bool is_state = false) {
    void* p = nullptr;
    if (count == 0) count = 1;
    if (cudaMalloc(&p, count * sizeof(T)) != cudaSuccess) throw std::bad_alloc();
    d->allocs.push_back(p);
    (is_state ? d->state_bytes : d->weight_bytes) += count * sizeof(T);
    return static_cast<T*>(p);
}

unsigned blocks_for(size_t n, int per) { return static_cast<unsigned>((n + per - 1) / per); }

uint64_t next_seed(Dec* d) { return d->seed = d->seed * 6364136223846793005ULL + 1442695040888963407ULL; }

Linear make_linear(Dec* d, int64_t n, int64_t k) {
    Linear l;
    l.n = n;
    l.k = k;
    const size_t wb = static_cast<size_t>(n) * (k / 2), sc = static_cast<size_t>(n) * (k / 128);
    l.w = dalloc<uint8_t>(d, wb);
    l.s = dalloc<__half>(d, sc);
    init_bytes_kernel<<<blocks_for((wb + 3) / 4, 256), 256>>>(l.w, wb, next_seed(d));
    init_half_kernel<<<blocks_for(sc, 256), 256>>>(l.s, sc, next_seed(d), 0, 0.f, 0.02f);
    return l;
}
float* make_floats(Dec* d, size_t n, float mean, float sigma) {
    float* p = dalloc<float>(d, n);
    init_float_kernel<<<blocks_for(n, 256), 256>>>(p, n, next_seed(d), mean, sigma);
    return p;
}

void make_layer(Dec* d, Layer& L, bool full) {
    const auto& c = d->cfg;
    const int64_t H = c.hidden_size, F = c.intermediate_size;
    L.full = full;
    L.input_norm = make_floats(d, H, 1.0f, 0.02f);
    L.post_norm = make_floats(d, H, 1.0f, 0.02f);
    L.gate = make_linear(d, F, H);
    L.up = make_linear(d, F, H);
    L.down = make_linear(d, H, F);
    if (full) {
        L.q_proj = make_linear(d, c.num_attention_heads * 512, H);
        L.k_proj = make_linear(d, c.num_key_value_heads * 256, H);
        L.v_proj = make_linear(d, c.num_key_value_heads * 256, H);
        L.o_proj = make_linear(d, H, c.num_attention_heads * 256);
        L.q_norm = make_floats(d, 256, 1.0f, 0.02f);
        L.k_norm = make_floats(d, 256, 1.0f, 0.02f);
        const size_t kv = static_cast<size_t>(d->batch) * d->max_seq * c.num_key_value_heads * 256;
        L.k_cache = dalloc<__half>(d, kv, true);
        L.v_cache = dalloc<__half>(d, kv, true);
    } else {
        const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads;
        const int64_t ch = 2 * hk * 128 + hv * 128;
        L.in_qkv = make_linear(d, ch, H);
        L.in_z = make_linear(d, hv * 128, H);
        L.in_b = make_linear(d, hv, H);
        L.in_a = make_linear(d, hv, H);
        L.out_proj = make_linear(d, H, hv * 128);
        L.conv_w = make_floats(d, ch * 4, 0.0f, 0.5f);
        L.A_log = make_floats(d, hv, 0.5f, 0.5f);
        L.dt_bias = make_floats(d, hv, 0.0f, 0.5f);
        L.gdn_norm = make_floats(d, 128, 1.0f, 0.02f);
        L.S = dalloc<float>(d, static_cast<size_t>(d->batch) * hv * 128 * 128, true);
        L.pend_k = dalloc<float>(d, static_cast<size_t>(d->batch) * hv * 8 * 128, true);
        L.pend_d = dalloc<float>(d, static_cast<size_t>(d->batch) * hv * 8 * 128, true);
        L.pend_g = dalloc<float>(d, static_cast<size_t>(d->batch) * hv * 8, true);
        L.conv_state = dalloc<float>(d, static_cast<size_t>(d->batch) * 3 * ch, true);
        L.conv_pend = dalloc<float>(d, static_cast<size_t>(d->batch) * 8 * ch, true);
    }
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

void account(Dec* d, const Linear& l, int M, int out_bytes, bool count_x) {
    d->linear_bytes += static_cast<double>(l.n) * (l.k / 2) + static_cast<double>(l.n) * (l.k / 128) * 2 +
                       (count_x ? static_cast<double>(M) * l.k * 2 : 0.0) + static_cast<double>(M) * l.n * out_bytes;
}

int lin(Dec* d, cudaStream_t s, __half* y, const __half* x, const Linear& l, int M) {
    ++d->launches_per_step;
    ++d->linear_launches;
    account(d, l, M, 2, true);
    return xinfer_linear_int4_f16f16(s, y, x, l.w, l.s, nullptr, M, l.n, l.k, 128);
}

// One decoder layer on M = batch * R rows; `x` is updated in place (the second residual add is folded
// into the next layer's norm by the caller through `pending_delta`).
int layer_forward(Dec* d, cudaStream_t s, Layer& L, int R, const int* ctx, const int* n_commit, int prev_rows,
                  bool first, const float* next_norm_unused) {
    (void)next_norm_unused;
    const auto& c = d->cfg;
    const int B = d->batch, M = B * R;
    const int H = static_cast<int>(c.hidden_size);
    // x += previous layer's MLP output (none for the first layer), then input RMSNorm
    if (first) NL(xb::rmsnorm_rows(s, d->normed, H, d->x, L.input_norm, M, H, c.rms_norm_eps));
    else NL(xb::add_rmsnorm_rows(s, d->normed, d->x, d->proj_out, L.input_norm, M, H, c.rms_norm_eps));
    ++d->launches_per_step;
    if (L.full) {
        xinfer_fused_desc fd[3] = {{d->q_gate, L.q_proj.w, L.q_proj.s, nullptr, L.q_proj.n},
                                   {d->kbuf, L.k_proj.w, L.k_proj.s, nullptr, L.k_proj.n},
                                   {d->vbuf, L.v_proj.w, L.v_proj.s, nullptr, L.v_proj.n}};
        CK(xinfer_linear_int4_fused_f16(s, d->normed, fd, 3, M, H, 128));
        ++d->linear_launches;
        account(d, L.q_proj, M, 2, true);
        account(d, L.k_proj, M, 2, false);
        account(d, L.v_proj, M, 2, false);
        NL(xb::attn_prep(s, d->qbuf, L.k_cache, L.v_cache, d->q_gate, d->kbuf, d->vbuf, L.q_norm, L.k_norm, ctx, B, R,
                         static_cast<int>(c.num_attention_heads), static_cast<int>(c.num_key_value_heads), d->max_seq,
                         c.rms_norm_eps, c.rope_theta, c.rope_dim));
        NL(xb::attn_decode(s, d->attn_out, d->qbuf, d->q_gate, L.k_cache, L.v_cache, ctx, B, R,
                           static_cast<int>(c.num_attention_heads), static_cast<int>(c.num_key_value_heads), d->max_seq,
                           d->attn_splits, d->attn_scratch));
        d->launches_per_step += 4;
        CK(lin(d, s, d->proj_out, d->attn_out, L.o_proj, M));
    } else {
        const int hv = static_cast<int>(c.linear_num_v_heads), hk = static_cast<int>(c.linear_num_k_heads);
        const int ch = 2 * hk * 128 + hv * 128;
        xinfer_fused_desc fd[4] = {{d->qkv_raw, L.in_qkv.w, L.in_qkv.s, nullptr, L.in_qkv.n},
                                   {d->zbuf, L.in_z.w, L.in_z.s, nullptr, L.in_z.n},
                                   {d->bbuf, L.in_b.w, L.in_b.s, nullptr, L.in_b.n},
                                   {d->abuf, L.in_a.w, L.in_a.s, nullptr, L.in_a.n}};
        CK(xinfer_linear_int4_fused_f16(s, d->normed, fd, 4, M, H, 128));
        ++d->linear_launches;
        account(d, L.in_qkv, M, 2, true);
        account(d, L.in_z, M, 2, false);
        account(d, L.in_b, M, 2, false);
        account(d, L.in_a, M, 2, false);
        NL(xb::conv1d_spec(s, d->qkv_conv, d->qkv_raw, L.conv_w, L.conv_state, L.conv_pend, n_commit, B, R, prev_rows, ch));
        NL(xb::gdn_spec(s, d->delta_out, d->qkv_conv, d->zbuf, d->bbuf, d->abuf, L.A_log, L.dt_bias, L.gdn_norm, L.S,
                        L.pend_k, L.pend_d, L.pend_g, n_commit, B, R, prev_rows, hv, hk));
        d->launches_per_step += 3;
        CK(lin(d, s, d->proj_out, d->delta_out, L.out_proj, M));
    }
    // x += mixer output, post-attention RMSNorm
    NL(xb::add_rmsnorm_rows(s, d->normed, d->x, d->proj_out, L.post_norm, M, H, c.rms_norm_eps));
    CK(xinfer_mlp_gate_up_swiglu_int4_f16(s, d->mlp, d->normed, L.gate.w, L.gate.s, L.up.w, L.up.s, M, L.gate.n, H, 128));
    ++d->linear_launches;
    account(d, L.gate, M, 2, true);
    d->linear_bytes += static_cast<double>(L.up.n) * (L.up.k / 2) + static_cast<double>(L.up.n) * (L.up.k / 128) * 2;
    d->launches_per_step += 2;
    CK(lin(d, s, d->proj_out, d->mlp, L.down, M));  // the caller adds proj_out into x
    return 0;
}

// final: x += last MLP output, final RMSNorm, LM head -> fp32 logits
int head_forward(Dec* d, cudaStream_t s, int M) {
    const auto& c = d->cfg;
    const int H = static_cast<int>(c.hidden_size);
    NL(xb::add_rmsnorm_rows(s, d->normed, d->x, d->proj_out, d->final_norm, M, H, c.rms_norm_eps));
    CK(xinfer_linear_int4_f16f32(s, d->logits, d->normed, d->lm_head.w, d->lm_head.s, nullptr, M, d->lm_head.n,
                                 d->lm_head.k, 128));
    ++d->linear_launches;
    account(d, d->lm_head, M, 4, true);
    d->launches_per_step += 2;
    return 0;
}

int draft_pass(Dec* d, cudaStream_t s, int i) {
    const auto& c = d->cfg;
    const int B = d->batch, H = static_cast<int>(c.hidden_size);
    const long long* tok = (i == 0) ? d->cur_tok : d->argmax_out;
    const __half* hprev = (i == 0) ? d->h_last : d->mtp_hidden;
    // cat = [rmsnorm(embed(tok)) ; rmsnorm(h_prev)]  ->  fc  ->  x
    NL(xb::embed_rows(s, d->x, d->embed, tok, B, H, c.vocab_size));
    NL(xb::rmsnorm_rows(s, d->cat, 2 * H, d->x, d->mtp_enorm, B, H, c.rms_norm_eps));
    NL(xb::rmsnorm_rows(s, d->cat + H, 2 * H, hprev, d->mtp_hnorm, B, H, c.rms_norm_eps));
    CK(lin(d, s, d->x, d->cat, d->mtp_fc, B));
    if (!d->linears_only) add_int_kernel<<<1, 64, 0, s>>>(d->ctx_draft, d->ctx, B, i);
    d->launches_per_step += 4;
    CK(layer_forward(d, s, d->mtp_layer, 1, d->ctx_draft, d->n_commit_zero, 0, true, nullptr));
    // keep the head's output hidden for the next draft pass: x + proj_out (pre final norm)
    NL(xb::add_rmsnorm_rows(s, d->normed, d->x, d->proj_out, d->final_norm, B, H, c.rms_norm_eps));
    if (!d->linears_only)
        cudaMemcpyAsync(d->mtp_hidden, d->x, static_cast<size_t>(B) * H * sizeof(__half), cudaMemcpyDeviceToDevice, s);
    CK(xinfer_linear_int4_f16f32(s, d->logits, d->normed, d->lm_head.w, d->lm_head.s, nullptr, B, d->lm_head.n,
                                 d->lm_head.k, 128));
    ++d->linear_launches;
    account(d, d->lm_head, B, 4, true);
    NL(xinfer_argmax_rows(s, d->logits, c.vocab_size, B, c.vocab_size, reinterpret_cast<int64_t*>(d->argmax_out)));
    NL(xb::copy_token_column(s, d->draft, d->argmax_out, B, d->k, i));
    d->launches_per_step += 6;
    return 0;
}

int target_pass(Dec* d, cudaStream_t s, int R, const long long* tokens) {
    const auto& c = d->cfg;
    const int M = d->batch * R, H = static_cast<int>(c.hidden_size);
    NL(xb::embed_rows(s, d->x, d->embed, tokens, M, H, c.vocab_size));
    ++d->launches_per_step;
    for (size_t l = 0; l < d->layers.size(); ++l)
        CK(layer_forward(d, s, d->layers[l], R, d->ctx, d->n_commit, d->prev_rows, l == 0, nullptr));
    CK(head_forward(d, s, M));
    if (!d->linears_only) d->prev_rows = R;
    return 0;
}

int enqueue_step(Dec* d, cudaStream_t s) {
    const auto& c = d->cfg;
    const int B = d->batch, k = d->k, R = k + 1;
    d->launches_per_step = 0;
    d->linear_launches = 0;
    d->linear_bytes = 0;
    xb::tc_plan_rewind();  // the step's linears come in the recorded order (if a plan was recorded at capture)
    for (int i = 0; i < k; ++i) CK(draft_pass(d, s, i));
    if (d->override_armed && !d->linears_only)
        cudaMemcpyAsync(d->draft, d->draft_override, static_cast<size_t>(B) * k * sizeof(long long), cudaMemcpyDeviceToDevice, s);
    NL(xb::build_verify_tokens(s, d->verify_tokens, d->cur_tok, d->draft, B, k));
    CK(target_pass(d, s, R, d->verify_tokens));
    NL(xinfer_speculative_accept_reject_batched(s, reinterpret_cast<const int64_t*>(d->draft), d->logits, c.vocab_size,
                                                c.vocab_size, nullptr, nullptr, 1.0f, B, k, R, k, d->records));
    // x still holds the pre-norm hidden rows of the verify pass (head_forward added the last MLP output)
    NL(xb::spec_commit(s, d->records, d->draft, B, k, R, d->ctx, d->n_commit, d->cur_tok, d->emitted, d->emitted_n,
                       d->h_last, d->x, static_cast<int>(c.hidden_size)));
    d->launches_per_step += 5;
    return 0;
}

}  // namespace

extern "C" {

int xinfer_spec_decoder_create(const xinfer_model_config* cfg, int batch, int k, int64_t max_seq, uint64_t seed,
                               xinfer_spec_decoder** out) {
    if (!cfg || !out || batch < 1 || k < 1 || k > 7 || max_seq < 8) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    const auto& c = *cfg;
    if (c.hidden_size % 128 || c.intermediate_size % 128 || c.num_key_value_heads < 1 ||
        c.num_attention_heads % c.num_key_value_heads || (c.num_attention_heads / c.num_key_value_heads) * (k + 1) > 32 ||
        c.linear_num_k_heads < 1 || c.linear_num_v_heads % c.linear_num_k_heads || batch * (k + 1) > 32 ||
        c.rope_dim > 256 || c.rope_dim % 2)
        return XINFER_ERR_INVALID_ARGUMENT;
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
    cudaGetDevice(&d->device);
    try {
        const int64_t H = c.hidden_size, V = c.vocab_size;
        const int M = batch * (k + 1);
        d->layers.resize(static_cast<size_t>(c.num_hidden_layers));
        const int interval = c.full_attention_interval > 0 ? c.full_attention_interval : 4;
        for (int64_t l = 0; l < c.num_hidden_layers; ++l) make_layer(d, d->layers[l], (l % interval) == interval - 1);
        make_layer(d, d->mtp_layer, true);
        d->mtp_fc = make_linear(d, H, 2 * H);
        d->lm_head = make_linear(d, V, H);
        d->mtp_enorm = make_floats(d, H, 1.0f, 0.02f);
        d->mtp_hnorm = make_floats(d, H, 1.0f, 0.02f);
        d->final_norm = make_floats(d, H, 1.0f, 0.02f);
        d->embed = dalloc<uint16_t>(d, static_cast<size_t>(V) * H);
        init_bf16_kernel<<<blocks_for(static_cast<size_t>(V) * H, 256), 256>>>(d->embed, static_cast<size_t>(V) * H,
                                                                                next_seed(d), 1.0f);
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
        const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads, ch = 2 * hk * 128 + hv * 128;
        d->x = dalloc<__half>(d, static_cast<size_t>(M) * H, true);
        d->normed = dalloc<__half>(d, static_cast<size_t>(M) * H, true);
        d->proj_out = dalloc<__half>(d, static_cast<size_t>(M) * H, true);
        d->mlp = dalloc<__half>(d, static_cast<size_t>(M) * c.intermediate_size, true);
        d->q_gate = dalloc<__half>(d, static_cast<size_t>(M) * c.num_attention_heads * 512, true);
        d->qbuf = dalloc<__half>(d, static_cast<size_t>(M) * c.num_attention_heads * 256, true);
        d->kbuf = dalloc<__half>(d, static_cast<size_t>(M) * c.num_key_value_heads * 256, true);
        d->vbuf = dalloc<__half>(d, static_cast<size_t>(M) * c.num_key_value_heads * 256, true);
        d->attn_out = dalloc<__half>(d, static_cast<size_t>(M) * c.num_attention_heads * 256, true);
        d->qkv_raw = dalloc<__half>(d, static_cast<size_t>(M) * ch, true);
        d->qkv_conv = dalloc<__half>(d, static_cast<size_t>(M) * ch, true);
        d->zbuf = dalloc<__half>(d, static_cast<size_t>(M) * hv * 128, true);
        d->bbuf = dalloc<__half>(d, static_cast<size_t>(M) * hv, true);
        d->abuf = dalloc<__half>(d, static_cast<size_t>(M) * hv, true);
        d->delta_out = dalloc<__half>(d, static_cast<size_t>(M) * hv * 128, true);
        d->cat = dalloc<__half>(d, static_cast<size_t>(batch) * 2 * H, true);
        d->logits = dalloc<float>(d, static_cast<size_t>(M) * V, true);
        {
            // KV splits: with one attention CTA per SM, two waves of CTAs over (split, kv head, sequence)
            int sms = 148;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->device);
            const int units = batch * static_cast<int>(c.num_key_value_heads);
            int splits = (2 * sms) / (units > 0 ? units : 1);
            d->attn_splits = splits < 1 ? 1 : (splits > 16 ? 16 : splits);
        }
        d->attn_scratch = dalloc<float>(
            d, xb::attn_scratch_bytes(batch, static_cast<int>(c.num_key_value_heads), d->attn_splits) / sizeof(float), true);
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

void xinfer_spec_decoder_destroy(xinfer_spec_decoder* d) {
    if (!d) return;
    xb::tc_plan_clear();  // the recorded plan points into this decoder's weights
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    for (void* p : d->allocs) cudaFree(p);
    if (d->h_emitted) cudaFreeHost(d->h_emitted);
    if (d->h_emitted_n) cudaFreeHost(d->h_emitted_n);
    delete d;
}

int xinfer_spec_decoder_reset(xinfer_spec_decoder* d, int64_t context_len, uint64_t seed) {
    if (!d || context_len < 0 || context_len + 2 * (d->k + 1) > d->max_seq) return XINFER_ERR_INVALID_ARGUMENT;
    const auto& c = d->cfg;
    const int B = d->batch;
    uint64_t sd = seed * 0x9E3779B97F4A7C15ULL + 777;
    auto nxt = [&]() { return sd = sd * 6364136223846793005ULL + 1442695040888963407ULL; };
    auto fill_layer = [&](Layer& L) {
        if (L.full) {
            const size_t kv = static_cast<size_t>(B) * d->max_seq * c.num_key_value_heads * 256;
            init_half_kernel<<<blocks_for(kv, 256), 256>>>(L.k_cache, kv, nxt(), 1, 0.f, 1.0f);
            init_half_kernel<<<blocks_for(kv, 256), 256>>>(L.v_cache, kv, nxt(), 1, 0.f, 1.0f);
        } else {
            const int64_t hv = c.linear_num_v_heads, hk = c.linear_num_k_heads, ch = 2 * hk * 128 + hv * 128;
            const size_t sn = static_cast<size_t>(B) * hv * 128 * 128;
            const float sig = context_len > 0 ? 0.05f : 0.0f;  // an empty context starts from zero state
            init_float_kernel<<<blocks_for(sn, 256), 256>>>(L.S, sn, nxt(), 0.f, sig);
            init_float_kernel<<<blocks_for(static_cast<size_t>(B) * 3 * ch, 256), 256>>>(
                L.conv_state, static_cast<size_t>(B) * 3 * ch, nxt(), 0.f, context_len > 0 ? 1.0f : 0.0f);
            cudaMemset(L.pend_k, 0, static_cast<size_t>(B) * hv * 8 * 128 * sizeof(float));
            cudaMemset(L.pend_d, 0, static_cast<size_t>(B) * hv * 8 * 128 * sizeof(float));
            cudaMemset(L.pend_g, 0, static_cast<size_t>(B) * hv * 8 * sizeof(float));
            cudaMemset(L.conv_pend, 0, static_cast<size_t>(B) * 8 * ch * sizeof(float));
        }
    };
    for (auto& L : d->layers) fill_layer(L);
    fill_layer(d->mtp_layer);
    xb::fill_int(nullptr, d->ctx, B, static_cast<int>(context_len));
    xb::fill_int(nullptr, d->n_commit, B, 0);
    xb::fill_int(nullptr, d->n_commit_zero, B, 0);
    init_tokens_kernel<<<1, 64>>>(d->cur_tok, B, nxt(), c.vocab_size);
    init_half_kernel<<<blocks_for(static_cast<size_t>(B) * c.hidden_size, 256), 256>>>(
        d->h_last, static_cast<size_t>(B) * c.hidden_size, nxt(), 1, 0.f, 1.0f);
    d->prev_rows = 0;
    return cudaDeviceSynchronize() == cudaSuccess ? XINFER_OK : XINFER_ERR_CUDA;
}

int xinfer_spec_decoder_step(xinfer_spec_decoder* d, xinfer_stream_t stream) {
    if (!d) return XINFER_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d->graph_exec) {
        return cudaGraphLaunch(d->graph_exec, s) == cudaSuccess ? XINFER_OK : XINFER_ERR_CUDA;
    }
    const int prev = d->prev_rows;
    (void)prev;
    return enqueue_step(d, s);
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
        xb::tc_plan_record_begin();
        int rc = enqueue_step(d, s);
        xb::tc_plan_record_end();
        if (rc < 0) return rc;
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
    cudaMemcpyAsync(d->h_emitted, d->emitted, static_cast<size_t>(M) * sizeof(long long), cudaMemcpyDeviceToHost, s);
    cudaMemcpyAsync(d->h_emitted_n, d->emitted_n, static_cast<size_t>(d->batch) * sizeof(int), cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) return XINFER_ERR_CUDA;
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
        default: return -1;
    }
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
        if (n == "logits") { nb = M * c.vocab_size * 4; return d->logits; }
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
        const int64_t kv = B * d->max_seq * c.num_key_value_heads * 256 * 2;
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
        if (n == "S") { nb = B * hv * 128 * 128 * 4; return L->S; }
        if (n == "conv_state") { nb = B * 3 * ch * 4; return L->conv_state; }
    }
    return nullptr;
}

const char* xinfer_spec_decoder_error(const xinfer_spec_decoder* d) { return d ? d->error.c_str() : ""; }

}  // extern "C"
