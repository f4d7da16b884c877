// CPU oracle for the per-layer glue of the decode / verify step.  TEST INFRASTRUCTURE ONLY (see the
// header of xinfer_oracle.cpp).  Literal single-sequence restatements of the reference's kernels, with
// `_Float16` for sycl::half and every fp16 rounding point kept.
//
// Parity status: pinned.  Each function restates one reference kernel; the reference's own tests for those
// kernels (tests/test_ops_oracle.cpp:50-285, 797-906; tests/test_decode_graph.cpp:208-284; tests/test_kv_cache.cpp:
// 286-314) hold no stored vectors, they recompute inline fp64 expectations from seeded inputs, so the pin is the
// same recipe: tests/test_mixer_oracle_pins.py regenerates those inputs (std::mt19937 streams, checked by CRC-64
// against tests/golden/mixer_streams.json), recomputes the expectations with the tests' own formulas
// (tests/ref_recipes.py) and holds these functions to the reference's tolerances.  For the gated delta rule the
// reference tests argument validation only (tests/test_decode_graph.cpp:37-49); its arithmetic here is a
// line-by-line restatement of src/targets/qwen3_8/linear_attn.cpp:144-343.  The speculative batching and the lazy state commit around these ops are
// additions of this repository and are checked against these functions applied sequence by sequence, token by token.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

typedef _Float16 half_t;

extern "C" {

// embed_tokens_lookup, src/targets/qwen3_8/forward.cpp:17-64: bf16 row -> float = bits << 16 -> fp16;
// token < 0 or >= vocab -> zeros.
void oracle_embed(uint16_t* out_f16, const uint16_t* table_bf16, const int64_t* tokens, int64_t n, int64_t hidden,
                  int64_t vocab) {
    half_t* out = reinterpret_cast<half_t*>(out_f16);
    for (int64_t t = 0; t < n; ++t) {
        int64_t tok = tokens[t];
        for (int64_t d = 0; d < hidden; ++d) {
            float v = 0.0f;
            if (!(tok < 0 || (vocab > 0 && tok >= vocab))) {
                uint32_t bits = static_cast<uint32_t>(table_bf16[tok * hidden + d]) << 16;
                std::memcpy(&v, &bits, 4);
            }
            out[t * hidden + d] = static_cast<half_t>(v);
        }
    }
}

// rmsnorm (fp16), src/ops/rmsnorm.cpp:15-82: y = half(x * (1/sqrt(mean(x^2) + eps)) * w), fp32 inside.
void oracle_rmsnorm_f16(uint16_t* out_f16, const uint16_t* in_f16, const float* w, int64_t tokens, int64_t hidden,
                        float eps) {
    half_t* out = reinterpret_cast<half_t*>(out_f16);
    const half_t* in = reinterpret_cast<const half_t*>(in_f16);
    for (int64_t t = 0; t < tokens; ++t) {
        double ss = 0.0;  // the reference sums in fp32 across 256 lanes; fp64 here is the tighter oracle
        for (int64_t i = 0; i < hidden; ++i) {
            float v = static_cast<float>(in[t * hidden + i]);
            ss += static_cast<double>(v) * v;
        }
        float mean_sq = static_cast<float>(ss) / static_cast<float>(hidden);
        float r = 1.0f / std::sqrt(mean_sq + eps);
        for (int64_t i = 0; i < hidden; ++i) {
            float v = static_cast<float>(in[t * hidden + i]);
            out[t * hidden + i] = static_cast<half_t>(v * r * w[i]);
        }
    }
}

// add_inplace (fp16), src/ops/elementwise.cpp:213-236.
void oracle_add_inplace_f16(uint16_t* a_f16, const uint16_t* b_f16, int64_t n) {
    half_t* a = reinterpret_cast<half_t*>(a_f16);
    const half_t* b = reinterpret_cast<const half_t*>(b_f16);
    for (int64_t i = 0; i < n; ++i) a[i] = static_cast<half_t>(static_cast<float>(a[i]) + static_cast<float>(b[i]));
}

// rope (fp16, in place), src/ops/rope.cpp:12-62: pairs (p, p + rot/2) of the first `rotary_dim` dims.
static void rope_heads(half_t* ptr, int64_t tokens, int64_t heads, int64_t head_dim, const int64_t* positions,
                       float theta, int64_t rotary_dim) {
    if (!ptr || heads <= 0) return;
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    int64_t half_rot = rotary_dim / 2;
    float log_theta = std::log(theta);
    float inv_rot = 1.0f / static_cast<float>(rotary_dim);
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t h = 0; h < heads; ++h)
            for (int64_t p = 0; p < half_rot; ++p) {
                float freq = std::exp(-static_cast<float>(2 * p) * inv_rot * log_theta);
                float angle = static_cast<float>(positions[t]) * freq;
                float c = std::cos(angle), s = std::sin(angle);
                half_t* base = ptr + (t * heads + h) * head_dim;
                float v0 = static_cast<float>(base[p]);
                float v1 = static_cast<float>(base[p + half_rot]);
                base[p] = static_cast<half_t>(v0 * c - v1 * s);
                base[p + half_rot] = static_cast<half_t>(v1 * c + v0 * s);
            }
}
void oracle_rope_f16(uint16_t* q, uint16_t* k, int64_t tokens, int64_t hq, int64_t hkv, int64_t head_dim,
                     const int64_t* positions, float theta, int64_t rotary_dim) {
    rope_heads(reinterpret_cast<half_t*>(q), tokens, hq, head_dim, positions, theta, rotary_dim);
    rope_heads(reinterpret_cast<half_t*>(k), tokens, hkv, head_dim, positions, theta, rotary_dim);
}

// attention_write_kv_cache, src/ops/attention.cpp:84-116: caches are [pos][kv_head][head_dim] fp16.
void oracle_kv_write(uint16_t* k_cache, uint16_t* v_cache, const uint16_t* k_in, const uint16_t* v_in,
                     int64_t start_pos, int64_t tokens, int64_t hkv, int64_t head_dim, int64_t max_seq) {
    if (tokens <= 0) return;
    if (max_seq > 0) {
        if (start_pos >= max_seq || start_pos < 0) return;
        if (start_pos + tokens > max_seq) tokens = max_seq - start_pos;
    }
    int64_t stride = hkv * head_dim;
    std::memcpy(k_cache + start_pos * stride, k_in, static_cast<size_t>(tokens * stride) * 2);
    std::memcpy(v_cache + start_pos * stride, v_in, static_cast<size_t>(tokens * stride) * 2);
}

// sdpa_causal_cached, src/ops/attention.cpp:151-243: query token i of head h sees keys 0 .. start_pos + i,
// kv head h / (hq / hkv), scale 1/sqrt(head_dim) when the passed scale <= 0, sequential online softmax
// in fp32, fp16 output.
void oracle_sdpa_cached(uint16_t* out_f16, const uint16_t* q_f16, const uint16_t* k_cache_f16,
                        const uint16_t* v_cache_f16, int64_t start_pos, int64_t nq, int64_t hq, int64_t hkv,
                        int64_t head_dim, float scale, int64_t max_seq) {
    half_t* out = reinterpret_cast<half_t*>(out_f16);
    const half_t* Q = reinterpret_cast<const half_t*>(q_f16);
    const half_t* kc = reinterpret_cast<const half_t*>(k_cache_f16);
    const half_t* vc = reinterpret_cast<const half_t*>(v_cache_f16);
    if (scale <= 0.0f) scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
    int64_t ratio = hq / hkv;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < nq; ++i)
        for (int64_t h = 0; h < hq; ++h) {
            int64_t kvh = h / ratio;
            const half_t* qv = Q + (i * hq + h) * head_dim;
            half_t* ov = out + (i * hq + h) * head_dim;
            int64_t total_keys = start_pos + i + 1;
            if (max_seq > 0 && total_keys > max_seq) total_keys = max_seq;
            if (total_keys <= 0) continue;
            float max_score = -std::numeric_limits<float>::infinity();
            float sum_exp = 0.0f;
            std::vector<float> acc(static_cast<size_t>(head_dim), 0.0f);
            for (int64_t j = 0; j < total_keys; ++j) {
                const half_t* kp = kc + (j * hkv + kvh) * head_dim;
                const half_t* vp = vc + (j * hkv + kvh) * head_dim;
                float dot = 0.0f;
                for (int64_t d = 0; d < head_dim; ++d) dot += static_cast<float>(qv[d]) * static_cast<float>(kp[d]);
                float score = dot * scale;
                float new_max = std::max(max_score, score);
                float exp_old = (max_score == -std::numeric_limits<float>::infinity()) ? 0.0f : std::exp(max_score - new_max);
                float exp_new = std::exp(score - new_max);
                sum_exp = sum_exp * exp_old + exp_new;
                for (int64_t d = 0; d < head_dim; ++d) acc[d] = acc[d] * exp_old + exp_new * static_cast<float>(vp[d]);
                max_score = new_max;
            }
            float inv_sum = 1.0f / (sum_exp > 0.0f ? sum_exp : 1.0f);
            for (int64_t d = 0; d < head_dim; ++d) ov[d] = static_cast<half_t>(acc[d] * inv_sum);
        }
}

// causal_conv1d_silu (fp16 in/out, fp32 state [3][channels]), src/targets/qwen3_8/linear_attn.cpp:37-122.
void oracle_conv1d_silu(uint16_t* out_f16, const uint16_t* in_f16, const float* conv_w, int64_t seq_len,
                        float* conv_state, int64_t channels) {
    half_t* out = reinterpret_cast<half_t*>(out_f16);
    const half_t* in = reinterpret_cast<const half_t*>(in_f16);
    if (seq_len <= 0) return;
    for (int64_t t = 0; t < seq_len; ++t)
        for (int64_t c = 0; c < channels; ++c) {
            float sum = 0.0f;
            for (int k = 0; k < 4; ++k) {
                int64_t src_t = t - (3 - k);
                float val = 0.0f;
                if (src_t >= 0) val = static_cast<float>(in[src_t * channels + c]);
                else if (conv_state) {
                    int64_t si = 3 + src_t;
                    if (si >= 0 && si < 3) val = conv_state[si * channels + c];
                }
                sum += conv_w[c * 4 + k] * val;
            }
            out[t * channels + c] = static_cast<half_t>(sum / (1.0f + std::exp(-sum)));
        }
    if (conv_state) {
        for (int64_t c = 0; c < channels; ++c) {
            float h[3] = {conv_state[c], conv_state[channels + c], conv_state[2 * channels + c]};
            // window of the last three inputs after seq_len more tokens
            float seq3[3];
            for (int r = 0; r < 3; ++r) {
                int64_t src = seq_len - 3 + r;  // index into the new inputs, negative -> old state
                seq3[r] = src >= 0 ? static_cast<float>(in[src * channels + c]) : h[3 + src];
            }
            conv_state[c] = seq3[0];
            conv_state[channels + c] = seq3[1];
            conv_state[2 * channels + c] = seq3[2];
        }
    }
}

// recurrent_gated_delta_net (fp16 in/out, fp32 state [hv][128][128]),
// src/targets/qwen3_8/linear_attn.cpp:144-343; head dims are 128 as in the reference.
void oracle_gdn(uint16_t* out_f16, const uint16_t* qkv_f16, const uint16_t* z_f16, const uint16_t* b_f16,
                const uint16_t* a_f16, const float* A_log, const float* dt_bias, const float* norm_w, float* state,
                int64_t seq_len, int zero_state, int64_t hv, int64_t hk) {
    half_t* out = reinterpret_cast<half_t*>(out_f16);
    const half_t* qkv = reinterpret_cast<const half_t*>(qkv_f16);
    const half_t* z = reinterpret_cast<const half_t*>(z_f16);
    const half_t* bb = reinterpret_cast<const half_t*>(b_f16);
    const half_t* aa = reinterpret_cast<const half_t*>(a_f16);
    const int64_t D = 128;
    const int64_t channels = 2 * hk * D + hv * D;
    const int64_t value_dim = hv * D;
#pragma omp parallel for schedule(static)
    for (int64_t h = 0; h < hv; ++h) {
        int64_t h_k = h / (hv / hk);
        float* S = state + h * D * D;
        if (zero_state) std::fill(S, S + D * D, 0.0f);
        float exp_a_log = std::exp(A_log[h]);
        float qn[128], kn[128], attn[128];
        for (int64_t t = 0; t < seq_len; ++t) {
            const half_t* cur = qkv + t * channels;
            const half_t* q_in = cur + h_k * D;
            const half_t* k_in = cur + hk * D + h_k * D;
            const half_t* v_in = cur + 2 * hk * D + h * D;
            float q_sq = 0.0f, k_sq = 0.0f;
            for (int64_t j = 0; j < D; ++j) {
                float rq = static_cast<float>(q_in[j]), rk = static_cast<float>(k_in[j]);
                q_sq += rq * rq;
                k_sq += rk * rk;
            }
            float inv_q = 1.0f / std::sqrt(q_sq + 1e-6f);
            float inv_k = 1.0f / std::sqrt(k_sq + 1e-6f);
            for (int64_t j = 0; j < D; ++j) {
                qn[j] = (static_cast<float>(q_in[j]) * inv_q) * 0.08838834764f;
                kn[j] = static_cast<float>(k_in[j]) * inv_k;
            }
            float b_val = static_cast<float>(bb[t * hv + h]);
            float beta = 1.0f / (1.0f + std::exp(-b_val));
            float a_val = static_cast<float>(aa[t * hv + h]) + dt_bias[h];
            float softplus = (a_val > 20.0f) ? a_val : std::log(1.0f + std::exp(a_val));
            float g = -exp_a_log * softplus;
            float exp_g = std::exp(g);
            float attn_sq = 0.0f;
            for (int64_t j = 0; j < D; ++j) {
                float kv_mem = 0.0f;
                for (int64_t i = 0; i < D; ++i) {
                    float s_val = S[i * D + j] * exp_g;
                    S[i * D + j] = s_val;
                    kv_mem += s_val * kn[i];
                }
                float delta = (static_cast<float>(v_in[j]) - kv_mem) * beta;
                float a_j = 0.0f;
                for (int64_t i = 0; i < D; ++i) {
                    float ns = S[i * D + j] + kn[i] * delta;
                    S[i * D + j] = ns;
                    a_j += ns * qn[i];
                }
                attn[j] = a_j;
                attn_sq += a_j * a_j;
            }
            float inv_std = 1.0f / std::sqrt(attn_sq / 128.0f + 1e-6f);
            for (int64_t j = 0; j < D; ++j) {
                float normed = attn[j] * inv_std * norm_w[j];
                float zv = static_cast<float>(z[t * value_dim + h * D + j]);
                float silu_z = zv / (1.0f + std::exp(-zv));
                out[t * value_dim + h * D + j] = static_cast<half_t>(normed * silu_z);
            }
        }
    }
}

// q / gate de-interleave and sigmoid output gate, src/targets/qwen3_8/forward.cpp:145-151, 217-226.
void oracle_split_q(uint16_t* q_out, const uint16_t* q_gate, int64_t tokens, int64_t hq, int64_t head_dim) {
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t h = 0; h < hq; ++h)
            std::memcpy(q_out + (t * hq + h) * head_dim, q_gate + (t * hq + h) * 2 * head_dim,
                        static_cast<size_t>(head_dim) * 2);
}
void oracle_gate_output(uint16_t* attn_f16, const uint16_t* q_gate_f16, int64_t tokens, int64_t hq, int64_t head_dim) {
    half_t* attn = reinterpret_cast<half_t*>(attn_f16);
    const half_t* qg = reinterpret_cast<const half_t*>(q_gate_f16);
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t h = 0; h < hq; ++h)
            for (int64_t d = 0; d < head_dim; ++d) {
                float gate = static_cast<float>(qg[(t * hq + h) * 2 * head_dim + head_dim + d]);
                float sig = 1.0f / (1.0f + std::exp(-gate));
                float cur = static_cast<float>(attn[(t * hq + h) * head_dim + d]);
                attn[(t * hq + h) * head_dim + d] = static_cast<half_t>(cur * sig);
            }
}

}  // extern "C"
