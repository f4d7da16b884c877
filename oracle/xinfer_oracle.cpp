// CPU oracle for the speculative-decode hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++ (g++ >= 13, `_Float16` stands in for sycl::half),
// the reference's own numerical oracles for the path.  It is never linked into or
// called by the product library; only the test-suite, the smoke check and the
// benchmark's cpu_baseline / reference arm load it.
//
// Parity status: PINNED for int4 unpacking, linear_int4 (all variants), fused
// projections, gate/up/SwiGLU, argmax and speculative_accept_reject -- each is
// checked against the reference tests' own deterministic input recipes and expected
// values (see tests/golden).  The reference ships no stored output files: its tests
// recompute the expectation inline each run, and so does this oracle.
// UNPINNED: the MTP draft head as a unit and the Philox/temperature front end, which
// do not exist in the reference (its tests reject temperature != 0).
//
// Every function cites the reference file:line it follows.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

typedef _Float16 half_t;

extern "C" {

// ---------------------------------------------------------------------------------
// int4 unpack.  Follows tools/convert/qwen3_8_27b/convert.py:129-148
// (dequantize_int4_symmetric) and src/ops/linear.cpp:708-714: low nibble = even k,
// high nibble = odd k, two's-complement 4 bit.
// ---------------------------------------------------------------------------------
void oracle_unpack_int4(const uint8_t* packed, int64_t n_bytes, int8_t* out) {
    for (int64_t i = 0; i < n_bytes; ++i) {
        uint8_t b = packed[i];
        int8_t lo = static_cast<int8_t>(b & 0x0F);
        if (lo >= 8) lo = static_cast<int8_t>(lo - 16);
        int8_t hi = static_cast<int8_t>((b >> 4) & 0x0F);
        if (hi >= 8) hi = static_cast<int8_t>(hi - 16);
        out[2 * i] = lo;
        out[2 * i + 1] = hi;
    }
}

// Same unpack through the production kernel's arithmetic-shift form,
// src/ops/linear.cpp:100-110: a little-endian u32 holds 8 consecutive k, nibble i <-> k+i,
// value = (int32(word) << (28 - 4 i)) >> 28.
void oracle_unpack_int4_shift(const uint8_t* packed, int64_t n_bytes, int8_t* out) {
    for (int64_t w = 0; w + 4 <= n_bytes; w += 4) {
        uint32_t p;
        std::memcpy(&p, packed + w, 4);
        int32_t sp = static_cast<int32_t>(p);
        for (int i = 0; i < 8; ++i) {
            int32_t v = static_cast<int32_t>(static_cast<uint32_t>(sp) << (28 - 4 * i)) >> 28;
            out[2 * w + i] = static_cast<int8_t>(v);
        }
    }
}

// Quantiser, tools/convert/qwen3_8_27b/convert.py:93-121: scale = max|x|/7 clamped to
// >= 1e-8, q = clamp(round_half_even(x/scale), -8, 7), packed low = even, high = odd.
void oracle_quantize_int4(const float* w, int64_t rows, int64_t K, int group_size,
                          uint8_t* packed, uint16_t* scales_f16_bits) {
    int64_t G = K / group_size;
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t g = 0; g < G; ++g) {
            const float* x = w + r * K + g * group_size;
            float mx = 0.f;
            for (int i = 0; i < group_size; ++i) mx = std::max(mx, std::fabs(x[i]));
            float scale = std::max(mx / 7.0f, 1e-8f);
            for (int i = 0; i < group_size; i += 2) {
                int q0 = static_cast<int>(std::nearbyint(x[i] / scale));
                int q1 = static_cast<int>(std::nearbyint(x[i + 1] / scale));
                q0 = std::min(7, std::max(-8, q0));
                q1 = std::min(7, std::max(-8, q1));
                packed[r * (K / 2) + (g * group_size + i) / 2] =
                    static_cast<uint8_t>((q0 & 0x0F) | ((q1 & 0x0F) << 4));
            }
            half_t hs = static_cast<half_t>(scale);
            std::memcpy(&scales_f16_bits[r * G + g], &hs, 2);
        }
    }
}

static inline void nibbles(uint8_t b, int& lo, int& hi) {
    lo = b & 0x0F; if (lo >= 8) lo -= 16;
    hi = (b >> 4) & 0x0F; if (hi >= 8) hi -= 16;
}

// ---------------------------------------------------------------------------------
// linear_int4, fp64 accumulate.  Follows the inline oracle of
// tests/test_ops_oracle.cpp:318-348 (also :410-439, :529-557, :730-754):
//   acc(double) += x[k] * (double(q) * double(scale));  Y = float(acc)  (+ bias).
// X is fp32 (an fp16 activation is widened by the caller, as the test does at :719).
// ---------------------------------------------------------------------------------
void oracle_linear_int4_f64(float* Y, const float* X, const uint8_t* W, const uint16_t* scales_bits,
                            const float* bias, int64_t M, int64_t N, int64_t K, int group_size) {
    if (M <= 0 || N <= 0 || K <= 0) return;
    const half_t* scales = reinterpret_cast<const half_t*>(scales_bits);
    int64_t G = K / group_size;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* rw = W + n * (K / 2);
        const half_t* rs = scales + n * G;
        for (int64_t m = 0; m < M; ++m) {
            const float* rx = X + m * K;
            double acc = 0.0;
            for (int64_t g = 0; g < G; ++g) {
                float scale = static_cast<float>(rs[g]);
                int64_t base_k = g * group_size;
                for (int64_t b = 0; b < group_size / 2; ++b) {
                    int lo, hi;
                    nibbles(rw[base_k / 2 + b], lo, hi);
                    acc += static_cast<double>(rx[base_k + 2 * b]) *
                           (static_cast<double>(lo) * static_cast<double>(scale));
                    acc += static_cast<double>(rx[base_k + 2 * b + 1]) *
                           (static_cast<double>(hi) * static_cast<double>(scale));
                }
            }
            float y = static_cast<float>(acc);
            if (bias) y += bias[n];
            Y[m * N + n] = y;
        }
    }
}

// ---------------------------------------------------------------------------------
// linear_int4_naive, the reference's "FP32 dequant oracle", src/ops/linear.cpp:681-730:
//   acc(float) += x[k] * (float(q) * scale), k ascending, bias added last.
// ---------------------------------------------------------------------------------
void oracle_linear_int4_naive_f32(float* Y, const float* X, const uint8_t* W, const uint16_t* scales_bits,
                                  const float* bias, int64_t M, int64_t N, int64_t K, int group_size) {
    if (M <= 0 || N <= 0 || K <= 0) return;
    const half_t* scales = reinterpret_cast<const half_t*>(scales_bits);
    int64_t G = K / group_size;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* rw = W + n * (K / 2);
        const half_t* rs = scales + n * G;
        for (int64_t m = 0; m < M; ++m) {
            const float* rx = X + m * K;
            float acc = 0.0f;
            for (int64_t g = 0; g < G; ++g) {
                float scale = static_cast<float>(rs[g]);
                int64_t base_k = g * group_size;
                for (int64_t b = 0; b < group_size / 2; ++b) {
                    int lo, hi;
                    nibbles(rw[base_k / 2 + b], lo, hi);
                    acc += rx[base_k + 2 * b] * (static_cast<float>(lo) * scale);
                    acc += rx[base_k + 2 * b + 1] * (static_cast<float>(hi) * scale);
                }
            }
            if (bias) acc += bias[n];
            Y[m * N + n] = acc;
        }
    }
}

// Production association, src/ops/linear.cpp:239-298: per 128-k group an fp32 dot of
// x*q (exact small integers), then acc += dot * scale; bias last.  (The reference
// splits each group over 16 lanes and tree-sums them; this restatement sums a group in
// k order, which is the same association up to the lane order of an fp32 sum.)
void oracle_linear_int4_grouped_f32(float* Y, const float* X, const uint8_t* W, const uint16_t* scales_bits,
                                    const float* bias, int64_t M, int64_t N, int64_t K, int group_size) {
    if (M <= 0 || N <= 0 || K <= 0) return;
    const half_t* scales = reinterpret_cast<const half_t*>(scales_bits);
    int64_t G = K / group_size;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* rw = W + n * (K / 2);
        const half_t* rs = scales + n * G;
        for (int64_t m = 0; m < M; ++m) {
            const float* rx = X + m * K;
            float acc = 0.0f;
            for (int64_t g = 0; g < G; ++g) {
                float scale = static_cast<float>(rs[g]);
                int64_t base_k = g * group_size;
                float dot = 0.0f;
                for (int64_t b = 0; b < group_size / 2; ++b) {
                    int lo, hi;
                    nibbles(rw[base_k / 2 + b], lo, hi);
                    dot += rx[base_k + 2 * b] * static_cast<float>(lo);
                    dot += rx[base_k + 2 * b + 1] * static_cast<float>(hi);
                }
                acc += dot * scale;
            }
            if (bias) acc += bias[n];
            Y[m * N + n] = acc;
        }
    }
}

// ---------------------------------------------------------------------------------
// Fused gate/up/SwiGLU.  Follows tests/test_ops_oracle.cpp:625-670: fp64 accumulate of
// gate and up, each narrowed to float, silu(g) = g / (1 + exp(-g)) in fp32, y = silu*u.
// Kernel contract: src/ops/linear.cpp:594-597.
// ---------------------------------------------------------------------------------
void oracle_mlp_gate_up_swiglu_f64(float* Y, const float* X, const uint8_t* Wg, const uint16_t* sg_bits,
                                   const uint8_t* Wu, const uint16_t* su_bits,
                                   int64_t M, int64_t N, int64_t K, int group_size) {
    if (M <= 0 || N <= 0 || K <= 0) return;
    std::vector<float> g(static_cast<size_t>(M * N)), u(static_cast<size_t>(M * N));
    oracle_linear_int4_f64(g.data(), X, Wg, sg_bits, nullptr, M, N, K, group_size);
    oracle_linear_int4_f64(u.data(), X, Wu, su_bits, nullptr, M, N, K, group_size);
    for (int64_t i = 0; i < M * N; ++i) {
        float gv = g[i];
        float silu = gv / (1.0f + std::exp(-gv));
        Y[i] = silu * u[i];
    }
}

// fp16 round-trip helpers so numpy callers and the oracle agree on RNE narrowing.
void oracle_f32_to_f16(const float* in, uint16_t* out_bits, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        half_t h = static_cast<half_t>(in[i]);
        std::memcpy(&out_bits[i], &h, 2);
    }
}
void oracle_f16_to_f32(const uint16_t* in_bits, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        half_t h;
        std::memcpy(&h, &in_bits[i], 2);
        out[i] = static_cast<float>(h);
    }
}

// ---------------------------------------------------------------------------------
// argmax.  Follows src/ops/sampling.cpp:12-92: null/empty -> 0, vocab==1 -> 0, per-256
// block maxima then a scan over blocks, both with strict '>' so the lowest index of a
// tie wins and NaN never wins (tests/test_ops_oracle.cpp:925-934 is the same scan).
// ---------------------------------------------------------------------------------
int64_t oracle_argmax(const float* logits, int64_t vocab) {
    if (vocab <= 0 || !logits) return 0;
    if (vocab == 1) return 0;
    float best_val = -std::numeric_limits<float>::infinity();
    int64_t best_idx = -1;
    const int64_t WG = 256;
    int64_t blocks = (vocab + WG - 1) / WG;
    for (int64_t b = 0; b < blocks; ++b) {
        // stage 1: block maximum (tree in the reference; strict '>' keeps the lowest index)
        float bv = -std::numeric_limits<float>::infinity();
        int64_t bi = -1;
        int64_t end = std::min(vocab, (b + 1) * WG);
        for (int64_t i = b * WG; i < end; ++i) {
            if (bi < 0) { bv = logits[i]; bi = i; continue; }
            if (logits[i] > bv) { bv = logits[i]; bi = i; }
        }
        // stage 2: host scan over partials, seeded with block 0
        if (b == 0) { best_val = bv; best_idx = bi; }
        else if (bv > best_val) { best_val = bv; best_idx = bi; }
    }
    return best_idx;
}

// ---------------------------------------------------------------------------------
// softmax probability of one token, as speculative_accept_reject evaluates it on the
// host: src/ops/sampling.cpp:139-154 (fp32, sequential, std::exp; 0 if the token is out
// of range or the sum is not positive).
// ---------------------------------------------------------------------------------
float oracle_token_prob_f32(const float* logits, int64_t vocab, int64_t tok) {
    float max_val = -std::numeric_limits<float>::infinity();
    for (int64_t v = 0; v < vocab; ++v) if (logits[v] > max_val) max_val = logits[v];
    float sum_exp = 0.0f;
    for (int64_t v = 0; v < vocab; ++v) sum_exp += std::exp(logits[v] - max_val);
    float p = 0.0f;
    if (tok >= 0 && tok < vocab && sum_exp > 0.0f) p = std::exp(logits[tok] - max_val) / sum_exp;
    return p;
}

// fp64 variant of the same quantity, used only to classify near-ties.
double oracle_token_prob_f64(const float* logits, int64_t vocab, int64_t tok) {
    double mx = -std::numeric_limits<double>::infinity();
    for (int64_t v = 0; v < vocab; ++v) if (logits[v] > mx) mx = logits[v];
    double s = 0.0;
    for (int64_t v = 0; v < vocab; ++v) s += std::exp(static_cast<double>(logits[v]) - mx);
    if (!(tok >= 0 && tok < vocab) || !(s > 0.0)) return 0.0;
    return std::exp(static_cast<double>(logits[tok]) - mx) / s;
}

// POD form of SpeculativeAcceptanceResult (src/ops/sampling.h:27-36).
struct OracleAcceptResult {
    int64_t accepted_tokens[64];
    int64_t bonus_or_resampled_token;
    int64_t rejected_token;
    int64_t num_accepted;
    int64_t num_rejected;
    int64_t num_resampled;
    int64_t num_remaining;
    int32_t has_rejected_token;
    int32_t contract_violated;  // the reference throws std::logic_error here
};

// ---------------------------------------------------------------------------------
// speculative_accept_reject, literal restatement of src/ops/sampling.cpp:94-199.
// `inv_temperature` is an addition in front of the reference contract: logits are
// multiplied by it before the reference rule is applied (1.0 reproduces the reference
// exactly; argmax is unchanged by a positive factor).
// ---------------------------------------------------------------------------------
void oracle_speculative_accept_reject(const int64_t* draft_tokens, int64_t num_draft_tokens,
                                      const float* target_logits, int64_t vocab,
                                      const float* draft_probs, const float* rand_uniform,
                                      float inv_temperature, OracleAcceptResult* out) {
    OracleAcceptResult r;
    std::memset(&r, 0, sizeof(r));
    r.bonus_or_resampled_token = -1;
    r.rejected_token = -1;
    if (num_draft_tokens <= 0 || !draft_tokens || !target_logits || vocab <= 0 || num_draft_tokens > 64) {
        *out = r;
        return;
    }
    bool rejection = false;
    std::vector<float> scaled;
    for (int64_t i = 0; i < num_draft_tokens; ++i) {
        int64_t draft_tok = draft_tokens[i];
        const float* cur = target_logits + i * vocab;
        int64_t t = oracle_argmax(cur, vocab);
        bool accepted = false;
        if (!draft_probs) {
            accepted = (draft_tok == t);
        } else {
            float p_draft = draft_probs[i];
            float rr = rand_uniform ? rand_uniform[i] : 0.0f;
            if (p_draft <= 0.0f) {
                accepted = (draft_tok == t);
            } else if (draft_tok == t && rr <= 0.0f) {
                accepted = true;
            } else {
                const float* src = cur;
                if (inv_temperature != 1.0f) {
                    scaled.resize(static_cast<size_t>(vocab));
                    for (int64_t v = 0; v < vocab; ++v) scaled[v] = cur[v] * inv_temperature;
                    src = scaled.data();
                }
                float p_target = oracle_token_prob_f32(src, vocab, draft_tok);
                float ratio = p_target / p_draft;
                accepted = (rr < ratio);
            }
        }
        if (accepted) {
            r.accepted_tokens[r.num_accepted++] = draft_tok;
        } else {
            rejection = true;
            r.has_rejected_token = 1;
            r.rejected_token = draft_tok;
            r.num_rejected = 1;
            r.bonus_or_resampled_token = t;
            r.num_resampled = 1;
            r.num_remaining = num_draft_tokens - (r.num_accepted + 1);
            break;
        }
    }
    if (rejection) {
        if (r.num_accepted + r.num_rejected + r.num_remaining != num_draft_tokens) r.contract_violated = 1;
    } else {
        if (r.num_accepted != num_draft_tokens) r.contract_violated = 1;
        r.bonus_or_resampled_token = oracle_argmax(target_logits + (num_draft_tokens - 1) * vocab, vocab);
    }
    *out = r;
}

// Row softmax, src/ops/softmax.cpp:13-44 (three passes, fp32).
void oracle_softmax(float* out, const float* in, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* x = in + r * cols;
        float* y = out + r * cols;
        float mx = -std::numeric_limits<float>::infinity();
        for (int64_t c = 0; c < cols; ++c) mx = std::max(mx, x[c]);
        float s = 0.0f;
        for (int64_t c = 0; c < cols; ++c) { y[c] = std::exp(x[c] - mx); s += y[c]; }
        for (int64_t c = 0; c < cols; ++c) y[c] /= s;
    }
}

// ---------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
// Not in the reference: it is the uniform source the stochastic acceptance test feeds to
// both sides.  Uniform i of stream (seed, subsequence) is word (i & 3) of the block with
// counter = {lo32(i>>2), hi32(i>>2), lo32(subsequence), hi32(subsequence)},
// key = {lo32(seed), hi32(seed)}, mapped to [0,1) as (word >> 8) * 2^-24.
// ---------------------------------------------------------------------------------
static inline void philox_round(uint32_t c[4], const uint32_t k[2]) {
    const uint64_t M0 = 0xD2511F53ull, M1 = 0xCD9E8D57ull;
    uint64_t p0 = M0 * c[0], p1 = M1 * c[2];
    uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
    uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
    uint32_t n0 = hi1 ^ c[1] ^ k[0];
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c[3] ^ k[1];
    uint32_t n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
    uint32_t k[2] = {key[0], key[1]};
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k);
        k[0] += 0x9E3779B9u;
        k[1] += 0xBB67AE85u;
    }
    out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

void oracle_philox_uniform(float* out, int64_t n, uint64_t seed, uint64_t subsequence) {
    uint32_t key[2] = {static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)};
    for (int64_t i = 0; i < n; ++i) {
        uint64_t blk = static_cast<uint64_t>(i) >> 2;
        uint32_t ctr[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32),
                           static_cast<uint32_t>(subsequence), static_cast<uint32_t>(subsequence >> 32)};
        uint32_t o[4];
        oracle_philox4x32_10(ctr, key, o);
        out[i] = static_cast<float>(o[i & 3] >> 8) * (1.0f / 16777216.0f);
    }
}

// CRC-64 (reflected ECMA-182 polynomial 0xC96C5795D7870F42, init and xor-out all ones),
// src/artifact/checksum.cpp:8-55; null or empty input -> 0 as src/artifact/c_api.cpp:9-12.
uint64_t oracle_crc64(const void* data, size_t length) {
    if (!data || length == 0) return 0;
    uint64_t crc = ~0ull;
    const uint8_t* p = static_cast<const uint8_t*>(data);
    for (size_t i = 0; i < length; ++i) {
        crc ^= p[i];
        for (int b = 0; b < 8; ++b) crc = (crc & 1) ? (crc >> 1) ^ 0xC96C5795D7870F42ull : (crc >> 1);
    }
    return ~crc;
}

int oracle_num_threads() {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
