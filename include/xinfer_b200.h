/* C-ABI of libxinfer_b200.so: the speculative-decode hot path of xInfer on NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only.  Every compute entry point takes a CUDA stream where the reference
 * takes `sycl::queue&`, raw DEVICE pointers owned by the caller (row-major, no strides) exactly as the
 * reference's ops do, and returns an int status instead of throwing (0 = ok).  Entry points are
 * asynchronous on the stream unless stated otherwise.  One stream per device at a time: the library
 * keeps per-device scratch that concurrent launches on different streams would share, which mirrors
 * the reference's single in-order queue (src/core/device.cpp:54-58).
 *
 * Each declaration names the reference interface it replaces (path within the reference project).
 */
#ifndef XINFER_B200_H_
#define XINFER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XINFER_EXPORT __attribute__((visibility("default")))

typedef void* xinfer_stream_t; /* a cudaStream_t; NULL is the default stream */

/* ---- status codes ------------------------------------------------------------------------------ */
enum {
    XINFER_OK = 0,
    XINFER_NOOP_INVALID_SHAPE = 1,   /* the reference returns silently (src/ops/linear.cpp:176,359); so do
                                        we, but the caller is told */
    XINFER_ERR_CUDA = -1,            /* a CUDA runtime call failed; see xinfer_last_cuda_error() */
    XINFER_ERR_INVALID_ARGUMENT = -2,/* std::invalid_argument in the reference */
    XINFER_ERR_OUT_OF_MEMORY = -3,   /* std::bad_alloc in the reference */
    XINFER_ERR_CONTRACT = -4,        /* std::logic_error in the reference (fail-loud accounting) */
    XINFER_ERR_DEVICE_TIMEOUT = -5,  /* a bounded device-side wait gave up (see xinfer_device_status) */
    XINFER_ERR_NO_DEVICE = -6        /* no CUDA device / sm_100a code cannot run here */
};

/* ---- library / device set-up ------------------------------------------------------------------- */
/* Allocates this device's scratch (split-K partials, tile counters, sampling partials, status word).
 * Called implicitly by the first compute call on a device; call it explicitly before any stream
 * capture, because it allocates.  No counterpart in the reference (SYCL USM is allocated per call there). */
XINFER_EXPORT int xinfer_b200_init(int device);
XINFER_EXPORT int xinfer_b200_init_current(void); /* the same for the calling thread's current device */
/* 0 when no bounded device-side wait has given up on `device` since the last call, else
 * XINFER_ERR_DEVICE_TIMEOUT.  Covers every entry point, xinfer_linear_int4_f16f16_noalloc included; reading
 * clears the record.  The output of a launch that reported a timeout is undefined. */
XINFER_EXPORT int xinfer_device_status(int device);
XINFER_EXPORT const char* xinfer_last_cuda_error(void);
XINFER_EXPORT const char* xinfer_b200_version(void);
/* Which kernel family the last linear call on this thread used: 0 none, 1 tcgen05 (M <= 32, the decode and verify
 * kernel), 2 CUDA cores (fp32 activations, odd shapes), 3 tcgen05 GEMM (M > 32: prefill chunks through the same entry
 * points, forward_prefill_chunk of src/targets/qwen3_8/forward.cpp:402-554). */
XINFER_EXPORT int xinfer_last_linear_path(void);
/* Test hook for the bounded device-side waits of the tcgen05 linear kernel.  limit_clocks: SM clocks after
 * which a wait gives up (<= 0 restores the default, about one second).  withhold_x_from_stage >= 0: the
 * kernel's loader never requests the activation stages from that index on, so the waits for them run out,
 * the kernel returns through its abort path and xinfer_device_status reports the timeout (-1: off).
 * Process-wide; applies to launches enqueued afterwards.  No counterpart in the reference. */
XINFER_EXPORT void xinfer_debug_set_wait_hooks(int64_t limit_clocks, int withhold_x_from_stage);
/* Force a kernel family for the linear entry points on the current device: 0 = automatic (fp16 activations: the
 * tcgen05 decode kernel up to 32 rows, 32-row slices of it up to 128 rows, the tcgen05 GEMM above), 1 = the same,
 * 2 = CUDA cores only, 3 = the GEMM for every M > 32.  For measurements and tests. */
XINFER_EXPORT void xinfer_set_linear_path(int path);

/* ---- INT4-G128-SYM W4A16 linear:  Y[M,N] = X[M,K] * W^T + bias ---------------------------------
 * W_int4  [N][K/2] bytes, low nibble = even k, two's-complement int4
 * scales  [N][K/group_size] fp16
 * bias    [N] fp32 or NULL
 * Replaces xinfer::ops::linear_int4, src/ops/linear.h:30-63 (impl src/ops/linear.cpp:165-348,
 * split-K variant :33-163). */
XINFER_EXPORT int xinfer_linear_int4_f16f16(xinfer_stream_t s, void* Y_f16, const void* X_f16, const uint8_t* W_int4,
                                            const void* scales_f16, const float* bias, int64_t M, int64_t N,
                                            int64_t K, int group_size);
XINFER_EXPORT int xinfer_linear_int4_f16f32(xinfer_stream_t s, float* Y, const void* X_f16, const uint8_t* W_int4,
                                            const void* scales_f16, const float* bias, int64_t M, int64_t N,
                                            int64_t K, int group_size);
XINFER_EXPORT int xinfer_linear_int4_f32f32(xinfer_stream_t s, float* Y, const float* X, const uint8_t* W_int4,
                                            const void* scales_f16, const float* bias, int64_t M, int64_t N,
                                            int64_t K, int group_size);

/* Up to 4 projections sharing X and K.  Replaces xinfer::ops::linear_int4_fused and
 * FusedProjectionDesc / FusedProjectionDescFP32, src/ops/linear.h:66-111 (impl src/ops/linear.cpp:351-498).
 * num_descs outside [1,4] is a no-op as in the reference (src/ops/linear.cpp:359). */
typedef struct xinfer_fused_desc {
    void* Y;                /* [M][N] fp16 (or fp32 for the _f32 entry point) */
    const uint8_t* W_int4;  /* [N][K/2] */
    const void* scales;     /* [N][K/group_size] fp16 */
    const float* bias;      /* [N] or NULL */
    int64_t N;
} xinfer_fused_desc;
XINFER_EXPORT int xinfer_linear_int4_fused_f16(xinfer_stream_t s, const void* X_f16, const xinfer_fused_desc* descs,
                                               int num_descs, int64_t M, int64_t K, int group_size);
XINFER_EXPORT int xinfer_linear_int4_fused_f32(xinfer_stream_t s, const float* X, const xinfer_fused_desc* descs,
                                               int num_descs, int64_t M, int64_t K, int group_size);

/* Y[m,n] = silu(gate . x) * (up . x); gate and up never reach memory.  Replaces
 * xinfer::ops::mlp_gate_up_swiglu_int4, src/ops/linear.h:117-139 (impl src/ops/linear.cpp:501-632). */
XINFER_EXPORT int xinfer_mlp_gate_up_swiglu_int4_f16(xinfer_stream_t s, void* Y_f16, const void* X_f16,
                                                     const uint8_t* W_gate, const void* scales_gate,
                                                     const uint8_t* W_up, const void* scales_up, int64_t M,
                                                     int64_t N, int64_t K, int group_size);
XINFER_EXPORT int xinfer_mlp_gate_up_swiglu_int4_f32(xinfer_stream_t s, float* Y, const float* X,
                                                     const uint8_t* W_gate, const void* scales_gate,
                                                     const uint8_t* W_up, const void* scales_up, int64_t M,
                                                     int64_t N, int64_t K, int group_size);

/* Column-sliced variant for N-split tensor parallelism: the output row stride `ldy` (elements) may
 * exceed N so that a rank writes its slice of a wider activation.  No counterpart in the reference
 * (it has no multi-GPU code). */
XINFER_EXPORT int xinfer_linear_int4_f16f16_ld(xinfer_stream_t s, void* Y_f16, int64_t ldy, const void* X_f16,
                                               const uint8_t* W_int4, const void* scales_f16, const float* bias,
                                               int64_t M, int64_t N, int64_t K, int group_size);

/* The same fp16 -> fp16 linear for callers that must not allocate device memory: a serving process that has
 * already given all free HBM to its cache pool, a job under a fixed memory quota, code that runs while a
 * CUDA graph is being captured.  This entry point calls no cudaMalloc / cudaFree and no allocating library
 * routine: its scratch (split-K partials, tile counters, status word; 10.5 MB) is a fixed array inside the
 * library image, held by every GPU that loads the library until the process exits.  It has no counterpart
 * in the reference.
 *   - Limits: 1 <= M <= 32, K a multiple of 128, group_size 128, 16-byte aligned X and W, N <= 2,097,152,
 *     at most 160 SMs.  Anything else returns XINFER_ERR_INVALID_ARGUMENT (there is no fallback path).
 *   - The first call on a device resolves the array's device address and configures the kernel (all three
 *     row-count variants); make that first call before any stream capture.  Later calls only enqueue work
 *     on `s`.
 *   - Every call uses the same array.  Counters are cleared at the start of each call, on `s`; two calls
 *     that overlap on the GPU (different streams, or graphs replayed concurrently) race on it.
 *   - A bounded wait that gives up inside this entry point is reported by xinfer_device_status(), like
 *     any other launch's; the record is kept across later calls until it has been read. */
XINFER_EXPORT int xinfer_linear_int4_f16f16_noalloc(xinfer_stream_t s, void* Y_f16, const void* X_f16,
                                                    const uint8_t* W_int4, const void* scales_f16, const float* bias,
                                                    int64_t M, int64_t N, int64_t K, int group_size);

/* Launch plan for callers that issue the same sequence of fp16-activation linears again and again (a decode or
 * verify pass).  Record one round of the sequence between record_begin() and record_end(); call rewind() at the
 * start of every later round.  Each launch of a recorded round then also asks the L2 cache for the first weight
 * tiles of the launch that follows it, so that launch starts from L2 instead of HBM.  The plan is a hint: results
 * are unchanged, and a call that does not match the recorded sequence switches the hints off until the next
 * recording.  These four calls act on the process-wide plan (a decoder object keeps a plan of its own);
 * clear() drops it (call it before freeing the recorded weights).
 * No counterpart in the reference (its queue has no cross-kernel prefetch). */
XINFER_EXPORT void xinfer_linear_plan_record_begin(void);
XINFER_EXPORT void xinfer_linear_plan_record_end(void);
XINFER_EXPORT void xinfer_linear_plan_rewind(void);
XINFER_EXPORT void xinfer_linear_plan_clear(void);

/* ---- sampling ---------------------------------------------------------------------------------- */
/* Replaces xinfer::ops::argmax_scratch_size, src/ops/sampling.h:11-15. */
XINFER_EXPORT size_t xinfer_argmax_scratch_size(int64_t vocab_size);
/* Synchronous greedy argmax of one fp32 logit row on the device; ties -> lowest index; vocab <= 0 or
 * NULL -> 0.  partial_max / partial_idx are optional caller scratch (device or managed memory, at
 * least xinfer_argmax_scratch_size entries).  Replaces xinfer::ops::argmax, src/ops/sampling.h:17-25. */
XINFER_EXPORT int64_t xinfer_argmax(xinfer_stream_t s, const float* logits, int64_t vocab_size, float* partial_max,
                                    int64_t* partial_idx);
/* Asynchronous, batched, result stays on the device: out_dev[r] = argmax(logits[r*row_stride ..]).
 * The graph-capturable form of the same op (the reference's argmax blocks the host,
 * src/ops/sampling.cpp:73). */
XINFER_EXPORT int xinfer_argmax_rows(xinfer_stream_t s, const float* logits, int64_t row_stride, int64_t rows,
                                     int64_t vocab_size, int64_t* out_dev);

/* POD form of xinfer::ops::SpeculativeAcceptanceResult, src/ops/sampling.h:27-36. */
#define XINFER_MAX_DRAFT_TOKENS 64
typedef struct xinfer_accept_result {
    int64_t accepted_tokens[XINFER_MAX_DRAFT_TOKENS];
    int64_t bonus_or_resampled_token; /* -1 for empty / invalid input */
    int64_t rejected_token;           /* -1 when none */
    int64_t num_accepted;
    int64_t num_rejected;
    int64_t num_resampled;
    int64_t num_remaining;
    int32_t has_rejected_token;
    int32_t reserved;
} xinfer_accept_result;

/* Synchronous.  draft_tokens / draft_probs / rand_uniform are HOST pointers, target_logits is a DEVICE
 * pointer [num_draft_tokens][vocab_size] fp32, as in the reference.  draft_probs == NULL selects the
 * greedy rule.  Returns XINFER_ERR_CONTRACT where the reference throws std::logic_error.
 * Replaces xinfer::ops::speculative_accept_reject, src/ops/sampling.h:42-49 (impl sampling.cpp:94-199). */
XINFER_EXPORT int xinfer_speculative_accept_reject(xinfer_stream_t s, const int64_t* draft_tokens,
                                                   size_t num_draft_tokens, const float* target_logits,
                                                   int64_t vocab_size, const float* draft_probs,
                                                   const float* rand_uniform, xinfer_accept_result* out);

/* Device-side, batched, asynchronous form for `batch` independent sequences: all pointers are DEVICE
 * pointers.  Sequence b owns logit rows b*rows_per_seq + i (row stride `row_stride` floats), verifies
 * draft token i against row i for i < num_draft, and on full acceptance takes its bonus token from row
 * `bonus_row` (num_draft-1 reproduces the reference; num_draft is the (k+1)-row convention).
 * Logits are multiplied by inv_temperature before the stochastic rule (1.0 reproduces the reference;
 * the reference has no temperature, src/runtime/engine.cpp:279-303).  out_dev: one record per sequence. */
typedef struct xinfer_accept_record {
    int64_t bonus_or_resampled_token;
    int64_t rejected_token;
    int32_t num_accepted;
    int32_t num_rejected;
    int32_t num_resampled;
    int32_t num_remaining;
    int32_t has_rejected_token;
    int32_t reserved;
} xinfer_accept_record;
XINFER_EXPORT int xinfer_speculative_accept_reject_batched(xinfer_stream_t s, const int64_t* draft_tokens_dev,
                                                           const float* target_logits_dev, int64_t row_stride,
                                                           int64_t vocab_size, const float* draft_probs_dev,
                                                           const float* rand_uniform_dev, float inv_temperature,
                                                           int batch, int num_draft, int rows_per_seq, int bonus_row,
                                                           xinfer_accept_record* out_dev);

/* One token per row drawn from softmax(logits * inv_temperature) at the row's uniform in [0, 1) (inverse of the
 * cumulative distribution, a fixed two-level fp32 summation: the same (logits, u) always gives the same token), and the
 * token's probability - the draft token and the p_draft that xinfer_speculative_accept_reject_batched takes.  No
 * counterpart in the reference, whose drafter is greedy (src/runtime/engine.cpp:279-303 rejects temperature).
 * Asynchronous; all pointers device memory. */
XINFER_EXPORT int xinfer_sample_tokens(xinfer_stream_t s, const float* logits_dev, int64_t row_stride, int64_t vocab_size,
                                       int rows, float inv_temperature, const float* rand_uniform_dev, int64_t* tokens_out_dev,
                                       float* probs_out_dev);
/* The same draw from the row's nucleus: the smallest set of highest-probability tokens of softmax(logits *
 * inv_temperature) whose probabilities reach top_p (ties at the threshold all in), renormalised.  Weights are the
 * integers rn(exp(s - max) * 2^32), so every sum is exact and order-free; the token is the first, in index order, at which
 * the running nucleus weight exceeds floor(u * Z_nucleus); probs_out is its weight / Z_nucleus.  0 < top_p <= 1.
 * GenerationConfig::top_p of the reference (include/xinfer/engine.h:20), which its engine refuses
 * (src/runtime/engine.cpp:294-303).  Asynchronous; all pointers device memory. */
XINFER_EXPORT int xinfer_sample_tokens_top_p(xinfer_stream_t s, const float* logits_dev, int64_t row_stride,
                                             int64_t vocab_size, int rows, float inv_temperature, float top_p,
                                             const float* uniforms_dev, int64_t* tokens_out_dev, float* probs_out_dev);

/* Philox4x32-10 uniforms in [0,1): out[i] = (word(i&3) of block(i>>2) >> 8) * 2^-24 with counter
 * {lo(i>>2), hi(i>>2), lo(subsequence), hi(subsequence)} and key {lo(seed), hi(seed)}.  No counterpart
 * in the reference (its acceptance op takes caller-supplied uniforms). */
XINFER_EXPORT int xinfer_philox_uniform(xinfer_stream_t s, float* out_dev, int64_t n, uint64_t seed,
                                        uint64_t subsequence);

/* ---- speculative decode runtime -------------------------------------------------------------------
 * A random-init Qwen-hybrid target (Gated-DeltaNet + full-attention layers, INT4-G128 weights), one MTP
 * draft head, and the step   k draft passes -> batched verify (k+1 rows per sequence) -> acceptance ->
 * commit   for `batch` independent sequences.  Stands in for the speculative loop of Engine::generate
 * (src/runtime/engine.cpp:400-525), draft_decode_loop / forward_verify
 * (src/targets/qwen3_8/forward.cpp:600-734) and DecodeGraph (src/targets/qwen3_8/decode_graph.h:18-60;
 * xinfer_spec_decoder_capture records the whole step into one CUDA graph, token ids and positions
 * living in device memory as in the reference).  The MTP head has no counterpart in the reference. */
typedef struct xinfer_model_config {   /* the shape fields of ModelConfig, src/targets/qwen3_8_27b/weights.h:58-107 */
    int64_t hidden_size;
    int64_t intermediate_size;
    int64_t num_hidden_layers;
    int64_t num_attention_heads;       /* head_dim is 256 */
    int64_t num_key_value_heads;
    int64_t vocab_size;
    int64_t linear_num_v_heads;        /* Gated-DeltaNet head dims are 128 */
    int64_t linear_num_k_heads;
    int32_t full_attention_interval;   /* layer l is full attention iff l % interval == interval - 1 */
    int32_t rope_dim;
    float rms_norm_eps;
    float rope_theta;
} xinfer_model_config;
typedef struct xinfer_spec_decoder xinfer_spec_decoder;
XINFER_EXPORT int xinfer_spec_decoder_create(const xinfer_model_config* cfg, int batch, int k, int64_t max_seq,
                                             uint64_t seed, xinfer_spec_decoder** out);
XINFER_EXPORT void xinfer_spec_decoder_destroy(xinfer_spec_decoder* d);
/* Synthetic context of `context_len` positions per sequence: random KV cache and recurrent state. */
XINFER_EXPORT int xinfer_spec_decoder_reset(xinfer_spec_decoder* d, int64_t context_len, uint64_t seed);
XINFER_EXPORT int xinfer_spec_decoder_set_tokens(xinfer_spec_decoder* d, const int64_t* cur_tokens_host);
/* Enqueues one speculative step (replays the captured graph when there is one).  Returns
 * XINFER_ERR_INVALID_ARGUMENT, enqueuing nothing, when another step could run past max_seq (the reference's
 * KVCache throws when it is full). */
XINFER_EXPORT int xinfer_spec_decoder_step(xinfer_spec_decoder* d, xinfer_stream_t stream);
XINFER_EXPORT int xinfer_spec_decoder_capture(xinfer_spec_decoder* d, xinfer_stream_t stream);
/* Synchronous: emitted_host [batch][k+1] (accepted drafts, then the bonus token, then -1), counts_host [batch]. */
XINFER_EXPORT int xinfer_spec_decoder_results(xinfer_spec_decoder* d, xinfer_stream_t stream, int64_t* emitted_host,
                                              int* counts_host);
/* Test hook (eager steps only): the next steps verify `drafts_host` [batch][k] instead of the MTP head's
 * tokens; the draft passes still run.  NULL disarms it. */
XINFER_EXPORT int xinfer_spec_decoder_override_drafts(xinfer_spec_decoder* d, const int64_t* drafts_host);
/* Measurement entry: enqueues only the W4A16 linear launches of one step (same order, same weights). */
XINFER_EXPORT int xinfer_spec_decoder_enqueue_linears(xinfer_spec_decoder* d, xinfer_stream_t stream);
/* what: 0 weight bytes, 1 state bytes, 2 kernel launches per step, 3 graph captured,
 * 4 algorithmic bytes of the step's linear launches (this rank's), 5 number of linear launches per step,
 * 6 inter-rank exchanges per step, 7 bytes of the decoder's one device block */
XINFER_EXPORT int64_t xinfer_spec_decoder_info(const xinfer_spec_decoder* d, int what);
XINFER_EXPORT void* xinfer_spec_decoder_tensor(xinfer_spec_decoder* d, int layer, const char* name, int64_t* bytes);
XINFER_EXPORT const char* xinfer_spec_decoder_error(const xinfer_spec_decoder* d);

/* ---- per-layer mixer ops (fp16 overloads of the reference's ops; head_dim 256) -----------------------
 * The kernels the speculative step uses between its projections, exported one by one so that each can be
 * checked against the reference's own op tests.  They keep the reference's fp16 rounding points; reductions
 * are fp32.  The stateful ones allocate a small per-device scratch on their first call (make it before any
 * stream capture). */
/* out = in * rsqrt(mean(in^2) + eps) * weight.  Replaces ops::rmsnorm (half), src/ops/rmsnorm.h:17-23. */
XINFER_EXPORT int xinfer_rmsnorm_f16(xinfer_stream_t s, void* out_f16, const void* in_f16, const float* weight,
                                     int64_t num_tokens, int64_t hidden_size, float eps);
/* residual += in (fp16); out = rmsnorm(residual).  Replaces ops::rmsnorm_residual (half), rmsnorm.h:35-42. */
XINFER_EXPORT int xinfer_rmsnorm_residual_f16(xinfer_stream_t s, void* out_f16, void* residual_f16, const void* in_f16,
                                              const float* weight, int64_t num_tokens, int64_t hidden_size, float eps);
/* In-place partial rotary embedding of Q [tokens][q_heads][256] and K [tokens][kv_heads][256]: pairs
 * (p, p + rotary_dim/2) of the first rotary_dim dims, angle = position * theta^(-2p/rotary_dim); positions is a
 * DEVICE array [tokens].  Replaces ops::rope (half), src/ops/rope.h:25-34. */
XINFER_EXPORT int xinfer_rope_f16(xinfer_stream_t s, void* q_f16, void* k_f16, int64_t num_tokens, int64_t num_q_heads,
                                  int64_t num_kv_heads, int64_t head_dim, const int64_t* positions_dev, float theta,
                                  int64_t rotary_dim);
/* Copies K, V rows into the fp16 cache [pos][kv_head][256] at start_pos...  Rows that do not fit a bounded
 * cache (max_seq_len > 0) are an error, as in the reference.  Replaces ops::attention_write_kv_cache (half),
 * src/ops/attention.h:49-58. */
XINFER_EXPORT int xinfer_attention_write_kv_cache_f16(xinfer_stream_t s, void* k_cache_f16, void* v_cache_f16,
                                                      const void* K_in_f16, const void* V_in_f16, int64_t start_pos,
                                                      int64_t num_tokens, int64_t num_kv_heads, int64_t head_dim,
                                                      int64_t max_seq_len);
/* Causal GQA attention of num_q_tokens query rows at positions start_pos... over the cache: row i sees keys
 * 0 .. start_pos + i.  scale <= 0 means 1/sqrt(head_dim).  Replaces ops::sdpa_causal_cached (half),
 * src/ops/attention.h:102-113 (also the body of sdpa_causal_verify). */
XINFER_EXPORT int xinfer_sdpa_causal_cached_f16(xinfer_stream_t s, void* out_f16, const void* Q_f16,
                                                const void* k_cache_f16, const void* v_cache_f16, int64_t start_pos,
                                                int64_t num_q_tokens, int64_t num_q_heads, int64_t num_kv_heads,
                                                int64_t head_dim, float scale, int64_t max_seq_len);
/* Depthwise causal conv (width 4) + SiLU over [seq_len][channels]; conv_state [3][channels] fp32 holds the last
 * three inputs and is updated by the call (NULL: zeros for the past, nothing kept).  Replaces
 * targets::qwen3_8::causal_conv1d_silu (half), src/targets/qwen3_8/linear_attn.h:15-21. */
XINFER_EXPORT int xinfer_causal_conv1d_silu_f16(xinfer_stream_t s, void* out_f16, const void* in_f16, const float* conv_w,
                                                int64_t seq_len, float* conv_state, int64_t num_channels);
/* Gated delta rule + gated RMSNorm, head dims 128, state [v_heads][128][128] fp32 updated by the call.
 * Replaces targets::qwen3_8::recurrent_gated_delta_net (half), src/targets/qwen3_8/linear_attn.h:41-58. */
XINFER_EXPORT int xinfer_recurrent_gated_delta_net_f16(xinfer_stream_t s, void* out_f16, const void* qkv_f16,
                                                       const void* z_f16, const void* b_f16, const void* a_f16,
                                                       const float* A_log, const float* dt_bias, const float* norm_weight,
                                                       float* state_buffer, int64_t seq_len, int zero_state,
                                                       int64_t num_v_heads, int64_t num_k_heads);

/* ---- N-split tensor parallelism over the GPUs of one box (one process per GPU) -------------------------
 * No counterpart in the reference (it has no multi-GPU code).  Rank r holds the output rows
 * [r N/g, (r+1) N/g) of every split projection, computes that slice for all activation rows and stores it
 * into every rank's activation buffer straight from the GEMM epilogue (plain peer stores over NVLink), then
 * one flag per (receiver, sender); device-side waits are bounded and report through xinfer_tp_status.
 *
 * Every rank owns an exchange region of `bytes` (the same on all ranks).  Set-up: create -> handle ->
 * all-gather the xinfer_tp_handle_bytes()-sized blobs among the ranks by any means -> connect. */
typedef struct xinfer_tp xinfer_tp;
XINFER_EXPORT int xinfer_tp_create(int rank, int world, size_t bytes, xinfer_tp** out);
XINFER_EXPORT void xinfer_tp_destroy(xinfer_tp* tp);
XINFER_EXPORT size_t xinfer_tp_handle_bytes(void);
XINFER_EXPORT int xinfer_tp_handle(xinfer_tp* tp, void* out_blob);
/* all_handles: world blobs in rank order (this rank's own is ignored). */
XINFER_EXPORT int xinfer_tp_connect(xinfer_tp* tp, const void* all_handles);
XINFER_EXPORT int xinfer_tp_rank(const xinfer_tp* tp);
XINFER_EXPORT int xinfer_tp_world(const xinfer_tp* tp);
/* Carves `bytes` out of the region (256-byte aligned).  Ranks that allocate in the same order get the same
 * offsets, and an offset names the same logical buffer on every rank. */
XINFER_EXPORT int xinfer_tp_alloc(xinfer_tp* tp, size_t bytes, size_t* offset_out);
XINFER_EXPORT void* xinfer_tp_ptr(xinfer_tp* tp, size_t offset);
/* Y[M][ldy] lives at y_offset of every rank's region; this rank computes the columns [col0, col0 + N_local)
 * from its slice of W / scales and stores them into EVERY rank's Y (rows_per_rank == 0), or row j only into
 * rank j / rows_per_rank's Y (the rank that owns the row's sequence).  When the launch completes on a
 * rank, every rank's columns have arrived there.  Shapes the tcgen05 kernel does not take are refused. */
XINFER_EXPORT int xinfer_tp_linear_int4_f16f16(xinfer_tp* tp, xinfer_stream_t s, size_t y_offset, int64_t ldy,
                                               int64_t col0, const void* X_f16, const uint8_t* W_int4,
                                               const void* scales_f16, const float* bias, int64_t M, int64_t N_local,
                                               int64_t K, int group_size, int rows_per_rank);
/* Copies [offset, offset + bytes) of this rank's region to the same place on every other rank, then the same
 * handshake (an all-gather when every rank pushes its own part of a buffer).  16-byte granularity. */
XINFER_EXPORT int xinfer_tp_push(xinfer_tp* tp, xinfer_stream_t s, size_t offset, size_t bytes);
XINFER_EXPORT int xinfer_tp_barrier(xinfer_tp* tp, xinfer_stream_t s);
/* Clock limit of the exchange waits (<= 0: the default, about one second), and whether one has run out
 * since the last call (XINFER_ERR_DEVICE_TIMEOUT; the data of that exchange is incomplete). */
XINFER_EXPORT void xinfer_tp_set_wait_limit(xinfer_tp* tp, int64_t limit_clocks);
XINFER_EXPORT int xinfer_tp_status(xinfer_tp* tp);

/* The speculative decoder over `tp` (connected): projections N-split, KV caches and recurrent state split by
 * sequence (batch % world == 0), LM head split by vocabulary with (max, index) partials exchanged, the whole
 * step one CUDA graph per rank.  Every rank must create its decoder with the same arguments and run the
 * same calls.  tp == NULL or world 1: the single-GPU decoder.  exchange_bytes: region size it needs. */
XINFER_EXPORT size_t xinfer_spec_decoder_exchange_bytes(const xinfer_model_config* cfg, int batch, int k, int world);
XINFER_EXPORT int xinfer_spec_decoder_create_tp(const xinfer_model_config* cfg, int batch, int k, int64_t max_seq,
                                                uint64_t seed, xinfer_tp* tp, xinfer_spec_decoder** out);

/* ---- device arena ------------------------------------------------------------------------------
 * cudaMalloc-backed bump allocator.  Replaces xinfer::core::DeviceArena, src/core/arena.h:14-66
 * (impl src/core/arena.cpp:84-139): 64-byte default alignment, allocate(0) -> NULL, overflow ->
 * XINFER_ERR_OUT_OF_MEMORY (std::bad_alloc there), persistent allocations survive reset(), one
 * persistent buffer that refuses to grow (XINFER_ERR_INVALID_ARGUMENT). */
typedef struct xinfer_arena xinfer_arena;
XINFER_EXPORT int xinfer_arena_create(size_t capacity_bytes, size_t default_alignment, xinfer_arena** out);
XINFER_EXPORT void xinfer_arena_destroy(xinfer_arena* a);
XINFER_EXPORT int xinfer_arena_allocate(xinfer_arena* a, size_t bytes, size_t alignment, void** out);
XINFER_EXPORT int xinfer_arena_allocate_persistent(xinfer_arena* a, size_t bytes, size_t alignment, void** out);
XINFER_EXPORT int xinfer_arena_persistent_buffer(xinfer_arena* a, size_t bytes, size_t alignment, void** out);
XINFER_EXPORT void xinfer_arena_reset(xinfer_arena* a);
XINFER_EXPORT size_t xinfer_arena_capacity(const xinfer_arena* a);
XINFER_EXPORT size_t xinfer_arena_allocated_bytes(const xinfer_arena* a);
XINFER_EXPORT size_t xinfer_arena_remaining_bytes(const xinfer_arena* a);
XINFER_EXPORT size_t xinfer_arena_peak_allocated_bytes(const xinfer_arena* a);
XINFER_EXPORT void* xinfer_arena_base_ptr(const xinfer_arena* a);

/* Plain device memory, streams and synchronous copies for hosts that do not link the CUDA runtime
 * themselves.  The reference's counterparts are members of DeviceContext, src/core/device.h:26-72. */
XINFER_EXPORT int xinfer_device_alloc(size_t bytes, void** out);   /* DeviceContext::allocate_device */
XINFER_EXPORT void xinfer_device_free(void* dev_ptr);              /* DeviceContext::free_device */
XINFER_EXPORT int xinfer_stream_create(xinfer_stream_t* out);      /* stands in for DeviceContext::queue() */
XINFER_EXPORT void xinfer_stream_destroy(xinfer_stream_t s);
XINFER_EXPORT int xinfer_stream_synchronize(xinfer_stream_t s);    /* DeviceContext::synchronize */
XINFER_EXPORT int xinfer_copy_device_to_host(void* dst_host, const void* src_dev, size_t bytes);
XINFER_EXPORT int xinfer_copy_host_to_device(void* dst_dev, const void* src_host, size_t bytes);

/* ---- artifact checksum (kept unchanged) -------------------------------------------------------
 * The two exports of the reference's xinfer_artifact_c library, src/artifact/c_api.h:12-20:
 * CRC-64 with reflected polynomial 0xC96C5795D7870F42, init and xor-out all ones; NULL or empty -> 0;
 * file variant reads at most max_bytes (0 = whole file), unreadable file -> 0. */
XINFER_EXPORT uint64_t xinfer_crc64(const void* data, size_t length);
XINFER_EXPORT uint64_t xinfer_crc64_file(const char* filepath, uint64_t max_bytes);
/* Incremental form of the same CRC for data that arrives in pieces: start from state ~0 (all ones), feed the
 * pieces in order, complement the final state; xinfer_crc64(d, n) == ~xinfer_crc64_update(~0, d, n).  No
 * counterpart in the C-ABI of the reference (its Crc64 class is C++ only, src/artifact/checksum.h). */
XINFER_EXPORT uint64_t xinfer_crc64_update(uint64_t state, const void* data, size_t length);

/* ---- `.xinfer` artifacts ------------------------------------------------------------------------------
 * Reader of the reference's container (docs/artifact-format.md; src/artifact/container.h:20-63) and loader of
 * its tensors into device memory.  open() applies the checks of ArtifactReader::open (src/artifact/reader.cpp:
 * 59-196: magics, version, header size, file size, bounds of metadata / section table / every section) and,
 * on request, the whole-file CRC-64 (reader.cpp:266-310).  Section payloads stream through pinned staging
 * buffers; their CRC-64 is checked while they stream.  XINFER_ERR_CONTRACT = checksum mismatch. */
typedef struct xinfer_artifact xinfer_artifact;
XINFER_EXPORT int xinfer_artifact_open(const char* path, int verify_file_checksum, xinfer_artifact** out);
XINFER_EXPORT void xinfer_artifact_close(xinfer_artifact* a);
XINFER_EXPORT int xinfer_artifact_section_count(const xinfer_artifact* a);
XINFER_EXPORT int xinfer_artifact_find(const xinfer_artifact* a, const char* name); /* index, or -1 */
XINFER_EXPORT int xinfer_artifact_section_info(const xinfer_artifact* a, int index, const char** name, uint32_t* type_tag,
                                               uint64_t* offset, uint64_t* size, uint64_t* checksum);
XINFER_EXPORT const char* xinfer_artifact_metadata(const xinfer_artifact* a, uint64_t* size); /* the JSON block */
XINFER_EXPORT const char* xinfer_artifact_error(const xinfer_artifact* a);
/* Whole section into host memory, checksum verified.  Replaces ArtifactReader::read_section, reader.h:44-47. */
XINFER_EXPORT int xinfer_artifact_read_section(xinfer_artifact* a, const char* name, void* dst_host, uint64_t capacity);
/* Bytes [offset, offset + bytes) of a section into device memory (synchronous).  verify != 0 reads the whole
 * section and checks its CRC-64 even when only a part is kept. */
XINFER_EXPORT int xinfer_artifact_load_section(xinfer_artifact* a, const char* name, uint64_t offset, uint64_t bytes,
                                               void* dst_dev, int verify);
/* One INT4 projection: sections `weight_name` ([out][in/2] bytes) and `weight_name`.scales ([out][in/group]
 * fp16) with the size checks of load_linear (src/targets/qwen3_8_27b/weights.cpp:252-304); rows
 * [row0, row0 + rows) of both go to the device: the whole projection, or the N-split shard of one rank. */
XINFER_EXPORT int xinfer_artifact_load_linear(xinfer_artifact* a, const char* weight_name, int64_t out_features,
                                              int64_t in_features, int group_size, int64_t row0, int64_t rows,
                                              void* dst_weights_dev, void* dst_scales_dev, int verify);
/* Sampling mode of the step.  temperature <= 0 (default): greedy drafting and the greedy accept rule, what the
 * reference's engine runs.  temperature > 0: draft tokens are drawn from softmax(head logits / T) and the verify pass
 * applies the reference's stochastic rule (src/ops/sampling.cpp:129-171) to target logits / T with the draft token's
 * probability; uniforms are Philox4x32-10 of (seed, step index) - element b * k + i picks draft i of sequence b,
 * element batch * k + b * k + i is its acceptance uniform - and the step index lives in device memory, so a replayed
 * graph draws fresh numbers.  Call before capture.  One GPU only. */
XINFER_EXPORT int xinfer_spec_decoder_set_sampling(xinfer_spec_decoder* d, float temperature, uint64_t seed);
/* Nucleus sampling inside the stochastic step: with 0 < top_p < 1 (and temperature > 0) the draft tokens are drawn from the
 * nucleus of the head's distribution (xinfer_sample_tokens_top_p) and the acceptance rule takes the target's probability
 * inside the target row's own nucleus (zero outside it).  top_p = 1 (default) is the whole distribution.  Call before
 * capture. */
XINFER_EXPORT int xinfer_spec_decoder_set_top_p(xinfer_spec_decoder* d, float top_p);
/* Builds the context from a prompt, tokens[batch][T] on the host (every sequence the same length), starting from the
 * empty context of xinfer_spec_decoder_reset(d, 0, seed): positions 0 .. T-2 go through the target in chunks of up to
 * 512 rows over all sequences (the projections of a chunk run as one M = 512 GEMM each, attention, convolution and the
 * gated delta rule take it in one launch each), the MTP head's KV slots of those positions are filled, the last prompt
 * token becomes the current token; ctx = T - 1 afterwards and xinfer_spec_decoder_step continues from there.  Stands
 * where the reference's chunked prefill does (forward_prefill_chunk, src/targets/qwen3_8/forward.cpp:402-554;
 * prefill_chunk_size = 512, include/xinfer/engine.h:34; engine.cpp:330-398).  Synchronous; one GPU only. */
XINFER_EXPORT int xinfer_spec_decoder_prefill(xinfer_spec_decoder* d, xinfer_stream_t stream, const int64_t* prompt_host,
                                              int64_t T);
/* The device side of Engine::generate's speculative loop (src/runtime/engine.cpp:262-560) for `batch` prompts of one
 * length T (host, [batch][T]): the reference's argument checks (max_new_tokens > 0, temperature >= 0, 0 < top_p <= 1 and top_p < 1 only with temperature > 0,
 * prompt + completion within the cache; messages in xinfer_spec_decoder_error), reset to the empty context, prefill,
 * then steps until every sequence has stopped.  A sequence stops on eos_token_id / im_end_token_id (a negative id
 * matches nothing; the stop token is not returned; finish 0 = "stop") or with max_new_tokens tokens (finish 1 =
 * "length"; also when the cache runs out).  temperature > 0 runs the stochastic step (the reference's engine
 * refuses it, engine.cpp:285-293; its acceptance rule exists in src/ops/sampling.cpp and is what the step applies);
 * top_p < 1 adds nucleus sampling on both sides of that rule (xinfer_spec_decoder_set_top_p).
 * token_ids_out is [batch][max_new_tokens], generated_out and finish_out are [batch]; stats may be NULL.
 * Sequences run in lockstep; a stopped one keeps its lane until the last has finished.  Uses the captured graph
 * when there is one.  Synchronous; one GPU only. */
typedef struct xinfer_generation_config {   /* GenerationConfig, include/xinfer/engine.h:17-25 */
    int32_t max_new_tokens;
    float temperature;          /* 0 = greedy */
    float top_p;                /* 1 = whole distribution; < 1 needs temperature > 0 */
    int64_t eos_token_id;
    int64_t im_end_token_id;
    uint64_t seed;              /* Philox seed of the stochastic step */
} xinfer_generation_config;
typedef struct xinfer_generation_stats {    /* the counters of GenerationResult, include/xinfer/engine.h:44-57 */
    int64_t prompt_tokens;      /* per sequence */
    int64_t generated_tokens;   /* over all sequences */
    int64_t steps;
    double time_to_first_token_sec;   /* reset + prefill + the first step */
    double decode_tokens_per_sec;     /* tokens kept after the first step / time after it, all sequences */
    double total_time_sec;
} xinfer_generation_stats;
XINFER_EXPORT int xinfer_spec_decoder_generate(xinfer_spec_decoder* d, xinfer_stream_t stream, const int64_t* prompt_host,
                                               int64_t T, const xinfer_generation_config* config, int64_t* token_ids_out,
                                               int32_t* generated_out, int32_t* finish_out,
                                               xinfer_generation_stats* stats);
/* Replaces a decoder's (synthetic) weights by the tensors of an artifact, under the section names of the reference's
 * loader (src/targets/qwen3_8_27b/weights.cpp:358-640); under tensor parallelism every rank loads its own row range of
 * each split projection.  The MTP head's tensors (`mtp.fc.weight`, `mtp.pre_fc_norm_{embedding,hidden}.weight`,
 * `mtp.layers.0.*`) are loaded when the file has them.  Call between create and the first step / capture.
 * XINFER_ERR_CONTRACT: a layer's kind in the file differs from the decoder's, or a checksum mismatch. */
XINFER_EXPORT int xinfer_spec_decoder_load_artifact(xinfer_spec_decoder* d, xinfer_artifact* a, int verify);
/* A BF16 vector as fp32 on the device, with the checkpoint's "1 + w" RMSNorm convention when add_unit_offset
 * (src/targets/qwen3_8_27b/weights.cpp:319-347). */
XINFER_EXPORT int xinfer_artifact_load_bf16_as_f32(xinfer_artifact* a, const char* name, int64_t num_elements,
                                                   int add_unit_offset, float* dst_dev);

#ifdef __cplusplus
}
#endif
#endif /* XINFER_B200_H_ */
