// Internal interface of the per-layer glue kernels (mixers.cu).  Rows are (sequence b, position i),
// i < rows_per_seq; every function is asynchronous on the stream and returns 0 or a negative code.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace xb {

int embed_rows(cudaStream_t s, __half* out, const void* table_bf16, const long long* tokens, int rows, int hidden,
               long long vocab);
// perm_out (here and below): write the output with every block of eight features in the order the int4 unpack of
// the W4A16 kernel yields them, (0,4,1,5,2,6,3,7): such a buffer is only good as the X of a projection launched
// with kTcXPermuted (w4a16.h).
int rmsnorm_rows(cudaStream_t s, __half* out, long long ld_out, const __half* in, const float* w, int rows, int hidden,
                 float eps, int perm_out = 0);
// x = half(x + delta) in place, out = rmsnorm(x) * w
int add_rmsnorm_rows(cudaStream_t s, __half* out, __half* x, const __half* delta, const float* w, int rows, int hidden,
                     float eps, int perm_out = 0);

// q/k head RMSNorm + partial RoPE + KV-cache write.  Caches are [batch][max_seq][hkv][256] fp16.
int attn_prep(cudaStream_t s, __half* q_out, __half* k_cache, __half* v_cache, const __half* q_gate, const __half* k_in,
              const __half* v_in, const float* q_norm_w, const float* k_norm_w, const int* ctx, int batch,
              int rows_per_seq, int hq, int hkv, long long max_seq, float eps, float rope_theta, int rope_dim);
// The same kernel with its optional pieces spelled out (the stand-alone op entry points): query heads
// `q_head_stride` halves apart in q_in, null norm weights skip the head norm, `positions` (per row) or `ctx_base`
// (when ctx is null) give the positions, null caches skip the write and the rotated keys go to `k_out`.
int attn_prep_ex(cudaStream_t s, __half* q_out, __half* k_cache, __half* v_cache, const __half* q_in, const __half* k_in,
                 const __half* v_in, const float* q_norm_w, const float* k_norm_w, const int* ctx, int batch,
                 int rows_per_seq, int hq, int hkv, long long max_seq, float eps, float rope_theta, int rope_dim,
                 int q_head_stride, const long long* positions, int ctx_base, __half* k_out, int cache_batch = 0);
size_t attn_scratch_bytes(int batch, int hkv, int nsplit);
// causal GQA attention over the cache (row i of sequence b sees keys below ctx[b] + i + 1), then * sigmoid(gate)
int attn_decode(cudaStream_t s, __half* out, const __half* q, const __half* q_gate, const __half* k_cache,
                const __half* v_cache, const int* ctx, int batch, int rows_per_seq, int hq, int hkv, long long max_seq,
                int nsplit, float* scratch);
// with an explicit softmax scale, a host-side context length when ctx is null, and no output gate when q_gate is null.
// cache_batch > 0 (here and in attn_prep_ex): entry e of the `batch` entries works on the cache of sequence
// e % cache_batch with its own ctx[e], so one launch can take several row groups of every sequence (prefill).
int attn_decode_ex(cudaStream_t s, __half* out, const __half* q, const __half* q_gate, const __half* k_cache,
                   const __half* v_cache, const int* ctx, int batch, int rows_per_seq, int hq, int hkv, long long max_seq,
                   int nsplit, float* scratch, float scale, int ctx_base, int perm_out = 0, int cache_batch = 0);

// state [batch][3][channels], pending [batch][8][channels] fp32.  The first min(n_commit[b], prev_rows) pending
// inputs of the previous call are committed to the state before the new rows are processed (n_commit null:
// nc_base of them).  rows_per_seq = 0 only commits.  early_state = 1 (both kernels): state, pending updates and
// weights were NOT written by the launch directly in front of this one in the stream, so the kernel may fetch
// them while that launch is still running (programmatic dependent launch).
int conv1d_spec(cudaStream_t s, __half* out, const __half* in, const float* conv_w, float* state, float* pending,
                const int* n_commit, int batch, int rows_per_seq, int prev_rows, int channels, int nc_base = 0,
                int early_state = 0);
// state [batch][hv][128][128], pend_k / pend_d [batch][hv][8][128], pend_g [batch][hv][8] fp32
int gdn_spec(cudaStream_t s, __half* out, const __half* qkv, const __half* z, const __half* b, const __half* a,
             const float* A_log, const float* dt_bias, const float* norm_w, float* state, float* pend_k, float* pend_d,
             float* pend_g, const int* n_commit, int batch, int rows_per_seq, int prev_rows, int hv, int hk, int nc_base = 0,
             int early_state = 0, int perm_out = 0);

// Row of (position p, sequence b) in a prefill chunk of rc positions per sequence.  The step's mixer kernels take at
// most a few rows per sequence and launch, laid out [sequence][row]; a projection does not care about the order of its
// rows.  So a chunk's rows are stored group by group: group j holds positions 4j .. 4j+3 of every sequence as one
// contiguous [sequence][row] block, which such a launch takes as it is.
__host__ __device__ inline long long chunk_row(int p, int b, int batch, int rc) {
    const int j = p >> 2, i = p & 3;
    const int rj = (rc - 4 * j) < 4 ? (rc - 4 * j) : 4;
    return static_cast<long long>(j) * batch * 4 + static_cast<long long>(b) * rj + i;
}
// The convolution and the gated delta rule over all rc positions of a prefill chunk in one launch each (rows in
// chunk_row order, every row kept, the state read once and written back once; nothing pending afterwards).
int conv1d_chunk(cudaStream_t s, __half* out, const __half* in, const float* conv_w, float* state, int batch, int rc,
                 int channels);
int gdn_chunk(cudaStream_t s, __half* out, const __half* qkv, const __half* z, const __half* b, const __half* a,
              const float* A_log, const float* dt_bias, const float* norm_w, float* state, int batch, int rc, int hv, int hk);

int spec_commit(cudaStream_t s, const void* accept_records, const long long* draft_tokens, int batch, int k,
                int rows_per_seq, int* ctx, int* n_commit, long long* cur_tok, long long* emitted, int* emitted_n,
                __half* h_last, const __half* hidden_rows, int hidden);
int build_verify_tokens(cudaStream_t s, long long* out, const long long* cur_tok, const long long* draft, int batch,
                        int k);
int fill_int(cudaStream_t s, int* p, int n, int v);
int copy_token_column(cudaStream_t s, long long* draft, const long long* argmax_out, int batch, int k, int col);

}  // namespace xb
