// Internal interface of the sampling / acceptance kernels (sampling.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace xb {

// Device-side form of SpeculativeAcceptanceResult (src/ops/sampling.h:27-36 of the reference); the
// accepted tokens are the first num_accepted draft tokens and are not repeated here.
struct AcceptOut {
    long long bonus_or_resampled_token;
    long long rejected_token;
    int num_accepted;
    int num_rejected;
    int num_resampled;
    int num_remaining;
    int has_rejected_token;
    int pad;
};

// What the acceptance rule needs to know of a row's nucleus (top-p): the order-preserving key of the smallest scaled
// logit inside it, the row's maximum scaled logit, and the sum of the integer weights rn(exp(s - max) * 2^32) inside.
struct Nucleus {
    unsigned long long z;
    float max_scaled;
    uint32_t thr_key;
};

int sampling_chunks(long long vocab);
size_t sampling_scratch_bytes(long long rows, long long vocab);

// The two halves of the calls below, for an LM head whose vocabulary is split over ranks: every rank runs
// sampling_partials over its slice (idx_offset = first token id of the slice), the partial blocks are
// exchanged, and the finish kernels merge `nslices` blocks that lie `slice_stride` entries apart.
int sampling_partials(cudaStream_t stream, const float* logits, long long row_stride, int rows, long long vocab,
                      float inv_temperature, bool want_sum, long long idx_offset, void* partials_out);
int argmax_finish(cudaStream_t stream, const void* partials, int chunks, int nslices, long long slice_stride, int rows,
                  long long* out_dev);
int accept_finish(cudaStream_t stream, const void* partials, int chunks, int nslices, long long slice_stride,
                  const float* logits, long long row_stride, long long vocab, float inv_temperature,
                  const long long* draft_tokens, const float* draft_probs, const float* uniforms, int batch,
                  int num_draft, int rows_per_seq, int bonus_row, AcceptOut* out_dev, const Nucleus* nucleus = nullptr);
// Per row: the nucleus of softmax(logits * inv_temperature) at top_p (nucleus_out, may be null) and, with uniforms,
// one token drawn from it (token ids to tok_out[row], its probability inside the nucleus to
// prob_out[row * prob_stride]).
int nucleus_rows(cudaStream_t stream, const float* logits, long long row_stride, int rows, long long vocab,
                 float inv_temperature, float top_p, const float* uniforms, int u_stride, Nucleus* nucleus_out,
                 long long* tok_out, float* prob_out, int prob_stride);

int argmax_rows(cudaStream_t stream, const float* logits, long long row_stride, int rows, long long vocab,
                void* scratch, long long* out_dev, float* partial_max, long long* partial_idx);

int accept_reject_batched(cudaStream_t stream, const float* logits, long long row_stride, long long vocab,
                          float inv_temperature, const long long* draft_tokens, const float* draft_probs,
                          const float* uniforms, int batch, int num_draft, int rows_per_seq, int bonus_row,
                          void* scratch, AcceptOut* out_dev);

int philox_uniform(cudaStream_t stream, float* out, long long n, unsigned long long seed, unsigned long long subseq);
// the subsequence read from device memory at run time (a counter that add_counter advances): graph-replay safe
int philox_uniform_counter(cudaStream_t stream, float* out, long long n, unsigned long long seed,
                           const unsigned long long* subseq_dev);
int add_counter(cudaStream_t stream, unsigned long long* counter_dev, unsigned long long v);
// One token per row from softmax(logits * inv_temperature) at the row's uniform (uniforms[row * u_stride]), from the
// partials of sampling_partials(..., want_sum = true): token ids to tok_out[row], probabilities to
// prob_out[row * prob_stride].
int sample_finish(cudaStream_t stream, const void* partials, int chunks, const float* logits, long long row_stride,
                  long long vocab, float inv_temperature, const float* uniforms, int u_stride, int rows, long long* tok_out,
                  float* prob_out, int prob_stride);

}  // namespace xb
