// C++ launchers of the non-GEMM kernels (LayerNorm over column-sharded features, GeLU,
// AdamW, vocab-parallel cross-entropy, embedding, gradient norm).  All tensors are row-major;
// bf16 activations/parameters, fp32 statistics and optimizer state.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace msb {

// ---- exchange of a few floats per row among the GPUs of a mesh row ------------------------
// Replaces the `psum` over the mesh columns of ShardedLayers.py:129-131 (and of the vocabulary-
// parallel cross-entropy) by traffic inside the kernels around it.  The PRODUCING kernel (the
// statistics pass) writes its rows' partial values into its slot on EVERY GPU of the group (plain
// stores into peer memory) and, per CTA, bumps one arrival counter on every peer; the CONSUMING
// kernel (the apply pass) waits (bounded) until all CTAs of all peers have arrived and sums the n
// slots of a row in fixed order.  Producer and consumer are separate launches, so no CTA ever
// waits for a CTA that may not be resident.  Counters only grow; the host hands out the cumulative
// target and alternates between two slot / counter sets, so that a GPU that is one call ahead
// never overwrites slots that a slower peer is still reading.
constexpr int kExMaxPeers = 8;
struct RowExchange {
  int n;                            // GPUs in the group
  int me;                           // this GPU's index in the group
  float* dst[kExMaxPeers];          // GPU p's slot area for THIS GPU's contributions ([rows * width])
  const float* slots;               // local slot areas of all n sources
  int64_t stride;                   // floats between consecutive sources' areas
  uint32_t* counter[kExMaxPeers];   // GPU p's arrival counter
  const uint32_t* my_counter;
  uint32_t target;                  // value of my_counter once every CTA of every peer has arrived
  uint64_t timeout_ns;
  uint32_t* status;                 // [4]: 20 (LayerNorm fwd) / 21 (bwd) / 22 (cross-entropy), CTA, seen, wanted
};
// CTAs the LayerNorm kernels launch for `rows` rows of `cols` local columns (0: widest case): with an exchange
// every CTA of the producing pass counts one arrival, so the host needs this number for the consumers' targets.
int ln_grid(int backward, int rows, int cols = 0);

// ---- LayerNorm over a feature dimension that may be split across the mesh columns --------
// Replaces ShardedLayerNorm (ShardedLayers.py:123-138) plus the residual adds (:178,:184);
// unlike the reference the affine parameters are applied.
// mode 0: single GPU holds the whole feature dim: h = x (+ res); y = LN(h)*gamma + beta
// mode 1: first pass of the sharded case: h = x (+ res); stats[row] = (sum h, sum h^2)
// mode 2: second pass: y from h and the all-reduced stats
// With `exch`, mode 1 publishes the statistics to the GPUs of the mesh row and mode 2 reads them
// from there (stats is unused): no all-reduce in between.
// `h_out` may alias x; `res` and `h_out` may be null (no residual add: h == x).
// mean_rstd receives (mean, rstd) per row (modes 0 and 2).
cudaError_t ln_fwd(int mode, const void* x, const void* res, void* h_out, void* y,
                   const void* gamma, const void* beta, float* stats, float* mean_rstd,
                   int rows, int cols, int total_cols, float eps, cudaStream_t stream,
                   const RowExchange* exch = nullptr);

// Backward.  g = dy * gamma, xhat = (h - mean) * rstd.
// mode 0: everything local: dx = rstd * (g - mean_D(g) - xhat * mean_D(g * xhat)) (+ dres)
// mode 1: stats[row] = (sum g, sum g * xhat) over the local columns; also accumulates
//         dgamma / dbeta (fp32, atomically, must be zeroed by the caller)
// mode 2: dx from the all-reduced stats
// With `exch`, modes 1 and 2 exchange the sums as in ln_fwd.
// mode 0 accumulates dgamma / dbeta as mode 1 does.
cudaError_t ln_bwd(int mode, const void* dy, const void* h, const void* gamma,
                   const float* mean_rstd, const void* dres, void* dx, float* stats,
                   float* dgamma, float* dbeta, int rows, int cols, int total_cols,
                   cudaStream_t stream, const RowExchange* exch = nullptr);

// ---- GeLU (tanh approximation, the jax.nn.gelu default used at ShardedLayers.py:182) -----
cudaError_t gelu_fwd(const void* x, void* y, int64_t n, cudaStream_t stream);
cudaError_t gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, cudaStream_t stream);

// ---- elementwise add (bf16): out = a + b -------------------------------------------------
cudaError_t add_bf16(const void* a, const void* b, void* out, int64_t n, cudaStream_t stream);

// ---- AdamW over flat buffers -------------------------------------------------------------
// param (bf16) and master/m/v (fp32) are updated in place from grad (bf16 or fp32).
// grad_scale multiplies the gradient first (loss scaling / clipping).
cudaError_t adamw_step(void* param, float* master, float* m, float* v, const void* grad,
                       int grad_fp32, int64_t n, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float bias_corr1, float bias_corr2,
                       const float* grad_scale, cudaStream_t stream);

// out[0] += sum of squares of x (bf16 or fp32), fp32 atomics.
cudaError_t sumsq(const void* x, int is_fp32, int64_t n, float* out, cudaStream_t stream);

// ---- vocab-parallel softmax cross-entropy -------------------------------------------------
// logits: bf16 [rows, cols] = this GPU's vocabulary slice [col_offset, col_offset + cols);
// columns with global index >= vocab are padding and ignored.
// pass 1: row_max[row], row_sumexp[row] (relative to row_max), tgt_logit[row] (0 if the
//         target is not in this slice)
// With `exch` the three values per row go to every GPU of the mesh row instead (width 3).
cudaError_t ce_partial(const void* logits, int64_t ld, const int64_t* targets, int rows, int cols,
                       int col_offset, int vocab, float* row_max, float* row_sumexp,
                       float* tgt_logit, cudaStream_t stream, const RowExchange* exch = nullptr);
int ce_grid(int rows);   // CTAs of ce_partial (each counts one arrival in an exchange)
// pass 2: logits <- (softmax - onehot) * scale, in place, using the global max / sumexp.
// With `exch` the global max / sumexp are combined from the mesh row's published partials (gmax /
// gsumexp unused) and row_loss[row] = log(sumexp) + max - target logit is written when non-null.
cudaError_t ce_grad(void* logits, int64_t ld, const int64_t* targets, int rows, int cols,
                    int col_offset, int vocab, const float* gmax, const float* gsumexp,
                    float scale, cudaStream_t stream, float* row_loss = nullptr,
                    const RowExchange* exch = nullptr);

// ---- embedding ----------------------------------------------------------------------------
// out[t, :] = tok_table[token[t], :] + pos_table[t % seq, :]   (tables bf16 [*, cols])
cudaError_t embedding_fwd(const int64_t* tokens, const void* tok_table, const void* pos_table,
                          void* out, int n_tokens, int seq, int cols, cudaStream_t stream);
// dtok[token[t], :] += dout[t, :]; dpos[t % seq, :] += dout[t, :]   (fp32 accumulators)
cudaError_t embedding_bwd(const int64_t* tokens, const void* dout, float* dtok, float* dpos,
                          int n_tokens, int seq, int cols, cudaStream_t stream);

// out(bf16)[i] = (accumulate ? out[i] : 0) + in(fp32)[i]
cudaError_t cast_f32_to_bf16(const float* in, void* out, int64_t n, int accumulate,
                             cudaStream_t stream);

}  // namespace msb
