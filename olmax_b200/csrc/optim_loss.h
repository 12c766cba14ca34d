// C interface of the loss / optimizer kernels (optim_loss.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Fused cross-entropy forward + gradient over fp32 logits [rows, V] (row stride ld).  labels int64; rows whose
// label equals ignore_index (or is out of range) contribute neither loss nor gradient.
//   stats[0] += sum of per-row losses, stats[1] += sum of lse^2 over valid rows
//   dlogits (bf16, row stride ld_d, may be null) = grad_scale * (*inv_count) * d(sum loss + z_loss * sum lse^2)/dlogits
//   softcap > 0: logits are first mapped to softcap * tanh(logits / softcap)
int ob_ce_fwd_bwd(const float* logits, long long ld, const long long* labels, void* dlogits, long long ld_d,
                  float* lse_out, float* stats, const float* inv_count, long long rows, int V, int ignore_index,
                  float softcap, float z_loss, float grad_scale, cudaStream_t stream);
// out[0] = 1 / max(1, count), out[1] = count of labels that are valid; counter: zero-initialised device int[2]
int ob_count_valid(const long long* labels, long long n, int ignore_index, int V, float* out, int* counter,
                   cudaStream_t stream);
// Vocabulary-parallel cross entropy (each member of a group holds the logits of its vocabulary slice for the same
// rows; see optim_loss.cu).  stats: [rows, 4] floats (max, sum exp, target logit, unused), 16-byte aligned.
int ob_ce_vp_stats(const float* logits, long long ld, const long long* labels, float* stats, long long rows, int V,
                   long long vocab_offset, float softcap, cudaStream_t stream);
// peer_stats: DEVICE array of the n_peers members' statistics buffers for these rows (peer memory allowed: plain loads);
// inv_counts[src] = 1 / counted labels of source `src`; row r of the chunk is row (row0 + r) of the gathered batch and
// belongs to source (row0 + r) / rows_per_src; loss_sums[0] += lse - target, loss_sums[1] += lse^2 over the rows of
// source my_src.  dlogits (bf16, may be null) = d(loss) / d(local logits) * grad_scale.
int ob_ce_vp_grad(const float* logits, long long ld, const long long* labels, void* dlogits, long long ld_d,
                  const float* const* peer_stats, int n_peers, const float* inv_counts, long long rows_per_src,
                  long long row0, int my_src, float* loss_sums, long long rows, int V, long long vocab_offset,
                  long long V_total, int ignore_index, float softcap, float z_loss, float grad_scale, cudaStream_t stream);
// AdamW on a flat fp32 shard; g_eff = g * (*gscale) when gscale (device scalar) is given.  bias_corr = 1 - beta^t.
// Also writes the bf16 copy `shadow` (optional) and clears g when zero_grad != 0.
int ob_adamw(float* p, float* m, float* v, float* g, void* shadow, long long n, float lr, float b1, float b2, float eps,
             float wd, float bias_corr1, float bias_corr2, const float* gscale, int zero_grad, cudaStream_t stream);
// *out (double, device) += sum x^2
int ob_sumsq(const float* x, long long n, double* out, cudaStream_t stream);
// out[1] = norm = sqrt(*sumsq) * pre_scale; out[0] = pre_scale * (max_norm > 0 ? max_norm / max(max_norm, norm) : 1)
int ob_clip_coef(const double* sumsq, float max_norm, float pre_scale, float* out, cudaStream_t stream);
int ob_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
