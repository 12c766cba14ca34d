// C interface of the bandwidth-bound kernels (elementwise.cu).  All tensors bf16 unless noted; every pointer must be
// 16-byte aligned and every row length a multiple of 8 elements.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Rows are addressed as base + (row / heads) * ld + (row % heads) * d; heads = 1 and ld = d is a plain [rows, d] tensor,
// heads > 1 normalises every head of a [tokens, heads * d (+ more)] buffer separately (QK-norm).
//   t = x (+ res if add_before); sum_out = t (optional, same layout as y); y = t * rstd * w (+ res if !add_before)
int ob_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd, long long rows,
                   int d, int heads, long long ld_x, long long ld_res, long long ld_y, int add_before, float eps,
                   cudaStream_t stream);
// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dsum, same layout as dx); dw (fp32) += dw_scale * sum_rows dy * xhat
int ob_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dsum, void* dx,
                   float* dw, long long rows, int d, int heads, long long ld_dy, long long ld_x, long long ld_dx,
                   float dw_scale, cudaStream_t stream);
// LayerNorm over plain [rows, d] tensors: y = (x - mean) * rstd * w (+ b); w / b may be null.  mean / rstd fp32 [rows].
int ob_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, long long rows,
                     int d, float eps, cudaStream_t stream);
// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = w * dy; dw / db (fp32, may be null) += scale * column sums
int ob_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                     float* dw, float* db, long long rows, int d, float scale, cudaStream_t stream);
// rotate-half RoPE on [B, S, H, D] with element strides; cos/sin fp32 [>= S + pos_offset, D/2]; sign -1 = backward
int ob_rope(const void* x, void* y, const float* cos_t, const float* sin_t, int B, int S, int H, int D, long long sb,
            long long ss, long long sh, long long ysb, long long yss, long long ysh, float sign, int pos_offset,
            cudaStream_t stream);
// y = rope(rmsnorm(x) * w) in one pass (q / k normalisation followed by the rotary embedding).  A row of d
// elements is d / hd heads; rows are addressed like ob_rmsnorm_fwd; the table row of a row is (row / heads) % S.
int ob_rmsnorm_rope_fwd(const void* x, const void* w, void* y, float* rstd, const float* cos_t, const float* sin_t,
                        long long rows, int d, int hd, int heads, long long ld_x, long long ld_y, int S, float eps,
                        cudaStream_t stream);
// backward of the fused op: the rotation's transpose, then the RMS-norm backward; dw (fp32) += dw_scale * ...
int ob_rmsnorm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                        const float* cos_t, const float* sin_t, long long rows, int d, int hd, int heads,
                        long long ld_dy, long long ld_x, long long ld_dx, int S, float dw_scale, cudaStream_t stream);
// a = act(g) * u with act = silu (gelu = 0) or tanh-gelu (gelu = 1)
int ob_glu_fwd(const void* g, const void* u, void* a, long long n, int gelu, cudaStream_t stream);
int ob_glu_bwd(const void* g, const void* u, const void* da, void* dg, void* du, void* a_out, long long n, int gelu,
               cudaStream_t stream);
// Embedding over n_shards row-shards of rows_per_shard rows each; `shards` / `grad_shards` are DEVICE arrays of
// pointers that may address peer GPUs' memory.  ids int64.  Gradients are fp32 and accumulated with red.add.
int ob_embed_gather(const long long* ids, const void* const* shards, int rows_per_shard, int n_shards, void* out,
                    long long tokens, int d, float scale, cudaStream_t stream);
int ob_embed_scatter(const long long* ids, float* const* grad_shards, int rows_per_shard, int n_shards,
                     const void* dout, long long tokens, int d, float scale, cudaStream_t stream);

// Small-tensor helpers over R shards whose base pointers (DEVICE array) may address peer GPUs (plain loads / red.add):
// gather 16-bit elements of every shard but `skip` into dst (shard r at dst + r*stride), and add a full fp32 vector
// into the shards that own its slices.
int ob_gather_shards(const void* const* src_shards, void* dst, long long stride, long long n_per_shard, int n_shards,
                     int skip, cudaStream_t stream);
int ob_scatter_add_shards(const float* src, float* const* dst_shards, long long n_per_shard, int n_shards, float scale,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
