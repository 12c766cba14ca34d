// Cross-entropy over fp32 logits (fused forward + gradient, soft-cap, ignore_index, z-loss), fused fp32 AdamW over a
// flat shard (also writes the bf16 compute copy and can clear the gradient), squared-norm reduction and the clip
// coefficient, fp32 -> bf16 cast.
//
// Math follows the reference: cross entropy = -log_softmax(logits)[label], labels equal to ignore_index excluded
// from numerator and denominator (`olmax/nn/functional.py:70-121`); AdamW with bias correction, decoupled weight
// decay and eps outside the square root, gradient clipping g * max_norm / max(max_norm, |g|)
// (`olmax/optim/config.py:125-156`, `olmax/optim/utils.py:15-38`).
#include "optim_loss.h"
#include "host_common.h"
#include "sm100.cuh"

namespace ob {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return MaxSum{m, 0.f};
  return MaxSum{m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}

// One block per row.  logits fp32 [rows, ld]; dlogits bf16 [rows, ld_d] = d(mean loss)/d(logits) * grad_scale.
//   stats[0] += sum over valid rows of loss;  stats[1] += sum over valid rows of lse^2 (z-loss numerator)
//   inv_count: device float, 1 / (number of valid labels in the whole batch)
__global__ void __launch_bounds__(CE_THREADS)
    ce_fwd_bwd_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                      bf16* __restrict__ dlogits, long long ld_d, float* __restrict__ lse_out,
                      float* __restrict__ stats, const float* __restrict__ inv_count, int V, int ignore_index,
                      float softcap, float z_loss, float grad_scale) {
  __shared__ MaxSum red[CE_THREADS / 32];
  __shared__ MaxSum total;
  const long long row = blockIdx.x;
  const float* lrow = logits + row * ld;
  const long long label = labels[row];
  // `counted` rows enter the mean and the z-loss; only rows whose label is a real class have a cross-entropy term (the
  // one-hot of an out-of-range class is all zero: `olmax/nn/functional.py:94-121` of the reference)
  const bool counted = label != (long long)ignore_index;
  const bool in_range = counted && label >= 0 && label < V;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const int nvec = V / 4;
  MaxSum acc{-INFINITY, 0.f};
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float4 v = *reinterpret_cast<const float4*>(lrow + i * 4);
    float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float x = e[j];
      if (softcap > 0.f) x = softcap * tanh_fast(x * inv_cap);
      if (x > acc.m) {
        acc.s = acc.s * __expf(acc.m - x) + 1.f;
        acc.m = x;
      } else {
        acc.s += __expf(x - acc.m);
      }
    }
  }
  for (int i = nvec * 4 + threadIdx.x; i < V; i += CE_THREADS) {
    float x = lrow[i];
    if (softcap > 0.f) x = softcap * tanh_fast(x * inv_cap);
    acc = combine(acc, MaxSum{x, 1.f});
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    MaxSum o{__shfl_xor_sync(0xffffffffu, acc.m, off), __shfl_xor_sync(0xffffffffu, acc.s, off)};
    acc = combine(acc, o);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    MaxSum t = red[0];
    for (int i = 1; i < CE_THREADS / 32; ++i) t = combine(t, red[i]);
    total = t;
  }
  __syncthreads();
  const float lse = total.m + __logf(total.s);
  if (threadIdx.x == 0) {
    if (lse_out != nullptr) lse_out[row] = lse;
    if (in_range) {
      float tl = lrow[label];
      if (softcap > 0.f) tl = softcap * tanh_fast(tl * inv_cap);
      atomicAdd(&stats[0], lse - tl);
    }
    if (counted) atomicAdd(&stats[1], lse * lse);
  }
  if (dlogits == nullptr) return;
  bf16* drow = dlogits + row * ld_d;
  // d/dz of [ (lse - z_label) + z_loss * lse^2 ] / count  = softmax * (1 + 2 z_loss lse) - onehot, all / count
  const float gs = in_range ? grad_scale * (*inv_count) : 0.f;
  const float gz = counted ? grad_scale * (*inv_count) * 2.f * z_loss * lse : 0.f;
  const float sm_scale = gs + gz;
  const int nvec8 = V / 8;
  for (int i = threadIdx.x; i < nvec8; i += CE_THREADS) {
    const float4 a = *reinterpret_cast<const float4*>(lrow + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(lrow + i * 8 + 4);
    float e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float x = e[j], dcap = 1.f;
      if (softcap > 0.f) {
        const float t = tanh_fast(x * inv_cap);
        x = softcap * t;
        dcap = 1.f - t * t;
      }
      float g = __expf(x - lse) * sm_scale;
      if ((long long)(i * 8 + j) == label) g -= gs;
      o[j] = g * dcap;
    }
    uint4 pk;
    pk.x = pack_bf16x2(o[0], o[1]);
    pk.y = pack_bf16x2(o[2], o[3]);
    pk.z = pack_bf16x2(o[4], o[5]);
    pk.w = pack_bf16x2(o[6], o[7]);
    *reinterpret_cast<uint4*>(drow + i * 8) = pk;
  }
  for (int i = nvec8 * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float x = lrow[i], dcap = 1.f;
    if (softcap > 0.f) {
      const float t = tanh_fast(x * inv_cap);
      x = softcap * t;
      dcap = 1.f - t * t;
    }
    float g = __expf(x - lse) * sm_scale;
    if ((long long)i == label) g -= gs;
    drow[i] = __float2bfloat16(g * dcap);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Vocabulary-parallel cross entropy: every member of a group holds the logits of ITS slice of the vocabulary
// ([rows, V_local], global class = vocab_offset + column) for the same rows.
//   stats kernel: per row (max, sum exp(z - max), target logit if the label falls in this slice else 0) of the local slice;
//   grad kernel:  reads every member's statistics (plain loads; the buffers may live in peer GPUs' memory), combines
//                 them into the row's global log-sum-exp and target logit, and writes d(loss)/d(local logits).
// Rows come from `n_src` sources (the members' own token shards, `rows_per_src` rows each); a row is normalised by the
// number of counted labels of its source, and a member adds to its loss sums only the rows of its own source.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(CE_THREADS)
    ce_vp_stats_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                       float* __restrict__ stats, int V, long long vocab_offset, float softcap) {
  __shared__ MaxSum red[CE_THREADS / 32];
  const long long row = blockIdx.x;
  const float* lrow = logits + row * ld;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  MaxSum acc{-INFINITY, 0.f};
  for (int i = threadIdx.x; i < V; i += CE_THREADS) {
    float x = lrow[i];
    if (softcap > 0.f) x = softcap * tanh_fast(x * inv_cap);
    acc = combine(acc, MaxSum{x, 1.f});
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    MaxSum o{__shfl_xor_sync(0xffffffffu, acc.m, off), __shfl_xor_sync(0xffffffffu, acc.s, off)};
    acc = combine(acc, o);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    MaxSum t = red[0];
    for (int i = 1; i < CE_THREADS / 32; ++i) t = combine(t, red[i]);
    const long long local = labels[row] - vocab_offset;
    float tl = 0.f;
    if (local >= 0 && local < V) {
      tl = lrow[local];
      if (softcap > 0.f) tl = softcap * tanh_fast(tl * inv_cap);
    }
    float4 out = make_float4(t.m, t.s, tl, 0.f);
    *reinterpret_cast<float4*>(stats + row * 4) = out;
  }
}

__global__ void __launch_bounds__(CE_THREADS)
    ce_vp_grad_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                      bf16* __restrict__ dlogits, long long ld_d, const float* const* __restrict__ peer_stats, int n_peers,
                      const float* __restrict__ inv_counts, long long rows_per_src, long long row0, int my_src,
                      float* __restrict__ loss_sums, int V, long long vocab_offset, long long V_total, int ignore_index,
                      float softcap, float z_loss, float grad_scale) {
  __shared__ float sh[3];
  const long long row = blockIdx.x;
  const float* lrow = logits + row * ld;
  const long long label = labels[row];
  const bool counted = label != (long long)ignore_index;
  const bool in_range = counted && label >= 0 && label < V_total;
  if (threadIdx.x == 0) {
    float m = -INFINITY;
    for (int r = 0; r < n_peers; ++r) m = fmaxf(m, peer_stats[r][row * 4]);
    float ssum = 0.f, t = 0.f;
    for (int r = 0; r < n_peers; ++r) {
      const float4 st = *reinterpret_cast<const float4*>(peer_stats[r] + row * 4);
      ssum += st.y * __expf(st.x - m);
      t += st.z;
    }
    const float lse = m + __logf(ssum);
    const int src = (int)((row0 + row) / rows_per_src);
    sh[0] = lse;
    sh[1] = inv_counts[src];
    if (src == my_src) {
      if (in_range) atomicAdd(&loss_sums[0], lse - t);
      if (counted) atomicAdd(&loss_sums[1], lse * lse);
    }
  }
  __syncthreads();
  if (dlogits == nullptr) return;
  const float lse = sh[0];
  const float gs = in_range ? grad_scale * sh[1] : 0.f;
  const float gz = counted ? grad_scale * sh[1] * 2.f * z_loss * lse : 0.f;
  const float sm_scale = gs + gz;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const long long local_label = label - vocab_offset;
  bf16* drow = dlogits + row * ld_d;
  for (int i = threadIdx.x; i < V; i += CE_THREADS) {
    float x = lrow[i], dcap = 1.f;
    if (softcap > 0.f) {
      const float t = tanh_fast(x * inv_cap);
      x = softcap * t;
      dcap = 1.f - t * t;
    }
    float g = __expf(x - lse) * sm_scale;
    if ((long long)i == local_label) g -= gs;
    drow[i] = __float2bfloat16(g * dcap);
  }
}

// out[0] = 1 / max(1, #labels != ignore_index), out[1] = that count
__global__ void count_valid_kernel(const long long* __restrict__ labels, long long n, int ignore_index, int V,
                                   float* __restrict__ out, int* __restrict__ counter) {
  int local = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long l = labels[i];
    local += (l != (long long)ignore_index) ? 1 : 0;  // out-of-range labels still count in the mean
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
  if ((threadIdx.x & 31) == 0 && local) atomicAdd(&counter[0], local);
  __syncthreads();
  __threadfence();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&counter[1], 1);
    if (done == (int)gridDim.x - 1) {
      const int c = atomicAdd(&counter[0], 0);
      out[0] = 1.f / (float)(c > 0 ? c : 1);
      out[1] = (float)c;
      counter[0] = 0;
      counter[1] = 0;
    }
  }
}

// p, m, v, g: fp32 [n]; shadow: bf16 [n] (optional).  g_eff = g * (*gscale) (gscale optional, device scalar).
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ g,
                             bf16* __restrict__ shadow, long long n, float lr, float b1, float b2, float eps, float wd,
                             float inv_bc1, float inv_bc2, const float* __restrict__ gscale, int zero_grad) {
  const float gs = gscale != nullptr ? *gscale : 1.f;
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    // streaming accesses: nothing of the optimizer state is read again before it has left the L2
    float4 pv = __ldcs(reinterpret_cast<const float4*>(p) + i);
    float4 mv = __ldcs(reinterpret_cast<const float4*>(m) + i);
    float4 vv = __ldcs(reinterpret_cast<const float4*>(v) + i);
    float4 gv = __ldcs(reinterpret_cast<const float4*>(g) + i);
    float pa[4] = {pv.x, pv.y, pv.z, pv.w}, ma[4] = {mv.x, mv.y, mv.z, mv.w}, va[4] = {vv.x, vv.y, vv.z, vv.w},
          ga[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gg = ga[j] * gs;
      ma[j] = b1 * ma[j] + (1.f - b1) * gg;
      va[j] = b2 * va[j] + (1.f - b2) * gg * gg;
      const float mh = ma[j] * inv_bc1, vh = va[j] * inv_bc2;
      pa[j] -= lr * (mh / (sqrtf(vh) + eps) + wd * pa[j]);
    }
    __stcs(reinterpret_cast<float4*>(p) + i, make_float4(pa[0], pa[1], pa[2], pa[3]));
    __stcs(reinterpret_cast<float4*>(m) + i, make_float4(ma[0], ma[1], ma[2], ma[3]));
    __stcs(reinterpret_cast<float4*>(v) + i, make_float4(va[0], va[1], va[2], va[3]));
    if (zero_grad) __stcs(reinterpret_cast<float4*>(g) + i, make_float4(0.f, 0.f, 0.f, 0.f));
    if (shadow != nullptr) {
      uint2 s;
      s.x = pack_bf16x2(pa[0], pa[1]);
      s.y = pack_bf16x2(pa[2], pa[3]);
      __stcs(reinterpret_cast<uint2*>(shadow) + i, s);
    }
  }
  // tail (n not a multiple of 4)
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gg = g[i] * gs;
    const float mm = b1 * m[i] + (1.f - b1) * gg;
    const float vv2 = b2 * v[i] + (1.f - b2) * gg * gg;
    float pp = p[i];
    pp -= lr * ((mm * inv_bc1) / (sqrtf(vv2 * inv_bc2) + eps) + wd * pp);
    p[i] = pp; m[i] = mm; v[i] = vv2;
    if (zero_grad) g[i] = 0.f;
    if (shadow != nullptr) shadow[i] = __float2bfloat16(pp);
  }
}

__global__ void sumsq_kernel(const float* __restrict__ x, long long n, double* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    acc += x[i] * x[i];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    if (threadIdx.x == 0) atomicAdd(out, (double)t);
  }
}

// norm = sqrt(sumsq) * pre_scale; coef = pre_scale * (max_norm > 0 ? max_norm / max(max_norm, norm) : 1)
__global__ void clip_coef_kernel(const double* __restrict__ sumsq, float max_norm, float pre_scale,
                                 float* __restrict__ out) {
  const float norm = (float)sqrt(*sumsq) * pre_scale;
  float coef = pre_scale;
  if (max_norm > 0.f) coef *= max_norm / fmaxf(max_norm, norm);
  out[0] = coef;
  out[1] = norm;
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long long n) {
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 s;
    s.x = pack_bf16x2(v.x, v.y);
    s.y = pack_bf16x2(v.z, v.w);
    reinterpret_cast<uint2*>(dst)[i] = s;
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

static inline int blocks_for(long long items, int threads, int per_sm) {
  long long b = (items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * per_sm;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace ob

using namespace ob;

extern "C" int ob_ce_fwd_bwd(const float* logits, long long ld, const long long* labels, void* dlogits, long long ld_d,
                             float* lse_out, float* stats, const float* inv_count, long long rows, int V,
                             int ignore_index, float softcap, float z_loss, float grad_scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (ld % 4 != 0 || (dlogits != nullptr && ld_d % 8 != 0)) OB_FAIL(-1, "cross entropy: row strides must be multiples of 4 (fp32) / 8 (bf16)");
  ce_fwd_bwd_kernel<<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, ld, labels, (bf16*)dlogits, ld_d, lse_out, stats,
                                                              inv_count, V, ignore_index, softcap, z_loss, grad_scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_count_valid(const long long* labels, long long n, int ignore_index, int V, float* out, int* counter,
                              cudaStream_t stream) {
  count_valid_kernel<<<blocks_for(n, 256, 2), 256, 0, stream>>>(labels, n, ignore_index, V, out, counter);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_ce_vp_stats(const float* logits, long long ld, const long long* labels, float* stats, long long rows,
                              int V, long long vocab_offset, float softcap, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(stats) & 15) OB_FAIL(-3, "vocab-parallel statistics need a 16-byte aligned buffer");
  ce_vp_stats_kernel<<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, ld, labels, stats, V, vocab_offset, softcap);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_ce_vp_grad(const float* logits, long long ld, const long long* labels, void* dlogits, long long ld_d,
                             const float* const* peer_stats, int n_peers, const float* inv_counts, long long rows_per_src,
                             long long row0, int my_src, float* loss_sums, long long rows, int V, long long vocab_offset,
                             long long V_total, int ignore_index, float softcap, float z_loss, float grad_scale,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (n_peers < 1 || rows_per_src <= 0) OB_FAIL(-3, "vocab-parallel loss: bad group description");
  ce_vp_grad_kernel<<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, ld, labels, reinterpret_cast<bf16*>(dlogits), ld_d,
                                                              peer_stats, n_peers, inv_counts, rows_per_src, row0, my_src,
                                                              loss_sums, V, vocab_offset, V_total, ignore_index, softcap,
                                                              z_loss, grad_scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_adamw(float* p, float* m, float* v, float* g, void* shadow, long long n, float lr, float b1, float b2,
                        float eps, float wd, float bias_corr1, float bias_corr2, const float* gscale, int zero_grad,
                        cudaStream_t stream) {
  if (n <= 0) return 0;
  adamw_kernel<<<blocks_for((n + 3) / 4, 256, 8), 256, 0, stream>>>(p, m, v, g, (bf16*)shadow, n, lr, b1, b2, eps, wd,
                                                                    1.f / bias_corr1, 1.f / bias_corr2, gscale, zero_grad);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_sumsq(const float* x, long long n, double* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<blocks_for((n + 3) / 4, 256, 8), 256, 0, stream>>>(x, n, out);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_clip_coef(const double* sumsq, float max_norm, float pre_scale, float* out, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, pre_scale, out);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<blocks_for((n + 3) / 4, 256, 8), 256, 0, stream>>>(src, (bf16*)dst, n);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}
