// Bandwidth-bound kernels of the train step for sm_100a: RMSNorm forward/backward (with fused residual adds and a
// strided "per-head" addressing mode for QK-norm), rotary embedding, gated-MLP activation forward/backward,
// embedding gather / gradient scatter over (possibly peer-resident) vocabulary shards.
//
// All kernels move 16 bytes per thread per access, keep the row in registers between the reduction and the
// normalisation (one read, one write of every tensor), and compute in fp32 with bf16 storage, matching the
// reference's "upcast, compute, cast back" rule (`olmax/nn/functional.py:51-67`, `olmax/nn/rope.py:99-115`,
// `olmax/nn/mlp.py:69-73`, `olmax/nn/embedding.py:30-32`).
#include "elementwise.h"
#include "host_common.h"
#include "sm100.cuh"

namespace ob {

struct __align__(16) bf16x8 {
  uint32_t v[4];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const bf16x8 raw = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(raw.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 load_raw8(const bf16* p) { return *reinterpret_cast<const bf16x8*>(p); }
__device__ __forceinline__ void unpack8(const bf16x8& raw, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(raw.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  bf16x8 raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) raw.v[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = raw;
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Sum over the TPR threads that share a row (TPR = 16 or 32: shuffles; TPR = 256: shuffles + shared memory).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* red) {
  if (TPR <= 32) {
#pragma unroll
    for (int off = TPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
  } else {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < TPR / 32; ++i) t += red[i];
    return t;
  }
}

constexpr int NORM_THREADS = 256;
constexpr int MAX_VPT = 4;  // most 8-element vectors per thread kept in registers (kernels are instantiated for 1, 2, 4)

// Rows are addressed as  base + (row / heads) * ld + (row % heads) * d   (heads = 1, ld = d: plain 2-D tensor).
__device__ __forceinline__ long long row_offset(long long row, int heads, long long ld, int d) {
  return heads == 1 ? row * ld : (row / heads) * ld + (row % heads) * (long long)d;
}

// t = x (+ res if add_before);  sum_out = t (optional);  y = t * rstd * w (+ res if !add_before and res given)
// The elements of the NEXT row group are fetched (as raw bf16) before the current one is reduced, so that loads stay
// in flight across the two barriers of the block-wide sum.
template <int TPR, int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
    rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const bf16* __restrict__ w,
                       bf16* __restrict__ y, bf16* __restrict__ sum_out, float* __restrict__ rstd_out, long long rows,
                       int d, int heads, long long ld_x, long long ld_res, long long ld_y, int add_before, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  constexpr int ROWS_PER_BLOCK = NORM_THREADS / TPR;
  const int sub = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int nvec = d / 8;
  const long long stride = (long long)gridDim.x * ROWS_PER_BLOCK;
  const bool with_res = res != nullptr;
  bf16x8 nx[VPT], nr[VPT];
  auto fetch = [&](long long row0) {
    const long long row = row0 + sub;
    if (row < rows) {
      const long long ox = row_offset(row, heads, ld_x, d), ores = row_offset(row, heads, ld_res, d);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tr + i * TPR;
        if (vi < nvec) {
          nx[i] = load_raw8(x + ox + vi * 8);
          if (with_res) nr[i] = load_raw8(res + ores + vi * 8);
        }
      }
    }
  };
  long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK;
  if (row0 < rows) fetch(row0);
  for (; row0 < rows; row0 += stride) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long oy = live ? row_offset(row, heads, ld_y, d) : 0;
    float t[VPT][8];
    bf16x8 cr[VPT];   // this row's residual, raw (the fetch below overwrites nr)
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        unpack8(nx[i], t[i]);
        if (with_res) cr[i] = nr[i];
        if (with_res && add_before) {
          float r[8];
          unpack8(cr[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) t[i][j] = __bfloat162float(__float2bfloat16(t[i][j] + r[j]));
          if (sum_out != nullptr) store8(sum_out + oy + vi * 8, t[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += t[i][j] * t[i][j];
      }
    }
    if (row0 + stride < rows) fetch(row0 + stride);
    ss = row_sum<TPR>(ss, red);
    const float rstd = rsqrtf(ss / (float)d + eps);
    if (live && tr == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        float wv[8], o[8];
        load8(w + vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = t[i][j] * rstd * wv[j];
        if (with_res && !add_before) {
          float r[8];
          unpack8(cr[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = __bfloat162float(__float2bfloat16(o[j])) + r[j];
        }
        store8(y + oy + vi * 8, o);
      }
    }
  }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dsum);  dw += sum_rows dy * xhat  (fp32 atomics, accumulating)
// (next row group fetched before the current one is reduced, as in the forward kernel)
template <int TPR, int VPT>
__global__ void __launch_bounds__(NORM_THREADS, VPT <= 1 ? 4 : (VPT <= 2 ? 3 : 2))
    rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                       const float* __restrict__ rstd_in, const bf16* __restrict__ dsum, bf16* __restrict__ dx,
                       float* __restrict__ dw, long long rows, int d, int heads, long long ld_dy, long long ld_x,
                       long long ld_dx, float dw_scale) {
  __shared__ float red[NORM_THREADS / 32];
  extern __shared__ float dw_part[];  // [d] per-block partial of dw
  constexpr int ROWS_PER_BLOCK = NORM_THREADS / TPR;
  const int sub = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int nvec = d / 8;
  const long long stride = (long long)gridDim.x * ROWS_PER_BLOCK;
  float dwacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  bf16x8 ng[VPT], nx[VPT];
  float nrstd = 0.f;
  auto fetch = [&](long long row0) {
    const long long row = row0 + sub;
    if (row < rows) {
      const long long ody = row_offset(row, heads, ld_dy, d), ox = row_offset(row, heads, ld_x, d);
      nrstd = rstd_in[row];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tr + i * TPR;
        if (vi < nvec) {
          ng[i] = load_raw8(dy + ody + vi * 8);
          nx[i] = load_raw8(x + ox + vi * 8);
        }
      }
    }
  };
  long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK;
  if (row0 < rows) fetch(row0);
  for (; row0 < rows; row0 += stride) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long odx = live ? row_offset(row, heads, ld_dx, d) : 0;
    const float rstd = live ? nrstd : 0.f;
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        float wv[8];
        unpack8(ng[i], g[i]);
        unpack8(nx[i], xh[i]);
        load8(w + vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          dwacc[i][j] += g[i][j] * xh[i][j];
          g[i][j] *= wv[j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    if (row0 + stride < rows) fetch(row0 + stride);
    dot = row_sum<TPR>(dot, red) / (float)d;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (dsum != nullptr) {
          float e[8];
          load8(dsum + odx + vi * 8, e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        store8(dx + odx + vi * 8, o);
      }
    }
  }
  if (dw == nullptr) return;
  // combine the row groups of this block in shared memory, then one atomic per element per block
  for (int i = threadIdx.x; i < d; i += NORM_THREADS) dw_part[i] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tr + i * TPR;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (ROWS_PER_BLOCK > 1) atomicAdd(&dw_part[vi * 8 + j], dwacc[i][j]);
        else dw_part[vi * 8 + j] = dwacc[i][j];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += NORM_THREADS) atomicAdd(dw + i, dw_part[i] * dw_scale);
}

// LayerNorm (`olmax/nn/functional.py:30-49`): y = (x - mean) * rstd * w (+ b), statistics over the row in fp32 (the
// variance is taken around the mean from the registers that hold the row, not as E[x^2] - mean^2).
template <int TPR, int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
    layernorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                         bf16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                         long long rows, int d, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  constexpr int ROWS_PER_BLOCK = NORM_THREADS / TPR;
  const int sub = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int nvec = d / 8;
  for (long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK; row0 < rows; row0 += (long long)gridDim.x * ROWS_PER_BLOCK) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long off = live ? row * (long long)d : 0;
    float t[VPT][8];
    float s1 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        load8(x + off + vi * 8, t[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s1 += t[i][j];
      }
    }
    const float mean = row_sum<TPR>(s1, red) / (float)d;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          t[i][j] -= mean;
          s2 += t[i][j] * t[i][j];
        }
      }
    }
    const float rstd = rsqrtf(row_sum<TPR>(s2, red) / (float)d + eps);
    if (live && tr == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        float wv[8], o[8];
        if (w != nullptr) load8(w + vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = t[i][j] * rstd * (w != nullptr ? wv[j] : 1.f);
        if (b != nullptr) {
          float bv[8];
          load8(b + vi * 8, bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += bv[j];
        }
        store8(y + off + vi * 8, o);
      }
    }
  }
}

// g = w*dy;  dx = rstd * (g - mean(g) - xhat * mean(g*xhat));  dw += scale * sum_rows dy*xhat;  db += scale * sum_rows dy
template <int TPR, int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
    layernorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                         const float* __restrict__ mean_in, const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                         float* __restrict__ dw, float* __restrict__ db, long long rows, int d, float scale) {
  __shared__ float red[NORM_THREADS / 32];
  extern __shared__ float part[];  // [2][d] per-block partials of dw and db
  constexpr int ROWS_PER_BLOCK = NORM_THREADS / TPR;
  const int sub = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int nvec = d / 8;
  float dwacc[VPT][8], dbacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = dbacc[i][j] = 0.f;
  for (long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK; row0 < rows; row0 += (long long)gridDim.x * ROWS_PER_BLOCK) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long off = live ? row * (long long)d : 0;
    const float mean = live ? mean_in[row] : 0.f;
    const float rstd = live ? rstd_in[row] : 0.f;
    float g[VPT][8], xh[VPT][8];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        float wv[8];
        load8(dy + off + vi * 8, g[i]);
        load8(x + off + vi * 8, xh[i]);
        if (w != nullptr) load8(w + vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          dwacc[i][j] += g[i][j] * xh[i][j];
          dbacc[i][j] += g[i][j];
          if (w != nullptr) g[i][j] *= wv[j];
          sg += g[i][j];
          sgx += g[i][j] * xh[i][j];
        }
      }
    }
    sg = row_sum<TPR>(sg, red) / (float)d;
    sgx = row_sum<TPR>(sgx, red) / (float)d;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (live && vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - sg - xh[i][j] * sgx);
        store8(dx + off + vi * 8, o);
      }
    }
  }
  if (dw == nullptr && db == nullptr) return;
  for (int i = threadIdx.x; i < 2 * d; i += NORM_THREADS) part[i] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tr + i * TPR;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&part[vi * 8 + j], dwacc[i][j]);
        atomicAdd(&part[d + vi * 8 + j], dbacc[i][j]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += NORM_THREADS) {
    if (dw != nullptr) atomicAdd(dw + i, part[i] * scale);
    if (db != nullptr) atomicAdd(db + i, part[d + i] * scale);
  }
}

// Rotary embedding, rotate-half convention: out = x * cos + rotate_half(x) * sin, cos/sin tables [S, D/2] fp32.
// sign = +1 forward, -1 backward (the transpose of a rotation).  One thread per 8 elements of the first half.
__global__ void rope_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int B, int S, int H, int D, long long sb, long long ss,
                            long long sh, long long ysb, long long yss, long long ysh, float sign, int pos_offset) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const long long total = (long long)B * S * H * vec_per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int vi = (int)(idx % vec_per_head);
    const int h = (int)((idx / vec_per_head) % H);
    const int s = (int)((idx / ((long long)vec_per_head * H)) % S);
    const int b = (int)(idx / ((long long)vec_per_head * H * S));
    const bf16* px = x + b * sb + s * ss + h * sh + vi * 8;
    bf16* py = y + b * ysb + s * yss + h * ysh + vi * 8;
    float lo[8], hi[8], c[8], sn[8], olo[8], ohi[8];
    load8(px, lo);
    load8(px + half, hi);
    load8f(cos_t + (long long)(s + pos_offset) * half + vi * 8, c);
    load8f(sin_t + (long long)(s + pos_offset) * half + vi * 8, sn);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = sn[j] * sign;
      olo[j] = lo[j] * c[j] - hi[j] * sj;
      ohi[j] = hi[j] * c[j] + lo[j] * sj;
    }
    store8(py, olo);
    store8(py + half, ohi);
  }
}

// q / k normalisation fused with the rotary embedding:  y = rope(rmsnorm(x) * w).
// A row (d elements, the span of one RMS statistic) is d / hd heads of hd elements: d == hd for a head-wise norm,
// d == n_heads * hd for a norm over the whole projection.  A thread owns PPT "pairs": 8 elements of the first half
// of a head and the 8 elements of the second half that rotate with them, so the rotation needs no exchange.
// Position of a row on the table axis: (row / heads) % S.  The normalised value stays in fp32 until the rotation is
// done (the two separate kernels round it to bf16 in between).  Replaces the q_norm / k_norm + rotary sequence of
// `olmax/nn/attention.py:270-300` for RMS norms.
// Both kernels fetch the NEXT row group's elements (as raw bf16, 4 registers per 8 elements) before they reduce the
// current one: the block-wide sum costs two barriers per row, and without loads in flight across them the kernel
// runs at the latency of a row, not at the memory bandwidth.
template <int TPR, int PPT>
__global__ void __launch_bounds__(NORM_THREADS)
    rmsnorm_rope_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                            float* __restrict__ rstd_out, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long rows, int d, int hd, int heads, long long ld_x,
                            long long ld_y, int S, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  constexpr int ROWS_PER_BLOCK = NORM_THREADS / TPR;
  const int sub = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int half = hd / 2, pph = hd / 16, npair = d / 16;
  const long long stride = (long long)gridDim.x * ROWS_PER_BLOCK;
  int e_of[PPT];
#pragma unroll
  for (int i = 0; i < PPT; ++i) {
    const int pi = tr + i * TPR;
    e_of[i] = pi < npair ? (pi / pph) * hd + (pi % pph) * 8 : -1;
  }
  bf16x8 nlo[PPT], nhi[PPT];
  auto fetch = [&](long long row0) {
    const long long row = row0 + sub;
    if (row < rows) {
      const long long ox = row_offset(row, heads, ld_x, d);
#pragma unroll
      for (int i = 0; i < PPT; ++i)
        if (e_of[i] >= 0) {
          nlo[i] = load_raw8(x + ox + e_of[i]);
          nhi[i] = load_raw8(x + ox + e_of[i] + half);
        }
    }
  };
  long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK;
  if (row0 < rows) fetch(row0);
  for (; row0 < rows; row0 += stride) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long oy = live ? row_offset(row, heads, ld_y, d) : 0;
    const unsigned pos = live ? ((unsigned)row / (unsigned)heads) % (unsigned)S : 0u;   // rows < 2^31 (checked by the launcher)
    float lo[PPT][8], hi[PPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      if (live && e_of[i] >= 0) {
        unpack8(nlo[i], lo[i]);
        unpack8(nhi[i], hi[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += lo[i][j] * lo[i][j] + hi[i][j] * hi[i][j];
      }
    }
    if (row0 + stride < rows) fetch(row0 + stride);
    ss = row_sum<TPR>(ss, red);
    const float rstd = rsqrtf(ss / (float)d + eps);
    if (live && tr == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      if (live && e_of[i] >= 0) {
        const int e = e_of[i], c0 = e % hd;   // e % hd < half: the pair's position inside the head's first half
        float wl[8], wh[8], c[8], sn[8], olo[8], ohi[8];
        load8(w + e, wl);
        load8(w + e + half, wh);
        load8f(cos_t + (size_t)pos * half + c0, c);
        load8f(sin_t + (size_t)pos * half + c0, sn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float nl = lo[i][j] * rstd * wl[j], nh = hi[i][j] * rstd * wh[j];
          olo[j] = nl * c[j] - nh * sn[j];
          ohi[j] = nh * c[j] + nl * sn[j];
        }
        store8(y + oy + e, olo);
        store8(y + oy + e + half, ohi);
      }
    }
  }
}

// Backward of the fused op: g = rope^T(dy), then the RMS-norm backward with g as the incoming gradient.
template <int TPR, int PPT>
__global__ void __launch_bounds__(NORM_THREADS, PPT <= 1 ? 3 : 2)
    rmsnorm_rope_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                            const float* __restrict__ rstd_in, bf16* __restrict__ dx, float* __restrict__ dw,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, long long rows, int d,
                            int hd, int heads, long long ld_dy, long long ld_x, long long ld_dx, int S,
                            float dw_scale) {
  __shared__ float red[NORM_THREADS / 32];
  extern __shared__ float dw_part[];  // [d] per-block partial of dw
  constexpr int ROWS_PER_BLOCK = NORM_THREADS / TPR;
  const int sub = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int half = hd / 2, pph = hd / 16, npair = d / 16;
  const long long stride = (long long)gridDim.x * ROWS_PER_BLOCK;
  int e_of[PPT];
#pragma unroll
  for (int i = 0; i < PPT; ++i) {
    const int pi = tr + i * TPR;
    e_of[i] = pi < npair ? (pi / pph) * hd + (pi % pph) * 8 : -1;
  }
  float dwl[PPT][8], dwh[PPT][8];
#pragma unroll
  for (int i = 0; i < PPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwl[i][j] = dwh[i][j] = 0.f;
  bf16x8 ndl[PPT], ndh[PPT], nxl[PPT], nxh[PPT];
  float nrstd = 0.f;
  auto fetch = [&](long long row0) {
    const long long row = row0 + sub;
    if (row < rows) {
      const long long ody = row_offset(row, heads, ld_dy, d), ox = row_offset(row, heads, ld_x, d);
      nrstd = rstd_in[row];
#pragma unroll
      for (int i = 0; i < PPT; ++i)
        if (e_of[i] >= 0) {
          ndl[i] = load_raw8(dy + ody + e_of[i]);
          ndh[i] = load_raw8(dy + ody + e_of[i] + half);
          nxl[i] = load_raw8(x + ox + e_of[i]);
          nxh[i] = load_raw8(x + ox + e_of[i] + half);
        }
    }
  };
  long long row0 = (long long)blockIdx.x * ROWS_PER_BLOCK;
  if (row0 < rows) fetch(row0);
  for (; row0 < rows; row0 += stride) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long odx = live ? row_offset(row, heads, ld_dx, d) : 0;
    const unsigned pos = live ? ((unsigned)row / (unsigned)heads) % (unsigned)S : 0u;   // rows < 2^31 (checked by the launcher)
    const float rstd = live ? nrstd : 0.f;
    float gl[PPT][8], gh[PPT][8], xl[PPT][8], xh[PPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      if (live && e_of[i] >= 0) {
        const int e = e_of[i], c0 = e % hd;
        float dl[8], dh[8], c[8], sn[8], wl[8], wh[8];
        unpack8(ndl[i], dl);
        unpack8(ndh[i], dh);
        unpack8(nxl[i], xl[i]);
        unpack8(nxh[i], xh[i]);
        load8f(cos_t + (size_t)pos * half + c0, c);
        load8f(sin_t + (size_t)pos * half + c0, sn);
        load8(w + e, wl);
        load8(w + e + half, wh);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float a = dl[j] * c[j] + dh[j] * sn[j];   // transpose of the rotation
          float b = dh[j] * c[j] - dl[j] * sn[j];
          xl[i][j] *= rstd;
          xh[i][j] *= rstd;
          dwl[i][j] += a * xl[i][j];
          dwh[i][j] += b * xh[i][j];
          a *= wl[j];
          b *= wh[j];
          dot += a * xl[i][j] + b * xh[i][j];
          gl[i][j] = a;
          gh[i][j] = b;
        }
      }
    }
    if (row0 + stride < rows) fetch(row0 + stride);
    dot = row_sum<TPR>(dot, red) / (float)d;
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      if (live && e_of[i] >= 0) {
        const int e = e_of[i];
        float ol[8], oh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ol[j] = rstd * (gl[i][j] - xl[i][j] * dot);
          oh[j] = rstd * (gh[i][j] - xh[i][j] * dot);
        }
        store8(dx + odx + e, ol);
        store8(dx + odx + e + half, oh);
      }
    }
  }
  if (dw == nullptr) return;
  for (int i = threadIdx.x; i < d; i += NORM_THREADS) dw_part[i] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < PPT; ++i) {
    if (e_of[i] >= 0) {
      const int e = e_of[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (ROWS_PER_BLOCK > 1) {
          atomicAdd(&dw_part[e + j], dwl[i][j]);
          atomicAdd(&dw_part[e + half + j], dwh[i][j]);
        } else {
          dw_part[e + j] = dwl[i][j];
          dw_part[e + half + j] = dwh[i][j];
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += NORM_THREADS) atomicAdd(dw + i, dw_part[i] * dw_scale);
}

__device__ __forceinline__ float act_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float act_silu_grad(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}
__device__ __forceinline__ float act_gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float act_gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

// a = act(g) * u
__global__ void glu_fwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u, bf16* __restrict__ a,
                               long long n8, int gelu) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float gv[8], uv[8], o[8];
    load8(g + i * 8, gv);
    load8(u + i * 8, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = (gelu ? act_gelu_tanh(gv[j]) : act_silu(gv[j])) * uv[j];
    store8(a + i * 8, o);
  }
}
// dg = da * u * act'(g); du = da * act(g); optionally a = act(g) * u recomputed (for the down-projection wgrad)
__global__ void glu_bwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u, const bf16* __restrict__ da,
                               bf16* __restrict__ dg, bf16* __restrict__ du, bf16* __restrict__ a_out, long long n8,
                               int gelu) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float gv[8], uv[8], dv[8], og[8], ou[8], oa[8];
    load8(g + i * 8, gv);
    load8(u + i * 8, uv);
    load8(da + i * 8, dv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float act = gelu ? act_gelu_tanh(gv[j]) : act_silu(gv[j]);
      const float dact = gelu ? act_gelu_tanh_grad(gv[j]) : act_silu_grad(gv[j]);
      og[j] = dv[j] * uv[j] * dact;
      ou[j] = dv[j] * act;
      oa[j] = act * uv[j];
    }
    store8(dg + i * 8, og);
    store8(du + i * 8, ou);
    if (a_out != nullptr) store8(a_out + i * 8, oa);
  }
}

// out[t, :] = scale * W[ids[t], :], the table being R row-shards (pointers in `shards`, rows_per_shard rows each);
// a shard pointer may address another GPU's memory (plain loads over NVLink).  One warp per token.
__global__ void embed_gather_kernel(const long long* __restrict__ ids, const bf16* const* __restrict__ shards,
                                    int rows_per_shard, int n_shards, bf16* __restrict__ out, long long tokens, int d,
                                    float scale) {
  const long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  long long id = ids[t];
  const long long vocab = (long long)rows_per_shard * n_shards;
  if (id < 0 || id >= vocab) id = 0;  // out-of-range ids read row 0 instead of faulting
  const bf16* src = shards[id / rows_per_shard] + (id % rows_per_shard) * (long long)d;
  bf16* dst = out + t * d;
  for (int v = lane; v < d / 8; v += 32) {
    float f[8];
    load8(src + v * 8, f);
    if (scale != 1.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= scale;
    }
    store8(dst + v * 8, f);
  }
}
// dW[ids[t], :] += scale * dout[t, :] into fp32 gradient shards (red.global.add, possibly to a peer GPU)
__global__ void embed_scatter_kernel(const long long* __restrict__ ids, float* const* __restrict__ grad_shards,
                                     int rows_per_shard, int n_shards, const bf16* __restrict__ dout, long long tokens,
                                     int d, float scale) {
  const long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const long long id = ids[t];
  const long long vocab = (long long)rows_per_shard * n_shards;
  if (id < 0 || id >= vocab) return;
  float* dst = grad_shards[id / rows_per_shard] + (id % rows_per_shard) * (long long)d;
  const bf16* src = dout + t * d;
  for (int v = lane; v < d / 8; v += 32) {
    float f[8];
    load8(src + v * 8, f);
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + v * 8), "f"(f[0] * scale),
                 "f"(f[1] * scale), "f"(f[2] * scale), "f"(f[3] * scale)
                 : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + v * 8 + 4), "f"(f[4] * scale),
                 "f"(f[5] * scale), "f"(f[6] * scale), "f"(f[7] * scale)
                 : "memory");
  }
}

// dst[r * stride + i] = src_shards[r][i] for every shard r != skip (small tensors: norm weights, biases)
__global__ void gather_shards_kernel(const uint16_t* const* __restrict__ src_shards, uint16_t* __restrict__ dst,
                                     long long stride, long long n_per_shard, int n_shards, int skip) {
  const long long total = n_per_shard * n_shards;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n_per_shard);
    const long long j = i % n_per_shard;
    if (r == skip) continue;
    dst[r * stride + j] = src_shards[r][j];
  }
}
// dst_shards[r][i] += scale * src[r * n_per_shard + i]  (fp32, red.add; destinations may be peer GPUs)
__global__ void scatter_add_shards_kernel(const float* __restrict__ src, float* const* __restrict__ dst_shards,
                                          long long n_per_shard, int n_shards, float scale) {
  const long long total = n_per_shard * n_shards;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n_per_shard);
    const long long j = i % n_per_shard;
    atomicAdd(dst_shards[r] + j, src[i] * scale);
  }
}

static inline int grid_for(long long work_items, int threads, int max_blocks_per_sm = 8) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = (long long)sm_count() * max_blocks_per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace ob

using namespace ob;

// Grid of a grid-stride normalisation kernel: exactly the number of blocks that are resident at once (occupancy x
// SMs), never more -- a second, partly filled wave of blocks would run at a fraction of the memory parallelism.
template <typename Kernel>
static inline int resident_grid(Kernel kernel, long long work_blocks, size_t smem) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, NORM_THREADS, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  long long cap = (long long)sm_count() * per_sm;
  return (int)(work_blocks < cap ? (work_blocks < 1 ? 1 : work_blocks) : cap);
}

// Thread layout of the normalisation kernels for a row of d elements: TPR threads share a row and each keeps VPT
// 8-element vectors of it in registers.  Instantiating the smallest VPT that covers d keeps the register count (and
// with it the number of resident blocks, i.e. the bytes in flight) right for the common widths.
template <int T, int V>
struct NormShape {
  static constexpr int TPR = T, VPT = V;
};
template <typename F>
static inline int norm_dispatch(int d, const char* what, F&& launch) {
  if (d % 8 != 0) OB_FAIL(-1, "%s: d (%d) must be a multiple of 8", what, d);
  if (d <= 128) launch(NormShape<16, 1>{});
  else if (d <= 512) launch(NormShape<16, 4>{});
  else if (d <= 2048) launch(NormShape<NORM_THREADS, 1>{});
  else if (d <= 4096) launch(NormShape<NORM_THREADS, 2>{});
  else if (d <= NORM_THREADS * 8 * MAX_VPT) launch(NormShape<NORM_THREADS, 4>{});
  else OB_FAIL(-2, "%s: d (%d) too large (max %d)", what, d, NORM_THREADS * 8 * MAX_VPT);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd,
                              long long rows, int d, int heads, long long ld_x, long long ld_res, long long ld_y,
                              int add_before, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  return norm_dispatch(d, "rmsnorm", [&](auto shape) {
    using S = decltype(shape);
    const int rpb = NORM_THREADS / S::TPR;
    auto kernel = rmsnorm_fwd_kernel<S::TPR, S::VPT>;
    kernel<<<resident_grid(kernel, (rows + rpb - 1) / rpb, 0), NORM_THREADS, 0, stream>>>(
        (const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)sum_out, rstd, rows, d, heads, ld_x, ld_res,
        ld_y, add_before, eps);
  });
}

extern "C" int ob_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dsum,
                              void* dx, float* dw, long long rows, int d, int heads, long long ld_dy, long long ld_x,
                              long long ld_dx, float dw_scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)d * sizeof(float);
  return norm_dispatch(d, "rmsnorm", [&](auto shape) {
    using S = decltype(shape);
    const int rpb = NORM_THREADS / S::TPR;
    auto kernel = rmsnorm_bwd_kernel<S::TPR, S::VPT>;
    kernel<<<resident_grid(kernel, (rows + rpb - 1) / rpb, smem), NORM_THREADS, smem, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dsum, (bf16*)dx, dw, rows, d, heads, ld_dy,
        ld_x, ld_dx, dw_scale);
  });
}

extern "C" int ob_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long rows, int d, float eps, cudaStream_t stream) {
  if (mean == nullptr || rstd == nullptr) OB_FAIL(-3, "layernorm: the mean and rstd outputs are required");
  if (rows <= 0) return 0;
  return norm_dispatch(d, "layernorm", [&](auto shape) {
    using S = decltype(shape);
    const int rpb = NORM_THREADS / S::TPR;
    auto kernel = layernorm_fwd_kernel<S::TPR, S::VPT>;
    kernel<<<resident_grid(kernel, (rows + rpb - 1) / rpb, 0), NORM_THREADS, 0, stream>>>(
        (const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, mean, rstd, rows, d, eps);
  });
}

extern "C" int ob_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                void* dx, float* dw, float* db, long long rows, int d, float scale,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)2 * d * sizeof(float);   // up to 64 KB for the widest rows
  return norm_dispatch(d, "layernorm", [&](auto shape) {
    using S = decltype(shape);
    const int rpb = NORM_THREADS / S::TPR;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_bwd_kernel<S::TPR, S::VPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    auto kernel = layernorm_bwd_kernel<S::TPR, S::VPT>;
    kernel<<<resident_grid(kernel, (rows + rpb - 1) / rpb, smem), NORM_THREADS, smem, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, mean, rstd, (bf16*)dx, dw, db, rows, d, scale);
  });
}

extern "C" int ob_rope(const void* x, void* y, const float* cos_t, const float* sin_t, int B, int S, int H, int D,
                       long long sb, long long ss, long long sh, long long ysb, long long yss, long long ysh,
                       float sign, int pos_offset, cudaStream_t stream) {
  if (D % 16 != 0) OB_FAIL(-1, "rope: head dim (%d) must be a multiple of 16", D);
  const long long total = (long long)B * S * H * (D / 16);
  if (total <= 0) return 0;
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const bf16*)x, (bf16*)y, cos_t, sin_t, B, S, H, D, sb, ss, sh,
                                                        ysb, yss, ysh, sign, pos_offset);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Thread layout of the fused norm + rotary kernels for a row of d / 16 pairs.
template <typename F>
static inline int norm_rope_dispatch(int d, int hd, const char* what, F&& launch) {
  if (hd % 16 != 0 || hd <= 0 || d % hd != 0) OB_FAIL(-1, "%s: d (%d) must be a multiple of the head dim (%d), itself a multiple of 16", what, d, hd);
  const int npair = d / 16;
  if (npair <= 8) launch(NormShape<8, 1>{});
  else if (npair <= 32) launch(NormShape<32, 1>{});
  else if (npair <= 64) launch(NormShape<32, 2>{});
  else if (npair <= 128) launch(NormShape<32, 4>{});
  else if (npair <= 256) launch(NormShape<NORM_THREADS, 1>{});
  else if (npair <= 512) launch(NormShape<NORM_THREADS, 2>{});
  else if (npair <= 1024) launch(NormShape<NORM_THREADS, 4>{});
  else OB_FAIL(-2, "%s: d (%d) too large (max %d)", what, d, NORM_THREADS * 16 * 4);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_rmsnorm_rope_fwd(const void* x, const void* w, void* y, float* rstd, const float* cos_t,
                                   const float* sin_t, long long rows, int d, int hd, int heads, long long ld_x,
                                   long long ld_y, int S, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (S <= 0 || rows >= (1LL << 31)) OB_FAIL(-3, "rmsnorm_rope: sequence length must be positive and rows below 2^31");
  return norm_rope_dispatch(d, hd, "rmsnorm_rope", [&](auto shape) {
    using Sh = decltype(shape);
    const int rpb = NORM_THREADS / Sh::TPR;
    auto kernel = rmsnorm_rope_fwd_kernel<Sh::TPR, Sh::VPT>;
    kernel<<<resident_grid(kernel, (rows + rpb - 1) / rpb, 0), NORM_THREADS, 0, stream>>>(
        (const bf16*)x, (const bf16*)w, (bf16*)y, rstd, cos_t, sin_t, rows, d, hd, heads, ld_x, ld_y, S, eps);
  });
}

extern "C" int ob_rmsnorm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                                   const float* cos_t, const float* sin_t, long long rows, int d, int hd, int heads,
                                   long long ld_dy, long long ld_x, long long ld_dx, int S, float dw_scale,
                                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (S <= 0 || rows >= (1LL << 31)) OB_FAIL(-3, "rmsnorm_rope: sequence length must be positive and rows below 2^31");
  const size_t smem = (size_t)d * sizeof(float);
  return norm_rope_dispatch(d, hd, "rmsnorm_rope", [&](auto shape) {
    using Sh = decltype(shape);
    const int rpb = NORM_THREADS / Sh::TPR;
    auto kernel = rmsnorm_rope_bwd_kernel<Sh::TPR, Sh::VPT>;
    kernel<<<resident_grid(kernel, (rows + rpb - 1) / rpb, smem), NORM_THREADS, smem, stream>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (bf16*)dx, dw, cos_t, sin_t, rows, d, hd, heads, ld_dy,
        ld_x, ld_dx, S, dw_scale);
  });
}

extern "C" int ob_glu_fwd(const void* g, const void* u, void* a, long long n, int gelu, cudaStream_t stream) {
  if (n % 8 != 0) OB_FAIL(-1, "glu: element count must be a multiple of 8");
  if (n == 0) return 0;
  glu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const bf16*)g, (const bf16*)u, (bf16*)a, n / 8, gelu);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_glu_bwd(const void* g, const void* u, const void* da, void* dg, void* du, void* a_out, long long n,
                          int gelu, cudaStream_t stream) {
  if (n % 8 != 0) OB_FAIL(-1, "glu: element count must be a multiple of 8");
  if (n == 0) return 0;
  glu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const bf16*)g, (const bf16*)u, (const bf16*)da, (bf16*)dg,
                                                           (bf16*)du, (bf16*)a_out, n / 8, gelu);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_embed_gather(const long long* ids, const void* const* shards, int rows_per_shard, int n_shards,
                               void* out, long long tokens, int d, float scale, cudaStream_t stream) {
  if (d % 8 != 0) OB_FAIL(-1, "embedding: d must be a multiple of 8");
  if (tokens == 0) return 0;
  const int threads = 256;
  const long long blocks = (tokens * 32 + threads - 1) / threads;
  embed_gather_kernel<<<(unsigned)blocks, threads, 0, stream>>>(ids, (const bf16* const*)shards, rows_per_shard,
                                                                n_shards, (bf16*)out, tokens, d, scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_embed_scatter(const long long* ids, float* const* grad_shards, int rows_per_shard, int n_shards,
                                const void* dout, long long tokens, int d, float scale, cudaStream_t stream) {
  if (d % 8 != 0) OB_FAIL(-1, "embedding: d must be a multiple of 8");
  if (tokens == 0) return 0;
  const int threads = 256;
  const long long blocks = (tokens * 32 + threads - 1) / threads;
  embed_scatter_kernel<<<(unsigned)blocks, threads, 0, stream>>>(ids, grad_shards, rows_per_shard, n_shards,
                                                                 (const bf16*)dout, tokens, d, scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_gather_shards(const void* const* src_shards, void* dst, long long stride, long long n_per_shard,
                                int n_shards, int skip, cudaStream_t stream) {
  if (n_per_shard <= 0) return 0;
  gather_shards_kernel<<<grid_for(n_per_shard * n_shards, 256), 256, 0, stream>>>(
      (const uint16_t* const*)src_shards, (uint16_t*)dst, stride, n_per_shard, n_shards, skip);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_scatter_add_shards(const float* src, float* const* dst_shards, long long n_per_shard, int n_shards,
                                     float scale, cudaStream_t stream) {
  if (n_per_shard <= 0) return 0;
  scatter_add_shards_kernel<<<grid_for(n_per_shard * n_shards, 256), 256, 0, stream>>>(src, dst_shards, n_per_shard,
                                                                                       n_shards, scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}
