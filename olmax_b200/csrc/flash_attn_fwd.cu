// Flash-attention forward for sm_100a (head_dim 128, bf16 in/out, fp32 softmax statistics).
//
// One CTA handles one 128-row query tile of one (batch, head).  S = Q K^T and O += P V run on tcgen05 tensor
// cores with accumulators in TMEM: S occupies 128 fp32 columns, O another 128; P (bf16) is written back over the
// S columns and is consumed from TMEM as the A operand of the second MMA, so P never touches shared memory.
// The softmax is done by 256 threads, two per query row (TMEM lane == row; the two column halves exchange their row
// maximum through shared memory, no shuffles).  The running maximum is only raised when it grows by more than 2^8 ("lazy rescale"), which keeps the
// O correction (a TMEM read-modify-write) off most iterations.  A CTA uses 256 TMEM columns and ~97 KiB of shared
// memory so that two CTAs share an SM: while one is in its softmax the other one's MMAs keep the tensor cores busy.
//
// Supports: causal masking, grouped-query attention (H a multiple of Hkv), a left sliding window, tanh soft-capping
// of the logits, arbitrary element strides for Q/K/V (so they can be slices of one fused QKV buffer) and sequence
// lengths that are not a multiple of the tile.  Writes O (bf16) and the log-sum-exp of every row (natural log).
//
// Takes the place of the cuDNN / TransformerEngine fused attention the reference calls in
// `olmax/nn/attention.py:52-109`; soft-cap has no counterpart there.
#include "flash_attn.h"
#include "host_common.h"
#include "sm100.cuh"

namespace ob {

namespace fa_fwd {

constexpr int TQ = 128;   // query rows per CTA
constexpr int TK = 128;   // keys per iteration
constexpr int HD = 128;   // head dim
constexpr int BLK = 128 * 64 * 2;            // one [128 rows][64 elems] swizzled block: 16 KiB
constexpr int TILE_BYTES = 2 * BLK;          // [128][128] bf16 as two blocks
constexpr int SMEM_BYTES = 3 * TILE_BYTES + 1024 + 128 + 1024;  // + row-statistics exchange [2][128] floats
constexpr int THREADS = 320;   // TMA warp, MMA warp, 8 softmax warps
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0;      // S (fp32, 128 cols); P (bf16x2, 64 cols) is written over its first 64 columns
constexpr int O_COL = 128;    // O (fp32, 128 cols)

struct Params {
  int B, S, H, Hkv;
  int Sk, q_off;               // key length; position of query row 0 on the key axis (query i sits at q_off + i)
  int causal, window;          // window < 0: none; else keys with kv >= q - window
  float scale_log2;            // softmax scale * log2(e)            (no soft-cap)
  float softcap;               // 0: none
  float scale_over_cap;        // softmax scale / softcap
  float cap_log2;              // softcap * log2(e)
  bf16* o;
  long long o_sb, o_ss, o_sh;  // element strides of O
  float* lse;                  // [B, H, S]
  int* status;
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(THREADS, 2)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;
  uint8_t* sV = smem + 2 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(bars + 16);   // [2][128] exchange between the two column halves of a row

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_q_tiles = (p.S + TQ - 1) / TQ;
  const int q_tile = n_q_tiles - 1 - (int)blockIdx.x;  // heaviest (longest causal row) tiles first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / (p.H / p.Hkv);
  const int q0 = q_tile * TQ;

  // key-tile range for this query tile
  int kv_tile_lo = 0;
  const int qp0 = p.q_off + q0;   // key-axis position of this tile's first query row
  int kv_tile_hi = (p.Sk + TK - 1) / TK - 1;
  if (p.causal) kv_tile_hi = min(kv_tile_hi, (qp0 + TQ - 1) / TK);
  if (p.window >= 0) kv_tile_lo = max(0, (qp0 - p.window) / TK);
  const int n_iters = kv_tile_hi - kv_tile_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);      // one arrival per softmax warp (lane 0, after the warp has synchronised)
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // The TMA and MMA warps run their loops with all 32 lanes so that the loop state stays warp-uniform; one elected
  // lane issues.  A wait that gives up marks the warp `dead`: the loop then runs out without issuing anything.
  if (warp == 0) {
    const bool leader = elect_one();
    bool dead = false;
    if (leader) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
      tma_load_4d(sQ, &tmQ, q_full, 0, h, q0, b);
      tma_load_4d(sQ + BLK, &tmQ, q_full, 64, h, q0, b);
    }
    for (int j = 0; j < n_iters; ++j) {
      const int kv0 = (kv_tile_lo + j) * TK;
      const uint32_t ph = (uint32_t)j & 1u;
      if (!dead) dead = !mbar_wait(k_empty, ph ^ 1u, abort_flag, p.status, 400);
      if (leader && !dead) {
        mbar_arrive_expect_tx(k_full, TILE_BYTES);
        tma_load_4d(sK, &tmK, k_full, 0, hkv, kv0, b);
        tma_load_4d(sK + BLK, &tmK, k_full, 64, hkv, kv0, b);
      }
      if (!dead) dead = !mbar_wait(v_empty, ph ^ 1u, abort_flag, p.status, 401);
      if (leader && !dead) {
        mbar_arrive_expect_tx(v_full, TILE_BYTES);
        tma_load_4d(sV, &tmV, v_full, 0, hkv, kv0, b);
        tma_load_4d(sV + BLK, &tmV, v_full, 64, hkv, kv0, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc_bf16(TQ, TK, 0, 0);
    constexpr uint32_t idesc_o = make_idesc_bf16(TQ, HD, 0, 1);
    // shared-memory descriptors: constant high words, low words (start address in 16-byte units) advanced per k step
    const uint64_t dQ = make_smem_desc(smem_u32(sQ), 0, 1024), dK = make_smem_desc(smem_u32(sK), 0, 1024);
    const uint64_t dV = make_smem_desc(smem_u32(sV), BLK, 1024);
    const uint32_t q_lo = (uint32_t)dQ, k_lo = (uint32_t)dK, v_lo = (uint32_t)dV;
    const uint32_t kk_hi = (uint32_t)(dQ >> 32), v_hi = (uint32_t)(dV >> 32);
    bool dead = !mbar_wait(q_full, 0, abort_flag, p.status, 500);
    for (int j = 0; j < n_iters; ++j) {
      const uint32_t ph = (uint32_t)j & 1u;
      if (!dead) dead = !mbar_wait(k_full, ph, abort_flag, p.status, 501);
      tc_fence_after_sync();
      if (leader && !dead) {
        // S = Q K^T.  In-order execution of this thread's MMAs keeps it behind the previous P V, which read P
        // from the same columns.
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = ((uint32_t)(kk >> 2) * BLK + (uint32_t)(kk & 3) * 32) >> 4;
          umma_ss_lohi(tmem_base + S_COL, q_lo + off, kk_hi, k_lo + off, kk_hi, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(k_empty);
        umma_commit(s_full);
      }
      if (!dead) dead = !mbar_wait(p_full, ph, abort_flag, p.status, 502);
      if (!dead) dead = !mbar_wait(v_full, ph, abort_flag, p.status, 503);
      tc_fence_after_sync();
      if (leader && !dead) {
        // O += P V: A = P from TMEM (128 x 16 bf16 per step = 8 columns), B = V as an MN-major operand
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk) {
          umma_ts_lohi(tmem_base + O_COL, tmem_base + S_COL + (uint32_t)kk * 8, v_lo + (uint32_t)kk * 128u, v_hi, idesc_o,
                       (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(v_empty);
        umma_commit(o_done);
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax + output: 8 warps, thread <-> (query row, 64-column half) ----------------
    // Two warps share each TMEM lane quarter and split the 128 score columns; the halves exchange their row maxima
    // through shared memory once per tile.  With two CTAs per SM every scheduler then has four softmax warps to hide
    // TMEM and MUFU latency.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = qd * 32 + lane;
    const int col0 = half * 64;
    const int q_idx = q0 + row;
    const int q_pos = p.q_off + q_idx;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const bool capped = p.softcap > 0.f;
    float m_run = -INFINITY;  // running max, log2 domain (identical in both halves of a row)
    float l_run = 0.f;        // this half's share of the running sum
    bool ok = true;
    for (int j = 0; j < n_iters && ok; ++j) {
      const uint32_t ph = (uint32_t)j & 1u;
      const int kv0 = (kv_tile_lo + j) * TK;
      ok = mbar_wait(s_full, ph, abort_flag, p.status, 600);
      if (!ok) break;
      tc_fence_after_sync();
      const bool need_mask = (kv0 + TK > p.Sk) || (p.causal && kv0 + TK - 1 > qp0) ||
                             (p.window >= 0 && kv0 < qp0 + TQ - 1 - p.window);
      const int kv_hi = p.causal ? min(q_pos, p.Sk - 1) : p.Sk - 1;  // last visible key
      const int kv_lo = p.window >= 0 ? q_pos - p.window : 0;        // first visible key
      // this thread's 64 scores, kept in registers for both the max and the exponentials
      uint32_t r0[32], r1[32];
      tmem_ld32(t_lane + S_COL + (uint32_t)col0, r0);
      tmem_ld32(t_lane + S_COL + (uint32_t)(col0 + 32), r1);
      tmem_ld_wait();
      if (capped) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          r0[i] = __float_as_uint(p.cap_log2 * fast_tanh(__uint_as_float(r0[i]) * p.scale_over_cap));
          r1[i] = __float_as_uint(p.cap_log2 * fast_tanh(__uint_as_float(r1[i]) * p.scale_over_cap));
        }
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + col0 + i;
          if (kv > kv_hi || kv < kv_lo) r0[i] = __float_as_uint(-INFINITY);
          if (kv + 32 > kv_hi || kv + 32 < kv_lo) r1[i] = __float_as_uint(-INFINITY);
        }
      }
      // four independent chains: a single running maximum (or sum, below) would serialise 32 dependent operations
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float sc = capped ? 1.0f : p.scale_log2;   // soft-capped scores are already in the log2 domain
      mx *= sc;                                        // sc > 0: max commutes with the scaling
      xch[half * 128 + row] = mx;
      asm volatile("bar.sync 2, 256;" ::: "memory");
      const float m_new = fmaxf(m_run, fmaxf(mx, xch[(half ^ 1) * 128 + row]));
      // lazy rescale: raise the running max only when it grows by more than 8 (factor 256); warp-uniform decision
      const bool want = (m_new > m_run + 8.0f) || (m_run == -INFINITY && m_new > -INFINITY);
      if (__any_sync(0xffffffffu, want)) {
        const float m_next = want ? m_new : m_run;
        const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_next);
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 64; c += 16) {
            uint32_t o[16];
            tmem_ld16(t_lane + O_COL + (uint32_t)(col0 + c), o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st16(t_lane + O_COL + (uint32_t)(col0 + c), o);
          }
          tmem_st_wait();
        }
        l_run *= alpha;
        m_run = m_next;
      }
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
      // P = exp2(s - m) as bf16 pairs, written over the S columns (both halves hold their scores in registers by now)
      float lsum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float s0 = __uint_as_float(hh ? r1[i] : r0[i]), s1 = __uint_as_float(hh ? r1[i + 1] : r0[i + 1]);
          const float e0 = fast_exp2(fmaf(s0, sc, neg_m)), e1 = fast_exp2(fmaf(s1, sc, neg_m));
          lsum4[(i >> 1) & 3] += e0 + e1;
          pk[i >> 1] = pack_bf16x2(e0, e1);
        }
        tmem_st16(t_lane + S_COL + (uint32_t)(half * 32 + hh * 16), pk);
      }
      l_run += (lsum4[0] + lsum4[1]) + (lsum4[2] + lsum4[3]);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // epilogue: wait for the last P V, combine the halves' sums, normalise, store
    if (ok) ok = mbar_wait(o_done, (uint32_t)(n_iters - 1) & 1u, abort_flag, p.status, 601);
    xch[half * 128 + row] = l_run;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (ok) {
      tc_fence_after_sync();
      const float l_tot = l_run + xch[(half ^ 1) * 128 + row];
      const float inv_l = l_tot > 0.f ? 1.0f / l_tot : 0.f;
      const bool row_ok = q_idx < p.S;
      bf16* orow = p.o + (long long)b * p.o_sb + (long long)q_idx * p.o_ss + (long long)h * p.o_sh + col0;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t r[32];
        tmem_ld32(t_lane + O_COL + (uint32_t)(col0 + c), r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]) * inv_l, __uint_as_float(r[g * 8 + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * inv_l, __uint_as_float(r[g * 8 + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * inv_l, __uint_as_float(r[g * 8 + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * inv_l, __uint_as_float(r[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + g * 8) = v;
          }
        }
      }
      if (row_ok && half == 0) {
        const float lse = l_tot > 0.f ? (m_run + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
        p.lse[((long long)b * p.H + h) * p.S + q_idx] = lse;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace fa_fwd

// [B, S, H, 128] tensor with element strides -> 4-D map (d, h, s, b), box 64 x 1 x 128 x 1, 128-byte swizzle
int encode_bshd_map(CUtensorMap* m, const void* ptr, int B, int S, int H, long long sb, long long ss, long long sh,
                    int box_rows) {
  uint64_t dims[4] = {128, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t str[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace ob

using namespace ob;

extern "C" int ob_flash_attn_fwd(const ObAttnArgs* a, cudaStream_t stream) {
  if (a == nullptr) OB_FAIL(-1, "null args");
  if (a->D != 128) OB_FAIL(-2, "flash attention kernels are built for head_dim 128 (got %d)", a->D);
  if (a->H % a->Hkv != 0) OB_FAIL(-3, "H (%d) must be a multiple of Hkv (%d)", a->H, a->Hkv);
  if (a->B <= 0 || a->S <= 0) OB_FAIL(-4, "empty problem");
  int Sk = 0;
  if (int g = ob_attn_check_geometry(a, &Sk))
    OB_FAIL(-5, "unsupported attention geometry (rule %d): S %d Sk %d q_off %d causal %d window %d", g, a->S, Sk,
            a->q_off, a->causal, a->window);
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = encode_bshd_map(&tq, a->q, a->B, a->S, a->H, a->q_sb, a->q_ss, a->q_sh, 128))) return rc;
  if ((rc = encode_bshd_map(&tk, a->k, a->B, Sk, a->Hkv, a->k_sb, a->k_ss, a->k_sh, 128))) return rc;
  if ((rc = encode_bshd_map(&tv, a->v, a->B, Sk, a->Hkv, a->v_sb, a->v_ss, a->v_sh, 128))) return rc;
  fa_fwd::Params p;
  p.B = a->B; p.S = a->S; p.H = a->H; p.Hkv = a->Hkv;
  p.Sk = Sk; p.q_off = a->q_off;
  p.causal = a->causal; p.window = a->window;
  const float LOG2E = 1.4426950408889634f;
  p.scale_log2 = a->scale * LOG2E;
  p.softcap = a->softcap;
  p.scale_over_cap = a->softcap > 0.f ? a->scale / a->softcap : 0.f;
  p.cap_log2 = a->softcap * LOG2E;
  p.o = reinterpret_cast<bf16*>(a->o);
  p.o_sb = a->o_sb; p.o_ss = a->o_ss; p.o_sh = a->o_sh;
  p.lse = a->lse;
  p.status = a->status;
  // the shared-memory opt-in is a per-device attribute of the function
  static bool attr_set[64] = {};
  int dev = 0;
  OB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) OB_FAIL(-6, "device ordinal %d outside the supported range [0, 64)", dev);
  if (!attr_set[dev]) {
    OB_CUDA_OK(cudaFuncSetAttribute(fa_fwd::flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    fa_fwd::SMEM_BYTES));
    attr_set[dev] = true;
  }
  dim3 grid((a->S + 127) / 128, a->H, a->B);
  fa_fwd::flash_fwd_kernel<<<grid, fa_fwd::THREADS, fa_fwd::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}
