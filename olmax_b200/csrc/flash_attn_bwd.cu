// Flash-attention backward for sm_100a (head_dim 128).
//
// One CTA owns one 128-key tile of one (batch, kv-head) and loops over every query head of the group and every
// query tile that can see those keys.  Per (query tile, key tile) it runs five tcgen05 MMAs:
//     S  = Q K^T          dP = dO V^T          dV += P^T dO          dK += dS^T Q          dQ_part = dS K
// with S / dP / dK / dV in the four 128-column quarters of TMEM.  dK and dV stay in TMEM for the whole CTA lifetime
// (no atomics, GQA heads accumulate in place); the dQ partial is produced in the S columns once S has been consumed
// and is added to an fp32 scratch tensor with a TMA reduce-add from shared memory (staged in the Q / dO buffers of the
// iteration, which are idle by then), which a small kernel converts to bf16 at the end.
// P and dS are formed by 256 threads (two per query row, 64 columns each), written as bf16 to one shared 32 KiB buffer in
// the 128-byte-swizzled layout the MMAs read (P^T / dS^T as an MN-major A operand, dS as a K-major A operand).
// Q and dO tiles stream through a 2-stage TMA ring; K and V stay resident in shared memory.
//
// The math is the standard recompute form: P = exp(S - lse), dS = P * (dP - delta) * scale, with
// delta = rowsum(dO * O) from a pre-pass; a tanh soft-cap multiplies dS by (1 - tanh^2).
//
// Counterpart of the autodiff of `olmax/nn/attention.py:96-103` (cuDNN backward in the reference).
#include "flash_attn.h"
#include "flash_attn_noalloc.h"
#include "host_common.h"
#include "sm100.cuh"

namespace ob {

int encode_bshd_map(CUtensorMap* m, const void* ptr, int B, int S, int H, long long sb, long long ss, long long sh,
                    int box_rows);

namespace fa_bwd {

constexpr int T = 128;    // tile (queries and keys)
constexpr int HD = 128;
constexpr int BLK = 128 * 64 * 2;   // 16 KiB swizzled block [128 rows][64 elems]
constexpr int TILE = 2 * BLK;       // 32 KiB
constexpr int STAGES = 2;   // the loops below index stages with (it & 1)
constexpr int OFF_K = 0;
constexpr int OFF_V = TILE;
constexpr int OFF_Q = 2 * TILE;                    // STAGES tiles
constexpr int OFF_DO = OFF_Q + STAGES * TILE;      // STAGES tiles
constexpr int OFF_P = OFF_DO + STAGES * TILE;      // P, later dS
constexpr int OFF_BAR = OFF_P + TILE;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int THREADS = 352;   // TMA warp, MMA warp, 8 compute warps, dQ store warp
constexpr int TMEM_COLS = 512;
constexpr int C_S = 0, C_DP = 128, C_DK = 256, C_DV = 384;

struct Params {
  int B, S, H, Hkv;
  int Sk, q_off;   // key length; key-axis position of query row 0
  int causal, window;
  float scale, scale_log2, softcap, scale_over_cap, cap_log2;
  const float* lse;
  const float* delta;
  float* dq_accum;   // [B, S, H, 128] fp32 contiguous
  bf16* dk; long long dk_sb, dk_ss, dk_sh;
  bf16* dv; long long dv_sb, dv_ss, dv_sh;
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

__global__ void __launch_bounds__(THREADS, 1)
    flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmDQ, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* full = bars + 1;       // [STAGES]
  uint64_t* empty = bars + 3;      // [STAGES]
  uint64_t* s_full = bars + 5;
  uint64_t* dp_full = bars + 6;
  uint64_t* p_ready = bars + 7;    // 8 arrivals (one per compute warp)
  uint64_t* pv_done = bars + 8;
  uint64_t* ds_ready = bars + 9;   // 8 arrivals
  uint64_t* dq_full = bars + 10;
  uint64_t* dq_read = bars + 11;   // 8 arrivals
  uint64_t* all_done = bars + 12;
  uint64_t* dq_staged = bars + 13; // 8 arrivals: the fp32 dQ partial tile is in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (p.S + T - 1) / T;
  const int kv_tile = blockIdx.x;
  const int hkv = blockIdx.y;
  const int b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int kv0 = kv_tile * T;

  // query tiles that see this key tile: rows i with kv0 <= q_off + i (causal) and q_off + i <= kv0 + T - 1 + window
  int i_lo = 0, i_hi = n_tiles - 1;
  if (p.causal) i_lo = max(0, kv0 - p.q_off) / T;
  if (p.window >= 0) {
    const int last = kv0 + T - 1 + p.window - p.q_off;
    i_hi = last < 0 ? -1 : min(i_hi, last / T);
  }
  const int n_q = max(0, i_hi - i_lo + 1);
  const int n_iters = n_q * G;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 8);     // one arrival per compute warp (lane 0, after the warp has synchronised)
    mbar_init(pv_done, 1);
    mbar_init(ds_ready, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, 8);
    mbar_init(all_done, 1);
    mbar_init(dq_staged, 8);
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

  // The TMA, MMA and dQ-store warps run their loops with all 32 lanes so that the loop state stays warp-uniform; one
  // elected lane issues.  A wait that gives up marks the warp `dead`: the loop then runs out without issuing anything.
  if (warp == 0) {
    const bool leader = elect_one();
    bool dead = false;
    if (leader && n_iters > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_arrive_expect_tx(kv_full, 2 * TILE);
      tma_load_4d(smem + OFF_K, &tmK, kv_full, 0, hkv, kv0, b);
      tma_load_4d(smem + OFF_K + BLK, &tmK, kv_full, 64, hkv, kv0, b);
      tma_load_4d(smem + OFF_V, &tmV, kv_full, 0, hkv, kv0, b);
      tma_load_4d(smem + OFF_V + BLK, &tmV, kv_full, 64, hkv, kv0, b);
    }
    int hq = 0, iq = 0;   // query head within the group, query tile within [i_lo, i_hi]
    for (int it = 0; it < n_iters; ++it) {
      const int s = it & 1;
      const uint32_t ph = (uint32_t)(it >> 1) & 1u;
      const int h = hkv * G + hq;
      const int q0 = (i_lo + iq) * T;
      if (!dead) dead = !mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 700);
      if (leader && !dead) {
        mbar_arrive_expect_tx(&full[s], 2 * TILE);
        uint8_t* sq = smem + OFF_Q + s * TILE;
        uint8_t* sdo = smem + OFF_DO + s * TILE;
        tma_load_4d(sq, &tmQ, &full[s], 0, h, q0, b);
        tma_load_4d(sq + BLK, &tmQ, &full[s], 64, h, q0, b);
        tma_load_4d(sdo, &tmDO, &full[s], 0, h, q0, b);
        tma_load_4d(sdo + BLK, &tmDO, &full[s], 64, h, q0, b);
      }
      if (++iq == n_q) {
        iq = 0;
        ++hq;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    const bool leader = elect_one();
    if (n_iters > 0) {
      constexpr uint32_t id_kk = make_idesc_bf16(T, T, 0, 0);    // both K-major
      constexpr uint32_t id_mm = make_idesc_bf16(T, HD, 1, 1);   // both MN-major
      constexpr uint32_t id_km = make_idesc_bf16(T, HD, 0, 1);   // A K-major, B MN-major
      // Shared-memory descriptors: the high word depends only on the operand's major-ness, the low word is the start
      // address in 16-byte units.  A K-major [128][128] tile is two [128][64] blocks: k step kk sits at
      // (kk / 4) * BLK + (kk % 4) * 32 bytes; in an MN-major tile k step kk sits at kk * 2048 bytes.
      const uint64_t d_k = make_smem_desc(0, 0, 1024), d_mn = make_smem_desc(0, BLK, 1024);
      const uint32_t hi_k = (uint32_t)(d_k >> 32), hi_mn = (uint32_t)(d_mn >> 32);
      const uint32_t lo_flags_k = (uint32_t)d_k, lo_flags_mn = (uint32_t)d_mn;   // low-word bits above the address
      auto lo = [](uint32_t addr) { return (addr & 0x3FFFFu) >> 4; };
      const uint32_t aK = lo(smem_u32(smem + OFF_K)), aV = lo(smem_u32(smem + OFF_V)), aP = lo(smem_u32(smem + OFF_P));
      const uint32_t aQ0 = lo(smem_u32(smem + OFF_Q)), aDO0 = lo(smem_u32(smem + OFF_DO));
      constexpr uint32_t TILE16 = TILE >> 4;
      bool dead = !mbar_wait(kv_full, 0, abort_flag, p.status, 800);
      auto koff = [](int kk) { return ((uint32_t)(kk >> 2) * BLK + (uint32_t)(kk & 3) * 32) >> 4; };
      auto issue_s = [&](uint32_t aQ) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_ss_lohi(tmem_base + C_S, lo_flags_k | (aQ + koff(kk)), hi_k, lo_flags_k | (aK + koff(kk)), hi_k, id_kk,
                       kk != 0 ? 1u : 0u);
      };
      auto issue_dp = [&](uint32_t aDO) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_ss_lohi(tmem_base + C_DP, lo_flags_k | (aDO + koff(kk)), hi_k, lo_flags_k | (aV + koff(kk)), hi_k, id_kk,
                       kk != 0 ? 1u : 0u);
      };
      if (!dead) dead = !mbar_wait(&full[0], 0, abort_flag, p.status, 801);
      tc_fence_after_sync();
      if (leader && !dead) {
        issue_s(aQ0);
        umma_commit(s_full);
        issue_dp(aDO0);
        umma_commit(dp_full);
      }
      for (int it = 0; it < n_iters; ++it) {
        const int s = it & 1;
        const uint32_t ph1 = (uint32_t)it & 1u;
        const uint32_t aQ = aQ0 + (uint32_t)s * TILE16;
        const uint32_t aDO = aDO0 + (uint32_t)s * TILE16;
        // dV += P^T dO
        if (!dead) dead = !mbar_wait(p_ready, ph1, abort_flag, p.status, 802);
        tc_fence_after_sync();
        if (leader && !dead) {
#pragma unroll
          for (int kk = 0; kk < T / 16; ++kk)
            umma_ss_lohi(tmem_base + C_DV, lo_flags_mn | (aP + (uint32_t)kk * 128u), hi_mn,
                         lo_flags_mn | (aDO + (uint32_t)kk * 128u), hi_mn, id_mm, (it | kk) != 0 ? 1u : 0u);
          umma_commit(pv_done);
        }
        // dK += dS^T Q ; dQ_part = dS K
        if (!dead) dead = !mbar_wait(ds_ready, ph1, abort_flag, p.status, 803);
        tc_fence_after_sync();
        if (leader && !dead) {
#pragma unroll
          for (int kk = 0; kk < T / 16; ++kk)
            umma_ss_lohi(tmem_base + C_DK, lo_flags_mn | (aP + (uint32_t)kk * 128u), hi_mn,
                         lo_flags_mn | (aQ + (uint32_t)kk * 128u), hi_mn, id_mm, (it | kk) != 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < T / 16; ++kk)
            umma_ss_lohi(tmem_base + C_S, lo_flags_k | (aP + koff(kk)), hi_k, lo_flags_mn | (aK + (uint32_t)kk * 128u), hi_mn,
                         id_km, kk != 0 ? 1u : 0u);
          umma_commit(dq_full);   // also tells the compute warps that every MMA reading stage s has finished
        }
        if (it + 1 < n_iters) {
          const int s2 = (it + 1) & 1;
          const uint32_t ph2 = (uint32_t)((it + 1) >> 1) & 1u;
          if (!dead) dead = !mbar_wait(&full[s2], ph2, abort_flag, p.status, 804);
          tc_fence_after_sync();
          if (leader && !dead) {
            issue_dp(aDO0 + (uint32_t)s2 * TILE16);
            umma_commit(dp_full);
          }
          if (!dead) dead = !mbar_wait(dq_read, ph1, abort_flag, p.status, 805);
          tc_fence_after_sync();
          if (leader && !dead) {
            issue_s(aQ0 + (uint32_t)s2 * TILE16);
            umma_commit(s_full);
          }
        }
      }
      if (leader && !dead) umma_commit(all_done);
    }
    __syncwarp();
  } else if (warp == 10) {
    // ---------------- dQ store warp: fp32 partial tile (in the Q / dO stage) += into global memory ----------------
    const bool leader = elect_one();
    bool dead = false;
    int hq = 0, iq = 0;
    for (int it = 0; it < n_iters; ++it) {
      const int s = it & 1;
      const int h = hkv * G + hq;
      const int q0 = (i_lo + iq) * T;
      if (!dead) dead = !mbar_wait(dq_staged, (uint32_t)it & 1u, abort_flag, p.status, 950);
      if (leader && !dead) {
        // columns [0, 64) sit in the Q stage, [64, 128) in the dO stage, 32 columns (128 bytes) per chunk
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const uint8_t* src = smem + (cc < 2 ? OFF_Q : OFF_DO) + s * TILE + (cc & 1) * 16384;
          tma_reduce_add_4d(&tmDQ, src, cc * 32, h, q0, b);
        }
        tma_store_commit();
        tma_store_wait_read<0>();      // the stage has been read: hand it back to the TMA producer
        mbar_arrive(&empty[s]);
      }
      if (++iq == n_q) {
        iq = 0;
        ++hq;
      }
    }
    if (leader) tma_store_wait<0>();
    __syncwarp();
  } else {
    // ---------------- P / dS / dQ / dK / dV: 8 warps, thread <-> (row, 64-column half) ----------------
    // Two warps share each TMEM lane quarter and split the 128 columns, so that every scheduler has two compute warps
    // to hide TMEM-load, MUFU and shared-memory latencies behind each other.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = qd * 32 + lane;
    const int col0 = half * 64;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    uint8_t* sP = smem + OFF_P + half * BLK + row * 128;   // this thread's 128-byte row of key block `half`
    const int sw = row & 7;
    const float LOG2E = 1.4426950408889634f;
    const bool capped = p.softcap > 0.f;
    bool ok = true;
    // Row statistics (log-sum-exp, delta) of the NEXT iteration's query row are fetched one iteration ahead: the loads
    // (global memory, hundreds of cycles) then complete under the current iteration's work instead of stalling the
    // exponentials right after S arrives.
    int hq = 0, iq = 0;          // query head within the group / query tile within [i_lo, i_hi] of iteration `it`
    // (only the loads are issued ahead; nothing computes on the loaded values until the next iteration, so that no
    // instruction of this iteration waits for them)
    float lse_next = INFINITY, dl_next = 0.f;
    auto fetch_stats = [&](int hq_, int iq_) {
      const int q_idx_ = min((i_lo + iq_) * T + row, p.S - 1);   // clamped: rows beyond S are masked by q_ok below
      const long long idx = ((long long)b * p.H + (hkv * G + hq_)) * p.S + q_idx_;
      lse_next = __ldg(p.lse + idx);
      dl_next = __ldg(p.delta + idx);
    };
    if (n_iters > 0) fetch_stats(0, 0);
    for (int it = 0; it < n_iters && ok; ++it) {
      const uint32_t ph1 = (uint32_t)it & 1u;
      const int q0 = (i_lo + iq) * T;
      const int q_idx = q0 + row;
      const bool q_ok = q_idx < p.S;
      const float lse2 = q_ok ? lse_next * LOG2E : INFINITY;
      const float dl = q_ok ? dl_next : 0.f;
      if (++iq == n_q) {
        iq = 0;
        ++hq;
      }
      if (it + 1 < n_iters) fetch_stats(hq, iq);
      const int qp0 = p.q_off + q0, q_pos = p.q_off + q_idx;   // positions on the key axis
      const bool need_mask = (kv0 + T > p.Sk) || (p.causal && kv0 + T - 1 > qp0) ||
                             (p.window >= 0 && kv0 < qp0 + T - 1 - p.window);
      const int kv_hi = p.causal ? min(q_pos, p.Sk - 1) : p.Sk - 1;
      const int kv_lo = p.window >= 0 ? q_pos - p.window : 0;

      ok = mbar_wait(s_full, ph1, abort_flag, p.status, 900);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t pp[32];  // P of this half row, bf16x2
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(t_lane + C_S + (uint32_t)col0, r0);
        tmem_ld32(t_lane + C_S + (uint32_t)(col0 + 32), r1);
        tmem_ld_wait();
        // P = exp2(s * scale * log2e - lse2), in place over the loaded scores.  The soft-cap and mask cases are
        // handled by loops of their own: a branch inside the hot loop would cut it into one basic block per element
        // pair and expose the FFMA -> EX2 -> pack latency of every pair instead of overlapping the pairs.
        if (capped) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            r0[i] = __float_as_uint(fast_exp2(p.cap_log2 * fast_tanh(__uint_as_float(r0[i]) * p.scale_over_cap) - lse2));
            r1[i] = __float_as_uint(fast_exp2(p.cap_log2 * fast_tanh(__uint_as_float(r1[i]) * p.scale_over_cap) - lse2));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            r0[i] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r0[i]), p.scale_log2, -lse2)));
            r1[i] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r1[i]), p.scale_log2, -lse2)));
          }
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kv = kv0 + col0 + i;
            if (kv > kv_hi || kv < kv_lo) r0[i] = 0u;
            if (kv + 32 > kv_hi || kv + 32 < kv_lo) r1[i] = 0u;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          pp[i >> 1] = pack_bf16x2(__uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
          pp[16 + (i >> 1)] = pack_bf16x2(__uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
        }
      }
      // eight 16-byte chunks of this row; the chunk index is XOR-swizzled by row % 8 (128-byte swizzle)
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(sP + ((ch ^ sw) << 4)) = make_uint4(pp[ch * 4], pp[ch * 4 + 1], pp[ch * 4 + 2], pp[ch * 4 + 3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      ok = mbar_wait(dp_full, ph1, abort_flag, p.status, 901);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t ds[32];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(t_lane + C_DP + (uint32_t)col0, r0);
        tmem_ld32(t_lane + C_DP + (uint32_t)(col0 + 32), r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float2 pv = unpack_bf16x2(pp[i >> 1]);
          const float g0 = __uint_as_float(i < 32 ? r0[i] : r1[i - 32]);
          const float g1 = __uint_as_float(i < 32 ? r0[i + 1] : r1[i - 31]);
          ds[i >> 1] = pack_bf16x2(pv.x * (g0 - dl) * p.scale, pv.y * (g1 - dl) * p.scale);
        }
      }
      if (capped) {  // dS *= 1 - tanh^2 (S is still intact: dQ overwrites it only after ds_ready)
        uint32_t r0[32], r1[32];
        tmem_ld32(t_lane + C_S + (uint32_t)col0, r0);
        tmem_ld32(t_lane + C_S + (uint32_t)(col0 + 32), r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float t0 = fast_tanh(__uint_as_float(i < 32 ? r0[i] : r1[i - 32]) * p.scale_over_cap);
          const float t1 = fast_tanh(__uint_as_float(i < 32 ? r0[i + 1] : r1[i - 31]) * p.scale_over_cap);
          const float2 d = unpack_bf16x2(ds[i >> 1]);
          ds[i >> 1] = pack_bf16x2(d.x * (1.f - t0 * t0), d.y * (1.f - t1 * t1));
        }
      }
      ok = mbar_wait(pv_done, ph1, abort_flag, p.status, 902);   // dV MMA has consumed P: the buffer may hold dS now
      if (!ok) break;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(sP + ((ch ^ sw) << 4)) = make_uint4(ds[ch * 4], ds[ch * 4 + 1], ds[ch * 4 + 2], ds[ch * 4 + 3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);

      ok = mbar_wait(dq_full, ph1, abort_flag, p.status, 903);
      if (!ok) break;
      tc_fence_after_sync();
      // dQ partial: TMEM -> registers -> the (now idle) Q/dO stage as an fp32 [128 x 128] tile made of four
      // [128 rows][128 B] swizzled chunks; the store warp adds it to global memory with TMA reduce-add.
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(t_lane + C_S + (uint32_t)col0, r0);
        tmem_ld32(t_lane + C_S + (uint32_t)(col0 + 32), r1);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_read);   // the S / dQ columns may be overwritten by the next S = Q K^T
        // columns [0, 64) go to this iteration's Q stage, [64, 128) to its dO stage (both idle since dq_full)
        uint8_t* c0p = (half == 0 ? smem + OFF_Q : smem + OFF_DO) + (it & 1) * TILE;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint8_t* crow = c0p + cc * 16384 + row * 128;
          const uint32_t* r = cc ? r1 : r0;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(crow + ((j ^ sw) << 4)) = make_uint4(r[j * 4], r[j * 4 + 1], r[j * 4 + 2], r[j * 4 + 3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_staged);
      }
    }
    // dK, dV out (thread <-> key row, 64-column half)
    const int kv_idx = kv0 + row;
    const bool kv_ok = kv_idx < p.Sk;
    bf16* dk_row = p.dk + (long long)b * p.dk_sb + (long long)kv_idx * p.dk_ss + (long long)hkv * p.dk_sh + col0;
    bf16* dv_row = p.dv + (long long)b * p.dv_sb + (long long)kv_idx * p.dv_ss + (long long)hkv * p.dv_sh + col0;
    if (n_iters == 0) {
      if (kv_ok) {
        for (int c = 0; c < 64; c += 8) {
          *reinterpret_cast<uint4*>(dk_row + c) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dv_row + c) = make_uint4(0, 0, 0, 0);
        }
      }
    } else {
      if (ok) ok = mbar_wait(all_done, 0, abort_flag, p.status, 904);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
          uint32_t r[32], r2[32];
          tmem_ld32(t_lane + C_DK + (uint32_t)(col0 + c), r);
          tmem_ld32(t_lane + C_DV + (uint32_t)(col0 + c), r2);
          tmem_ld_wait();
          if (kv_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 v, w;
              v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
              w.x = pack_bf16x2(__uint_as_float(r2[g * 8 + 0]), __uint_as_float(r2[g * 8 + 1]));
              w.y = pack_bf16x2(__uint_as_float(r2[g * 8 + 2]), __uint_as_float(r2[g * 8 + 3]));
              w.z = pack_bf16x2(__uint_as_float(r2[g * 8 + 4]), __uint_as_float(r2[g * 8 + 5]));
              w.w = pack_bf16x2(__uint_as_float(r2[g * 8 + 6]), __uint_as_float(r2[g * 8 + 7]));
              *reinterpret_cast<uint4*>(dk_row + c + g * 8) = v;
              *reinterpret_cast<uint4*>(dv_row + c + g * 8) = w;
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row
__global__ void attn_delta_kernel(const bf16* __restrict__ o, long long o_sb, long long o_ss, long long o_sh,
                                  const bf16* __restrict__ d_o, long long do_sb, long long do_ss, long long do_sh,
                                  float* __restrict__ delta, int B, int S, int H) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (gw >= total) return;
  const int h = (int)(gw % H);
  const int s = (int)((gw / H) % S);
  const int b = (int)(gw / ((long long)H * S));
  const uint2 a = *reinterpret_cast<const uint2*>(o + b * o_sb + s * o_ss + h * o_sh + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(d_o + b * do_sb + s * do_ss + h * do_sh + lane * 4);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
  float acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[((long long)b * H + h) * S + s] = acc;
}

// dq[b, s, h, :] (bf16, strided) = dq_accum[b, s, h, :] (fp32 contiguous); one warp per row
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, long long sb,
                                       long long ss, long long sh, int B, int S, int H) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (gw >= total) return;
  const int h = (int)(gw % H);
  const int s = (int)((gw / H) % S);
  const int b = (int)(gw / ((long long)H * S));
  const float4 v = *reinterpret_cast<const float4*>(acc + gw * 128 + lane * 4);
  uint2 o;
  o.x = pack_bf16x2(v.x, v.y);
  o.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(dq + b * sb + s * ss + h * sh + lane * 4) = o;
}

// fp32 dQ accumulator [B, S, H, 128] contiguous -> 4-D map (d, h, s, b), box 32 x 1 x 128 x 1 (128-byte rows)
static int encode_dq_map(CUtensorMap* m, float* acc, int B, int S, int H) {
  uint64_t dims[4] = {128, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t str[3] = {128 * 4, (uint64_t)H * 128 * 4, (uint64_t)S * H * 128 * 4};
  uint32_t box[4] = {32, 1, 128, 1};
  return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, acc, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace fa_bwd
}  // namespace ob

using namespace ob;

// Everything both entry points share: argument checks (all of them before the first enqueue), tensor maps, the delta
// pre-pass, clearing the dQ accumulator, the main kernel and the fp32 -> bf16 conversion of dQ.  `delta` ([B, H, S]) and
// `dq_accum` ([B, S, H, 128], fp32) are the two work buffers, whoever owns them.
static int launch_flash_bwd(const ObAttnArgs* a, float* delta, float* dq_accum, cudaStream_t stream) {
  if (a->D != 128) OB_FAIL(-2, "flash attention kernels are built for head_dim 128 (got %d)", a->D);
  if (a->B <= 0 || a->S <= 0 || a->H <= 0 || a->Hkv <= 0) OB_FAIL(-4, "empty problem");
  if (a->H % a->Hkv != 0) OB_FAIL(-3, "H (%d) must be a multiple of Hkv (%d)", a->H, a->Hkv);
  int Sk = 0;
  if (int g = ob_attn_check_geometry(a, &Sk))
    OB_FAIL(-5, "unsupported attention geometry (rule %d): S %d Sk %d q_off %d causal %d window %d", g, a->S, Sk,
            a->q_off, a->causal, a->window);
  CUtensorMap tq, tk, tv, tdo, tdq;
  int rc;
  if ((rc = encode_bshd_map(&tq, a->q, a->B, a->S, a->H, a->q_sb, a->q_ss, a->q_sh, 128))) return rc;
  if ((rc = encode_bshd_map(&tk, a->k, a->B, Sk, a->Hkv, a->k_sb, a->k_ss, a->k_sh, 128))) return rc;
  if ((rc = encode_bshd_map(&tv, a->v, a->B, Sk, a->Hkv, a->v_sb, a->v_ss, a->v_sh, 128))) return rc;
  if ((rc = encode_bshd_map(&tdo, a->d_o, a->B, a->S, a->H, a->do_sb, a->do_ss, a->do_sh, 128))) return rc;
  if ((rc = fa_bwd::encode_dq_map(&tdq, dq_accum, a->B, a->S, a->H))) return rc;
  // the shared-memory opt-in is a per-device attribute of the function
  static bool attr_set[64] = {};
  int dev = 0;
  OB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) OB_FAIL(-6, "device ordinal %d outside the supported range [0, 64)", dev);
  if (!attr_set[dev]) {
    OB_CUDA_OK(cudaFuncSetAttribute(fa_bwd::flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    fa_bwd::SMEM_BYTES));
    attr_set[dev] = true;
  }

  const long long rows = (long long)a->B * a->S * a->H;
  const int wpb = 8;  // warps per block
  const unsigned nblk = (unsigned)((rows + wpb - 1) / wpb);
  fa_bwd::attn_delta_kernel<<<nblk, wpb * 32, 0, stream>>>(
      reinterpret_cast<const bf16*>(a->o), a->o_sb, a->o_ss, a->o_sh, reinterpret_cast<const bf16*>(a->d_o), a->do_sb,
      a->do_ss, a->do_sh, delta, a->B, a->S, a->H);
  OB_CUDA_OK(cudaGetLastError());
  // the accumulator may hold a previous call's sums: clear the part this call uses
  OB_CUDA_OK(cudaMemsetAsync(dq_accum, 0, (size_t)rows * 128 * sizeof(float), stream));

  fa_bwd::Params p;
  p.B = a->B; p.S = a->S; p.H = a->H; p.Hkv = a->Hkv;
  p.Sk = Sk; p.q_off = a->q_off;
  p.causal = a->causal; p.window = a->window;
  const float LOG2E = 1.4426950408889634f;
  p.scale = a->scale;
  p.scale_log2 = a->scale * LOG2E;
  p.softcap = a->softcap;
  p.scale_over_cap = a->softcap > 0.f ? a->scale / a->softcap : 0.f;
  p.cap_log2 = a->softcap * LOG2E;
  p.lse = a->lse;
  p.delta = delta;
  p.dq_accum = dq_accum;
  p.dk = reinterpret_cast<bf16*>(a->dk); p.dk_sb = a->dk_sb; p.dk_ss = a->dk_ss; p.dk_sh = a->dk_sh;
  p.dv = reinterpret_cast<bf16*>(a->dv); p.dv_sb = a->dv_sb; p.dv_ss = a->dv_ss; p.dv_sh = a->dv_sh;
  p.status = a->status;
  dim3 grid((Sk + 127) / 128, a->Hkv, a->B);
  fa_bwd::flash_bwd_kernel<<<grid, fa_bwd::THREADS, fa_bwd::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, tdq, p);
  OB_CUDA_OK(cudaGetLastError());
  fa_bwd::attn_dq_convert_kernel<<<nblk, wpb * 32, 0, stream>>>(dq_accum, reinterpret_cast<bf16*>(a->dq), a->dq_sb,
                                                               a->dq_ss, a->dq_sh, a->B, a->S, a->H);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_flash_attn_bwd(const ObAttnArgs* a, cudaStream_t stream) {
  if (a == nullptr) OB_FAIL(-1, "null args");
  if (a->delta == nullptr || a->dq_accum == nullptr) OB_FAIL(-4, "backward needs the delta and dq_accum scratch buffers");
  return launch_flash_bwd(a, a->delta, a->dq_accum, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in flash_attn_noalloc.h)
// ---------------------------------------------------------------------------------------------------------------------
// The backward pass needs two work buffers besides its inputs and outputs: delta[B, H, S] and the fp32 dQ accumulator
// [B, S, H, 128].  ob_flash_attn_bwd() takes them from the caller.  The variant below keeps them in a fixed array that
// is part of the library image, for callers that have no way to obtain device memory of their own.
namespace ob {
namespace fa_bwd_static {

constexpr long long MAX_ROWS = OB_FLASH_BWD_STATIC_MAX_ROWS;             // B * S * H
constexpr long long SCRATCH_FLOATS = MAX_ROWS * 128 + MAX_ROWS;          // dQ accumulator, then delta

static __device__ __align__(256) float g_scratch[SCRATCH_FLOATS];

// In host code `g_scratch` is only a handle for the runtime, not an address a kernel may use; the device address is
// looked up once per device with cudaGetSymbolAddress and cached here.
constexpr int MAX_DEVICES = 64;
static float* g_scratch_dev[MAX_DEVICES] = {nullptr};

static int scratch_for_current_device(float** out) {
  int dev = -1;
  OB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) OB_FAIL(-21, "device ordinal %d outside the supported range [0, %d)", dev, MAX_DEVICES);
  if (g_scratch_dev[dev] == nullptr) {
    float* p = nullptr;
    OB_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch));
    if (p == nullptr) OB_FAIL(-22, "cudaGetSymbolAddress returned a null scratch address");
    g_scratch_dev[dev] = p;
  }
  *out = g_scratch_dev[dev];
  return 0;
}

}  // namespace fa_bwd_static
}  // namespace ob

extern "C" int ob_flash_attn_bwd_static(const ObAttnArgs* a, cudaStream_t stream) {
  using namespace ob::fa_bwd_static;
  if (a == nullptr) OB_FAIL(-1, "null args");
  if (a->B <= 0 || a->S <= 0 || a->H <= 0 || a->Hkv <= 0) OB_FAIL(-4, "empty problem");
  const long long rows = (long long)a->B * a->S * a->H;
  if (rows > MAX_ROWS)
    OB_FAIL(-20, "B*S*H = %lld exceeds the %lld rows the built-in work area holds; use ob_flash_attn_bwd with "
                 "caller-provided buffers for larger problems", rows, (long long)MAX_ROWS);
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  // dQ accumulator [rows, 128] first, delta [rows] after the accumulator's full-size region
  return launch_flash_bwd(a, scratch + MAX_ROWS * 128, scratch, stream);
}
