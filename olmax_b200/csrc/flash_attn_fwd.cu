// Flash-attention forward for sm_100a (head_dim 128, bf16 in/out, fp32 softmax statistics).
//
// A persistent CTA (one per SM) takes work items from a counter in global memory.  A work item is a pair of
// 128-row query tiles of one (batch, head).  S = Q K^T and O += P V run on tcgen05 tensor cores with accumulators in
// TMEM: each query tile owns 128 fp32 columns for S and 128 for O (512 columns in all); P (bf16) is written back
// over its S columns and is consumed from TMEM as the A operand of the second MMA, so P never touches shared
// memory.  Each query tile has its own softmax warpgroup (4 warps, one thread per query row, the whole 128-score
// row in registers, so no exchange between threads), and the MMA warp interleaves the two tiles:
//     P V (tile 0, keys j), Q K^T (tile 0, keys j+1), P V (tile 1, keys j), Q K^T (tile 1, keys j+1), ...
// so that the tensor cores work on one tile while the other tile is in its softmax.  P is announced in two halves, so
// that P V of the first 64 keys runs under the exponentials of the rest.  K and V tiles go through rings shared by
// both query tiles (three K stages, two V stages; K is loaded one tile ahead of V because the next Q K^T is issued
// before the current P V).  The softmax warpgroups take registers from the producer warpgroup (`setmaxnreg`), so that
// the 128-score row stays in registers without spills.  The running maximum is only raised when it grows by more
// than 2^8 ("lazy rescale"), which keeps the O correction (a TMEM read-modify-write) off most iterations.
//
// Work items are handed out heaviest first inside groups of eight (batch, head) slices, so that the CTAs that run
// at the same time read the K / V of few heads (L2 reuse) and the light items fill the tail.
//
// Supports: causal masking, grouped-query attention (H a multiple of Hkv), a left sliding window, tanh soft-capping
// of the logits, arbitrary element strides for Q/K/V (so they can be slices of one fused QKV buffer) and sequence
// lengths that are not a multiple of the tile.  Writes O (bf16) and the log-sum-exp of every row (natural log).
//
// Takes the place of the cuDNN / TransformerEngine fused attention the reference calls in
// `olmax/nn/attention.py:52-109`; soft-cap has no counterpart there.
#include <atomic>

#include "flash_attn.h"
#include "host_common.h"
#include "sm100.cuh"

namespace ob {

namespace fa_fwd {

constexpr int TQ = 128;   // query rows per tile; a work item has two tiles
constexpr int TK = 128;   // keys per iteration
constexpr int HD = 128;   // head dim
constexpr int BLK = 128 * 64 * 2;            // one [128 rows][64 elems] swizzled block: 16 KiB
constexpr int TILE_BYTES = 2 * BLK;          // [128][128] bf16 as two blocks
constexpr int STK = 3, STV = 2;             // K and V ring depths (K is needed one MMA group earlier than V)
constexpr int SMEM_BYTES = (2 + STK + STV) * TILE_BYTES + 1024 + 1024;   // Q pair, K ring, V ring, barriers, alignment
constexpr int THREADS = 384;   // warpgroup 0: TMA / scheduler warp, MMA warp, two idle warps; warpgroups 1, 2: softmax
constexpr int TMEM_COLS = 512;
constexpr int S_COL = 0;      // S of tile i: columns [128 i, 128 i + 128); P (bf16x2, 64 cols) over its first 64
constexpr int O_COL = 256;    // O of tile i: columns [256 + 128 i, ...)
constexpr int GROUP = 8;      // (batch, head) slices per scheduling group
constexpr int N_SCHED = 64;   // ring of work counters (one per launch in flight)

__device__ int g_sched[N_SCHED];

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
  int* sched;                  // work counter, zero at launch
  int n_pairs, n_items;        // query-tile pairs per (batch, head); items in the padded schedule
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// max of three in one instruction
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// The softmax warpgroups keep a whole 128-score row per thread: they take registers from warpgroup 0, whose two
// working warps need few (setmaxnreg moves the per-thread register limit of a whole warpgroup).
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Key-tile ranges of a work item.  Tile i covers query rows [q0 + 128 i, +128); it is inactive (lo > hi) when it
// starts beyond the sequence.  The union [ulo, uhi] is what the K / V rings carry.
struct Geo {
  int q0, h, b, hkv;
  int lo[2], hi[2], ulo, uhi;
};
__device__ __forceinline__ Geo item_geometry(const Params& p, int pair, int h, int b) {
  Geo g;
  g.q0 = pair * 2 * TQ;
  g.h = h;
  g.b = b;
  g.hkv = h / (p.H / p.Hkv);
  const int last = (p.Sk + TK - 1) / TK - 1;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int qp0 = p.q_off + g.q0 + i * TQ;
    int hi = last, lo = 0;
    if (p.causal) hi = min(hi, (qp0 + TQ - 1) / TK);
    if (p.window >= 0) lo = max(0, (qp0 - p.window) / TK);
    if (g.q0 + i * TQ >= p.S) { lo = 1; hi = 0; }
    g.lo[i] = lo;
    g.hi[i] = hi;
  }
  g.ulo = g.lo[0];
  g.uhi = g.hi[0];
  if (g.lo[1] <= g.hi[1]) g.uhi = max(g.uhi, g.hi[1]);   // lo[1] >= lo[0] always
  return g;
}

// schedule position -> (pair, h, b); false for the padding of the last group
__device__ __forceinline__ bool decode_item(const Params& p, int w, int& pair, int& h, int& b) {
  const int per_group = GROUP * p.n_pairs;
  const int g = w / per_group, r = w - g * per_group;
  pair = p.n_pairs - 1 - r / GROUP;          // heaviest (longest causal rows) first
  const int bh = g * GROUP + r % GROUP;
  if (bh >= p.B * p.H) return false;
  b = bh / p.H;
  h = bh - b * p.H;
  return true;
}

__global__ void __launch_bounds__(THREADS, 1)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                              // two tiles
  uint8_t* sK = smem + 2 * TILE_BYTES;             // STK tiles
  uint8_t* sV = smem + (2 + STK) * TILE_BYTES;     // STV tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + STK + STV) * TILE_BYTES);
  uint64_t* item_full = bars + 0;     // [2]
  uint64_t* item_empty = bars + 2;    // [2]  9 arrivals: MMA warp + 8 softmax warps
  uint64_t* q_full = bars + 4;
  uint64_t* q_empty = bars + 5;
  uint64_t* k_full = bars + 6;        // [STK]
  uint64_t* k_empty = bars + 6 + STK;
  uint64_t* v_full = bars + 6 + 2 * STK;   // [STV]
  uint64_t* v_empty = bars + 6 + 2 * STK + STV;
  uint64_t* s_full = bars + 6 + 2 * STK + 2 * STV;   // [2]
  uint64_t* p_full = s_full + 2;          // [2 tiles][2 halves of P]  4 arrivals (one per softmax warp of the tile)
  uint64_t* o_done = s_full + 6;          // [2]
  uint64_t* o_free = s_full + 8;          // [2]  4 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* item_slot = reinterpret_cast<volatile int*>(tmem_slot + 4);   // [2][4]: pair (< 0: end), h, b

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(item_full + i, 1);
      mbar_init(item_empty + i, 9);
      mbar_init(s_full + i, 1);
      mbar_init(p_full + 2 * i, 4);
      mbar_init(p_full + 2 * i + 1, 4);
      mbar_init(o_done + i, 1);
      mbar_init(o_free + i, 4);
    }
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < STK; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
    }
    for (int i = 0; i < STV; ++i) {
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
    }
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
  // lane issues.  A wait that gives up marks the warp `dead`: the loops then run out without issuing anything.
  if (warp == 0) {
    // ---------------- scheduler + TMA producer ----------------
    reg_dealloc<48>();
    const bool leader = elect_one();
    bool dead = false;
    if (leader) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
    }
    uint32_t n_item = 0, k_it = 0;
    while (!dead) {
      int pair = -1, h = 0, b = 0;
      for (;;) {
        int w = 0;
        if (lane == 0) w = atomicAdd(p.sched, 1);
        w = __shfl_sync(0xffffffffu, w, 0);
        if (w >= p.n_items) { pair = -1; break; }
        if (decode_item(p, w, pair, h, b)) break;
      }
      const uint32_t slot = n_item & 1u;
      dead = !mbar_wait(item_empty + slot, ((n_item >> 1) & 1u) ^ 1u, abort_flag, p.status, 400);
      if (dead) break;
      if (lane == 0) {
        item_slot[slot * 4 + 0] = pair;
        item_slot[slot * 4 + 1] = h;
        item_slot[slot * 4 + 2] = b;
        mbar_arrive(item_full + slot);
      }
      if (pair < 0) break;
      const Geo g = item_geometry(p, pair, h, b);
      // K runs one tile ahead of V: the MMA warp issues Q K^T of tile u + 1 before P V of tile u
      auto load_k = [&](int u, uint32_t it) {
        const uint32_t st = it % STK, ph = (it / STK) & 1u;
        if (!dead) dead = !mbar_wait(k_empty + st, ph ^ 1u, abort_flag, p.status, 402);
        if (leader && !dead) {
          mbar_arrive_expect_tx(k_full + st, TILE_BYTES);
          tma_load_4d(sK + st * TILE_BYTES, &tmK, k_full + st, 0, g.hkv, u * TK, b);
          tma_load_4d(sK + st * TILE_BYTES + BLK, &tmK, k_full + st, 64, g.hkv, u * TK, b);
        }
      };
      load_k(g.ulo, k_it);
      // Q after the first K tile: that one can already travel while the previous item's last Q K^T runs
      if (!dead) dead = !mbar_wait(q_empty, (n_item & 1u) ^ 1u, abort_flag, p.status, 401);
      if (leader && !dead) {
        mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
        tma_load_4d(sQ, &tmQ, q_full, 0, h, g.q0, b);
        tma_load_4d(sQ + BLK, &tmQ, q_full, 64, h, g.q0, b);
        tma_load_4d(sQ + TILE_BYTES, &tmQ, q_full, 0, h, g.q0 + TQ, b);
        tma_load_4d(sQ + TILE_BYTES + BLK, &tmQ, q_full, 64, h, g.q0 + TQ, b);
      }
      for (int u = g.ulo; u <= g.uhi; ++u, ++k_it) {
        if (u < g.uhi) load_k(u + 1, k_it + 1);
        const uint32_t st = k_it % STV, ph = (k_it / STV) & 1u;
        if (!dead) dead = !mbar_wait(v_empty + st, ph ^ 1u, abort_flag, p.status, 403);
        if (leader && !dead) {
          mbar_arrive_expect_tx(v_full + st, TILE_BYTES);
          tma_load_4d(sV + st * TILE_BYTES, &tmV, v_full + st, 0, g.hkv, u * TK, b);
          tma_load_4d(sV + st * TILE_BYTES + BLK, &tmV, v_full + st, 64, g.hkv, u * TK, b);
        }
      }
      ++n_item;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    reg_dealloc<48>();
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc_bf16(TQ, TK, 0, 0);
    constexpr uint32_t idesc_o = make_idesc_bf16(TQ, HD, 0, 1);
    // shared-memory descriptors: constant high words, low words (start address in 16-byte units) advanced per step
    const uint64_t dQ = make_smem_desc(smem_u32(sQ), 0, 1024), dK = make_smem_desc(smem_u32(sK), 0, 1024);
    const uint64_t dV = make_smem_desc(smem_u32(sV), BLK, 1024);
    const uint32_t q_lo = (uint32_t)dQ, k_lo = (uint32_t)dK, v_lo = (uint32_t)dV;
    const uint32_t kk_hi = (uint32_t)(dQ >> 32), v_hi = (uint32_t)(dV >> 32);
    constexpr uint32_t TILE16 = TILE_BYTES >> 4;
    bool dead = false;
    uint32_t n_item = 0, k_it = 0;
    uint32_t cs[2] = {0, 0};   // S tiles issued per query tile (phase of s_full / p_full)
    uint32_t ce[2] = {0, 0};   // items in which the query tile was active (phase of o_done / o_free)

    // S_i = Q_i K^T into the S columns of tile i.  In-order execution of this thread's MMAs keeps it behind the
    // previous P V of the same tile, which read P from these columns.
    auto issue_s = [&](int i, uint32_t st) {
      if (leader && !dead) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = ((uint32_t)(kk >> 2) * BLK + (uint32_t)(kk & 3) * 32) >> 4;
          umma_ss_lohi(tmem_base + S_COL + (uint32_t)i * 128u, q_lo + (uint32_t)i * TILE16 + off, kk_hi,
                       k_lo + st * TILE16 + off, kk_hi, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full + i);
      }
    };
    // O_i += P_i V: A = P from TMEM (128 x 16 bf16 per step = 8 columns), B = V as an MN-major operand
    // (issued in two halves of 64 keys, each as soon as its part of P has been written)
    auto issue_pv = [&](int i, int hf, uint32_t st, bool first) {
      if (leader && !dead) {
#pragma unroll
        for (int k4 = 0; k4 < TK / 32; ++k4) {
          const int kk = hf * (TK / 32) + k4;
          umma_ts_lohi(tmem_base + O_COL + (uint32_t)i * 128u, tmem_base + S_COL + (uint32_t)i * 128u + (uint32_t)kk * 8,
                       v_lo + st * TILE16 + (uint32_t)kk * 128u, v_hi, idesc_o, (!first || kk != 0) ? 1u : 0u);
        }
      }
    };

    while (!dead) {
      const uint32_t slot = n_item & 1u;
      dead = !mbar_wait(item_full + slot, (n_item >> 1) & 1u, abort_flag, p.status, 500);
      if (dead) break;
      const int pair = item_slot[slot * 4 + 0], h = item_slot[slot * 4 + 1], b = item_slot[slot * 4 + 2];
      __syncwarp();
      if (lane == 0) mbar_arrive(item_empty + slot);
      if (pair < 0) break;
      const Geo g = item_geometry(p, pair, h, b);
      const bool act1 = g.lo[1] <= g.hi[1];
      dead = !mbar_wait(q_full, n_item & 1u, abort_flag, p.status, 501);
      // first K tile: S of both query tiles
      {
        const uint32_t st = k_it % STK, ph = (k_it / STK) & 1u;
        if (!dead) dead = !mbar_wait(k_full + st, ph, abort_flag, p.status, 502);
        tc_fence_after_sync();
        issue_s(0, st);
        if (act1 && g.lo[1] == g.ulo) issue_s(1, st);
        if (leader && !dead) {
          umma_commit(k_empty + st);
          if (g.ulo == g.uhi) umma_commit(q_empty);
        }
      }
      for (int u = g.ulo; u <= g.uhi; ++u, ++k_it) {
        const uint32_t st = k_it % STV, ph = (k_it / STV) & 1u;                 // V stage of tile u
        const uint32_t st_n = (k_it + 1) % STK, ph_n = ((k_it + 1) / STK) & 1u;   // K stage of tile u + 1
        const bool more = u < g.uhi;
        const bool in0 = u <= g.hi[0];
        const bool in1 = act1 && u >= g.lo[1] && u <= g.hi[1];
        if (!dead) dead = !mbar_wait(v_full + st, ph, abort_flag, p.status, 503);
        if (in0) {
          if (u == g.lo[0] && !dead) dead = !mbar_wait(o_free, (ce[0] & 1u) ^ 1u, abort_flag, p.status, 504);
          if (!dead) dead = !mbar_wait(p_full, cs[0] & 1u, abort_flag, p.status, 505);
          tc_fence_after_sync();
          issue_pv(0, 0, st, u == g.lo[0]);
          if (!dead) dead = !mbar_wait(p_full + 1, cs[0] & 1u, abort_flag, p.status, 509);
          tc_fence_after_sync();
          issue_pv(0, 1, st, u == g.lo[0]);
          if (u == g.hi[0] && leader && !dead) umma_commit(o_done);
          ++cs[0];
        }
        if (more) {
          if (!dead) dead = !mbar_wait(k_full + st_n, ph_n, abort_flag, p.status, 506);
          tc_fence_after_sync();
          if (u + 1 <= g.hi[0]) issue_s(0, st_n);
        }
        if (in1) {
          if (u == g.lo[1] && !dead) dead = !mbar_wait(o_free + 1, (ce[1] & 1u) ^ 1u, abort_flag, p.status, 507);
          if (!dead) dead = !mbar_wait(p_full + 2, cs[1] & 1u, abort_flag, p.status, 508);
          tc_fence_after_sync();
          issue_pv(1, 0, st, u == g.lo[1]);
          if (!dead) dead = !mbar_wait(p_full + 3, cs[1] & 1u, abort_flag, p.status, 510);
          tc_fence_after_sync();
          issue_pv(1, 1, st, u == g.lo[1]);
          if (u == g.hi[1] && leader && !dead) umma_commit(o_done + 1);
          ++cs[1];
        }
        if (leader && !dead) umma_commit(v_empty + st);
        if (more) {
          if (act1 && u + 1 >= g.lo[1] && u + 1 <= g.hi[1]) issue_s(1, st_n);
          if (leader && !dead) {
            umma_commit(k_empty + st_n);
            if (u + 1 == g.uhi) umma_commit(q_empty);
          }
        }
      }
      ++ce[0];
      if (act1) ++ce[1];
      ++n_item;
    }
    __syncwarp();
  } else if (warp < 4) {
    reg_dealloc<48>();   // the rest of warpgroup 0 has no work; the instruction is per warpgroup
  } else {
    // ---------------- softmax + output: one warpgroup per query tile, thread <-> query row ----------------
    reg_alloc<224>();
    const int tile = (warp - 4) >> 2;          // 0: warps 4-7, 1: warps 8-11
    const int qd = warp & 3;                   // TMEM lane quarter this warp may access
    const int row = qd * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t t_s = t_lane + S_COL + (uint32_t)tile * 128u;
    const uint32_t t_o = t_lane + O_COL + (uint32_t)tile * 128u;
    const bool capped = p.softcap > 0.f;
    const float sc = capped ? 1.0f : p.scale_log2;   // soft-capped scores are already in the log2 domain
    bool ok = true;
    uint32_t n_item = 0, cs = 0, ce = 0;
    while (ok) {
      const uint32_t slot = n_item & 1u;
      ok = mbar_wait(item_full + slot, (n_item >> 1) & 1u, abort_flag, p.status, 600);
      if (!ok) break;
      const int pair = item_slot[slot * 4 + 0], h = item_slot[slot * 4 + 1], b = item_slot[slot * 4 + 2];
      __syncwarp();
      if (lane == 0) mbar_arrive(item_empty + slot);
      ++n_item;
      if (pair < 0) break;
      const Geo g = item_geometry(p, pair, h, b);
      if (g.lo[tile] > g.hi[tile]) continue;
      const int q0 = g.q0 + tile * TQ;
      const int qp0 = p.q_off + q0;
      const int q_idx = q0 + row;
      const int q_pos = p.q_off + q_idx;
      const int kv_hi = p.causal ? min(q_pos, p.Sk - 1) : p.Sk - 1;  // last visible key
      const int kv_lo = p.window >= 0 ? q_pos - p.window : 0;        // first visible key
      float m_run = -INFINITY;  // running max, log2 domain
      float l_run = 0.f;
      for (int u = g.lo[tile]; u <= g.hi[tile] && ok; ++u, ++cs) {
        const int kv0 = u * TK;
        ok = mbar_wait(s_full + tile, cs & 1u, abort_flag, p.status, 601);
        if (!ok) break;
        tc_fence_after_sync();
        const bool need_mask = (kv0 + TK > p.Sk) || (p.causal && kv0 + TK - 1 > qp0) ||
                               (p.window >= 0 && kv0 < qp0 + TQ - 1 - p.window);
        // the whole score row in registers, for both the maximum and the exponentials; the second half of the row is
        // still on its way from TMEM while the maximum of the first half is taken
        uint32_t r[4][32];
        tmem_ld32(t_s, r[0]);
        tmem_ld32(t_s + 32u, r[1]);
        tmem_ld_wait();
        tmem_ld32(t_s + 64u, r[2]);
        tmem_ld32(t_s + 96u, r[3]);
        float mx;
        if (!capped && !need_mask) {
          // eight independent chains: a single running maximum would serialise 128 dependent operations
          float m8[8];
#pragma unroll
          for (int k = 0; k < 8; ++k)
            m8[k] = fmax3(__uint_as_float(r[0][k]), __uint_as_float(r[0][k + 8]), __uint_as_float(r[0][k + 16]));
#pragma unroll
          for (int k = 0; k < 8; ++k)
            m8[k] = fmax3(m8[k], __uint_as_float(r[0][k + 24]), __uint_as_float(r[1][k]));
#pragma unroll
          for (int k = 0; k < 8; ++k)
            m8[k] = fmax3(m8[k], __uint_as_float(r[1][k + 8]), __uint_as_float(r[1][k + 16]));
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 8; ++k)
            m8[k] = fmax3(m8[k], __uint_as_float(r[1][k + 24]), __uint_as_float(r[2][k]));
#pragma unroll
          for (int c = 2; c < 4; ++c)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              m8[k] = fmax3(m8[k], __uint_as_float(r[c][k + 8]), __uint_as_float(r[c][k + 16]));
              if (c == 2) m8[k] = fmax3(m8[k], __uint_as_float(r[2][k + 24]), __uint_as_float(r[3][k]));
              else m8[k] = fmaxf(m8[k], __uint_as_float(r[3][k + 24]));
            }
          mx = fmax3(fmax3(m8[0], m8[1], m8[2]), fmax3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7]));
        } else {
          tmem_ld_wait();
          if (capped) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                r[c][i] = __float_as_uint(p.cap_log2 * fast_tanh(__uint_as_float(r[c][i]) * p.scale_over_cap));
          }
          if (need_mask) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int kv = kv0 + c * 32 + i;
                if (kv > kv_hi || kv < kv_lo) r[c][i] = __float_as_uint(-INFINITY);
              }
          }
          float m8[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) m8[k] = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 16)
#pragma unroll
              for (int k = 0; k < 8; ++k)
                m8[k] = fmax3(m8[k], __uint_as_float(r[c][i + k]), __uint_as_float(r[c][i + 8 + k]));
          mx = fmax3(fmax3(m8[0], m8[1], m8[2]), fmax3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7]));
        }
        mx *= sc;                                        // sc > 0: max commutes with the scaling
        const float m_new = fmaxf(m_run, mx);
        // lazy rescale: raise the running max only when it grows by more than 8 (factor 256); warp-uniform decision
        const bool want = (m_new > m_run + 8.0f) || (m_run == -INFINITY && m_new > -INFINITY);
        if (__any_sync(0xffffffffu, want)) {
          const float m_next = want ? m_new : m_run;
          const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_next);
          if (u > g.lo[tile]) {
#pragma unroll 1
            for (int c = 0; c < 128; c += 16) {
              uint32_t o[16];
              tmem_ld16(t_o + (uint32_t)c, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st16(t_o + (uint32_t)c, o);
            }
            tmem_st_wait();
          }
          l_run *= alpha;
          m_run = m_next;
        }
        const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
        // P = exp2(s - m) as bf16 pairs, written over the S columns (the scores are all in registers by now).  The
        // first half of P is announced while the third quarter is being computed, so that the first half of P V runs
        // under the rest of the exponentials.
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(r[c][i]), sc, neg_m));
            const float e1 = fast_exp2(fmaf(__uint_as_float(r[c][i + 1]), sc, neg_m));
            ls[(i >> 1) & 3] += e0 + e1;
            pk[i >> 1] = pack_bf16x2(e0, e1);
          }
          tmem_st16(t_s + (uint32_t)c * 16u, pk);
          if (c == 2) {
            // the stores of quarters 0 and 1 have had a quarter's worth of exponentials to land
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 2 * tile);
          }
        }
        l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 2 * tile + 1);
      }
      // epilogue: wait for the last P V, normalise, store
      if (ok) ok = mbar_wait(o_done + tile, ce & 1u, abort_flag, p.status, 602);
      ++ce;
      if (!ok) break;
      tc_fence_after_sync();
      const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
      const bool row_ok = q_idx < p.S;
      bf16* orow = p.o + (long long)b * p.o_sb + (long long)q_idx * p.o_ss + (long long)h * p.o_sh;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t o[32];
        tmem_ld32(t_o + (uint32_t)c, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * inv_l, __uint_as_float(o[q * 8 + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * inv_l, __uint_as_float(o[q * 8 + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * inv_l, __uint_as_float(o[q * 8 + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * inv_l, __uint_as_float(o[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + q * 8) = v;
          }
        }
      }
      // O of this tile has been read: the next item's first P V may overwrite it
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free + tile);
      if (row_ok) {
        const float lse = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
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
  // persistent CTAs, one per SM, fed from a work counter: a ring of counters so that launches in flight on different
  // streams never share one; the launch's counter is cleared in stream order just before the kernel
  static int n_sm[64] = {};
  static int* sched_base[64] = {};
  if (n_sm[dev] == 0) {
    int n = 0;
    OB_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    void* sym = nullptr;
    OB_CUDA_OK(cudaGetSymbolAddress(&sym, fa_fwd::g_sched));
    sched_base[dev] = static_cast<int*>(sym);
    n_sm[dev] = n;
  }
  static std::atomic<unsigned> launch_no{0};
  p.sched = sched_base[dev] + launch_no.fetch_add(1) % fa_fwd::N_SCHED;
  p.n_pairs = (a->S + 2 * fa_fwd::TQ - 1) / (2 * fa_fwd::TQ);
  const int groups = (a->B * a->H + fa_fwd::GROUP - 1) / fa_fwd::GROUP;
  p.n_items = groups * fa_fwd::GROUP * p.n_pairs;
  OB_CUDA_OK(cudaMemsetAsync(p.sched, 0, sizeof(int), stream));
  const int valid_items = a->B * a->H * p.n_pairs;
  dim3 grid(valid_items < n_sm[dev] ? valid_items : n_sm[dev]);
  fa_fwd::flash_fwd_kernel<<<grid, fa_fwd::THREADS, fa_fwd::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}
