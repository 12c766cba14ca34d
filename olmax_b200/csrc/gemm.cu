// bf16 GEMM for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with fp32 accumulators in TMEM, persistent
// CTAs (one per SM), warp-specialised (TMA producer / MMA issuer / 4 epilogue warps), double-buffered accumulators
// so that the epilogue of tile i overlaps the main loop of tile i+1.
//
// Two tile geometries share one kernel body (template parameter CG):
//   CG = 2 (default): a CTA PAIR (2-CTA cluster on the two SMs of a TPC) computes a 256 x 256 tile with
//          tcgen05.mma.cta_group::2.  Each CTA TMA-loads its own 128 rows of A and its own 128 columns of B per
//          k-block (32 KiB instead of 48 KiB per 128 x 256 x 64 of work), six stages deep; both CTAs' loads complete on
//          the leader's mbarrier, the leader's MMA thread issues for the pair and frees the stages / publishes the
//          accumulator in both CTAs with one tcgen05.commit per CTA (no multicast of any kind).  Each CTA's epilogue
//          drains its own 128 rows from its own TMEM.
//   CG = 1: one CTA computes a 128 x 256 tile (cta_group::1), four stages; used for problems with too few tiles to
//          fill the pairs, and selectable for comparison.
// Accumulating fp32 epilogues (weight gradients) get a split-K tail: the tiles of the last, partly filled wave are
// cut into k slices so that every SM stays busy; the slices meet in the output through the reduce-add epilogue.
//
// One kernel covers the three layouts a Linear layer needs (forward Y = X W^T, dgrad dX = dY W, wgrad dW = dY^T X)
// by letting either operand be K-major or MN-major in shared memory, and covers dim-0-sharded weights by giving
// the B operand / the output a third "shard" coordinate:
//   * forward with gathered weights:  B rows (output columns) come from R buffers `b_shard_stride` apart,
//   * dgrad:                          the contraction runs over R weight shards,
//   * wgrad with reduce-scatter:      output row block s goes to the buffer `c_shards[s]`, which may live in another
//                                     GPU's memory (staged in shared memory, then line-coalesced plain stores or
//                                     red.global over NVLink; never TMA).
// Tensor parallelism with sequence parallelism uses the same two mechanisms on the ACTIVATION side: the all-gather of
// the A operand's row shards is fused in (`ag_on_a`: the copy warps pull the peers' rows while the tensor cores work
// on the local rows), and the reduce-scatter of a row-parallel output is fused into the epilogue (row block s of
// the partial product, plus an optional local partial sum, is stored into GPU s's staging slot).
// Epilogues: bf16 store, fp32 store / accumulate / red.add, and the gated-MLP epilogue act(gate) * up computed from
// a tile whose 256 accumulator columns are 128 gate columns followed by 128 up columns.
//
// Replaces the library GEMM calls behind the reference's `olmax/nn/functional.py:14-27` (linear) and
// `olmax/nn/mlp.py:69-73` (gated MLP).
#include "gemm.h"

#include <stdlib.h>

#include "host_common.h"
#include "sm100.cuh"

namespace ob {

constexpr int BM = 128;   // output rows per CTA (the pair tile has CG * BM rows)
constexpr int BN = 256;   // accumulator columns (MMA N)
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int MN_BLOCK_BYTES = 64 * BK * 2;  // one 64(MN) x 64(K) MN-major block: 8 KiB
constexpr int TMEM_COLS = 512;
constexpr int GEMM_THREADS = 256;  // warp 0 TMA, 1 MMA, 2-5 epilogue, 6-7 peer-copy (fused all-gather)
constexpr int COPY_WARPS = 2;
constexpr int AG_BLOCK_ROWS = 256;  // granularity of the all-gather ready flags
constexpr int EPI_STAGE_BYTES = 128 * 128;  // one 128-row x 128-byte output chunk
constexpr int MAX_STAGES = 6;

// Per-CTA geometry of the two variants: B columns held per CTA, stage size, pipeline depth, shared-memory size.
template <int CG>
struct Geo {
  static constexpr int BNL = BN / CG;                    // B columns (rows of the K-major weight) per CTA
  static constexpr int B_STAGE_BYTES = BNL * BK * 2;     // 32 KiB / 16 KiB
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = CG == 1 ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * EPI_STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct KernelParams {
  int M, N, Kc;
  int M_s, N_s, Kc_s;
  int m_tiles_per_shard, n_tiles_per_shard, k_iters_per_shard;
  int m_shards, n_shards, k_shards;
  int bn_out;  // output columns per tile: 256, or 128 for the gated epilogue
  int epi;
  float alpha;
  void* c;
  void* c2;
  void* c3;
  void* const* c_shards;
  long long c_shard_stride;
  long long ldc;
  int* status;
  int split, full_items, total_items;   // split-K tail: work items [full_items, total_items) are k slices of tiles
  int group_m;                 // tile rasterisation group (M tiles)
  int m_rot;                   // rotation of the M tile order (tiles), see decode_tile
  int a_single, b_single;      // MN-major operand fetched with one 4-D TMA box per stage instead of 64-wide boxes
  int tma_epi;                 // 1: outputs leave through shared memory + TMA store / reduce-add (tmC valid)
  // FSDP all-gather fused into the GEMM: the B operand's remote shards are pulled from peer GPUs (plain loads over
  // NVLink) into the local staging buffer by the copy warps while the tensor cores work on tiles already present.
  int ag_shards;               // 0: off
  int ag_on_a;                 // 1: the gathered operand is A (row shards of a K-major activation), 0: B (weights)
  int ag_rank;                 // this GPU's shard index (its slot of the staging buffer is filled by the host)
  int ag_rows;                 // rows of one shard piece
  int ag_blocks;               // AG_BLOCK_ROWS-row blocks per shard piece
  long long ag_row_bytes;      // bytes of one piece row
  const uint8_t* const* ag_src;    // [ag_shards] piece base in each GPU's memory
  const uint8_t* const* ag_src2;   // second operand of the gated epilogue, or null
  uint8_t* ag_dst;             // staging piece of shard 0 (shard s at + s * ag_dst_stride)
  uint8_t* ag_dst2;
  long long ag_dst_stride;     // bytes
  unsigned* ag_flags;          // [ag_shards * ag_blocks] arrival counters, monotonic across launches
  unsigned ag_target;          // counter value that means "block present" for this launch
  // Prefetch for LATER launches: copy bytes [pf_off, pf_off + pf_bytes) of every remote shard's slice of the next
  // FSDP unit into that unit's staging buffer (consumers are later kernels in stream order, so no flags).
  int pf_shards;               // 0: off
  int pf_rank;
  const uint8_t* const* pf_src;    // [pf_shards] base of the unit slice in each GPU's memory
  uint8_t* pf_dst;             // staging slot of shard 0 (shard s at + s * pf_dst_stride)
  long long pf_dst_stride;
  long long pf_off, pf_bytes;  // multiples of 16
};

// One warp-interleaved copy of n16 16-byte words; cw = this copy warp's index among n_cw.
__device__ __forceinline__ void warp_copy16(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16, int cw,
                                            int n_cw, int lane) {
  long long i = (long long)cw * 32 + lane;
  const long long step = (long long)n_cw * 32;
  // COPY_UNROLL x 16 bytes per lane in flight (a 256-row block of a 4096-wide operand is ~14 words per lane)
  constexpr int COPY_UNROLL = 8;
  for (; i + (COPY_UNROLL - 1) * step < n16; i += COPY_UNROLL * step) {
    uint4 v[COPY_UNROLL];
#pragma unroll
    for (int u = 0; u < COPY_UNROLL; ++u) v[u] = __ldcg(src + i + u * step);
#pragma unroll
    for (int u = 0; u < COPY_UNROLL; ++u) dst[i + u * step] = v[u];
  }
  for (; i + 3 * step < n16; i += 4 * step) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcg(src + i + u * step);
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[i + u * step] = v[u];
  }
  for (; i < n16; i += step) dst[i] = __ldcg(src + i);
}

// Tile rasterisation: tiles are visited in groups of `group_m` consecutive M tiles, all N tiles of a group before the
// next group, M fastest inside.  A wave of ~148 concurrent CTAs then touches group_m A slabs and 148 / group_m B slabs
// instead of every A slab, which keeps the operands of a wave resident in L2.
__device__ __forceinline__ void decode_tile(int tile, int m_tiles, int n_tiles, int group_m, int n_rot, int m_rot,
                                            int& mt, int& nt) {
  const int per_group = group_m * n_tiles;
  const int g = tile / per_group;
  const int within = tile - g * per_group;
  const int gm = min(group_m, m_tiles - g * group_m);
  nt = (within / gm + n_rot) % n_tiles;
  // m_rot staggers the output row shards by rank, so that GPUs adding into each other's shards do not all target the
  // same owner (and the same addresses) at the same time
  mt = (g * group_m + within % gm + m_rot) % m_tiles;
}

// Bounded wait for an all-gather block; returns false (and records the error) when it does not arrive.
__device__ __forceinline__ bool ag_wait(const KernelParams& p, int shard, int block, volatile int* abort_flag) {
  if (p.ag_shards == 0 || shard == p.ag_rank) return true;
  const unsigned* f = p.ag_flags + shard * p.ag_blocks + block;
  for (unsigned it = 0; it < (1u << 26); ++it) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int)(v - p.ag_target) >= 0) {
      asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores -> async-proxy (TMA) reads
      return true;
    }
    if ((it & 255u) == 255u && *abort_flag) return false;
    __nanosleep(64);
  }
  *abort_flag = 1;
  report_error(p.status, ERR_PEER_TIMEOUT, 110, shard * 1000 + block);
  return false;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// Work item w of a launch: a whole tile, or (in the split-K tail) one k slice of a tile.
__device__ __forceinline__ void decode_work(const KernelParams& p, int w, int k_iters, int& tile, int& k_begin, int& k_count) {
  if (w < p.full_items) {
    tile = w;
    k_begin = 0;
    k_count = k_iters;
  } else {
    const int idx = w - p.full_items;
    tile = p.full_items + idx / p.split;
    const int sl = idx % p.split;
    k_begin = (int)((long long)k_iters * sl / p.split);
    k_count = (int)((long long)k_iters * (sl + 1) / p.split) - k_begin;
  }
}

template <bool A_MN, bool B_MN, int CG>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmB2,
                                          const CUtensorMap& tmC, const KernelParams& p) {
  using G = Geo<CG>;
  constexpr int STAGES = G::STAGES;
  constexpr int STAGE_BYTES = G::STAGE_BYTES;
  constexpr int BNL = G::BNL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;   // 2 x 16 KiB output staging, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + 2 * EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                           // [STAGES]  (CG = 2: only the leader's are used)
  uint64_t* empty_bar = bars + MAX_STAGES;             // [STAGES]
  uint64_t* tfull_bar = bars + 2 * MAX_STAGES;         // [2]
  uint64_t* tempty_bar = bars + 2 * MAX_STAGES + 2;    // [2]       (CG = 2: only the leader's are used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta_rank = CG == 2 ? (int)cluster_ctarank() : 0;   // 0 = leader
  const int worker = (int)blockIdx.x / CG;                     // index of this CTA (pair) among the persistent workers
  const int n_workers = (int)gridDim.x / CG;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4 * CG);   // lane 0 of every epilogue warp of the CTA (pair)
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    if (CG == 2) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if (CG == 2) cluster_sync_all(); else __syncthreads();   // barriers of BOTH CTAs exist before any remote signal
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // shared::cluster addresses of the leader's and the peer's barrier arrays (CG = 2)
  const uint32_t bars_leader = CG == 2 ? mapa_shared(smem_u32(bars), 0) : smem_u32(bars);
  const uint32_t bars_peer = CG == 2 ? mapa_shared(smem_u32(bars), 1) : smem_u32(bars);

  const int m_tiles = p.m_shards * p.m_tiles_per_shard;     // tiles of CG * BM rows
  const int n_tiles = p.n_shards * p.n_tiles_per_shard;
  const int k_iters = p.k_shards * p.k_iters_per_shard;
  const bool glu = (p.epi == EPI_SWIGLU || p.epi == EPI_GEGLU);
  // With a fused all-gather the tile order is rotated so that work on the local shard comes first and the other
  // shards follow in the order the copy warps fetch them (rank+1, rank+2, ...).
  const int n_rot = (p.ag_shards > 0 && !p.ag_on_a && !B_MN) ? p.ag_rank * p.n_tiles_per_shard : 0;
  const int k_rot = (p.ag_shards > 0 && !p.ag_on_a && B_MN) ? p.ag_rank * p.k_iters_per_shard : 0;

  // The producer and MMA warps run their loops with all 32 lanes (loop state stays warp-uniform); the one elected
  // lane issues the TMA / tcgen05 instructions.  A wait that gives up marks the warp `dead`: the loops then run to
  // their end without issuing anything, and the other roles give up at their own next wait.
  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (glu) tma_prefetch_desc(&tmB2);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool dead = false;
    // Fused all-gather: the copy warps of every CTA fetch the shards in the order rank+1, rank+2, ... and the blocks
    // of a shard in order, so arrival is monotone in  idx = ((shard - rank) mod S) * blocks + block.  The flag of a
    // block is polled (an L2 round trip with acquire semantics) only while idx is beyond the newest block seen
    // ready: once per block and CTA over the whole kernel instead of once per k-iteration.
    int ag_ready_idx = p.ag_blocks - 1;   // the local shard is always present
    for (int w = worker; w < p.total_items; w += n_workers) {
      int tile, k_begin, k_count, mt, nt;
      decode_work(p, w, k_iters, tile, k_begin, k_count);
      decode_tile(tile, m_tiles, n_tiles, p.group_m, n_rot, p.m_rot, mt, nt);
      const int m_local0 = (mt % p.m_tiles_per_shard) * (BM * CG) + cta_rank * BM;   // this CTA's rows in the shard
      const int m0 = (mt / p.m_tiles_per_shard) * p.M_s + m_local0;
      const int n_shard = nt / p.n_tiles_per_shard;
      const int n_local0 = (nt % p.n_tiles_per_shard) * p.bn_out;
      // k position, advanced without divisions inside the loop
      const int kit_first = (k_begin + k_rot) % k_iters;
      int k_shard = kit_first / p.k_iters_per_shard;
      int k_local = (kit_first % p.k_iters_per_shard) * BK;
      const int k_local_end = p.k_iters_per_shard * BK;
      for (int i = 0; i < k_count; ++i) {
        const int k_glob = k_shard * p.Kc_s + k_local;
        if (!dead) dead = !mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 100);
        if (p.ag_shards > 0 && !dead) {
          int ag_s, ag_b;
          if (p.ag_on_a) {
            ag_s = mt / p.m_tiles_per_shard;
            ag_b = min(m_local0, p.M_s - 1) / AG_BLOCK_ROWS;
          } else if (B_MN) {
            ag_s = k_shard;
            ag_b = k_local / AG_BLOCK_ROWS;
          } else {
            ag_s = n_shard;
            ag_b = n_local0 / AG_BLOCK_ROWS;
          }
          const int ag_idx = ((ag_s - p.ag_rank + p.ag_shards) % p.ag_shards) * p.ag_blocks + ag_b;
          if (ag_idx > ag_ready_idx) {
            dead = !ag_wait(p, ag_s, ag_b, abort_flag);
            ag_ready_idx = ag_idx;
          }
        }
        uint8_t* sa = smem + stage * STAGE_BYTES;
        uint8_t* sb = sa + A_STAGE_BYTES;
        if (leader && !dead) {
          if (CG == 1) {
            mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
            if (A_MN) {
              if (p.a_single) {
                // one 4-D box: (64 elements, 64 k-rows, 2 column blocks): lands as [block][k][128 B]
                tma_load_4d(sa, &tmA, &full_bar[stage], 0, k_glob, m0 >> 6, 0);
              } else {
                tma_load_3d(sa, &tmA, &full_bar[stage], m0, k_glob, 0);
                tma_load_3d(sa + MN_BLOCK_BYTES, &tmA, &full_bar[stage], m0 + 64, k_glob, 0);
              }
            } else {
              tma_load_3d(sa, &tmA, &full_bar[stage], k_glob, m0, 0);
            }
            if (B_MN) {
              // dims (N, Kc_s, k_shards): four 64-wide blocks along N
              const int n0 = n_local0;  // MN-major B is never N-sharded
              if (p.b_single) {
                tma_load_4d(sb, &tmB, &full_bar[stage], 0, k_local, n0 >> 6, k_shard);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  tma_load_3d(sb + j * MN_BLOCK_BYTES, &tmB, &full_bar[stage], n0 + j * 64, k_local, k_shard);
              }
            } else if (glu) {
              tma_load_3d(sb, &tmB, &full_bar[stage], k_glob, n_local0, n_shard);
              tma_load_3d(sb + G::B_STAGE_BYTES / 2, &tmB2, &full_bar[stage], k_glob, n_local0, n_shard);
            } else {
              tma_load_3d(sb, &tmB, &full_bar[stage], k_glob, n_local0, n_shard);
            }
          } else {
            // CTA pair: both CTAs' copies complete on the leader's barrier, which expects the bytes of both
            const uint32_t fb = bars_leader + (uint32_t)stage * 8u;
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
            if (A_MN) {
              if (p.a_single) {
                tma_load_4d_pair(sa, &tmA, fb, 0, k_glob, m0 >> 6, 0);
              } else {
                tma_load_3d_pair(sa, &tmA, fb, m0, k_glob, 0);
                tma_load_3d_pair(sa + MN_BLOCK_BYTES, &tmA, fb, m0 + 64, k_glob, 0);
              }
            } else {
              tma_load_3d_pair(sa, &tmA, fb, k_glob, m0, 0);
            }
            if (B_MN) {
              const int n0 = n_local0 + cta_rank * BNL;   // this CTA's half of the tile's columns: two 64-wide blocks
              if (p.b_single) {
                tma_load_4d_pair(sb, &tmB, fb, 0, k_local, n0 >> 6, k_shard);
              } else {
#pragma unroll
                for (int j = 0; j < BNL / 64; ++j)
                  tma_load_3d_pair(sb + j * MN_BLOCK_BYTES, &tmB, fb, n0 + j * 64, k_local, k_shard);
              }
            } else if (glu) {
              // accumulator columns [0,128) = gate (leader's B half), [128,256) = up (peer's B half)
              tma_load_3d_pair(sb, cta_rank == 0 ? &tmB : &tmB2, fb, k_glob, n_local0, n_shard);
            } else {
              tma_load_3d_pair(sb, &tmB, fb, k_glob, n_local0 + cta_rank * BNL, n_shard);
            }
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        k_local += BK;
        if (k_local == k_local_end) {
          k_local = 0;
          if (++k_shard == p.k_shards) k_shard = 0;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (CG = 2: the leader CTA issues for the pair) ----------------------
    const bool leader = elect_one();
    if (cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM * CG, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool dead = false;
      // descriptors of stage 0; the loop only adds to the low word (start address, 16-byte units, never carries out)
      const uint64_t da0 = A_MN ? make_smem_desc(smem_u32(smem), MN_BLOCK_BYTES, 1024) : make_smem_desc(smem_u32(smem), 0, 1024);
      const uint64_t db0 = B_MN ? make_smem_desc(smem_u32(smem) + A_STAGE_BYTES, MN_BLOCK_BYTES, 1024)
                                : make_smem_desc(smem_u32(smem) + A_STAGE_BYTES, 0, 1024);
      const uint32_t a_lo0 = (uint32_t)da0, a_hi = (uint32_t)(da0 >> 32);
      const uint32_t b_lo0 = (uint32_t)db0, b_hi = (uint32_t)(db0 >> 32);
      for (int w = worker; w < p.total_items; w += n_workers, ++it) {
        int tile, k_begin, k_count;
        decode_work(p, w, k_iters, tile, k_begin, k_count);
        const int buf = it & 1;
        const uint32_t tphase = (uint32_t)(it >> 1) & 1u;
        if (!dead) dead = !mbar_wait(&tempty_bar[buf], tphase ^ 1u, abort_flag, p.status, 200);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kit = 0; kit < k_count; ++kit) {
          if (!dead) dead = !mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 201);
          tc_fence_after_sync();
          if (leader && !dead) {
            const uint32_t a_lo = a_lo0 + (uint32_t)stage * (uint32_t)(STAGE_BYTES >> 4);
            const uint32_t b_lo = b_lo0 + (uint32_t)stage * (uint32_t)(STAGE_BYTES >> 4);
#pragma unroll
            for (int k4 = 0; k4 < BK / 16; ++k4) {
              // advancing 16 elements along K: 32 bytes inside the 128-byte swizzle row of a K-major tile, 16 rows of
              // 128 bytes in an MN-major tile; the start-address field counts 16-byte units
              const uint32_t al = a_lo + (uint32_t)k4 * (A_MN ? 128u : 2u);
              const uint32_t bl = b_lo + (uint32_t)k4 * (B_MN ? 128u : 2u);
              if (CG == 2) umma_ss_pair_lohi(d_tmem, al, a_hi, bl, b_hi, idesc, (kit | k4) != 0 ? 1u : 0u);
              else umma_ss_lohi(d_tmem, al, a_hi, bl, b_hi, idesc, (kit | k4) != 0 ? 1u : 0u);
            }
            // free the stage (in both CTAs) once these MMAs have read it
            if (CG == 2) {
              umma_commit_pair(bars_leader + (uint32_t)(MAX_STAGES + stage) * 8u);
              umma_commit_pair(bars_peer + (uint32_t)(MAX_STAGES + stage) * 8u);
            } else {
              umma_commit(&empty_bar[stage]);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (leader && !dead) {
          if (CG == 2) {
            umma_commit_pair(bars_leader + (uint32_t)(2 * MAX_STAGES + buf) * 8u);
            umma_commit_pair(bars_peer + (uint32_t)(2 * MAX_STAGES + buf) * 8u);
          } else {
            umma_commit(&tfull_bar[buf]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ------------------------------- peer-copy warps (fused all-gather) -------------------------------
    const int cw = (int)blockIdx.x * COPY_WARPS + (warp - 6);      // this copy warp's index
    const int n_cw = (int)gridDim.x * COPY_WARPS;
    if (p.ag_shards > 0) {
      for (int ds = 1; ds < p.ag_shards; ++ds) {
        const int s = (p.ag_rank + ds) % p.ag_shards;
        for (int b = 0; b < p.ag_blocks; ++b) {
          const int rows = min(AG_BLOCK_ROWS, p.ag_rows - b * AG_BLOCK_ROWS);
          const long long bytes = (long long)rows * p.ag_row_bytes;           // multiple of 16
          const long long off = (long long)b * AG_BLOCK_ROWS * p.ag_row_bytes;
          const long long n16 = bytes >> 4;
          // each copy warp moves an interleaved slice of the block, 4 x 16 bytes per lane in flight
          for (int which = 0; which < (p.ag_src2 != nullptr ? 2 : 1); ++which) {
            const uint4* src = reinterpret_cast<const uint4*>((which ? p.ag_src2[s] : p.ag_src[s]) + off);
            uint4* dst = reinterpret_cast<uint4*>((which ? p.ag_dst2 : p.ag_dst) + (long long)s * p.ag_dst_stride + off);
            warp_copy16(src, dst, n16, cw, n_cw, lane);
          }
          __syncwarp();
          if (lane == 0) {
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.ag_flags + s * p.ag_blocks + b) : "memory");
          }
        }
      }
    }
    if (p.pf_shards > 0 && p.pf_bytes > 0) {
      for (int ds = 1; ds < p.pf_shards; ++ds) {
        const int s = (p.pf_rank + ds) % p.pf_shards;
        warp_copy16(reinterpret_cast<const uint4*>(p.pf_src[s] + p.pf_off),
                    reinterpret_cast<uint4*>(p.pf_dst + (long long)s * p.pf_dst_stride + p.pf_off), p.pf_bytes >> 4, cw,
                    n_cw, lane);
      }
    }
  } else {
    // ------------------------------- epilogue (warps 2..5) -------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int row_in_tile = q * 32 + lane;
    int it = 0;
    bool ok = true;
    for (int w = worker; w < p.total_items && ok; w += n_workers, ++it) {
      const int buf = it & 1;
      const uint32_t tphase = (uint32_t)(it >> 1) & 1u;
      int tile, k_begin, k_count, mt, nt;
      decode_work(p, w, k_iters, tile, k_begin, k_count);
      decode_tile(tile, m_tiles, n_tiles, p.group_m, n_rot, p.m_rot, mt, nt);
      const int m_shard = mt / p.m_tiles_per_shard;
      const int m_local0 = (mt % p.m_tiles_per_shard) * (BM * CG) + cta_rank * BM;   // this CTA's 128 rows
      const int n_shard = nt / p.n_tiles_per_shard;
      const int n_local0 = (nt % p.n_tiles_per_shard) * p.bn_out;
      const int m_valid = max(0, min(BM, p.M_s - m_local0));
      const int n_valid = min(p.bn_out, p.N_s - n_local0);
      const int n_glob0 = n_shard * p.N_s + n_local0;
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(q * 32) << 16);
      const bool row_ok = row_in_tile < m_valid;
      // Row base pointers.  With c_shards the output rows of shard s live in buffer c_shards[s].
      long long row_off;
      uint8_t* cbase;
      if (p.c_shards != nullptr) {
        cbase = reinterpret_cast<uint8_t*>(p.c_shards[m_shard]);
        row_off = (long long)(m_local0 + row_in_tile) * p.ldc + n_glob0;
      } else if (p.c_shard_stride > 0) {
        cbase = reinterpret_cast<uint8_t*>(p.c);
        row_off = (long long)m_shard * p.c_shard_stride + (long long)(m_local0 + row_in_tile) * p.ldc + n_glob0;
      } else {
        cbase = reinterpret_cast<uint8_t*>(p.c);
        row_off = (long long)(m_shard * p.M_s + m_local0 + row_in_tile) * p.ldc + n_glob0;
      }
      if (p.tma_epi) {
        // Output through shared memory + TMA: each thread writes its row's 128 bytes of the chunk into a swizzled
        // staging tile, one thread issues a bulk tensor store (or reduce-add for the accumulating epilogue).  The
        // TMA clips at the tensor / shard boundary, so partial tiles need no per-element guards.
        const bool f32 = !(p.epi == EPI_BF16 || p.epi == EPI_BF16_ACC);
        const int cols = f32 ? 32 : 64;                      // columns per 128-byte chunk row
        // EPI_BF16_ACC towards c_shards: the LOCAL partial sum in p.c ([M, N], row stride ldc) is folded in first
        const bf16* prior_row = (p.epi == EPI_BF16_ACC && p.tma_epi == 2 && row_ok)
            ? reinterpret_cast<const bf16*>(p.c) + (long long)(m_shard * p.M_s + m_local0 + row_in_tile) * p.ldc + n_glob0
            : nullptr;
        const int out_row = (p.c_shard_stride > 0) ? m_local0 : m_shard * p.M_s + m_local0;
        const int out_z = (p.c_shard_stride > 0) ? m_shard : 0;
        const bool store_thread = (threadIdx.x == 64);
        int chunk = 0;
        for (int c0 = 0; c0 < BN; c0 += cols, ++chunk) {
          if (c0 >= n_valid) break;
          uint8_t* stage_buf = epi_smem + (chunk & 1) * EPI_STAGE_BYTES;
          if (store_thread && p.tma_epi == 1) tma_store_wait_read<1>();   // the store that last read this buffer is done
          asm volatile("bar.sync 1, 128;" ::: "memory");
          uint32_t r[32], r2[32];
          tmem_ld32(t_row + (uint32_t)c0, r);
          if (!f32) tmem_ld32(t_row + (uint32_t)(c0 + 32), r2);
          tmem_ld_wait();
          uint8_t* srow = stage_buf + row_in_tile * 128;
          const int sw = row_in_tile & 7;
          if (f32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v = make_float4(__uint_as_float(r[j * 4 + 0]) * p.alpha, __uint_as_float(r[j * 4 + 1]) * p.alpha,
                                     __uint_as_float(r[j * 4 + 2]) * p.alpha, __uint_as_float(r[j * 4 + 3]) * p.alpha);
              *reinterpret_cast<float4*>(srow + ((j ^ sw) << 4)) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t* src = (j < 4) ? &r[j * 8] : &r2[(j - 4) * 8];
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(src[e]) * p.alpha;
              if (prior_row != nullptr && c0 + j * 8 + 8 <= n_valid) {
                const uint4 o = *reinterpret_cast<const uint4*>(prior_row + c0 + j * 8);
                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 t = unpack_bf16x2(ow[e]);
                  f[2 * e] += t.x;
                  f[2 * e + 1] += t.y;
                }
              }
              uint4 v;
              v.x = pack_bf16x2(f[0], f[1]);
              v.y = pack_bf16x2(f[2], f[3]);
              v.z = pack_bf16x2(f[4], f[5]);
              v.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(srow + ((j ^ sw) << 4)) = v;
            }
          }
          if (p.tma_epi == 1) {
            fence_proxy_async();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (store_thread) {
              if (m_valid > 0) {   // a pair tile's second half may lie wholly below the shard
                if (p.epi == EPI_F32_ACC) tma_reduce_add_3d(&tmC, stage_buf, n_glob0 + c0, out_row, out_z);
                else tma_store_3d(&tmC, stage_buf, n_glob0 + c0, out_row, out_z);
              }
              tma_store_commit();
            }
          } else {
            // Destination may be another GPU's memory (no TMA there): the four epilogue warps write the staged chunk
            // out cooperatively, 8 lanes per 128-byte row segment, so that every store instruction covers whole
            // 128-byte lines (NVLink moves full lines far better than scattered 16-byte pieces).
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int et = (int)threadIdx.x - 64;          // 0..127
            const int piece = et & 7;
            uint8_t* dbase = reinterpret_cast<uint8_t*>(p.c_shards[m_shard]);
            const int nv_bytes = min(cols, n_valid - c0) * (f32 ? 4 : 2);
#pragma unroll
            for (int pass = 0; pass < 8; ++pass) {
              const int rr = pass * 16 + (et >> 3);
              if (rr < m_valid && piece * 16 < nv_bytes) {
                const uint4 v = *reinterpret_cast<const uint4*>(stage_buf + rr * 128 + ((piece ^ (rr & 7)) << 4));
                uint8_t* dst = dbase + ((long long)(m_local0 + rr) * p.ldc + n_glob0 + c0) * (f32 ? 4 : 2) + piece * 16;
                if (p.epi == EPI_F32_RED) {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v.x)),
                               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                               : "memory");
                } else {
                  *reinterpret_cast<uint4*>(dst) = v;
                }
              }
            }
          }
        }
      } else if (!glu) {
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (c0 >= n_valid) break;  // warp-uniform
          uint32_t r[32];
          tmem_ld32(t_row + (uint32_t)c0, r);
          tmem_ld_wait();
          if (row_ok) {
            const int nv = min(32, n_valid - c0);
            if (p.epi == EPI_BF16 || p.epi == EPI_BF16_ACC) {
              bf16* dst = reinterpret_cast<bf16*>(cbase) + row_off + c0;
              if (p.epi == EPI_BF16_ACC) {
                // fold the existing C into the accumulator registers, then fall through to the plain store
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  if (g * 8 + 8 <= nv) {
                    const uint4 o = *reinterpret_cast<const uint4*>(dst + g * 8);
                    const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const float2 f = unpack_bf16x2(ow[j]);
                      r[g * 8 + 2 * j] = __float_as_uint(__uint_as_float(r[g * 8 + 2 * j]) + f.x / p.alpha);
                      r[g * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(r[g * 8 + 2 * j + 1]) + f.y / p.alpha);
                    }
                  } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                      if (g * 8 + j < nv)
                        r[g * 8 + j] = __float_as_uint(__uint_as_float(r[g * 8 + j]) +
                                                       __bfloat162float(dst[g * 8 + j]) / p.alpha);
                  }
                }
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (g * 8 + 8 <= nv) {
                  uint4 v;
                  v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]) * p.alpha, __uint_as_float(r[g * 8 + 1]) * p.alpha);
                  v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * p.alpha, __uint_as_float(r[g * 8 + 3]) * p.alpha);
                  v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * p.alpha, __uint_as_float(r[g * 8 + 5]) * p.alpha);
                  v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * p.alpha, __uint_as_float(r[g * 8 + 7]) * p.alpha);
                  *reinterpret_cast<uint4*>(dst + g * 8) = v;
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (g * 8 + j < nv) dst[g * 8 + j] = __float2bfloat16(__uint_as_float(r[g * 8 + j]) * p.alpha);
                }
              }
            } else {
              float* dst = reinterpret_cast<float*>(cbase) + row_off + c0;
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                if (g * 4 + 4 <= nv) {
                  float4 v = make_float4(__uint_as_float(r[g * 4 + 0]) * p.alpha, __uint_as_float(r[g * 4 + 1]) * p.alpha,
                                         __uint_as_float(r[g * 4 + 2]) * p.alpha, __uint_as_float(r[g * 4 + 3]) * p.alpha);
                  float4* d4 = reinterpret_cast<float4*>(dst + g * 4);
                  if (p.epi == EPI_F32) {
                    *d4 = v;
                  } else if (p.epi == EPI_F32_ACC) {
                    float4 o = *d4;
                    o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
                    *d4 = o;
                  } else {  // EPI_F32_RED: the destination may be another GPU's memory
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d4), "f"(v.x), "f"(v.y),
                                 "f"(v.z), "f"(v.w)
                                 : "memory");
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (g * 4 + j < nv) {
                      float v = __uint_as_float(r[g * 4 + j]) * p.alpha;
                      if (p.epi == EPI_F32) dst[g * 4 + j] = v;
                      else if (p.epi == EPI_F32_ACC) dst[g * 4 + j] += v;
                      else atomicAdd(dst + g * 4 + j, v);
                    }
                  }
                }
              }
            }
          }
        }
      } else {
        // gated epilogue: columns [0,128) = gate, [128,256) = up
        bf16* cact = reinterpret_cast<bf16*>(p.c);
        bf16* cg = reinterpret_cast<bf16*>(p.c2);
        bf16* cu = reinterpret_cast<bf16*>(p.c3);
        for (int c0 = 0; c0 < 128; c0 += 16) {
          if (c0 >= n_valid) break;
          uint32_t g[16], u[16];
          tmem_ld16(t_row + (uint32_t)c0, g);
          tmem_ld16(t_row + (uint32_t)(128 + c0), u);
          tmem_ld_wait();
          if (row_ok) {
            const int nv = min(16, n_valid - c0);
            float a[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // round gate / up to bf16 first so that act(g)*u matches what a backward pass recomputes from them
              float gf = __bfloat162float(__float2bfloat16(__uint_as_float(g[j])));
              float uf = __bfloat162float(__float2bfloat16(__uint_as_float(u[j])));
              a[j] = (p.epi == EPI_SWIGLU ? silu(gf) : gelu_tanh(gf)) * uf;
            }
            const long long off = row_off + c0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (h * 8 + 8 <= nv) {
                uint4 va, vg, vu;
                va.x = pack_bf16x2(a[h * 8 + 0], a[h * 8 + 1]);
                va.y = pack_bf16x2(a[h * 8 + 2], a[h * 8 + 3]);
                va.z = pack_bf16x2(a[h * 8 + 4], a[h * 8 + 5]);
                va.w = pack_bf16x2(a[h * 8 + 6], a[h * 8 + 7]);
                *reinterpret_cast<uint4*>(cact + off + h * 8) = va;
                if (cg != nullptr) {
                  vg.x = pack_bf16x2(__uint_as_float(g[h * 8 + 0]), __uint_as_float(g[h * 8 + 1]));
                  vg.y = pack_bf16x2(__uint_as_float(g[h * 8 + 2]), __uint_as_float(g[h * 8 + 3]));
                  vg.z = pack_bf16x2(__uint_as_float(g[h * 8 + 4]), __uint_as_float(g[h * 8 + 5]));
                  vg.w = pack_bf16x2(__uint_as_float(g[h * 8 + 6]), __uint_as_float(g[h * 8 + 7]));
                  *reinterpret_cast<uint4*>(cg + off + h * 8) = vg;
                  vu.x = pack_bf16x2(__uint_as_float(u[h * 8 + 0]), __uint_as_float(u[h * 8 + 1]));
                  vu.y = pack_bf16x2(__uint_as_float(u[h * 8 + 2]), __uint_as_float(u[h * 8 + 3]));
                  vu.z = pack_bf16x2(__uint_as_float(u[h * 8 + 4]), __uint_as_float(u[h * 8 + 5]));
                  vu.w = pack_bf16x2(__uint_as_float(u[h * 8 + 6]), __uint_as_float(u[h * 8 + 7]));
                  *reinterpret_cast<uint4*>(cu + off + h * 8) = vu;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (h * 8 + j < nv) {
                    cact[off + h * 8 + j] = __float2bfloat16(a[h * 8 + j]);
                    if (cg != nullptr) {
                      cg[off + h * 8 + j] = __float2bfloat16(__uint_as_float(g[h * 8 + j]));
                      cu[off + h * 8 + j] = __float2bfloat16(__uint_as_float(u[h * 8 + j]));
                    }
                  }
                }
              }
            }
          }
        }
      }
      // hand the accumulator buffer back to the MMA thread (of the leader): one arrival per epilogue warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (CG == 2) mbar_arrive_cluster(bars_leader + (uint32_t)(2 * MAX_STAGES + 2 + buf) * 8u);
        else mbar_arrive(&tempty_bar[buf]);
      }
    }
  }

  // teardown: everyone meets here (also after an aborted wait; with CG = 2 both CTAs, so that neither leaves while
  // the other may still signal its barriers or read its shared memory), then the allocating warp frees TMEM
  if (threadIdx.x == 64) tma_store_wait<0>();
  tc_fence_before_sync();
  if (CG == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) {
    if (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC,
                     const KernelParams p) {
  gemm_body<A_MN, B_MN, 1>(tmA, tmB, tmB2, tmC, p);
}

// The CTA-pair variant: the grid is a whole number of 2-CTA clusters.
template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC,
                          const KernelParams p) {
  gemm_body<A_MN, B_MN, 2>(tmA, tmB, tmB2, tmC, p);
}

constexpr int MAX_DEVICES = 64;

template <bool A_MN, bool B_MN, int CG>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const CUtensorMap& tC,
                  const KernelParams& kp, int grid, cudaStream_t stream) {
  // the shared-memory opt-in is a per-device attribute of the function
  static bool attr_set[MAX_DEVICES] = {};
  int dev = 0;
  OB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) OB_FAIL(-20, "device index %d out of range", dev);
  if (CG == 2) {
    if (!attr_set[dev]) {
      OB_CUDA_OK(cudaFuncSetAttribute(gemm_bf16_pair_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Geo<2>::SMEM_BYTES));
      attr_set[dev] = true;
    }
    gemm_bf16_pair_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, Geo<2>::SMEM_BYTES, stream>>>(tA, tB, tB2, tC, kp);
  } else {
    if (!attr_set[dev]) {
      OB_CUDA_OK(cudaFuncSetAttribute(gemm_bf16_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Geo<1>::SMEM_BYTES));
      attr_set[dev] = true;
    }
    gemm_bf16_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, Geo<1>::SMEM_BYTES, stream>>>(tA, tB, tB2, tC, kp);
  }
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int CG>
static int launch_layout(bool a_mn, bool b_mn, const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2,
                         const CUtensorMap& tC, const KernelParams& kp, int grid, cudaStream_t stream) {
  if (a_mn) return b_mn ? launch<true, true, CG>(tA, tB, tB2, tC, kp, grid, stream)
                        : launch<true, false, CG>(tA, tB, tB2, tC, kp, grid, stream);
  return b_mn ? launch<false, true, CG>(tA, tB, tB2, tC, kp, grid, stream)
              : launch<false, false, CG>(tA, tB, tB2, tC, kp, grid, stream);
}

// 1: force single-CTA tiles, 2: force CTA pairs, 0: choose per problem (OLMAX_B200_GEMM_CTA_GROUP)
static int cta_group_override() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("OLMAX_B200_GEMM_CTA_GROUP");
    v = (e != nullptr && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
  }
  return v;
}
static bool split_k_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("OLMAX_B200_GEMM_SPLIT_K");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

}  // namespace ob

using namespace ob;

extern "C" int ob_gemm_bf16(const ObGemmArgs* a, cudaStream_t stream) {
  if (a == nullptr) OB_FAIL(-1, "null args");
  if (a->M <= 0 || a->N <= 0 || a->Kc <= 0) OB_FAIL(-2, "empty problem M=%d N=%d K=%d", a->M, a->N, a->Kc);
  const bool glu = (a->epi == EPI_SWIGLU || a->epi == EPI_GEGLU);
  const int M_s = a->M_s > 0 ? a->M_s : a->M;
  const int N_s = a->N_s > 0 ? a->N_s : a->N;
  const int Kc_s = a->Kc_s > 0 ? a->Kc_s : a->Kc;
  if (a->M % M_s || a->N % N_s || a->Kc % Kc_s) OB_FAIL(-3, "shard extents must divide M/N/K");
  if (a->Kc % 8 || Kc_s % 8 || N_s % 8 || M_s % 8) OB_FAIL(-4, "M_s, N_s, K_s must be multiples of 8");
  if (a->b_mn && N_s != a->N) OB_FAIL(-5, "an MN-major B operand cannot be N-sharded");
  if (!a->b_mn && Kc_s != a->Kc) OB_FAIL(-6, "a K-major B operand cannot be K-sharded");
  if (glu && (a->b_mn || a->a_mn || a->b2 == nullptr)) OB_FAIL(-7, "gated epilogue needs K-major A, B and b2");
  if (a->c_shards == nullptr && M_s != a->M && a->epi != EPI_F32_RED && false) OB_FAIL(-8, "unreachable");

  KernelParams kp;
  kp.M = a->M; kp.N = a->N; kp.Kc = a->Kc;
  kp.M_s = M_s; kp.N_s = N_s; kp.Kc_s = Kc_s;
  kp.bn_out = glu ? 128 : BN;
  kp.m_shards = a->M / M_s;
  kp.n_shards = a->N / N_s;
  kp.k_shards = a->Kc / Kc_s;
  const int cap = a->max_ctas > 0 ? a->max_ctas : sm_count();
  // Tile geometry: CTA pairs (256-row tiles) unless forced, or unless the problem has so few 256-row tiles that
  // 128-row tiles on single CTAs keep more SMs busy.
  int CG = cta_group_override();
  if (CG == 0) {
    const long long n_t = (long long)kp.n_shards * ((N_s + kp.bn_out - 1) / kp.bn_out);
    const long long pair_tiles = (long long)kp.m_shards * ((M_s + 2 * BM - 1) / (2 * BM)) * n_t;
    const long long single_tiles = (long long)kp.m_shards * ((M_s + BM - 1) / BM) * n_t;
    CG = (pair_tiles >= cap / 2 || single_tiles == pair_tiles) ? 2 : 1;
    // row shards of at most 128 rows (e.g. the k / v weight gradients of a grouped-query model over 8 GPUs): the
    // second CTA of every pair would have no rows at all
    if (kp.m_shards > 1 && M_s <= BM) CG = 1;
  }
  if (cap < 2) CG = 1;
  const int BMT = BM * CG;            // tile rows
  const int BNL = BN / CG;            // B columns held per CTA
  kp.m_tiles_per_shard = (M_s + BMT - 1) / BMT;
  kp.n_tiles_per_shard = (N_s + kp.bn_out - 1) / kp.bn_out;
  kp.k_iters_per_shard = (Kc_s + BK - 1) / BK;
  kp.epi = a->epi;
  kp.group_m = a->group_m > 0 ? a->group_m : (CG == 2 ? 8 : 16);
  kp.m_rot = (a->m_shard_rot > 0 ? a->m_shard_rot : 0) * kp.m_tiles_per_shard;
  if (kp.group_m > kp.m_shards * kp.m_tiles_per_shard) kp.group_m = kp.m_shards * kp.m_tiles_per_shard;
  kp.alpha = a->alpha;
  kp.c = a->c; kp.c2 = a->c2; kp.c3 = a->c3;
  kp.c_shards = a->c_shards;
  kp.c_shard_stride = a->c_shard_stride;
  kp.ldc = a->ldc;
  kp.status = a->status;
  kp.ag_shards = 0;
  kp.ag_on_a = 0;
  kp.ag_rank = 0; kp.ag_rows = 0; kp.ag_blocks = 0; kp.ag_row_bytes = 0;
  kp.ag_src = nullptr; kp.ag_src2 = nullptr; kp.ag_dst = nullptr; kp.ag_dst2 = nullptr; kp.ag_dst_stride = 0;
  kp.ag_flags = nullptr; kp.ag_target = 0;
  kp.pf_shards = 0; kp.pf_rank = 0; kp.pf_src = nullptr; kp.pf_dst = nullptr; kp.pf_dst_stride = 0; kp.pf_off = 0;
  kp.pf_bytes = 0;
  if (a->pf_src != nullptr && a->pf_bytes > 0) {
    if (a->pf_shards < 2 || a->pf_dst == nullptr) OB_FAIL(-14, "prefetch needs >= 2 shards and a destination");
    if ((a->pf_off | a->pf_bytes | a->pf_dst_stride) & 15) OB_FAIL(-15, "prefetch offsets must be multiples of 16 bytes");
    kp.pf_shards = a->pf_shards; kp.pf_rank = a->pf_rank;
    kp.pf_src = reinterpret_cast<const uint8_t* const*>(a->pf_src);
    kp.pf_dst = reinterpret_cast<uint8_t*>(a->pf_dst);
    kp.pf_dst_stride = a->pf_dst_stride; kp.pf_off = a->pf_off; kp.pf_bytes = a->pf_bytes;
  }

  CUtensorMap tA, tB, tB2;
  memset(&tB2, 0, sizeof(tB2));
  int rc;
  kp.a_single = kp.b_single = 0;
  // (every tile must start on a multiple of 64 along M: with row shards of M_s rows, tile starts are s * M_s + 128 t)
  if (a->a_mn && a->M % 64 == 0 && M_s % 64 == 0 && !a->multi_box_mn) {
    // view [Kc, M] as (64, Kc, M/64): a tile is ONE box of 64 x 64 x 2, which lands in shared memory as two
    // [64 k][128 B] blocks, the MN-major layout the MMA descriptor expects
    uint64_t dims[4] = {64, (uint64_t)a->Kc, (uint64_t)a->M / 64, 1};
    uint64_t str[3] = {(uint64_t)a->lda * 2, 128, (uint64_t)a->lda * 2 * (uint64_t)a->Kc};
    uint32_t box[4] = {64, (uint32_t)BK, 2, 1};
    rc = encode_tmap(&tA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    kp.a_single = 1;
  } else if (a->a_mn) {  // stored [Kc, M], M contiguous
    uint64_t dims[3] = {(uint64_t)a->M, (uint64_t)a->Kc, 1};
    uint64_t str[2] = {(uint64_t)a->lda * 2, (uint64_t)a->lda * 2 * (uint64_t)a->Kc};
    uint32_t box[3] = {64, (uint32_t)BK, 1};
    rc = encode_tmap(&tA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {  // stored [M, Kc], Kc contiguous
    uint64_t dims[3] = {(uint64_t)a->Kc, (uint64_t)a->M, 1};
    uint64_t str[2] = {(uint64_t)a->lda * 2, (uint64_t)a->lda * 2 * (uint64_t)a->M};
    uint32_t box[3] = {(uint32_t)BK, (uint32_t)BM, 1};
    rc = encode_tmap(&tA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc) return rc;
  const long long bss = a->b_shard_stride > 0 ? a->b_shard_stride : 0;
  if (a->b_mn && a->N % 64 == 0 && !a->multi_box_mn) {
    uint64_t sstride = kp.k_shards > 1 ? (uint64_t)bss * 2 : (uint64_t)a->ldb * 2 * (uint64_t)Kc_s;
    uint64_t dims[4] = {64, (uint64_t)Kc_s, (uint64_t)a->N / 64, (uint64_t)kp.k_shards};
    uint64_t str[3] = {(uint64_t)a->ldb * 2, 128, sstride};
    uint32_t box[4] = {64, (uint32_t)BK, (uint32_t)(BNL / 64), 1};
    rc = encode_tmap(&tB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    kp.b_single = 1;
  } else if (a->b_mn) {  // stored [Kc, N] per k-shard, N contiguous
    uint64_t dims[3] = {(uint64_t)a->N, (uint64_t)Kc_s, (uint64_t)kp.k_shards};
    uint64_t sstride = kp.k_shards > 1 ? (uint64_t)bss * 2 : (uint64_t)a->ldb * 2 * (uint64_t)Kc_s;
    uint64_t str[2] = {(uint64_t)a->ldb * 2, sstride};
    uint32_t box[3] = {64, (uint32_t)BK, 1};
    rc = encode_tmap(&tB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  } else {  // stored [N_s, Kc] per n-shard, Kc contiguous
    uint64_t dims[3] = {(uint64_t)a->Kc, (uint64_t)N_s, (uint64_t)kp.n_shards};
    uint64_t sstride = kp.n_shards > 1 ? (uint64_t)bss * 2 : (uint64_t)a->ldb * 2 * (uint64_t)N_s;
    uint64_t str[2] = {(uint64_t)a->ldb * 2, sstride};
    uint32_t box[3] = {(uint32_t)BK, (uint32_t)(glu ? 128 : BNL), 1};
    rc = encode_tmap(&tB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (glu) {
      rc = encode_tmap(&tB2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->b2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
    }
  }
  if ((kp.n_shards > 1 || kp.k_shards > 1) && bss <= 0) OB_FAIL(-9, "sharded B needs b_shard_stride");

  // Work list: whole tiles, then (accumulating fp32 epilogues only) the tiles of the last partial wave cut into k
  // slices that meet in the output through reduce-add.
  const int total = kp.m_shards * kp.m_tiles_per_shard * kp.n_shards * kp.n_tiles_per_shard;
  const int max_workers = cap / CG;
  const int k_iters_total = kp.k_shards * kp.k_iters_per_shard;
  kp.split = 1;
  kp.full_items = total;
  kp.total_items = total;
  const bool split_ok = split_k_enabled() && !a->no_split_k && a->ag_src == nullptr &&
                        ((a->epi == EPI_F32_ACC && a->c_shards == nullptr && !a->no_tma_epilogue) || a->epi == EPI_F32_RED);
  if (split_ok) {
    const int rem = total % max_workers;
    if (rem > 0 && max_workers / rem >= 2) {
      int split = max_workers / rem;
      if (split > 8) split = 8;
      while (split > 1 && k_iters_total / split < 16) --split;
      if (split > 1) {
        kp.split = split;
        kp.full_items = total - rem;
        kp.total_items = kp.full_items + rem * split;
      }
    }
  }
  const int workers = kp.total_items < max_workers ? kp.total_items : max_workers;
  const int grid = workers * CG;
  if (a->ag_src != nullptr && a->ag_on_a) {
    // all-gather of the A operand's row shards (sequence-parallel activations): shard s = rows [s*M_s, (s+1)*M_s)
    const int shards = kp.m_shards;
    if (a->a_mn) OB_FAIL(-16, "fused all-gather of A needs a K-major A operand");
    if (shards < 2) OB_FAIL(-10, "fused all-gather of A needs M_s < M");
    if (a->ag_flags == nullptr) OB_FAIL(-11, "fused all-gather needs a flags buffer");
    if (a->ag_rank < 0 || a->ag_rank >= shards) OB_FAIL(-12, "ag_rank %d outside [0, %d)", a->ag_rank, shards);
    if (a->ag_src2 != nullptr) OB_FAIL(-17, "fused all-gather of A has a single source table");
    kp.ag_shards = shards;
    kp.ag_on_a = 1;
    kp.ag_rank = a->ag_rank;
    kp.ag_rows = M_s;
    kp.ag_blocks = (M_s + AG_BLOCK_ROWS - 1) / AG_BLOCK_ROWS;
    kp.ag_row_bytes = (long long)a->lda * 2;
    if (kp.ag_row_bytes % 16 != 0) OB_FAIL(-13, "fused all-gather needs 16-byte aligned rows");
    kp.ag_src = reinterpret_cast<const uint8_t* const*>(a->ag_src);
    kp.ag_dst = reinterpret_cast<uint8_t*>(const_cast<void*>(a->a));
    kp.ag_dst_stride = (long long)M_s * kp.ag_row_bytes;
    kp.ag_flags = a->ag_flags;
    kp.ag_target = (unsigned)(grid * COPY_WARPS);
    if (a->m_shard_rot <= 0) kp.m_rot = a->ag_rank * kp.m_tiles_per_shard;   // local rows first, then rank+1, ...
    OB_CUDA_OK(cudaMemsetAsync(a->ag_flags, 0, sizeof(unsigned) * (size_t)shards * kp.ag_blocks, stream));
  } else if (a->ag_src != nullptr) {
    const int shards = a->b_mn ? kp.k_shards : kp.n_shards;
    if (shards < 2 || bss <= 0) OB_FAIL(-10, "fused all-gather needs a sharded B operand");
    if (a->ag_flags == nullptr) OB_FAIL(-11, "fused all-gather needs a flags buffer");
    if (a->ag_rank < 0 || a->ag_rank >= shards) OB_FAIL(-12, "ag_rank %d outside [0, %d)", a->ag_rank, shards);
    kp.ag_shards = shards;
    kp.ag_rank = a->ag_rank;
    kp.ag_rows = a->b_mn ? Kc_s : N_s;
    kp.ag_blocks = (kp.ag_rows + AG_BLOCK_ROWS - 1) / AG_BLOCK_ROWS;
    kp.ag_row_bytes = (long long)a->ldb * 2;
    if (kp.ag_row_bytes % 16 != 0) OB_FAIL(-13, "fused all-gather needs 16-byte aligned rows");
    kp.ag_src = reinterpret_cast<const uint8_t* const*>(a->ag_src);
    kp.ag_src2 = reinterpret_cast<const uint8_t* const*>(a->ag_src2);
    kp.ag_dst = reinterpret_cast<uint8_t*>(const_cast<void*>(a->b));
    kp.ag_dst2 = reinterpret_cast<uint8_t*>(const_cast<void*>(a->b2));
    kp.ag_dst_stride = bss * 2;
    kp.ag_flags = a->ag_flags;
    kp.ag_target = (unsigned)(grid * COPY_WARPS);
    OB_CUDA_OK(cudaMemsetAsync(a->ag_flags, 0, sizeof(unsigned) * (size_t)shards * kp.ag_blocks, stream));
  }
  // Output map for the TMA epilogue (local destinations only; peer destinations keep the direct red.add path).
  CUtensorMap tC;
  memset(&tC, 0, sizeof(tC));
  kp.tma_epi = 0;
  const bool tma_ok = (a->epi == EPI_BF16 || a->epi == EPI_F32 || a->epi == EPI_F32_ACC) && a->c_shards == nullptr &&
                      !a->no_tma_epilogue && (kp.m_shards == 1 || a->c_shard_stride > 0 || M_s % BM == 0) &&
                      // the store clips at the end of the matrix, not at a column shard's end: a shard's last tile may
                      // only be written in whole 64-column chunks
                      (kp.n_shards == 1 || N_s % 64 == 0);
  if (tma_ok) {
    const bool f32 = a->epi != EPI_BF16;
    const uint64_t es = f32 ? 4 : 2;
    const bool sharded = a->c_shard_stride > 0;
    uint64_t dims[3] = {(uint64_t)a->N, (uint64_t)(sharded ? M_s : a->M), (uint64_t)(sharded ? kp.m_shards : 1)};
    uint64_t str[2] = {(uint64_t)a->ldc * es, sharded ? (uint64_t)a->c_shard_stride * es : (uint64_t)a->ldc * es * (uint64_t)a->M};
    uint32_t box[3] = {(uint32_t)(f32 ? 32 : 64), (uint32_t)BM, 1};
    if ((reinterpret_cast<uintptr_t>(a->c) & 15) == 0 && str[0] % 16 == 0 && str[1] % 16 == 0) {
      rc = encode_tmap(&tC, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->c, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
      kp.tma_epi = 1;
    }
  }
  if (kp.split > 1 && a->epi == EPI_F32_ACC && kp.tma_epi != 1) {   // no atomic path for the slices: whole tiles only
    kp.split = 1;
    kp.full_items = kp.total_items = total;
  }
  // peer destinations: staged, line-coalesced stores / reductions (needs 16-byte aligned rows)
  if (kp.tma_epi == 0 && a->c_shards != nullptr && !a->no_tma_epilogue &&
      (a->epi == EPI_F32 || a->epi == EPI_F32_RED || a->epi == EPI_BF16 || (a->epi == EPI_BF16_ACC && a->c != nullptr)) &&
      (a->ldc * ((a->epi == EPI_BF16 || a->epi == EPI_BF16_ACC) ? 2 : 4)) % 16 == 0)
    kp.tma_epi = 2;
  if (a->c_shards != nullptr && a->epi == EPI_BF16_ACC && kp.tma_epi != 2)
    OB_FAIL(-18, "EPI_BF16_ACC towards c_shards needs the staged epilogue (16-byte aligned rows, local partial in c)");
  return CG == 2 ? launch_layout<2>(a->a_mn != 0, a->b_mn != 0, tA, tB, tB2, tC, kp, grid, stream)
                 : launch_layout<1>(a->a_mn != 0, a->b_mn != 0, tA, tB, tB2, tC, kp, grid, stream);
}

extern "C" const char* ob_last_error() { return ob::last_error_buf(); }
