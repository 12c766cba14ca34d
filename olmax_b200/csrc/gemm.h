// C interface of the tcgen05 bf16 GEMM (see gemm.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum ObGemmEpilogue {
  EPI_BF16 = 0,     // C(bf16)  = alpha * A.B
  EPI_F32 = 1,      // C(fp32)  = alpha * A.B
  EPI_F32_ACC = 2,  // C(fp32) += alpha * A.B        (read-modify-write, local memory)
  EPI_F32_RED = 3,  // C(fp32) += alpha * A.B        (red.global.add; destination may be a peer GPU's memory)
  EPI_SWIGLU = 4,   // C(bf16)  = silu(A.B) * (A.B2); optionally c2 = A.B, c3 = A.B2
  EPI_GEGLU = 5,    // C(bf16)  = gelu_tanh(A.B) * (A.B2)
  EPI_BF16_ACC = 6, // C(bf16) += alpha * A.B        (read-modify-write, local memory); with c_shards: row block s of
                    // c (the local partial sum, [M, N]) + alpha * A.B is STORED to c_shards[s] and c is left unchanged
};

// C[M, N] = A[M, Kc] . B[Kc, N]  with bf16 operands and fp32 accumulation.
//   a_mn = 0: A stored [M, Kc] (Kc contiguous), a_mn = 1: A stored [Kc, M] (M contiguous); lda = row stride, elements
//   b_mn = 0: B stored [N, Kc] (Kc contiguous), b_mn = 1: B stored [Kc, N] (N contiguous); ldb = row stride, elements
// Sharding (0 = unsharded):
//   N_s:  with b_mn = 0, output columns [s*N_s, (s+1)*N_s) use the B rows at b + s*b_shard_stride
//   Kc_s: with b_mn = 1, contraction block s uses the B rows at b + s*b_shard_stride
//   M_s:  output rows [s*M_s, (s+1)*M_s) are written to c_shards[s] (row index local to the shard) when c_shards is
//         given, to c + s*c_shard_stride when c_shard_stride > 0, otherwise to c as one [M, N] matrix
// All extents that are sharded, and lda/ldb/ldc, must be multiples of 8 elements; all base pointers 16-byte aligned.
typedef struct ObGemmArgs {
  const void* a;
  long long lda;
  const void* b;
  long long ldb;
  long long b_shard_stride;
  const void* b2;
  void* c;
  long long ldc;
  void* c2;
  void* c3;
  void* const* c_shards;  // DEVICE array of base pointers, one per M shard (or null)
  long long c_shard_stride;  // with c_shards null and M_s set: rows of shard s start at c + s * c_shard_stride elements
  int M, N, Kc;
  int M_s, N_s, Kc_s;
  int a_mn, b_mn;
  int epi;
  float alpha;
  int* status;   // device int[4]: a kernel-side wait that ran out writes its code here (may be null)
  int max_ctas;  // 0 = one CTA per SM
  // Fused FSDP all-gather (optional).  With ag_src set, B is a staging buffer of R shard slots (N_s / Kc_s rows each,
  // b_shard_stride apart) of which only slot ag_rank is filled; the kernel's copy warps fetch the other slots from
  // ag_src[s] (DEVICE array of R base pointers into the peer GPUs' memory, read with plain loads over NVLink) while
  // the tensor cores start on the local slot, and tiles of slot s wait for its blocks to land (bounded wait).
  const void* const* ag_src;
  const void* const* ag_src2;  // same for b2 (gated epilogue)
  unsigned* ag_flags;          // device scratch, >= R * ceil(rows_per_shard / 256) words; cleared by the launcher
  int ag_rank;
  // Prefetch for later launches (optional): while this GEMM computes, its copy warps also copy bytes
  // [pf_off, pf_off + pf_bytes) of every OTHER GPU's slice (pf_src[s], DEVICE array of pf_shards peer pointers) into
  // pf_dst + s * pf_dst_stride.  Used to stream the next FSDP unit's weights in under the current unit's GEMMs.
  const void* const* pf_src;
  void* pf_dst;
  long long pf_dst_stride, pf_off, pf_bytes;  // bytes, multiples of 16
  int pf_shards, pf_rank;
  int m_shard_rot;      // start the M tile order at output row shard m_shard_rot (stagger ranks that add into peers)
  int group_m;          // tile rasterisation group in M tiles (0 = default 16)
  int multi_box_mn;     // 1: fetch MN-major operands as 64-wide boxes even when one 4-D box per stage would do
  int no_tma_epilogue;  // 1: write outputs with per-thread stores instead of shared memory + TMA (for comparison)
  // 1: ag_src / ag_flags / ag_rank describe an all-gather of the A operand instead of B: A (K-major, [M, Kc]) is a
  // buffer of M / M_s row shards of which only shard ag_rank is filled; the copy warps fetch shard s from ag_src[s]
  // (a contiguous [M_s, Kc] piece with the same row stride in GPU s's memory) and the tiles of shard s wait for it.
  int ag_on_a;
  // 1: never cut the tiles of the last partial wave into k slices (accumulating fp32 epilogues do by default)
  int no_split_k;
} ObGemmArgs;

int ob_gemm_bf16(const ObGemmArgs* args, cudaStream_t stream);
const char* ob_last_error();

#ifdef __cplusplus
}
#endif
