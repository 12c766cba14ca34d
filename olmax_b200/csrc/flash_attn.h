// C interface of the sm_100a flash-attention kernels (flash_attn_fwd.cu, flash_attn_bwd.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Tensors are [B, S, H, D] (K/V: [B, S, Hkv, D]) bf16 with arbitrary element strides for batch (sb), sequence (ss)
// and head (sh); the head dimension is contiguous and D must be 128.  Strides must be multiples of 8 elements and
// base pointers 16-byte aligned (TMA requirement).
typedef struct ObAttnArgs {
  const void* q; long long q_sb, q_ss, q_sh;
  const void* k; long long k_sb, k_ss, k_sh;
  const void* v; long long v_sb, v_ss, v_sh;
  void* o;       long long o_sb, o_ss, o_sh;   // forward output / backward input
  float* lse;                                  // [B, H, S] natural-log sum-exp: forward output / backward input
  // backward only
  const void* d_o; long long do_sb, do_ss, do_sh;
  void* dq;      long long dq_sb, dq_ss, dq_sh;
  void* dk;      long long dk_sb, dk_ss, dk_sh;
  void* dv;      long long dv_sb, dv_ss, dv_sh;
  float* delta;     // scratch [B, H, S]: rowsum(dO * O)
  float* dq_accum;  // scratch [B, S, H, D] fp32, zero-filled by the launcher, dQ is reduced into it
  int B, S, H, Hkv, D;
  int causal;       // 1: key j visible to query i only if j <= i
  int window;       // < 0: no window; else key j visible only if j >= i - window
  float scale;      // softmax scale (usually 1/sqrt(D))
  float softcap;    // 0: off; else logits = softcap * tanh(scale * q.k / softcap)
  int* status;      // device int[4] error words (may be null)
  // Rectangular problems (context parallelism, blockwise / ring attention): K and V have Sk rows (0: Sk = S) and
  // query row i sits at position q_off + i of the key axis, so with `causal` key j is visible when j <= q_off + i.
  // The launchers accept only geometries in which every query row sees at least one key and every 128-row key tile
  // is seen by at least one query row: q_off >= 0; causal: Sk <= q_off + S; window >= 0: q_off <= window + 127 and
  // q_off + S - 1 - window <= Sk - 1.  lse / delta / dq are indexed by the S query rows, dk / dv by the Sk key rows.
  int Sk, q_off;
} ObAttnArgs;

int ob_flash_attn_fwd(const ObAttnArgs* args, cudaStream_t stream);
int ob_flash_attn_bwd(const ObAttnArgs* args, cudaStream_t stream);

#ifdef __cplusplus
}
// 0 when the geometry is one the kernels handle; otherwise the number of the violated rule (see ObAttnArgs)
static inline int ob_attn_check_geometry(const ObAttnArgs* a, int* Sk_out) {
  const int Sk = a->Sk > 0 ? a->Sk : a->S;
  *Sk_out = Sk;
  if (a->q_off < 0) return 1;
  if (a->causal && Sk > a->q_off + a->S) return 2;
  if (!a->causal && a->window >= 0) return 3;   // a window is only defined together with the causal mask
  if (a->window >= 0 && a->q_off > a->window + 127) return 4;
  if (a->window >= 0 && a->q_off + a->S - 1 - a->window > Sk - 1) return 5;
  return 0;
}
#endif
