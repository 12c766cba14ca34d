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
} ObAttnArgs;

int ob_flash_attn_fwd(const ObAttnArgs* args, cudaStream_t stream);
int ob_flash_attn_bwd(const ObAttnArgs* args, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
