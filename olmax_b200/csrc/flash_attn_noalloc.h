// Flash-attention backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference: the reference reaches attention through a compiler and a
// vendor library that manage their own workspaces.  It exists for programs that embed this library where device
// memory is not theirs to hand out: an inference or fine-tuning server whose memory was carved into a fixed arena at
// start-up, a plug-in running inside another framework's allocator, a job under a hard memory cap that must not grow
// after initialisation, or a latency-critical loop in which a cudaMalloc (which can synchronise the whole device)
// is not acceptable.  Such a caller still owns its input and output tensors, but has nowhere to get the two work
// buffers the backward pass needs (delta[B, H, S] and the fp32 dQ accumulator [B, S, H, 128]).
//
// ob_flash_attn_bwd_static() computes exactly what ob_flash_attn_bwd() computes, but takes those work buffers from a
// fixed array built into the library instead of from the caller (the `delta` and `dq_accum` fields of the argument
// struct are ignored).  It calls no cudaMalloc / cudaFree and no routine that allocates.
//
// Limits and rules:
//   * B * S * H must not exceed OB_FLASH_BWD_STATIC_MAX_ROWS (32768, e.g. batch 1 x 4096 tokens x 8 heads); larger
//     problems are rejected with an error message and must use ob_flash_attn_bwd().  The array occupies
//     32768 * 129 * 4 bytes = 16.1 MiB on every GPU that loads the library, for the life of the process.
//   * The first call on a device looks up the array's device address (with that device current) and caches it, and
//     opts the kernel in to its shared-memory size on that device.  Make that first call during start-up, outside any
//     stream capture, and from one host thread per device (the per-device cache is written without a lock).
//   * All calls on a device share the one array, which keeps whatever the previous call left in it.  The function
//     clears the part it accumulates into before use, so back-to-back calls on ONE stream are safe; calls that can
//     overlap on the GPU (different streams, different host threads) would race on it and must be serialised by the
//     caller.
#pragma once
#include "flash_attn.h"

#define OB_FLASH_BWD_STATIC_MAX_ROWS 32768

#ifdef __cplusplus
extern "C" {
#endif

int ob_flash_attn_bwd_static(const ObAttnArgs* args, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
