// C interface of the peer-memory all-reduce kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// In-place sum (times `scale`) of an fp32 buffer over `world` GPUs.  bufs: DEVICE array of the members' buffer
// addresses (peer-mapped), me: this GPU's index in that array.  The caller must barrier the members before (buffers
// complete) and after (results visible) the launch; the kernel itself never waits.
int ob_allreduce_p2p_f32(float* const* bufs, long long n, int me, int world, float scale, int max_blocks,
                         cudaStream_t stream);
// Same through an NVLS multicast address `mc` (multimem.ld_reduce / multimem.st); n must be a multiple of 4.
int ob_allreduce_multimem_f32(float* mc, long long n, int me, int world, int max_blocks, cudaStream_t stream);

// acc[i] += scale * sum over r < R of stage[r * slot_stride + i]   (fp32, local memory)
int ob_reduce_slots_f32(const float* stage, float* acc, long long n, int R, long long slot_stride, float scale,
                        cudaStream_t stream);

// out[i] = (accumulate ? out[i] : 0) + sum over slots r != skip of stage[r * slot_stride + i]  (bf16 storage, fp32
// sums, local memory): folds the staging slots of a fused GEMM -> reduce-scatter over a tensor-parallel group
int ob_fold_slots_bf16(void* out, const void* stage, long long n, int slots, long long slot_stride, int skip,
                       int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
