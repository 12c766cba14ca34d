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
// the same with bf16 slots (n and slot_stride multiples of 8 elements)
int ob_reduce_slots_bf16(const void* stage, float* acc, long long n, int R, long long slot_stride, float scale,
                        cudaStream_t stream);

// Stream-ordered barrier of n GPUs over peer memory: flags = DEVICE array of the members' flag arrays (n words each,
// zero-initialised, peer-mapped), epoch = 1, 2, 3, ... (the same sequence on every member).  A member that does not see
// all others within timeout_ns (<= 0: 30 s) writes ERR_PEER_TIMEOUT (site 500) to status and returns.
int ob_peer_barrier(unsigned* const* flags, int me, int n, unsigned epoch, long long timeout_ns, int* status,
                    cudaStream_t stream);
// The two halves of the barrier as separate launches, for members that publish an epoch when their stores are done
// and wait for the others' epoch only later (the same epoch sequence as ob_peer_barrier: every publish, whether from
// ob_peer_barrier or ob_peer_signal, takes the next number; a wait passes once every member's word is >= its epoch).
int ob_peer_signal(unsigned* const* flags, int me, int n, unsigned epoch, cudaStream_t stream);
int ob_peer_wait(unsigned* const* flags, int me, int n, unsigned epoch, long long timeout_ns, int* status,
                 cudaStream_t stream);
// dst = src (bytes, 16-byte multiples); either side may be peer memory.  blocks <= 0: 4 per SM; unroll 4 / 8 / 16 = 16-byte
// loads in flight per thread (matters when src is remote).
int ob_copy_bytes(void* dst, const void* src, long long bytes, int blocks, int unroll, cudaStream_t stream);
// dsts[s] = src for every s != skip (dsts: DEVICE array of n_dst destination addresses, typically one per GPU of a
// group: an all-gather as a push of the local piece into everybody's gathered buffer with posted remote stores)
int ob_push_copy(void* const* dsts, const void* src, long long bytes, int n_dst, int skip, int blocks, cudaStream_t stream);

// out[i] = (accumulate ? out[i] : 0) + sum over slots r != skip of stage[r * slot_stride + i]  (bf16 storage, fp32
// sums, local memory): folds the staging slots of a fused GEMM -> reduce-scatter over a tensor-parallel group
int ob_fold_slots_bf16(void* out, const void* stage, long long n, int slots, long long slot_stride, int skip,
                       int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
