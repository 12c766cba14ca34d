// All-reduce kernels over NVLink peer memory for the once-per-step gradient all-reduce of HSDP / DDP
// (the reference issues an NCCL all-reduce after EVERY micro-batch, `README.md:30` of the reference).
//
// Both kernels are two-shot and contain no waits: rank i reduces slice i of the buffer over all members and writes
// the result back to every member.  The caller brackets the launch with stream-ordered barriers (all members have
// finished producing their buffers / all slices have been written), so a missing peer can never hang a kernel.
//   * ob_allreduce_p2p_f32:      plain vector loads from / stores to the members' buffers (any group of GPUs);
//   * ob_allreduce_multimem_f32: NVSwitch in-network reduction, multimem.ld_reduce + multimem.st on a multicast address
//                                that maps the same buffer on every member.
#include "comm.h"
#include "host_common.h"
#include "sm100.cuh"

namespace ob {

constexpr int AR_THREADS = 512;

__global__ void __launch_bounds__(AR_THREADS)
    allreduce_p2p_kernel(float* const* __restrict__ bufs, long long n, int me, int world, float scale) {
  // slice of this rank, in float4 units
  const long long n4 = n / 4;
  const long long per = (n4 + world - 1) / world;
  const long long lo = per * me, hi = min(n4, lo + per);
  for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(bufs[(me + r) % world]) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(bufs[(me + r) % world])[i] = acc;
  }
  // tail elements (n not a multiple of 4) are handled by rank 0
  if (me == 0 && blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      float acc = 0.f;
      for (int r = 0; r < world; ++r) acc += bufs[r][i];
      acc *= scale;
      for (int r = 0; r < world; ++r) bufs[r][i] = acc;
    }
  }
}

__global__ void __launch_bounds__(AR_THREADS)
    allreduce_multimem_kernel(float* mc, long long n, int me, int world) {
  const long long n4 = n / 4;   // the caller pads n to a multiple of 4
  const long long per = (n4 + world - 1) / world;
  const long long lo = per * me, hi = min(n4, lo + per);
  for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
    float* addr = mc + i * 4;
    float x, y, z, w;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(x), "=f"(y), "=f"(z), "=f"(w)
                 : "l"(addr)
                 : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z), "f"(w)
                 : "memory");
  }
}

// acc[i] += scale * sum_r stage[r * slot_stride + i]: folds the R per-source slots that peers' weight-gradient GEMMs
// stored into this GPU's staging buffer into the fp32 gradient accumulator (all local memory).
__global__ void __launch_bounds__(AR_THREADS)
    reduce_slots_kernel(const float* __restrict__ stage, float* __restrict__ acc, long long n, int R,
                        long long slot_stride, float scale) {
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 a = reinterpret_cast<float4*>(acc)[i];
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < R; ++r) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(stage + r * slot_stride) + i);
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    a.x += scale * sum.x; a.y += scale * sum.y; a.z += scale * sum.z; a.w += scale * sum.w;
    reinterpret_cast<float4*>(acc)[i] = a;
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float sum = 0.f;
    for (int r = 0; r < R; ++r) sum += stage[r * slot_stride + i];
    acc[i] += scale * sum;
  }
}

// out[i] = (accumulate ? out[i] : 0) + sum over slots r != skip of stage[r * slot_stride + i], bf16 storage, fp32 sums
__global__ void __launch_bounds__(AR_THREADS)
    fold_slots_bf16_kernel(bf16* __restrict__ out, const bf16* __restrict__ stage, long long n8,
                           int slots, long long slot_stride, int skip, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (accumulate) {
      const uint4 o = *reinterpret_cast<const uint4*>(out + i * 8);
      const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 t = unpack_bf16x2(w[e]);
        acc[2 * e] = t.x;
        acc[2 * e + 1] = t.y;
      }
    }
    for (int r = 0; r < slots; ++r) {
      if (r == skip) continue;
      const uint4 o = *reinterpret_cast<const uint4*>(stage + (long long)r * slot_stride + i * 8);
      const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 t = unpack_bf16x2(w[e]);
        acc[2 * e] += t.x;
        acc[2 * e + 1] += t.y;
      }
    }
    uint4 v;
    v.x = pack_bf16x2(acc[0], acc[1]);
    v.y = pack_bf16x2(acc[2], acc[3]);
    v.z = pack_bf16x2(acc[4], acc[5]);
    v.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = v;
  }
}

}  // namespace ob

using namespace ob;

extern "C" int ob_fold_slots_bf16(void* out, const void* stage, long long n, int slots, long long slot_stride, int skip,
                                  int accumulate, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || slot_stride % 8 != 0) OB_FAIL(-4, "fold: element counts must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(stage)) & 15) OB_FAIL(-5, "fold: 16-byte alignment");
  long long blocks = (n / 8 + AR_THREADS - 1) / AR_THREADS;
  const long long cap = 8LL * sm_count();
  if (blocks > cap) blocks = cap;
  fold_slots_bf16_kernel<<<(unsigned)blocks, AR_THREADS, 0, stream>>>(
      reinterpret_cast<bf16*>(out), reinterpret_cast<const bf16*>(stage), n / 8, slots, slot_stride,
      skip, accumulate);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_allreduce_p2p_f32(float* const* bufs, long long n, int me, int world, float scale, int max_blocks,
                                    cudaStream_t stream) {
  if (n <= 0 || world <= 1) return 0;
  if (me < 0 || me >= world) OB_FAIL(-1, "allreduce: rank %d outside [0, %d)", me, world);
  const long long per = ((n / 4) + world - 1) / world;
  long long blocks = (per + AR_THREADS - 1) / AR_THREADS;
  const long long cap = max_blocks > 0 ? max_blocks : 2LL * sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  allreduce_p2p_kernel<<<(unsigned)blocks, AR_THREADS, 0, stream>>>(bufs, n, me, world, scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_allreduce_multimem_f32(float* mc, long long n, int me, int world, int max_blocks, cudaStream_t stream) {
  if (n <= 0 || world <= 1) return 0;
  if (mc == nullptr) OB_FAIL(-2, "allreduce: no multicast address");
  if (n % 4 != 0 || (reinterpret_cast<uintptr_t>(mc) & 15)) OB_FAIL(-3, "allreduce: need n %% 4 == 0 and 16-byte alignment");
  const long long per = ((n / 4) + world - 1) / world;
  long long blocks = (per + AR_THREADS - 1) / AR_THREADS;
  const long long cap = max_blocks > 0 ? max_blocks : 2LL * sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  allreduce_multimem_kernel<<<(unsigned)blocks, AR_THREADS, 0, stream>>>(mc, n, me, world);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_reduce_slots_f32(const float* stage, float* acc, long long n, int R, long long slot_stride, float scale,
                                   cudaStream_t stream) {
  if (n <= 0 || R <= 0) return 0;
  long long blocks = ((n + 3) / 4 + AR_THREADS - 1) / AR_THREADS;
  const long long cap = 8LL * sm_count();
  if (blocks > cap) blocks = cap;
  reduce_slots_kernel<<<(unsigned)blocks, AR_THREADS, 0, stream>>>(stage, acc, n, R, slot_stride, scale);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}
