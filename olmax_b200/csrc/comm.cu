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

// The same fold for bf16 slots (the reduce-scatter wire format that halves the bytes crossing NVLink and read here):
// acc[i] += scale * sum_r float(stage[r * slot_stride + i]); n8 groups of 8 elements, slot_stride in elements.
__global__ void __launch_bounds__(AR_THREADS)
    reduce_slots_bf16_kernel(const bf16* __restrict__ stage, float* __restrict__ acc, long long n8, int R,
                             long long slot_stride, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float sum[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) sum[e] = 0.f;
    for (int r = 0; r < R; ++r) {
      const uint4 v = __ldcs(reinterpret_cast<const uint4*>(stage + r * slot_stride) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(w[e]);
        sum[2 * e] += f.x;
        sum[2 * e + 1] += f.y;
      }
    }
    float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
    float4 a0 = a[0], a1 = a[1];
    a0.x += scale * sum[0]; a0.y += scale * sum[1]; a0.z += scale * sum[2]; a0.w += scale * sum[3];
    a1.x += scale * sum[4]; a1.y += scale * sum[5]; a1.z += scale * sum[6]; a1.w += scale * sum[7];
    a[0] = a0;
    a[1] = a1;
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

// Stream-ordered barrier of n GPUs through peer memory.  flags[r] is GPU r's flag array (n words, peer-mapped).  GPU
// `me` publishes `epoch` in word `me` of every member's array (system-scope release after a system fence: whatever its
// earlier kernels stored into peer memory is visible to a GPU that sees the flag), then waits until all n words of its
// own array show `epoch` -- with a time limit, after which it records ERR_PEER_TIMEOUT and returns, so a missing peer
// costs `timeout_ns` and an exception on the host, never a hung GPU.
//
// The two halves can also be launched on their own (`phases`: 1 = publish, 2 = wait, 3 = both): a member publishes when
// its stores are done and waits later, right before it needs the others' stores, so that the skew between the GPUs is
// absorbed by the work in between instead of being paid at every barrier.
__global__ void peer_barrier_kernel(unsigned* const* __restrict__ flags, int me, int n, unsigned epoch,
                                    long long timeout_ns, int* status, int phases) {
  const int t = (int)threadIdx.x;
  if (t >= n) return;
  if (phases & 1) {
    __threadfence_system();
    unsigned* remote = flags[t] + me;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  if (!(phases & 2)) return;
  const unsigned* own = flags[me] + t;
  long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned it = 0;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if ((it & 63u) == 63u) {
      long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > timeout_ns) {
        report_error(status, ERR_PEER_TIMEOUT, 500, t);
        break;
      }
    }
    __nanosleep(200);
  }
}

// dsts[s][i] = src[i] for every s != skip (16-byte words).  The destinations may be peer GPUs' memory: remote STORES
// are posted, so a push runs at link rate with few bytes in flight, whereas remote loads pay a round trip each.
template <int U>
__global__ void __launch_bounds__(AR_THREADS)
    push_copy_kernel(const uint4* __restrict__ src, uint4* const* __restrict__ dsts, int n_dst, int skip, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < n16; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = src[i + u * stride];
    for (int s = 0; s < n_dst; ++s) {
      if (s == skip) continue;
      uint4* d = dsts[s];
#pragma unroll
      for (int u = 0; u < U; ++u) d[i + u * stride] = v[u];
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = src[i];
    for (int s = 0; s < n_dst; ++s)
      if (s != skip) dsts[s][i] = v;
  }
}

// dst[i] = src[i] (16-byte words, U loads in flight per thread); either side may be a peer GPU's memory
template <int U>
__global__ void __launch_bounds__(AR_THREADS)
    copy16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < n16; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = __ldcg(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < n16; i += stride) dst[i] = __ldcg(src + i);
}

}  // namespace ob

using namespace ob;

extern "C" int ob_peer_barrier(unsigned* const* flags, int me, int n, unsigned epoch, long long timeout_ns, int* status,
                               cudaStream_t stream) {
  if (n <= 1) return 0;
  if (n > 64 || me < 0 || me >= n) OB_FAIL(-7, "barrier: rank %d / group of %d not supported (max 64)", me, n);
  if (timeout_ns <= 0) timeout_ns = 30LL * 1000 * 1000 * 1000;
  peer_barrier_kernel<<<1, 64, 0, stream>>>(flags, me, n, epoch, timeout_ns, status, 3);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_peer_signal(unsigned* const* flags, int me, int n, unsigned epoch, cudaStream_t stream) {
  if (n <= 1) return 0;
  if (n > 64 || me < 0 || me >= n) OB_FAIL(-7, "barrier: rank %d / group of %d not supported (max 64)", me, n);
  peer_barrier_kernel<<<1, 64, 0, stream>>>(flags, me, n, epoch, 0, nullptr, 1);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_peer_wait(unsigned* const* flags, int me, int n, unsigned epoch, long long timeout_ns, int* status,
                            cudaStream_t stream) {
  if (n <= 1) return 0;
  if (n > 64 || me < 0 || me >= n) OB_FAIL(-7, "barrier: rank %d / group of %d not supported (max 64)", me, n);
  if (timeout_ns <= 0) timeout_ns = 30LL * 1000 * 1000 * 1000;
  peer_barrier_kernel<<<1, 64, 0, stream>>>(flags, me, n, epoch, timeout_ns, status, 2);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_copy_bytes(void* dst, const void* src, long long bytes, int blocks, int unroll, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  if ((bytes | (long long)reinterpret_cast<uintptr_t>(dst) | (long long)reinterpret_cast<uintptr_t>(src)) & 15)
    OB_FAIL(-6, "copy: addresses and size must be multiples of 16 bytes");
  const long long n16 = bytes >> 4;
  if (blocks <= 0) blocks = 4 * sm_count();
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  if (unroll >= 16) copy16_kernel<16><<<blocks, AR_THREADS, 0, stream>>>(s, d, n16);
  else if (unroll >= 8) copy16_kernel<8><<<blocks, AR_THREADS, 0, stream>>>(s, d, n16);
  else copy16_kernel<4><<<blocks, AR_THREADS, 0, stream>>>(s, d, n16);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ob_push_copy(void* const* dsts, const void* src, long long bytes, int n_dst, int skip, int blocks,
                            cudaStream_t stream) {
  if (bytes <= 0 || n_dst <= 0) return 0;
  if ((bytes | (long long)reinterpret_cast<uintptr_t>(src)) & 15) OB_FAIL(-6, "push: source and size must be 16-byte multiples");
  if (blocks <= 0) blocks = 2 * sm_count();
  push_copy_kernel<4><<<blocks, AR_THREADS, 0, stream>>>(reinterpret_cast<const uint4*>(src),
                                                         reinterpret_cast<uint4* const*>(dsts), n_dst, skip, bytes >> 4);
  OB_CUDA_OK(cudaGetLastError());
  return 0;
}

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

extern "C" int ob_reduce_slots_bf16(const void* stage, float* acc, long long n, int R, long long slot_stride, float scale,
                                    cudaStream_t stream) {
  if (n <= 0 || R <= 0) return 0;
  if (n % 8 != 0 || slot_stride % 8 != 0) OB_FAIL(-1, "reduce_slots_bf16: element counts must be multiples of 8");
  long long blocks = (n / 8 + AR_THREADS - 1) / AR_THREADS;
  const long long cap = 8LL * sm_count();
  if (blocks > cap) blocks = cap;
  reduce_slots_bf16_kernel<<<(unsigned)blocks, AR_THREADS, 0, stream>>>((const bf16*)stage, acc, n / 8, R, slot_stride,
                                                                        scale);
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
