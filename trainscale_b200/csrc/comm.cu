// Collectives fused with their neighbouring compute, over peer-mapped (symmetric) memory on NVLink 5 / NVSwitch.
//
//   ts_symm_reduce_scatter   gradient reduce-scatter fused with cast + scale + squared-norm:
//                            every rank pulls ITS slice of all W ranks' gradient buffers with plain peer loads
//                            (or one multimem.ld_reduce through the switch), sums in fp32, scales by 1/W, writes
//                            the fp32 shard and accumulates sum(g^2) for the global clip - one kernel, no staging
//                            copies, no bf16 round trip.
//   ts_symm_adamw_bcast      sharded AdamW fused with the parameter all-gather: the update kernel writes each new
//                            bf16 weight straight into every rank's parameter buffer (peer stores / multimem.st).
//   ts_symm_all_gather       plain pull all-gather (used when another optimizer produced the shard).
//   ts_symm_gather_pull      one-sided parameter gather of ZeRO-3: every rank keeps its 1/W bf16 shard of a unit in
//                            symmetric memory and a consumer copies all W shards into a LOCAL full-size buffer with
//                            plain peer loads.  No rendezvous: shards only change in the optimizer step, which is
//                            fenced by the step's barriers, so a rank never waits for a peer to launch anything
//                            (an NCCL all-gather makes every rank wait for the slowest one, once per layer).
//   ts_symm_barrier          flag barrier over the signal pads (release/acquire at system scope, bounded waits).
//
// They replace the NCCL reduce_scatter_tensor / all_gather_into_tensor + separate cast / AdamW launches behind
// torch FSDP in the reference (data_pipeline/trainer/distributed/fsdp2.py:1594,1718-1785) and the unused helper
// kernels of data_pipeline/trainer/distributed/fsdp2.py:588-660.
//
// Waits are bounded (`wait_cycles`): on expiry the kernel records ERR_FLAG_TIMEOUT in the library's error word and
// returns without touching peer data, so a missing peer ends in a host-visible status, not a hang.
// No TMA and no cluster multicast is used anywhere in this file.
#include "common.cuh"
#include "host_common.h"

namespace ts {

constexpr int MAX_WORLD = 16;

struct PeerTable {
  void* ptr[MAX_WORLD];
};
struct PadTable {
  unsigned int* pad[MAX_WORLD];
};

// All ranks signal every peer's pad slot [slot0 + my_rank] = epoch, then wait for their own pad slots
// [slot0 + r] >= epoch.  Executed by the first warp(s) of a block; returns false on timeout.
__device__ __forceinline__ bool pad_barrier(const PadTable& pads, int rank, int world, unsigned int slot0,
                                            unsigned int epoch, long long wait_cycles, unsigned int site) {
  bool ok = true;
  if ((int)threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(pads.pad[threadIdx.x] + slot0 + rank, epoch);
    ok = flag_wait_geq_sys(pads.pad[rank] + slot0 + threadIdx.x, epoch, wait_cycles, site);
  }
  return ok;
}

// local wait only (peers signalled through pad_barrier executed by block 0 of every rank)
__device__ __forceinline__ bool pad_wait_all(const PadTable& pads, int rank, int world, unsigned int slot0,
                                             unsigned int epoch, long long wait_cycles, unsigned int site) {
  bool ok = true;
  if ((int)threadIdx.x < world) ok = flag_wait_geq_sys(pads.pad[rank] + slot0 + threadIdx.x, epoch, wait_cycles, site);
  return ok;
}

__global__ void symm_barrier_kernel(PadTable pads, int rank, int world, unsigned int slot0, unsigned int epoch,
                                    long long wait_cycles, unsigned int* status) {
  const bool ok = pad_barrier(pads, rank, world, slot0, epoch, wait_cycles, 900);
  if (!ok && status) atomicExch(status, 1u);
}

// ------------------------------------------------------------------------------------------------
// reduce-scatter + cast + scale + sum of squares
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load_vec8(const T* p, float* f);
template <>
__device__ __forceinline__ void load_vec8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y), c = unpack_bf16x2(r.z), d = unpack_bf16x2(r.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <>
__device__ __forceinline__ void load_vec8<float>(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// In-switch reduction of 8 bf16 values at a multicast address, accumulated in fp32 by the switch.
__device__ __forceinline__ void multimem_ld_reduce_bf16x8(const void* mc_ptr, float* f) {
  uint32_t r0, r1, r2, r3;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "l"(mc_ptr)
               : "memory");
  const float2 a = unpack_bf16x2(r0), b = unpack_bf16x2(r1), c = unpack_bf16x2(r2), d = unpack_bf16x2(r3);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void multimem_ld_reduce_f32x4(const void* mc_ptr, float* f) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(f[0]), "=f"(f[1]), "=f"(f[2]), "=f"(f[3])
               : "l"(mc_ptr)
               : "memory");
}

template <typename T>
__global__ void __launch_bounds__(512)
symm_reduce_scatter_kernel(PeerTable peers, PadTable pads, const void* mc_base, int rank, int world,
                           long long shard_start, long long shard_numel, float* __restrict__ out, float scale,
                           float* __restrict__ sumsq, float* __restrict__ nonfinite, unsigned int slot0,
                           unsigned int epoch, long long wait_cycles, unsigned int* status, long long buf_elems) {
  __shared__ float scratch[32];
  __shared__ int s_ok;
  // entry barrier: every rank's gradient buffer is complete before anyone reads it
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  bool ok = (blockIdx.x == 0) ? pad_barrier(pads, rank, world, slot0, epoch, wait_cycles, 910)
                              : pad_wait_all(pads, rank, world, slot0, epoch, wait_cycles, 911);
  if (!ok) s_ok = 0;
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && status) atomicExch(status, 1u);
    return;
  }
  float ss = 0.f;
  const long long nvec = shard_numel >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = shard_start + (i << 3);
    float acc[8];
    // debug build: the 8 elements must lie inside the symmetric buffer every rank registered (buf_elems of T)
    if (!TS_IN_BOUNDS(reinterpret_cast<const T*>(peers.ptr[rank]) + e, 8 * sizeof(T), peers.ptr[rank],
                      static_cast<size_t>(buf_elems) * sizeof(T), 7200))
      continue;
    if (mc_base) {
      if constexpr (sizeof(T) == 2) {
        multimem_ld_reduce_bf16x8(reinterpret_cast<const T*>(mc_base) + e, acc);
      } else {
        multimem_ld_reduce_f32x4(reinterpret_cast<const T*>(mc_base) + e, acc);
        multimem_ld_reduce_f32x4(reinterpret_cast<const T*>(mc_base) + e + 4, acc + 4);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
      // start with a different peer on every rank so that the W readers do not hit the same GPU at once
      for (int pi = 0; pi < world; ++pi) {
        const int pr = (rank + pi) % world;
        float f[8];
        load_vec8<T>(reinterpret_cast<const T*>(peers.ptr[pr]) + e, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += f[k];
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      acc[k] *= scale;
      ss += acc[k] * acc[k];
    }
    *reinterpret_cast<float4*>(out + (i << 3)) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(out + (i << 3) + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) {
    if (sumsq) atomicAdd(sumsq, ss);
    if (nonfinite && !isfinite(ss)) *nonfinite = 1.f;
  }
}

// ------------------------------------------------------------------------------------------------
// AdamW over this rank's shard; the bf16 result is stored into every rank's parameter buffer
// ------------------------------------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_mul, max_norm;
};

__device__ __forceinline__ void multimem_st_b64(void* mc_ptr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_ptr), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b))
               : "memory");
}

__global__ void __launch_bounds__(256)
symm_adamw_bcast_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                        const float* __restrict__ grad, PeerTable params, void* mc_params, int world,
                        long long param_offset, long long n, AdamArgs a, const float* __restrict__ sumsq,
                        const float* __restrict__ skip_flag) {
  if (skip_flag && *skip_flag != 0.f) return;
  float gm = a.grad_mul;
  if (sumsq && a.max_norm > 0.f) gm *= fminf(1.f, a.max_norm / (sqrtf(*sumsq) + 1e-6f));
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    float4 p = *reinterpret_cast<float4*>(master + i);
    float4 mm = *reinterpret_cast<float4*>(m + i);
    float4 vv = *reinterpret_cast<float4*>(v + i);
    const float4 g4 = *reinterpret_cast<const float4*>(grad + i);
    float* pp = reinterpret_cast<float*>(&p);
    float* pm = reinterpret_cast<float*>(&mm);
    float* pv = reinterpret_cast<float*>(&vv);
    const float g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * gm;
      pm[e] = a.beta1 * pm[e] + (1.f - a.beta1) * ge;
      pv[e] = a.beta2 * pv[e] + (1.f - a.beta2) * ge * ge;
      pp[e] = pp[e] * (1.f - a.lr * a.weight_decay) - a.lr * (pm[e] / a.bc1) / (sqrtf(pv[e] / a.bc2) + a.eps);
    }
    *reinterpret_cast<float4*>(master + i) = p;
    *reinterpret_cast<float4*>(m + i) = mm;
    *reinterpret_cast<float4*>(v + i) = vv;
    const uint32_t lo = pack_bf16x2(pp[0], pp[1]), hi = pack_bf16x2(pp[2], pp[3]);
    if (mc_params) {
      multimem_st_b64(reinterpret_cast<__nv_bfloat16*>(mc_params) + param_offset + i, lo, hi);
    } else {
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[r]) + param_offset + i) =
            make_uint2(lo, hi);
    }
  }
}

// pull all-gather: copy every peer's shard of the same symmetric buffer into the local buffer
__global__ void __launch_bounds__(512)
symm_all_gather_kernel(PeerTable peers, PadTable pads, int rank, int world, long long shard_bytes,
                       unsigned int slot0, unsigned int epoch, long long wait_cycles, unsigned int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  bool ok = (blockIdx.x == 0) ? pad_barrier(pads, rank, world, slot0, epoch, wait_cycles, 920)
                              : pad_wait_all(pads, rank, world, slot0, epoch, wait_cycles, 921);
  if (!ok) s_ok = 0;
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && status) atomicExch(status, 1u);
    return;
  }
  const long long nvec = shard_bytes >> 4;
  uint4* local = reinterpret_cast<uint4*>(peers.ptr[rank]);
  for (int pi = 1; pi < world; ++pi) {
    const int pr = (rank + pi) % world;
    const uint4* src = reinterpret_cast<const uint4*>(peers.ptr[pr]) + pr * nvec;
    uint4* dst = local + pr * nvec;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      dst[i] = src[i];
  }
}

// one-sided gather: dst[pr * shard .. (pr+1) * shard) = peer pr's shard, for every pr (this rank's included).
// Four 16-byte loads in flight per thread; the grid is kept small by the host so that the copy shares the SMs
// with the GEMMs it runs under.
__global__ void __launch_bounds__(512)
symm_gather_pull_kernel(PeerTable peers, uint4* __restrict__ dst, int rank, int world, long long nvec) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int pi = 0; pi < world; ++pi) {
    const int pr = (rank + 1 + pi) % world;          // remote shards first, a different peer first on every rank
    const uint4* __restrict__ src = reinterpret_cast<const uint4*>(peers.ptr[pr]);
    uint4* d = dst + pr * nvec;
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], e = src[i + 3 * stride];
      d[i] = a; d[i + stride] = b; d[i + 2 * stride] = c; d[i + 3 * stride] = e;
    }
    for (; i < nvec; i += stride) d[i] = src[i];
  }
}

static inline void fill_tables(PeerTable& pt, PadTable& pd, const unsigned long long* ptrs,
                               const unsigned long long* pads, int world, long long byte_offset) {
  for (int i = 0; i < MAX_WORLD; ++i) {
    pt.ptr[i] = (i < world && ptrs) ? reinterpret_cast<void*>(ptrs[i] + byte_offset) : nullptr;
    pd.pad[i] = (i < world && pads) ? reinterpret_cast<unsigned int*>(pads[i]) : nullptr;
  }
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_comm)

using namespace ts;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// peer_ptrs / pad_ptrs: host arrays of `world` device addresses (the same symmetric allocation on every rank and
// its signal pad).  byte_offset selects a sub-buffer of the allocation.  status: device word set to 1 on timeout.
extern "C" int ts_symm_barrier(const unsigned long long* pad_ptrs, int rank, int world, unsigned int slot0,
                               unsigned int epoch, long long wait_cycles, unsigned int* status, void* stream) {
  if (world > MAX_WORLD) return -10;
  PeerTable pt; PadTable pd;
  fill_tables(pt, pd, nullptr, pad_ptrs, world, 0);
  symm_barrier_kernel<<<1, 32, 0, ST(stream)>>>(pd, rank, world, slot0, epoch, wait_cycles, status);
  return (int)cudaGetLastError();
}

extern "C" int ts_symm_reduce_scatter(const unsigned long long* peer_ptrs, const unsigned long long* pad_ptrs,
                                      unsigned long long mc_ptr, long long byte_offset, int is_bf16, int rank,
                                      int world, long long shard_start, long long shard_numel, float* out,
                                      float scale, float* sumsq, float* nonfinite, unsigned int slot0,
                                      unsigned int epoch, long long wait_cycles, unsigned int* status, int max_blocks,
                                      long long buf_elems, void* stream) {
  // buf_elems: elements (of the gradient dtype) from byte_offset to the end of the symmetric allocation
  if (world > MAX_WORLD || shard_numel % 8 != 0 || shard_start < 0 || shard_start + shard_numel > buf_elems) return -10;
  PeerTable pt; PadTable pd;
  fill_tables(pt, pd, peer_ptrs, pad_ptrs, world, byte_offset);
  const void* mc = mc_ptr ? reinterpret_cast<const void*>(mc_ptr + byte_offset) : nullptr;
  long long blocks = (shard_numel / 8 + 511) / 512;
  const long long cap = max_blocks > 0 ? max_blocks : sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (is_bf16)
    symm_reduce_scatter_kernel<__nv_bfloat16><<<(unsigned)blocks, 512, 0, ST(stream)>>>(
        pt, pd, mc, rank, world, shard_start, shard_numel, out, scale, sumsq, nonfinite, slot0, epoch, wait_cycles,
        status, buf_elems);
  else
    symm_reduce_scatter_kernel<float><<<(unsigned)blocks, 512, 0, ST(stream)>>>(
        pt, pd, mc, rank, world, shard_start, shard_numel, out, scale, sumsq, nonfinite, slot0, epoch, wait_cycles,
        status, buf_elems);
  return (int)cudaGetLastError();
}

extern "C" int ts_symm_adamw_bcast(float* master, float* m, float* v, const float* grad,
                                   const unsigned long long* param_ptrs, unsigned long long mc_ptr,
                                   long long byte_offset, int world, long long param_offset, long long n, float lr,
                                   float beta1, float beta2, float eps, float weight_decay, int step, float grad_mul,
                                   const float* sumsq, float max_norm, const float* skip_flag, int max_blocks,
                                   void* stream) {
  if (world > MAX_WORLD || n % 4 != 0 || n <= 0) return n == 0 ? 0 : -10;
  PeerTable pt; PadTable pd;
  fill_tables(pt, pd, param_ptrs, nullptr, world, byte_offset);
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step); a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_mul = grad_mul; a.max_norm = max_norm;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = max_blocks > 0 ? max_blocks : (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  void* mc = mc_ptr ? reinterpret_cast<void*>(mc_ptr + byte_offset) : nullptr;
  symm_adamw_bcast_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(master, m, v, grad, pt, mc, world, param_offset, n,
                                                                    a, sumsq, skip_flag);
  return (int)cudaGetLastError();
}

extern "C" int ts_symm_all_gather(const unsigned long long* peer_ptrs, const unsigned long long* pad_ptrs,
                                  long long byte_offset, int rank, int world, long long shard_bytes,
                                  unsigned int slot0, unsigned int epoch, long long wait_cycles, unsigned int* status,
                                  void* stream) {
  if (world > MAX_WORLD || shard_bytes % 16 != 0) return -10;
  PeerTable pt; PadTable pd;
  fill_tables(pt, pd, peer_ptrs, pad_ptrs, world, byte_offset);
  symm_all_gather_kernel<<<sm_count(), 512, 0, ST(stream)>>>(pt, pd, rank, world, shard_bytes, slot0, epoch,
                                                             wait_cycles, status);
  return (int)cudaGetLastError();
}

// peer_ptrs: the W addresses of the symmetric shard store; byte_offset: this unit's shard inside it; dst: local buffer
// of world * shard_bytes.  Makes no flag traffic and waits for nobody.
extern "C" int ts_symm_gather_pull(const unsigned long long* peer_ptrs, long long byte_offset, void* dst, int rank,
                                   int world, long long shard_bytes, int max_blocks, void* stream) {
  if (world > MAX_WORLD || shard_bytes % 16 != 0 || (reinterpret_cast<unsigned long long>(dst) & 15ull) ||
      (byte_offset & 15ll))
    return -10;
  PeerTable pt; PadTable pd;
  fill_tables(pt, pd, peer_ptrs, nullptr, world, byte_offset);
  const long long nvec = shard_bytes >> 4;
  long long blocks = (nvec + 2047) / 2048;
  const long long cap = max_blocks > 0 ? max_blocks : 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  symm_gather_pull_kernel<<<(unsigned)blocks, 512, 0, ST(stream)>>>(pt, reinterpret_cast<uint4*>(dst), rank, world, nvec);
  return (int)cudaGetLastError();
}

// The same one-sided gather on the copy engines: one peer-to-peer cudaMemcpyAsync per remote shard (the peers' shards
// are mapped into this process's address space) plus one local copy.  No SM runs a single instruction for it, so a
// gather that is prefetched under a layer's GEMMs takes nothing from them but NVLink and HBM bandwidth.
extern "C" int ts_symm_gather_ce(const unsigned long long* peer_ptrs, long long byte_offset, void* dst, int rank,
                                 int world, long long shard_bytes, void* stream) {
  if (world > MAX_WORLD || shard_bytes <= 0) return -10;
  for (int pi = 0; pi < world; ++pi) {
    const int pr = (rank + 1 + pi) % world;          // remote shards first, a different peer first on every rank
    const void* src = reinterpret_cast<const void*>(peer_ptrs[pr] + byte_offset);
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(dst) + static_cast<long long>(pr) * shard_bytes, src,
                                    static_cast<size_t>(shard_bytes), cudaMemcpyDeviceToDevice, ST(stream));
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

// Single-GPU self-test of the bounded wait: one warp waits (system-scope acquire loads) on a flag that nothing
// sets, with the given limit.  `status` becomes 1 when the wait gave up, and the library's error word records
// ERR_FLAG_TIMEOUT; the context stays usable.
__global__ void wait_selftest_kernel(const unsigned int* flag, long long wait_cycles, unsigned int* status) {
  if (threadIdx.x == 0) {
    const bool ok = ts::flag_wait_geq_sys(flag, 1u, wait_cycles, 990);
    if (!ok) atomicExch(status, 1u);
  }
}
extern "C" int ts_symm_wait_selftest(const unsigned int* flag, long long wait_cycles, unsigned int* status,
                                     void* stream) {
  wait_selftest_kernel<<<1, 32, 0, ST(stream)>>>(flag, wait_cycles, status);
  return (int)cudaGetLastError();
}
