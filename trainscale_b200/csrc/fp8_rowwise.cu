// Row-scaled fp8 GEMM at the full fp8 tensor-core rate, and the quantisation kernels around it, for sm_100a.
//
//   C[m][n] = sa[m] * sb[n] * sum_k Aq[m][k] * Bq[n][k]   (+ C)
//
// Every scale is constant along the reduction axis, so it is applied once, in the epilogue: the main loop is the
// paired-CTA tcgen05 loop of the bf16 GEMM (a cluster of two CTAs per 256 x 256 tile, `tcgen05.mma.cta_group::2
// kind::f8f6f4`, 128 fp8 values of K per stage, double-buffered TMEM accumulators) with nothing between the MMAs.
// The 1 x 128 / 128 x 128 block-scaled kernel of fp8.cu pays a TMEM round trip per 128-deep block; this one does not.
//
// All three GEMMs of a linear layer run on it without a transpose pass, because either operand may be K-major or
// MN-major in memory:
//   forward   y [T][N]  = x  (row scales per token)        . W  (row scales per output feature)   K-major, K-major
//   dgrad     dx [T][K] = dy (row scales per token)        . W  (column scales per input feature) K-major, MN-major
//   wgrad     dW [N][K] = dy (column scales per feature n) . x  (column scales per feature k)     MN-major, MN-major
// "Row scale": one fp32 scale per row of the stored matrix; "column scale": one per column (amax over all rows).
// Operands are E4M3 or E5M2 (gradients), chosen per operand.
//
// Replaces _fp8_matmul_row_scaled_kernel, the fp8 quantisation kernels and the delayed-scaling bookkeeping of
// data_pipeline/trainer/kernels/fp8_kernels.py:144-196,472-620 (scales here are taken from the current tensor).
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_common.h"

namespace ts {

constexpr float E4M3_MAX = 448.f;
constexpr float E5M2_MAX = 57344.f;

template <int FMT>   // 0 = e4m3, 1 = e5m2
__device__ __forceinline__ uint32_t pack4_fp8(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t I = FMT == 0 ? __NV_E4M3 : __NV_E5M2;
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, I);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, I);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y), c = unpack_bf16x2(r.z), d = unpack_bf16x2(r.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// ---------------------------------------------------------------------------------------------------------------
// quantisation: one scale per row.  One CTA per row; rows of up to 256 * 4 * 8 = 8192 values stay in registers,
// wider rows are read a second time (an L2 hit).
// ---------------------------------------------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256) quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, long long ld,
                                                            uint8_t* __restrict__ q, float* __restrict__ scale,
                                                            int cols) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ld);
  const int nvec = cols >> 3;
  uint4 cache[4];
  float amax = 0.f;
  auto take = [&](const uint4& r) {
    float f[8];
    unpack8(r, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
  };
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int i = threadIdx.x + c * 256;
    cache[c] = i < nvec ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
    take(cache[c]);
  }
  for (int i = threadIdx.x + 1024; i < nvec; i += 256) take(xr[i]);
  amax = block_max(amax, scratch);
  const float fmax_ = FMT == 0 ? E4M3_MAX : E5M2_MAX;
  const float s = fmaxf(amax, 1e-12f) / fmax_;
  const float inv = 1.f / s;
  uint2* qr = reinterpret_cast<uint2*>(q + row * static_cast<size_t>(cols));
  auto put = [&](int i, const uint4& r) {
    float f[8];
    unpack8(r, f);
    uint2 o;
    o.x = pack4_fp8<FMT>(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
    o.y = pack4_fp8<FMT>(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
    qr[i] = o;
  };
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int i = threadIdx.x + c * 256;
    if (i < nvec) put(i, cache[c]);
  }
  for (int i = threadIdx.x + 1024; i < nvec; i += 256) put(i, xr[i]);
  if (threadIdx.x == 0) scale[row] = s;
}

// ---------------------------------------------------------------------------------------------------------------
// quantisation: one scale per column.  Pass 1 takes the column maxima (each CTA owns 2048 columns x a chunk of rows;
// non-negative floats order like their bit patterns, so the partial maxima meet in an integer atomicMax).  Pass 2
// divides.  Both passes read 4 KiB contiguous per row per CTA.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) col_amax_kernel(const __nv_bfloat16* __restrict__ x, long long ld,
                                                       unsigned int* __restrict__ amax_bits, long long rows, int cols,
                                                       int rows_per_cta) {
  const int col = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (col >= cols) return;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
  float m[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) m[e] = 0.f;
#pragma unroll 4
  for (long long r = r0; r < r1; ++r) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + col);
    float f[8];
    unpack8(v, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) m[e] = fmaxf(m[e], fabsf(f[e]));
  }
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (m[e] > 0.f) atomicMax(amax_bits + col + e, __float_as_uint(m[e]));
}

template <int FMT>
__global__ void __launch_bounds__(256) quant_colwise_kernel(const __nv_bfloat16* __restrict__ x, long long ld,
                                                            const unsigned int* __restrict__ amax_bits,
                                                            uint8_t* __restrict__ q, float* __restrict__ scale,
                                                            long long rows, int cols, int rows_per_cta) {
  const int col = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (col >= cols) return;
  const float fmax_ = FMT == 0 ? E4M3_MAX : E5M2_MAX;
  float inv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float s = fmaxf(__uint_as_float(amax_bits[col + e]), 1e-12f) / fmax_;
    inv[e] = 1.f / s;
    if (blockIdx.y == 0) scale[col + e] = s;
  }
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
#pragma unroll 4
  for (long long r = r0; r < r1; ++r) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + col);
    float f[8];
    unpack8(v, f);
    uint2 o;
    o.x = pack4_fp8<FMT>(f[0] * inv[0], f[1] * inv[1], f[2] * inv[2], f[3] * inv[3]);
    o.y = pack4_fp8<FMT>(f[4] * inv[4], f[5] * inv[5], f[6] * inv[6], f[7] * inv[7]);
    *reinterpret_cast<uint2*>(q + r * static_cast<long long>(cols) + col) = o;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------------------------------------------
constexpr int R8_THREADS = 192;              // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int R8_STAGES = 6;
constexpr int R8_STAGE_BYTES = 32768;        // A 128 x 128 B + this CTA's half of B 128 x 128 B
constexpr int R8_SMEM = R8_STAGES * R8_STAGE_BYTES + 256 + 1024;
constexpr int R8_GROUP_M = 8;

struct R8Params {
  int M, N, K, ldc;
  int a_mn, b_mn;            // 0: K-major operand ([rows][K]); 1: MN-major ([K][rows])
  int a_fmt, b_fmt;          // 0 e4m3, 1 e5m2
  int out_fp32, accumulate;
  const float* sa;           // [M]
  const float* sb;           // [N]
  void* C;
  size_t c_bytes;            // extent of C in bytes (checked per store in the debug build)
  int k_blocks;
};

__device__ __forceinline__ void umma_f8_ss_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 accumulator columns of one output row: apply sa[row] * sb[col], optionally add C, convert, store.
__device__ __forceinline__ void r8_store_chunk(const R8Params& p, const uint32_t* r, size_t row, int col0, float sa) {
  const bool full = (col0 + 32 <= p.N);
  {
    const size_t esz = p.out_fp32 ? 4 : 2;
    const int ncols = full ? 32 : p.N - col0;
    if (!TS_IN_BOUNDS(static_cast<const char*>(p.C) + (row * p.ldc + col0) * esz, ncols * esz, p.C, p.c_bytes, 7100))
      return;
  }
  float v[32];
  if (full && ((reinterpret_cast<uintptr_t>(p.sb + col0) & 15u) == 0)) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(p.sb + col0) + j);
      v[4 * j] = __uint_as_float(r[4 * j]) * sa * s.x;
      v[4 * j + 1] = __uint_as_float(r[4 * j + 1]) * sa * s.y;
      v[4 * j + 2] = __uint_as_float(r[4 * j + 2]) * sa * s.z;
      v[4 * j + 3] = __uint_as_float(r[4 * j + 3]) * sa * s.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (col0 + j < p.N) ? __uint_as_float(r[j]) * sa * __ldg(p.sb + col0 + j) : 0.f;
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
    if (full && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (p.accumulate) {
          const float4 c = *reinterpret_cast<const float4*>(dst + 4 * j);
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        *reinterpret_cast<float4*>(dst + 4 * j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
    if (full && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.accumulate) {
          const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * j);
          const float2 o0 = unpack_bf16x2(o.x), o1 = unpack_bf16x2(o.y), o2 = unpack_bf16x2(o.z),
                       o3 = unpack_bf16x2(o.w);
          v[8 * j] += o0.x; v[8 * j + 1] += o0.y; v[8 * j + 2] += o1.x; v[8 * j + 3] += o1.y;
          v[8 * j + 4] += o2.x; v[8 * j + 5] += o2.y; v[8 * j + 6] += o3.x; v[8 * j + 7] += o3.y;
        }
        uint4 w;
        w.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
        w.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
        w.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
        w.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
        *reinterpret_cast<uint4*>(dst + 8 * j) = w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = __float2bfloat16(p.accumulate ? __bfloat162float(dst[j]) + v[j] : v[j]);
    }
  }
}

__global__ void __launch_bounds__(R8_THREADS, 1)
fp8_rowwise_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             R8Params p) {
  constexpr int STAGES = R8_STAGES;
  constexpr int BN = 256;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * 16384;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * R8_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const bool leader = (crank == 0);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);     // the leader's copy is the one in use: one expect_tx, bytes from both CTAs
      mbar_init(&empty_bar[s], 1);    // one multicast commit per phase
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 8);     // 4 epilogue warps of each CTA arrive on the leader's copy
    mbar_init(&tempty_bar[1], 8);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TMEM_COLS);
    tmem_relinquish_2cta();
    tc_fence_before_sync();
  }
  __syncthreads();
  cluster_sync_all();                 // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (p.M + 255) / 256;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int tiles_per_group = R8_GROUP_M * n_tiles;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  bool alive = true;

  auto tile_coords = [&](int t, int& m0, int& n0) {
    const int g = t / tiles_per_group;
    const int first_m = g * R8_GROUP_M;
    const int gsz = min(m_tiles - first_m, R8_GROUP_M);
    const int r = t - g * tiles_per_group;
    m0 = (first_m + (r % gsz)) * 256 + (int)crank * 128;   // this CTA's 128 rows
    n0 = (r / gsz) * BN;
  };

  if (warp == 0) {
    if (elect_one_sync()) {
      uint32_t it = 0;
      for (int t = cluster_id; t < num_tiles && alive; t += num_clusters) {
        int m0, n0;
        tile_coords(t, m0, n0);
        const int nb0 = n0 + (int)crank * 128;             // this CTA's half of the B tile
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, alive, 1110)) break;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * R8_STAGE_BYTES);
          const int k0 = kb * 128;
          if (!p.a_mn) tma_load_2d_2cta(smem_a + s * 16384, &tmA, &full_bar[s], k0, m0);
          else         tma_load_2d_2cta(smem_a + s * 16384, &tmA, &full_bar[s], m0, k0);
          if (!p.b_mn) tma_load_2d_2cta(smem_b + s * 16384, &tmB, &full_bar[s], k0, nb0);
          else         tma_load_2d_2cta(smem_b + s * 16384, &tmB, &full_bar[s], nb0, k0);
        }
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one_sync()) {
      const uint32_t idesc = make_idesc(256, BN, (uint32_t)p.a_fmt, (uint32_t)p.b_fmt, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
      // one instruction reduces 32 values of K: 32 bytes along a K-major row, or 32 rows of 128 bytes when MN-major
      const uint32_t a_kstep = p.a_mn ? 4096u : 32u;
      const uint32_t b_kstep = p.b_mn ? 4096u : 32u;
      uint32_t it = 0, tile_it = 0;
      for (int t = cluster_id; t < num_tiles && alive; t += num_clusters, ++tile_it) {
        const uint32_t acc = tile_it & 1u;
        if (!mbar_wait(&tempty_bar[acc], ((tile_it >> 1) & 1u) ^ 1u, alive, 1210)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1u, alive, 1211)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * 16384);
          const uint32_t b_addr = smem_u32(smem_b + s * 16384);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8_ss_2cta(d_tmem, make_smem_desc_sw128(a_addr + k * a_kstep, 16, 1024),
                            make_smem_desc_sw128(b_addr + k * b_kstep, 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_2cta_mc(&empty_bar[s], 3);
        }
        if (!alive) break;
        umma_commit_2cta_mc(&tfull_bar[acc], 3);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tile_it = 0;
    for (int t = cluster_id; t < num_tiles && alive; t += num_clusters, ++tile_it) {
      int m0, n0;
      tile_coords(t, m0, n0);
      const int row = m0 + q * 32 + lane;
      const float sa = (row < p.M) ? __ldg(p.sa + row) : 0.f;
      const uint32_t acc = tile_it & 1u;
      if (!mbar_wait(&tfull_bar[acc], (tile_it >> 1) & 1u, alive, 1310)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) r8_store_chunk(p, r, static_cast<size_t>(row), col0, sa);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&tempty_bar[acc], 0);   // the leader's MMA thread owns the accumulators
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // nobody leaves (or frees TMEM) while the peer may still signal or read
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_fp8_rowwise)
using namespace ts;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// x [rows][ld] bf16 (cols used, cols % 8 == 0, 16-byte aligned rows) -> q fp8 [rows][cols], scale fp32 [rows].
// fmt: 0 = E4M3, 1 = E5M2.
extern "C" int ts_fp8_quant_rowwise(const void* x, long long ld, void* q, float* scale, long long rows, int cols,
                                    int fmt, void* stream) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15u)) return -10;
  if (fmt == 0)
    quant_rowwise_kernel<0><<<(unsigned)rows, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, scale, cols);
  else
    quant_rowwise_kernel<1><<<(unsigned)rows, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, scale, cols);
  return (int)cudaGetLastError();
}

// x [rows][ld] bf16 -> q fp8 [rows][cols] in the SAME layout, scale fp32 [cols] (amax over all rows of a column).
// `amax_work`: device u32 [cols] scratch (cleared here).
extern "C" int ts_fp8_quant_colwise(const void* x, long long ld, void* q, float* scale, unsigned int* amax_work,
                                    long long rows, int cols, int fmt, void* stream) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15u)) return -10;
  cudaError_t e = cudaMemsetAsync(amax_work, 0, sizeof(unsigned int) * (size_t)cols, ST(stream));
  if (e != cudaSuccess) return (int)e;
  const int gx = (cols + 2047) / 2048;
  // enough CTAs to fill the GPU a few times over, at least 16 rows each
  long long gy = (static_cast<long long>(sm_count()) * 8 + gx - 1) / gx;
  if (gy > (rows + 15) / 16) gy = (rows + 15) / 16;
  if (gy < 1) gy = 1;
  if (gy > 65535) gy = 65535;
  const int rpc = (int)((rows + gy - 1) / gy);
  gy = (rows + rpc - 1) / rpc;
  dim3 grid(gx, (unsigned)gy);
  col_amax_kernel<<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, ld, amax_work, rows, cols, rpc);
  if (fmt == 0)
    quant_colwise_kernel<0><<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, ld, amax_work, (uint8_t*)q, scale, rows,
                                                          cols, rpc);
  else
    quant_colwise_kernel<1><<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, ld, amax_work, (uint8_t*)q, scale, rows,
                                                          cols, rpc);
  return (int)cudaGetLastError();
}

// C[M][N] = sa[m] * sb[n] * (A . B^T) (+ C).
//   a_mn == 0: A stored [M][lda] (K contiguous);  a_mn == 1: A stored [K][lda] (M contiguous)
//   b_mn == 0: B stored [N][ldb] (K contiguous);  b_mn == 1: B stored [K][ldb] (N contiguous)
//   a_fmt / b_fmt: 0 = E4M3, 1 = E5M2.  Leading dimensions in bytes (= elements), multiples of 16.
extern "C" int ts_fp8_rowwise_gemm(const void* A, const float* sa, const void* B, const float* sb, void* C, int M, int N,
                                   int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int a_fmt, int b_fmt,
                                   int out_fp32, int accumulate, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (a_fmt | b_fmt) > 1) return -10;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128, 128);
  else       rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 128, 128);
  if (rc) return rc * 100 - 1;
  if (!b_mn) rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, 128);
  else       rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 128, 128);
  if (rc) return rc * 100 - 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fp8_rowwise_gemm_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, R8_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  R8Params p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.a_mn = a_mn; p.b_mn = b_mn; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.sa = sa; p.sb = sb; p.C = C;
  p.k_blocks = (K + 127) / 128;
  p.c_bytes = (static_cast<size_t>(M - 1) * ldc + N) * (out_fp32 ? 4 : 2);
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  int clusters = sm_count() / 2;
  if (tiles < clusters) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * 2);
  cfg.blockDim = dim3(R8_THREADS);
  cfg.dynamicSmemBytes = R8_SMEM;
  cfg.stream = ST(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, fp8_rowwise_gemm_2cta_kernel, tmA, tmB, p);
}
