// Block-scaled fp8 (E4M3) GEMM and the quantise / dequantise kernels around it, for sm_100a.
//
//   C[m][n] = sum_kb ( sum_{k in block kb} Aq[m][k] * Bq[n][k] ) * sa[kb][m] * sb[n / 128][kb]
//
// Activations carry one fp32 scale per 1 x 128 block, weights one per 128 x 128 block.  The tensor core reduces one
// 128-deep block at a time (tcgen05.mma kind::f8f6f4, four K=32 instructions) into one of four TMEM accumulators; eight
// epilogue warps drain the finished block, apply the two scales and add into fp32 registers ("promotion") while the MMA
// warp already fills the next accumulators.  B may be K-major ([N][K], forward) or MN-major ([K][N], dgrad: the same
// stored weight without a transpose pass).
//
// Replaces _fp8_matmul_block_scaled_kernel / _fp8_matmul_row_scaled_kernel and the quantisation kernels of
// data_pipeline/trainer/kernels/fp8_kernels.py:203-553.
#include <cuda_fp8.h>

#include "common.cuh"
#include "host_common.h"

namespace ts {

constexpr float FP8_E4M3_MAX = 448.f;

// ---------------------------------------------------------------------------------------------------------------
// quantisation
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// x [M][K] bf16 -> q [M][K] e4m3, scale [K/128][M] fp32 (one per 1 x 128 block, stored block-major so that the GEMM
// epilogue reads consecutive rows).  One warp per block, four elements per lane.
__global__ void fp8_quant_act_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                     float* __restrict__ scale, long long M, int K) {
  const int kblocks = K / 128;
  const long long total = M * kblocks;
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long w = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += warps) {
    const long long m = w / kblocks;
    const int kb = static_cast<int>(w - m * kblocks);
    const size_t off = static_cast<size_t>(m) * K + kb * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(x + off);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
    amax = warp_max(amax);
    const float s = fmaxf(amax, 1e-12f) / FP8_E4M3_MAX;
    const float inv = 1.f / s;
    *reinterpret_cast<uint32_t*>(q + off) = pack4_e4m3(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
    if (lane == 0) scale[static_cast<size_t>(kb) * M + m] = s;
  }
}

// w [N][K] bf16 -> q [N][K] e4m3, scale [ceil(N/128)][K/128] fp32 (one per 128 x 128 block).  One CTA per block.
__global__ void __launch_bounds__(256) fp8_quant_block_kernel(const __nv_bfloat16* __restrict__ w,
                                                              uint8_t* __restrict__ q, float* __restrict__ scale,
                                                              int N, int K) {
  __shared__ float scratch[32];
  const int nb = blockIdx.y, kb = blockIdx.x;
  const int kblocks = K / 128;
  // thread t: column group (t & 31) * 4, rows (t >> 5) + 8 * i
  const int c = (threadIdx.x & 31) * 4;
  float v[16][4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = nb * 128 + (threadIdx.x >> 5) + 8 * i;
    if (r < N) {
      const uint2 raw = *reinterpret_cast<const uint2*>(w + static_cast<size_t>(r) * K + kb * 128 + c);
      const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = b.x; v[i][3] = b.y;
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
    } else {
      v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    }
  }
  amax = block_max(amax, scratch);
  const float s = fmaxf(amax, 1e-12f) / FP8_E4M3_MAX;
  const float inv = 1.f / s;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = nb * 128 + (threadIdx.x >> 5) + 8 * i;
    if (r < N)
      *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(r) * K + kb * 128 + c) =
          pack4_e4m3(v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv);
  }
  if (threadIdx.x == 0) scale[static_cast<size_t>(nb) * kblocks + kb] = s;
}

// per-row (per-token) quantisation: scale [M]
__global__ void __launch_bounds__(256) fp8_quant_row_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                            float* __restrict__ scale, int K) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float amax = 0.f;
  for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + row * K + i);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
  }
  amax = block_max(amax, scratch);
  const float s = fmaxf(amax, 1e-12f) / FP8_E4M3_MAX;
  const float inv = 1.f / s;
  for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + row * K + i);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    *reinterpret_cast<uint32_t*>(q + row * K + i) = pack4_e4m3(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
  }
  if (threadIdx.x == 0) scale[row] = s;
}

// q [R][K] e4m3 -> out bf16 with scale index (r / rdiv) * s_r + (k / 128) * s_k (covers block, activation and row
// layouts: row scales use s_k = 0)
__global__ void fp8_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale,
                                   __nv_bfloat16* __restrict__ out, long long R, int K, int rdiv, long long s_r,
                                   long long s_k) {
  const long long total = R * (K / 4);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / (K / 4);
    const int k = static_cast<int>(i - r * (K / 4)) * 4;
    const float s = scale[(r / rdiv) * s_r + (k / 128) * s_k];
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(q + r * K + k);
    uint2 o;
    o.x = pack_bf16x2(e4m3_to_float(raw & 0xff) * s, e4m3_to_float((raw >> 8) & 0xff) * s);
    o.y = pack_bf16x2(e4m3_to_float((raw >> 16) & 0xff) * s, e4m3_to_float(raw >> 24) * s);
    *reinterpret_cast<uint2*>(out + r * K + k) = o;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------------------------------------------
constexpr int F8_THREADS = 320;       // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two per TMEM lane quarter)
constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
constexpr int F8_STAGES = 6;
constexpr int F8_STAGE_BYTES = 2 * 128 * 128;
constexpr int F8_SMEM = F8_STAGES * F8_STAGE_BYTES + 256 + 1024;

struct Fp8GemmParams {
  int M, N, K, ldc;
  int b_mn;                 // 0: B stored [N][K]; 1: B stored [K][N]
  int out_fp32;
  const float* sa;          // [K/128][M]
  const float* sb;          // index: (n / 128) * sb_n + kb * sb_k
  long long sb_n, sb_k;
  void* C;
  int num_m_tiles, num_n_tiles, k_blocks;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Fp8GemmParams p) {
  constexpr int STAGES = F8_STAGES;
  constexpr int NACC = 4;                     // 128-column accumulators in flight between MMA and promotion
  constexpr uint32_t TMEM_COLS = NACC * F8_BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * 16384;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * F8_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;            // [NACC]
  uint64_t* tempty_bar = bars + 2 * STAGES + NACC;     // [NACC]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NACC);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  bool alive = true;

  auto tile_coords = [&](int t, int& m0, int& n0) {   // M fastest: neighbouring CTAs share the weight tile in L2
    m0 = (t % p.num_m_tiles) * F8_BM;
    n0 = (t / p.num_m_tiles) * F8_BN;
  };

  if (warp == 0) {
    if (elect_one_sync()) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int m0, n0;
        tile_coords(t, m0, n0);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, alive, 900)) break;
          mbar_expect_tx(&full_bar[s], F8_STAGE_BYTES);
          tma_load_2d(smem_a + s * 16384, &tmA, &full_bar[s], kb * F8_BK, m0);
          if (!p.b_mn)
            tma_load_2d(smem_b + s * 16384, &tmB, &full_bar[s], kb * F8_BK, n0);
          else
            tma_load_2d(smem_b + s * 16384, &tmB, &full_bar[s], n0, kb * F8_BK);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      const uint32_t idesc = make_idesc(F8_BM, F8_BN, 0, 0, 0, (uint32_t)p.b_mn);   // e4m3 x e4m3
      const uint32_t b_kstep = p.b_mn ? 4096u : 32u;   // 32 reduction rows of 128 bytes, or 32 bytes along a row
      uint32_t it = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t acc = it % NACC;
          if (!mbar_wait(&tempty_bar[acc], ((it / NACC) & 1u) ^ 1u, alive, 910)) break;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1u, alive, 911)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * 16384), b_addr = smem_u32(smem_b + s * 16384);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8_ss(tmem_base + acc * F8_BN, make_smem_desc_sw128(a_addr + k * 32, 16, 1024),
                       make_smem_desc_sw128(b_addr + k * b_kstep, 16, 1024), idesc, k != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
          umma_commit(&tfull_bar[acc]);   // one 128-deep block is complete: hand it to the promotion warps
        }
      }
    }
  } else {
    const int q = warp & 3;               // TMEM lane quarter
    const int half = (warp - 2) >> 2;     // column half (64 columns)
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * 64;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
      int m0, n0;
      tile_coords(t, m0, n0);
      const int row = m0 + q * 32 + lane;
      const int rowc = row < p.M ? row : p.M - 1;
      float accum[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) accum[j] = 0.f;
      const float* sbp = p.sb + static_cast<long long>(n0 / 128) * p.sb_n;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        const uint32_t acc = it % NACC;
        const float sc = p.sa[static_cast<size_t>(kb) * p.M + rowc] * sbp[kb * p.sb_k];
        if (!mbar_wait(&tfull_bar[acc], (it / NACC) & 1u, alive, 920)) break;
        tc_fence_after_sync();
        uint32_t v[64];
        tmem_ld_32x32b_x32(t_lane + acc * F8_BN, v);
        tmem_ld_32x32b_x32(t_lane + acc * F8_BN + 32, v + 32);
        tc_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);   // the block is in registers: the accumulator may be refilled
#pragma unroll
        for (int j = 0; j < 64; ++j) accum[j] = fmaf(__uint_as_float(v[j]), sc, accum[j]);
      }
      if (!alive) break;
      if (row < p.M) {
        const int c0 = n0 + half * 64;
        if (p.out_fp32) {
          float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + c0;
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (c0 + j < p.N) dst[j] = accum[j];
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + c0;
          if (c0 + 64 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint4 o;
              o.x = pack_bf16x2(accum[8 * j], accum[8 * j + 1]);
              o.y = pack_bf16x2(accum[8 * j + 2], accum[8 * j + 3]);
              o.z = pack_bf16x2(accum[8 * j + 4], accum[8 * j + 5]);
              o.w = pack_bf16x2(accum[8 * j + 6], accum[8 * j + 7]);
              *reinterpret_cast<uint4*>(dst + 8 * j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j)
              if (c0 + j < p.N) dst[j] = __float2bfloat16(accum[j]);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_fp8)
using namespace ts;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

static int elem_grid(long long work_items, int per_block) {
  long long blocks = (work_items + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// x [M][K] bf16 -> q e4m3 [M][K], scale fp32 [K/128][M]
extern "C" int ts_fp8_quant_act(const void* x, void* q, float* scale, long long M, int K, void* stream) {
  if (M <= 0 || K <= 0 || K % 128 != 0) return -10;
  fp8_quant_act_kernel<<<elem_grid(M * (K / 128), 8), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (uint8_t*)q, scale,
                                                                            M, K);
  return (int)cudaGetLastError();
}

// w [N][K] bf16 -> q e4m3 [N][K], scale fp32 [ceil(N/128)][K/128]
extern "C" int ts_fp8_quant_block(const void* w, void* q, float* scale, int N, int K, void* stream) {
  if (N <= 0 || K <= 0 || K % 128 != 0) return -10;
  fp8_quant_block_kernel<<<dim3(K / 128, (N + 127) / 128), 256, 0, ST(stream)>>>((const __nv_bfloat16*)w, (uint8_t*)q,
                                                                                  scale, N, K);
  return (int)cudaGetLastError();
}

extern "C" int ts_fp8_quant_row(const void* x, void* q, float* scale, long long M, int K, void* stream) {
  if (M <= 0 || K <= 0 || K % 4 != 0) return -10;
  fp8_quant_row_kernel<<<(unsigned)M, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (uint8_t*)q, scale, K);
  return (int)cudaGetLastError();
}

// layout: 0 = 128x128 blocks (scale [R/128][K/128]), 1 = 1x128 activation blocks (scale [K/128][R]), 2 = per row
extern "C" int ts_fp8_dequant(const void* q, const float* scale, void* out, long long R, int K, int layout,
                              void* stream) {
  if (R <= 0 || K <= 0 || K % 4 != 0 || (layout != 2 && K % 128 != 0)) return -10;
  int rdiv = 1;
  long long s_r = 1, s_k = 0;
  if (layout == 0) { rdiv = 128; s_r = K / 128; s_k = 1; }
  else if (layout == 1) { rdiv = 1; s_r = 1; s_k = R; }
  fp8_dequant_kernel<<<elem_grid(R * (K / 4), 256), 256, 0, ST(stream)>>>((const uint8_t*)q, scale, (__nv_bfloat16*)out,
                                                                          R, K, rdiv, s_r, s_k);
  return (int)cudaGetLastError();
}

// C[M][N] = block-scaled Aq[M][K] * B.  b_mn = 0: Bq is [N][K] with scales sb[(n/128)*sb_n + (k/128)*sb_k];
// b_mn = 1: Bq is stored [K][N] (N contiguous).  sa is [K/128][M].  K must be a multiple of 128; A rows and B rows
// must be 16-byte aligned (lda, ldb in bytes == elements).
extern "C" int ts_fp8_gemm(const void* Aq, const float* sa, const void* Bq, const float* sb, long long sb_n,
                           long long sb_k, void* C, int M, int N, int K, int lda, int ldb, int ldc, int b_mn,
                           int out_fp32, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 128 != 0) return -10;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128, 128);
  if (rc) return rc * 100 - 1;
  if (!b_mn)
    rc = make_tmap_2d(&tmB, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, 128);
  else
    rc = make_tmap_2d(&tmB, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 128, 128);
  if (rc) return rc * 100 - 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  Fp8GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.b_mn = b_mn; p.out_fp32 = out_fp32;
  p.sa = sa; p.sb = sb; p.sb_n = sb_n; p.sb_k = sb_k; p.C = C;
  p.num_m_tiles = (M + F8_BM - 1) / F8_BM;
  p.num_n_tiles = (N + F8_BN - 1) / F8_BN;
  p.k_blocks = K / F8_BK;
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  fp8_gemm_kernel<<<grid, F8_THREADS, F8_SMEM, ST(stream)>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}
