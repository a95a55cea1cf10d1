// bf16 GEMM for sm_100a: C[M,N] = alpha * sum_k A[m,k] * B[n,k] (+ C), fp32 accumulation in TMEM.
//
// Design (one CTA per SM, persistent over output tiles):
//   warp 0      TMA producer   - streams 128x64 A tiles and BNx64 B tiles into a STAGES-deep shared-memory ring
//                                (128-byte swizzle, plain non-multicast tiled loads)
//   warp 1      MMA issuer     - one elected thread issues tcgen05.mma (128 x BN x 16) into one of two TMEM
//                                accumulators, tcgen05.commit releases ring slots / publishes the accumulator
//   warps 2..5  epilogue       - tcgen05.ld the finished accumulator (each warp owns its 32 TMEM lanes),
//                                scale / add / convert and store with 16-byte vector stores, while the MMA
//                                warp already works on the next tile in the other accumulator
// Operands may be K-major or MN-major in memory, so forward (X W^T), dgrad (dY W) and wgrad (dY^T X)
// all run without a transpose pass.
//
// Replaces the library GEMMs behind F.linear in the reference
// (data_pipeline/trainer/distributed/tensor_parallel.py:1061,1214) and the zero-bubble split-backward
// GEMMs (data_pipeline/trainer/distributed/zbpp.py:202,232).
#include <stdlib.h>

#include "common.cuh"
#include "host_common.h"

namespace ts {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 8;

struct GemmParams {
  int M, N, K;
  int ldc;
  int a_mn, b_mn;       // 0 = K-major operand, 1 = MN-major operand
  int out_fp32;         // C dtype: 0 = bf16, 1 = fp32
  int accumulate;       // 1: C = alpha*acc + C
  float alpha;
  void* C;
  int num_m_tiles, num_n_tiles, k_blocks;
  // grouped (mixture-of-experts) modes
  const int* tile_expert;   // MODE 1: expert of every 128-row tile of A / C (-1: tile unused)
  size_t c_bytes;           // extent of C in bytes (checked per store in the debug build)
  const int* seg_start;     // MODE 2: [E + 1] first row of every expert's (128-aligned) segment along the K axis
  int group_rows;           // MODE 1: rows (K-major B) or K extent (MN-major B) of one expert inside the stacked B
  int num_groups;           // MODE 2: E; C is [E][M][ldc]
};

// 32 consecutive fp32 accumulator columns of one output row: scale, optionally add to C, convert, store.
__device__ __forceinline__ void gemm_store_chunk(const GemmParams& p, const uint32_t* r, size_t row, int col0) {
  const bool full = (col0 + 32 <= p.N);
  {
    const size_t esz = p.out_fp32 ? 4 : 2;
    const int ncols = full ? 32 : p.N - col0;
    if (!TS_IN_BOUNDS(static_cast<const char*>(p.C) + (row * p.ldc + col0) * esz, ncols * esz, p.C, p.c_bytes, 7000))
      return;
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
    if (full && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v = make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                               __uint_as_float(r[4 * j + 2]) * p.alpha, __uint_as_float(r[4 * j + 3]) * p.alpha);
        if (p.accumulate) {
          const float4 o = *reinterpret_cast<const float4*>(dst + 4 * j);
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *reinterpret_cast<float4*>(dst + 4 * j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {   // static indices keep the accumulator chunk in registers
        if (col0 + j < p.N) {
          float v = __uint_as_float(r[j]) * p.alpha;
          if (p.accumulate) v += dst[j];
          dst[j] = v;
        }
      }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
    if (full && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]) * p.alpha;
        if (p.accumulate) {
          const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * j);
          const float2 o0 = unpack_bf16x2(o.x), o1 = unpack_bf16x2(o.y), o2 = unpack_bf16x2(o.z),
                       o3 = unpack_bf16x2(o.w);
          f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
          f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
        }
        uint4 v;
        v.x = pack_bf16x2(f[0], f[1]);
        v.y = pack_bf16x2(f[2], f[3]);
        v.z = pack_bf16x2(f[4], f[5]);
        v.w = pack_bf16x2(f[6], f[7]);
        *reinterpret_cast<uint4*>(dst + 8 * j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col0 + j < p.N) {
          float v = __uint_as_float(r[j]) * p.alpha;
          if (p.accumulate) v += __bfloat162float(dst[j]);
          dst[j] = __float2bfloat16(v);
        }
      }
    }
  }
}

struct GemmTile {
  int m0, n0;        // tile origin in the A-row / B-row (output) index spaces
  int b_off;         // MODE 1: offset of this tile's expert along B's row (K-major) or K (MN-major) coordinate
  int k0, k_blocks;  // MODE 2: first reduction row and number of 64-wide reduction blocks
  size_t c_row0;     // MODE 2: first output row of this expert's C slab
};

template <int BN>
struct GemmSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;   // 16 KiB
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;   // + alignment slack
};

// MODE 0: dense.  MODE 1: grouped rows - every 128-row tile of A/C belongs to one expert whose weight is a slab of
// the stacked B operand (forward and dgrad of a mixture-of-experts layer on an expert-sorted, 128-aligned token
// buffer).  MODE 2: grouped reduction - one output slab per expert, reduced over that expert's row segment (wgrad).
template <int BN, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : 2 * BN;   // two accumulators

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * S::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;      // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 4);
    mbar_init(&tempty_bar[1], 4);
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

  const int tiles_per_slab = p.num_m_tiles * p.num_n_tiles;
  const int num_tiles = tiles_per_slab * (MODE == 2 ? p.num_groups : 1);
  const int tiles_per_group = GEMM_GROUP_M * p.num_n_tiles;
  bool alive = true;

  // every role walks the same tile sequence and skips the same tiles (returns false), so their phase counters agree
  auto tile_info = [&](int t, GemmTile& ti) -> bool {
    int e = 0;
    if (MODE == 2) {
      e = t / tiles_per_slab;
      t -= e * tiles_per_slab;
    }
    const int g = t / tiles_per_group;
    const int first_m = g * GEMM_GROUP_M;
    const int gsz = min(p.num_m_tiles - first_m, GEMM_GROUP_M);
    const int r = t - g * tiles_per_group;
    ti.m0 = (first_m + (r % gsz)) * GEMM_BM;
    ti.n0 = (r / gsz) * BN;
    ti.b_off = 0;
    ti.k0 = 0;
    ti.k_blocks = p.k_blocks;
    ti.c_row0 = 0;
    if (MODE == 1) {
      const int ex = p.tile_expert[ti.m0 / GEMM_BM];
      if (ex < 0) return false;
      ti.b_off = ex * p.group_rows;
    } else if (MODE == 2) {
      const int s0 = p.seg_start[e], s1 = p.seg_start[e + 1];
      ti.k0 = s0;
      ti.k_blocks = (s1 - s0) / GEMM_BK;
      ti.c_row0 = static_cast<size_t>(e) * p.M;
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one_sync()) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        GemmTile ti;
        if (!tile_info(t, ti)) continue;
        const int m0 = ti.m0, n0 = ti.n0;
        for (int kb = 0; kb < ti.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, alive, 100)) break;
          mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
          uint8_t* a_dst = smem_a + s * S::A_BYTES;
          uint8_t* b_dst = smem_b + s * S::B_BYTES;
          const int k0 = ti.k0 + kb * GEMM_BK;
          if (!p.a_mn) {
            tma_load_2d(a_dst, &tmA, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[s], m0 + j * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(b_dst, &tmB, &full_bar[s], k0, n0 + ti.b_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[s], n0 + j * 64, k0 + ti.b_off);
          }
        }
      }
      if (!alive) {
        // tear-down after a failed wait: give the loads that are still in flight a bounded time to land
        const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
        for (uint32_t i = first; i < it; ++i) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1u) && clock64() - t0 < 2000000ll) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one_sync()) {
      const uint32_t idesc = make_idesc(GEMM_BM, BN, 1, 1, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      uint32_t it = 0, tile_it = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        GemmTile ti;
        if (!tile_info(t, ti) || ti.k_blocks == 0) continue;   // an empty reduction is zero-filled by the epilogue
        const uint32_t acc = tile_it & 1u;
        const uint32_t acc_ph = (tile_it >> 1) & 1u;
        ++tile_it;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1u, alive, 200)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < ti.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, alive, 201)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * S::A_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + s * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
            umma_f16_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);   // slot is free once these MMAs have read it
        }
        if (!alive) break;
        umma_commit(&tfull_bar[acc]);   // accumulator complete
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int q = warp & 3;   // TMEM lane quarter this warp may access
    uint32_t tile_it = 0;
    for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
      GemmTile ti;
      if (!tile_info(t, ti)) continue;
      const int m0 = ti.m0, n0 = ti.n0;
      const int row = m0 + q * 32 + lane;
      if (ti.k_blocks == 0) {
        // nothing to reduce (an expert without tokens): the slab is zero unless it accumulates
        if (!p.accumulate && row < p.M) {
          uint32_t z[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) z[j] = 0u;
          for (int c = 0; c < BN / 32; ++c)
            if (n0 + c * 32 < p.N) gemm_store_chunk(p, z, ti.c_row0 + row, n0 + c * 32);
        }
        continue;
      }
      const uint32_t acc = tile_it & 1u;
      const uint32_t acc_ph = (tile_it >> 1) & 1u;
      ++tile_it;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, alive, 300)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) gemm_store_chunk(p, r, ti.c_row0 + row, col0);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------------------
// cta_group::2 variant: a cluster of two CTAs computes one 256 x 256 tile.  Each CTA streams its own 128 rows of A
// and its own half (128 rows of N) of B, so the shared-memory fill per MMA is 2/3 of the single-CTA kernel's and the
// ring is 6 stages deep.  The leader (even cluster rank) issues the MMAs for both CTAs; every CTA drains its own
// 128 accumulator lanes.  Loads are plain tiled loads whose completion is signalled on the leader's barrier.
// ---------------------------------------------------------------------------------------------------------
constexpr int G2_STAGES = 6;
constexpr int G2_STAGE_BYTES = 32768;      // A 128x64 + B-half 128x64, bf16
constexpr int G2_SMEM = G2_STAGES * G2_STAGE_BYTES + 256 + 1024;

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  constexpr int STAGES = G2_STAGES;
  constexpr int BN = 256;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * 16384;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * G2_STAGE_BYTES);
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
      mbar_init(&full_bar[s], 1);     // leader's copy is the one in use: one arrive.expect_tx, bytes from both CTAs
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
  const int tiles_per_group = GEMM_GROUP_M * n_tiles;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  bool alive = true;

  auto tile_coords = [&](int t, int& m0, int& n0) {
    const int g = t / tiles_per_group;
    const int first_m = g * GEMM_GROUP_M;
    const int gsz = min(m_tiles - first_m, GEMM_GROUP_M);
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
          if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, alive, 110)) break;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * G2_STAGE_BYTES);
          uint8_t* a_dst = smem_a + s * 16384;
          uint8_t* b_dst = smem_b + s * 16384;
          const int k0 = kb * GEMM_BK;
          if (!p.a_mn) {
            tma_load_2d_2cta(a_dst, &tmA, &full_bar[s], k0, m0);
          } else {
            tma_load_2d_2cta(a_dst, &tmA, &full_bar[s], m0, k0);
            tma_load_2d_2cta(a_dst + 8192, &tmA, &full_bar[s], m0 + 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d_2cta(b_dst, &tmB, &full_bar[s], k0, nb0);
          } else {
            tma_load_2d_2cta(b_dst, &tmB, &full_bar[s], nb0, k0);
            tma_load_2d_2cta(b_dst + 8192, &tmB, &full_bar[s], nb0 + 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one_sync()) {
      const uint32_t idesc = make_idesc(256, BN, 1, 1, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      uint32_t it = 0, tile_it = 0;
      for (int t = cluster_id; t < num_tiles && alive; t += num_clusters, ++tile_it) {
        const uint32_t acc = tile_it & 1u;
        if (!mbar_wait(&tempty_bar[acc], ((tile_it >> 1) & 1u) ^ 1u, alive, 210)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1u, alive, 211)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * 16384);
          const uint32_t b_addr = smem_u32(smem_b + s * 16384);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k)
            umma_f16_ss_2cta(d_tmem, make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024),
                             make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
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
      const uint32_t acc = tile_it & 1u;
      if (!mbar_wait(&tfull_bar[acc], (tile_it >> 1) & 1u, alive, 310)) break;
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) gemm_store_chunk(p, r, static_cast<size_t>(row), col0);
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

static int launch_gemm_2cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  int clusters = sm_count() / 2;
  if (tiles < clusters) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * 2);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = G2_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_bf16_2cta_kernel, tmA, tmB, p);
}

template <int BN, int MODE = 0>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmSmem<BN>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles * (MODE == 2 ? p.num_groups : 1);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_bf16_kernel<BN, MODE><<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_gemm)

// C[M,N] = alpha * A . B^T (+ C).
//   a_mn == 0: A is stored [M][lda] (K contiguous);   a_mn == 1: A is stored [K][lda] (M contiguous)
//   b_mn == 0: B is stored [N][ldb] (K contiguous);   b_mn == 1: B is stored [K][ldb] (N contiguous)
//   out_fp32: C is fp32 (else bf16); accumulate: add into the existing C.
//   bn: N tile (256, 128 or 64; 0 = choose).
// Leading dimensions are in elements and must keep rows 16-byte aligned. Returns 0 on success.
extern "C" int ts_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                            int a_mn, int b_mn, int out_fp32, int accumulate, float alpha, int bn, void* stream) {
  using namespace ts;
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if (bn == 0) {
    // prefer the widest tile that still gives every SM work
    const int tiles256 = ((M + 127) / 128) * ((N + 255) / 256);
    bn = (N >= 256 && tiles256 >= sm_count()) ? 256 : (N >= 128 ? 128 : 64);
    if (N >= 256 && tiles256 < sm_count() && ((M + 127) / 128) * ((N + 127) / 128) < tiles256 * 2) bn = 128;
    // the paired-CTA kernel wins whenever every CTA pair gets at least one 256 x 256 tile
    if (N >= 256 && M >= 256 && ((M + 255) / 256) * ((N + 255) / 256) >= sm_count() / 2) bn = 512;
  }
  const bool two_cta = (bn == 512);
  if (two_cta) bn = 128;   // per-CTA B box: 128 rows of N
  if (bn != 256 && bn != 128 && bn != 64) return -11;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, GEMM_BM, 64);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 64);
  if (rc) return rc * 100 - 1;
  if (!b_mn)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)bn, 64);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
  if (rc) return rc * 100 - 2;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.a_mn = a_mn; p.b_mn = b_mn; p.out_fp32 = out_fp32;
  p.accumulate = accumulate; p.alpha = alpha; p.C = C;
  p.num_m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  p.num_n_tiles = (N + bn - 1) / bn;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.tile_expert = nullptr; p.seg_start = nullptr; p.group_rows = 0; p.num_groups = 1;
  p.c_bytes = (static_cast<size_t>(M - 1) * ldc + N) * (out_fp32 ? 4 : 2);
#ifdef TS_DEBUG
  // test hook of the debug build: pretend C ends `TS_DEBUG_SHRINK_C_ROWS` rows early, so that the bounds check (and
  // nothing else) keeps the kernel from writing them
  if (const char* e = getenv("TS_DEBUG_SHRINK_C_ROWS")) {
    const long long cut = atoll(e);
    if (cut > 0 && cut < M) p.c_bytes = (static_cast<size_t>(M - cut - 1) * ldc + N) * (out_fp32 ? 4 : 2);
  }
#endif
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (two_cta) return launch_gemm_2cta(tmA, tmB, p, st);
  if (bn == 256) return launch_gemm<256>(tmA, tmB, p, st);
  if (bn == 128) return launch_gemm<128>(tmA, tmB, p, st);
  return launch_gemm<64>(tmA, tmB, p, st);
}

// Grouped GEMM over an expert-sorted token buffer whose per-expert segments start on 128-row boundaries.
//   mode 1 (forward / dgrad): C[P][N] = A[P][K] * B_e, where e = tile_expert[row / 128] (-1 skips the tile) and B is
//     the stack of E expert matrices: K-major [E*N][ldb] (b_mn = 0) or MN-major [E*K][ldb] (b_mn = 1).  a_mn = 0.
//   mode 2 (wgrad): C[e][M][N] = sum over rows r in [seg_start[e], seg_start[e+1]) of A[r][m] * B[r][n]; both operands
//     MN-major (a_mn = b_mn = 1), K = P.  An empty segment gives a zero slab (or leaves C alone when accumulating).
// `groups` is the device int32 array tile_expert (mode 1, ceil(P/128) entries) or seg_start (mode 2, E + 1 entries).
// Serves the grouped expert GEMMs of data_pipeline/trainer/kernels/moe_kernels.py:219-785.
extern "C" int ts_gemm_grouped_bf16(const void* A, const void* B, void* C, int mode, int M, int N, int K, int lda,
                                    int ldb, int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, float alpha,
                                    const int* groups, int num_groups, void* stream) {
  using namespace ts;
  if (M <= 0 || N <= 0 || K <= 0 || num_groups <= 0 || groups == nullptr) return -10;
  if (mode == 1 && (a_mn != 0 || K % GEMM_BK != 0)) return -12;
  if (mode == 2 && (a_mn != 1 || b_mn != 1)) return -12;
  if (mode != 1 && mode != 2) return -11;
  const int bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, GEMM_BM, 64);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 64);
  if (rc) return rc * 100 - 1;
  const uint64_t eb = (mode == 1) ? (uint64_t)num_groups : 1u;   // mode 1: B stacks the experts along its row axis
  if (!b_mn)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, eb * N, (uint64_t)K, (uint64_t)ldb, (uint32_t)bn, 64);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, eb * K, (uint64_t)N, (uint64_t)ldb, 64, 64);
  if (rc) return rc * 100 - 2;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.a_mn = a_mn; p.b_mn = b_mn; p.out_fp32 = out_fp32;
  p.accumulate = accumulate; p.alpha = alpha; p.C = C;
  p.num_m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  p.num_n_tiles = (N + bn - 1) / bn;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.tile_expert = (mode == 1) ? groups : nullptr;
  p.seg_start = (mode == 2) ? groups : nullptr;
  p.group_rows = b_mn ? K : N;
  p.num_groups = num_groups;
  p.c_bytes = (static_cast<size_t>((mode == 2 ? num_groups : 1)) * M - 1) * ldc * (out_fp32 ? 4 : 2) +
              static_cast<size_t>(N) * (out_fp32 ? 4 : 2);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mode == 1) {
    if (bn == 256) return launch_gemm<256, 1>(tmA, tmB, p, st);
    if (bn == 128) return launch_gemm<128, 1>(tmA, tmB, p, st);
    return launch_gemm<64, 1>(tmA, tmB, p, st);
  }
  if (bn == 256) return launch_gemm<256, 2>(tmA, tmB, p, st);
  if (bn == 128) return launch_gemm<128, 2>(tmA, tmB, p, st);
  return launch_gemm<64, 2>(tmA, tmB, p, st);
}
