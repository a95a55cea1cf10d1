// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a, tcgen05 + TMEM + TMA).
//
//   mode GATHER  (all-gather -> GEMM):  A's rows are sharded over the W ranks (sequence parallelism).  Copier warps
//       of the same persistent kernel pull the remote row blocks into a local buffer with plain peer loads, in the
//       order the MMA tiles will need them (own rows first, then rank+1, rank+2, ...), and publish per-row-block
//       counters; the TMA producer waits on the counter of a row block (bounded) before it loads tiles from it.
//       The transfer overlaps the math tile by tile and every remote byte crosses NVLink once.
//   mode REDUCE  (GEMM -> reduce-scatter): the epilogue adds each 128-row tile of partial sums straight into the
//       owning rank's fp32 buffer with vector `red.global.add.v4.f32` over peer pointers; no partial-sum tensor is
//       ever written locally and nothing waits for the whole GEMM to finish before data moves.
// Both modes run the cross-rank hand-shakes inside the kernel: an entry barrier (peer operands are ready / the
// reduction buffers are cleared) performed by CTA 0 and published through a local flag, and an exit barrier
// performed by the last CTA to finish (so a rank's kernel completes only after every peer has finished touching
// its memory).  All waits are bounded and report through the error word / status word.
//
// TMA loads here are plain tiled loads (never cluster multicast), and they only ever read THIS GPU's memory: the
// remote rows are brought in by ordinary ld.global from peer pointers.
//
// Replaces the serial all_gather -> F.linear and F.linear -> reduce_scatter pairs of
// data_pipeline/trainer/distributed/tensor_parallel.py:1053-1061,1214-1219.
#include <cstdlib>

#include "common.cuh"
#include "host_common.h"

namespace ts {

constexpr int TP_BM = 128, TP_BK = 64, TP_GROUP_M = 8, TP_MAX_WORLD = 16;
constexpr int TP_THREADS = 320;          // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue, warps 6..9 copiers
constexpr int TP_SUB = 4;                // a remote row block is fetched as TP_SUB column slices

struct TpPeers {
  const void* src[TP_MAX_WORLD];         // GATHER: every rank's A shard ([rows_per_rank][K] bf16)
  void* dst[TP_MAX_WORLD];               // REDUCE: every rank's accumulation buffer ([rows_per_rank][N], fp32 or bf16)
  unsigned int* pad[TP_MAX_WORLD];       // signal pads
};

struct TpMaps {
  CUtensorMap m[TP_MAX_WORLD];           // REDUCE by bulk tensor reduction: rank r's [rows_per_rank][N] bf16 accumulation buffer
};

struct TpParams {
  int M, N, K, ldc;
  int b_mn;
  int mode;                              // 1 = GATHER (rows of A), 2 = REDUCE, 3 = GATHER_B (rows of the weight operand)
  int acc_bf16;                          // REDUCE: accumulate packed bf16 pairs (8 elements per 16-byte red) instead of fp32
  int tma_red;                           // REDUCE: epilogue tiles are added into the owner's bf16 buffer by bulk tensor reductions
  int push;                              // REDUCE: no atomics - partial sums are stored into slot `rank` of the owner's staging buffer
  int rank, world, rows_per_rank;
  void* C;                               // GATHER: bf16 output [M][ldc]
  __nv_bfloat16* a_full;                 // GATHER: local [M][K] buffer the remote rows are staged into
  int num_m_tiles, num_n_tiles, k_blocks;
  unsigned int* flags;                   // [0] entry flag, [1] done counter, [2 + m_block] staging counters
  unsigned int epoch, slot0;
  long long wait_cycles;
  unsigned int* status;
};

template <int BN>
struct TpSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = TP_BM * TP_BK * 2;
  static constexpr int B_BYTES = BN * TP_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 256 + 1024;
};

__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void red_add_v4_bf16x2(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
// one 32-column chunk of partial sums of `row` added into the owner's buffer
__device__ __forceinline__ void tp_reduce_chunk(const TpParams& p, const TpPeers& peers, const uint32_t* r, int row,
                                                int col0);
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

__device__ __forceinline__ void tp_reduce_chunk(const TpParams& p, const TpPeers& peers, const uint32_t* r, int row,
                                                int col0) {
  const int owner = row / p.rows_per_rank;
  const size_t off = static_cast<size_t>(row - owner * p.rows_per_rank) * p.N + col0;
  if (p.push && owner != p.rank) {
    // plain 16-byte stores of this rank's partial sums into its own slot of the owner's staging buffer
    // ([W][rows_per_rank][N] bf16): nothing is read-modify-written across NVLink, the owner adds the slots afterwards
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peers.dst[owner]) +
                         static_cast<size_t>(p.rank) * p.rows_per_rank * p.N + off;
    if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
        v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        *reinterpret_cast<uint4*>(dst + 8 * j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
    }
    return;
  }
  if ((p.acc_bf16 || p.push) && owner == p.rank && p.C != nullptr) {
    // this rank's own rows need no reduction traffic: the partial sum is stored into a private buffer and added to
    // what the peers reduced into the shared one after the kernel
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
    if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
        v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        *reinterpret_cast<uint4*>(dst + 8 * j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
    }
    return;
  }
  if (p.acc_bf16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peers.dst[owner]) + off;
    if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        red_add_v4_bf16x2(dst + 8 * j, pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                          pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                          pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                          pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) atomicAdd(dst + j, __float2bfloat16(__uint_as_float(r[j])));
    }
    return;
  }
  float* dst = reinterpret_cast<float*>(peers.dst[owner]) + off;
  if (col0 + 32 <= p.N) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      red_add_v4_f32(dst + 4 * j, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                     __uint_as_float(r[4 * j + 3]));
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) atomicAdd_system(dst + j, __uint_as_float(r[j]));
  }
}

template <int BN>
__global__ void __launch_bounds__(TP_THREADS, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, TpParams p,
               TpPeers peers) {
  using S = TpSmem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * S::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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

  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int tiles_per_group = TP_GROUP_M * p.num_n_tiles;
  const int m_tiles_per_rank = p.rows_per_rank / TP_BM;
  bool alive = true;

  // logical m index j -> physical row block: own rows first, then the next ranks' rows in ring order
  // REDUCE: the next ranks' rows first and the own rows last, so that remote additions start at once and the tail of
  // the kernel only touches local memory
  auto phys_m = [&](int j) {
    if (p.mode != 1) return (j + (p.rank + 1) * m_tiles_per_rank) % p.num_m_tiles;
    return (j + p.rank * m_tiles_per_rank) % p.num_m_tiles;
  };
  auto tile_coords = [&](int t, int& mt, int& n0) {
    const int g = t / tiles_per_group;
    const int first_m = g * TP_GROUP_M;
    const int gsz = min(p.num_m_tiles - first_m, TP_GROUP_M);
    const int r = t - g * tiles_per_group;
    mt = phys_m(first_m + (r % gsz));
    n0 = (r / gsz) * BN;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one_sync()) {
      uint32_t it = 0;
      int last_ready = -1;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int mt, n0;
        tile_coords(t, mt, n0);
        if (p.mode == 1 && mt / m_tiles_per_rank != p.rank && mt != last_ready) {
          // the rows of this block come from a peer: wait until the copiers have staged all of it
          if (!flag_wait_geq_gpu(p.flags + 2 + mt, p.epoch * TP_SUB, p.wait_cycles, 1000)) {
            alive = false;
            if (p.status) atomicExch(p.status, 1u);
            break;
          }
          fence_proxy_async_global();
          last_ready = mt;
        }
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, alive, 1001)) break;
          mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
          tma_load_2d(smem_a + s * S::A_BYTES, &tmA, &full_bar[s], kb * TP_BK, mt * TP_BM);
          uint8_t* b_dst = smem_b + s * S::B_BYTES;
          if (!p.b_mn) {
            tma_load_2d(b_dst, &tmB, &full_bar[s], kb * TP_BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[s], n0 + j * 64, kb * TP_BK);
          }
        }
      }
      if (!alive) {
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
      const uint32_t idesc = make_idesc(TP_BM, BN, 1, 1, 0u, (uint32_t)p.b_mn);
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      uint32_t it = 0, tile_it = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x, ++tile_it) {
        const uint32_t acc = tile_it & 1u;
        if (!mbar_wait(&tempty_bar[acc], ((tile_it >> 1) & 1u) ^ 1u, alive, 1010)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1u, alive, 1011)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * S::A_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + s * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < TP_BK / 16; ++k)
            umma_f16_ss(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 16, 1024),
                        make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (!alive) break;
        umma_commit(&tfull_bar[acc]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    uint32_t tile_it = 0;
    bool entry_ok = (p.mode != 2);
    for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x, ++tile_it) {
      int mt, n0;
      tile_coords(t, mt, n0);
      const uint32_t acc = tile_it & 1u;
      if (!mbar_wait(&tfull_bar[acc], (tile_it >> 1) & 1u, alive, 1020)) break;
      tc_fence_after_sync();
      if (!entry_ok) {
        // nobody may add into a peer's buffer before every rank has cleared it (entry barrier by CTA 0)
        if (!flag_wait_geq_gpu(p.flags, p.epoch, p.wait_cycles, 1021)) {
          alive = false;
          if (p.status) atomicExch(p.status, 1u);
          break;
        }
        entry_ok = true;
      }
      const int row = mt * TP_BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (row >= p.M || col0 >= p.N) continue;
        if (p.mode == 2) {
          tp_reduce_chunk(p, peers, r, row, col0);
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
          if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(dst + 8 * j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
    __threadfence_system();   // peer adds of this thread are ordered before the CTA's "done" count
  } else {
    // ------------------------------ copiers (warps 6..9) ------------------------------
    const int ct = threadIdx.x - 192;   // 0..127
    if (blockIdx.x == 0) {
      // entry barrier with the peers, then publish it to the other CTAs of this GPU through flags[0]
      if (ct < p.world) {
        __threadfence_system();
        st_release_sys(peers.pad[ct] + p.slot0 + p.rank, p.epoch);
        if (!flag_wait_geq_sys(peers.pad[p.rank] + p.slot0 + ct, p.epoch, p.wait_cycles, 1030) && p.status)
          atomicExch(p.status, 1u);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ct == 0) {
        const unsigned int bad = p.status ? atomicAdd(p.status, 0u) : 0u;
        if (!bad) st_release_gpu(p.flags, p.epoch);
      }
    }
    if (p.mode == 1) {
      if (!flag_wait_geq_gpu(p.flags, p.epoch, p.wait_cycles, 1031)) {
        if (ct == 0 && p.status) atomicExch(p.status, 1u);
      } else {
        // remote row blocks in the order the tiles need them; work item = (row block, column slice)
        const int remote_blocks = p.num_m_tiles - m_tiles_per_rank;
        const int items = remote_blocks * TP_SUB;
        const int vec_per_row = (p.K / TP_SUB) >> 3;   // 16-byte vectors per row slice
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
          const int jb = item / TP_SUB, sub = item - jb * TP_SUB;
          const int mt = (jb + (p.rank + 1) * m_tiles_per_rank) % p.num_m_tiles;
          const int owner = mt / m_tiles_per_rank;
          const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(peers.src[owner]) +
                                     static_cast<size_t>(mt - owner * m_tiles_per_rank) * TP_BM * p.K + sub * (p.K / TP_SUB);
          __nv_bfloat16* dst = p.a_full + static_cast<size_t>(mt) * TP_BM * p.K + sub * (p.K / TP_SUB);
          // eight independent 16-byte peer loads per thread are in flight before the first store: a remote load
          // takes microseconds, and one-at-a-time copies would leave the link idle
          const int nvec = TP_BM * vec_per_row;
          for (int v0 = ct; v0 < nvec; v0 += 128 * 8) {
            uint4 val[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int v = v0 + u * 128;
              if (v < nvec) {
                const int rr = v / vec_per_row, cc = v - rr * vec_per_row;
                val[u] = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(rr) * p.K + cc * 8);
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int v = v0 + u * 128;
              if (v < nvec) {
                const int rr = v / vec_per_row, cc = v - rr * vec_per_row;
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rr) * p.K + cc * 8) = val[u];
              }
            }
          }
          __threadfence();
          asm volatile("bar.sync 2, 128;" ::: "memory");
          if (ct == 0) atom_add_release_gpu(p.flags + 2 + mt, 1u);
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
  // ------------------------------ exit barrier: the last CTA to finish talks to the peers ------------------------------
  if (warp == 6) {
    unsigned int last = 0;
    if (lane == 0) {
      __threadfence_system();
      last = (atomicAdd(p.flags + 1, 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      bool ok = true;
      if (lane < p.world) {
        __threadfence_system();
        st_release_sys(peers.pad[lane] + p.slot0 + TP_MAX_WORLD + p.rank, p.epoch);
        ok = flag_wait_geq_sys(peers.pad[p.rank] + p.slot0 + TP_MAX_WORLD + lane, p.epoch, p.wait_cycles, 1040);
      }
      if (!ok && p.status) atomicExch(p.status, 1u);
      __syncwarp();
      if (lane == 0) p.flags[1] = 0u;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Paired-CTA variant (cta_group::2): a cluster of two CTAs owns a 256 x 256 tile, each CTA its own 128 rows of A and
// half of B; the leader issues the MMAs for both (same mainloop as the plain paired-CTA GEMM).  The cross-rank
// protocol is unchanged: copier warps of every CTA stage remote row blocks, the producer of a CTA waits for the
// staging counter of the 128-row block it loads, epilogues add into the owner's buffer, CTA 0 runs the entry barrier
// and the last CTA the exit barrier.  Requires rows_per_rank % 256 == 0.
// ---------------------------------------------------------------------------------------------------------------
constexpr int TP2_STAGES = 6;
constexpr int TP2_STAGE_BYTES = 32768;
constexpr int TP2_STG_BYTES = 128 * 64 * 2;        // one 128 x 64 bf16 epilogue tile (128-byte swizzled rows)
constexpr int TP2_SMEM = TP2_STAGES * TP2_STAGE_BYTES + 2 * TP2_STG_BYTES + 256 + 1024;

__global__ void __launch_bounds__(TP_THREADS, 1)
tp_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, TpParams p,
                    TpPeers peers, const __grid_constant__ TpMaps maps) {
  constexpr int STAGES = TP2_STAGES;
  constexpr int BN = 256;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * 16384;
  uint8_t* stg = smem + STAGES * TP2_STAGE_BYTES;      // two epilogue staging tiles (1024-byte aligned)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * TP2_STAGE_BYTES + 2 * TP2_STG_BYTES);
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
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 8);
    mbar_init(&tempty_bar[1], 8);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TMEM_COLS);
    tmem_relinquish_2cta();
    tc_fence_before_sync();
  }
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = p.M / 256;                       // 256-row super-blocks
  const int n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int tiles_per_group = TP_GROUP_M * n_tiles;
  const int sb_per_rank = p.rows_per_rank / 256;
  const int m_blocks_per_rank = p.rows_per_rank / TP_BM;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  bool alive = true;

  // logical super-block j -> physical: GATHER walks the own rows first, then the next ranks' rows in ring order
  auto tile_coords = [&](int t, int& mt, int& n0) {
    const int g = t / tiles_per_group;
    const int first_m = g * TP_GROUP_M;
    const int gsz = min(m_tiles - first_m, TP_GROUP_M);
    const int r = t - g * tiles_per_group;
    int sb = first_m + (r % gsz);
    int nt = r / gsz;
    if (p.mode == 3) {
      nt = (nt + p.rank * (n_tiles / p.world)) % n_tiles;       // GATHER_B: this rank's own weight rows first
    } else {
      sb = (sb + (p.mode == 1 ? p.rank : p.rank + 1) * sb_per_rank) % m_tiles;   // REDUCE: remote rows first, own last
    }
    mt = sb * 2 + (int)crank;                          // this CTA's 128-row block
    n0 = nt * BN;
  };

  if (warp == 0) {
    if (elect_one_sync()) {
      uint32_t it = 0;
      int last_ready = -1;
      for (int t = cluster_id; t < num_tiles && alive; t += num_clusters) {
        int mt, n0;
        tile_coords(t, mt, n0);
        if (p.mode == 1 && mt / m_blocks_per_rank != p.rank && mt != last_ready) {
          if (!flag_wait_geq_gpu(p.flags + 2 + mt, p.epoch * TP_SUB, p.wait_cycles, 1100)) {
            alive = false;
            if (p.status) atomicExch(p.status, 1u);
            break;
          }
          fence_proxy_async_global();
          last_ready = mt;
        }
        const int nb0 = n0 + (int)crank * 128;
        if (p.mode == 3) {
          // the 128 weight rows this CTA loads come from a peer: wait until the copiers have staged the block
          const int nblk = nb0 / TP_BM, n_blocks_per_rank = p.N / (TP_BM * p.world);
          if (nblk / n_blocks_per_rank != p.rank && nblk != last_ready) {
            if (!flag_wait_geq_gpu(p.flags + 2 + nblk, p.epoch * TP_SUB, p.wait_cycles, 1102)) {
              alive = false;
              if (p.status) atomicExch(p.status, 1u);
              break;
            }
            fence_proxy_async_global();
            last_ready = nblk;
          }
        }
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, alive, 1101)) break;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * TP2_STAGE_BYTES);
          tma_load_2d_2cta(smem_a + s * 16384, &tmA, &full_bar[s], kb * TP_BK, mt * TP_BM);
          uint8_t* b_dst = smem_b + s * 16384;
          if (!p.b_mn) {
            tma_load_2d_2cta(b_dst, &tmB, &full_bar[s], kb * TP_BK, nb0);
          } else {
            tma_load_2d_2cta(b_dst, &tmB, &full_bar[s], nb0, kb * TP_BK);
            tma_load_2d_2cta(b_dst + 8192, &tmB, &full_bar[s], nb0 + 64, kb * TP_BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one_sync()) {
      const uint32_t idesc = make_idesc(256, BN, 1, 1, 0u, (uint32_t)p.b_mn);
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      uint32_t it = 0, tile_it = 0;
      for (int t = cluster_id; t < num_tiles && alive; t += num_clusters, ++tile_it) {
        const uint32_t acc = tile_it & 1u;
        if (!mbar_wait(&tempty_bar[acc], ((tile_it >> 1) & 1u) ^ 1u, alive, 1110)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1u, alive, 1111)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * 16384), b_addr = smem_u32(smem_b + s * 16384);
#pragma unroll
          for (int k = 0; k < TP_BK / 16; ++k)
            umma_f16_ss_2cta(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 16, 1024),
                             make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_2cta_mc(&empty_bar[s], 3);
        }
        if (!alive) break;
        umma_commit_2cta_mc(&tfull_bar[acc], 3);
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    uint32_t tile_it = 0;
    bool entry_ok = (p.mode != 2);
    uint32_t stg_it = 0;
    for (int t = cluster_id; t < num_tiles && alive; t += num_clusters, ++tile_it) {
      int mt, n0;
      tile_coords(t, mt, n0);
      const uint32_t acc = tile_it & 1u;
      if (!mbar_wait(&tfull_bar[acc], (tile_it >> 1) & 1u, alive, 1120)) break;
      tc_fence_after_sync();
      if (!entry_ok) {
        if (!flag_wait_geq_gpu(p.flags, p.epoch, p.wait_cycles, 1121)) {
          alive = false;
          if (p.status) atomicExch(p.status, 1u);
          break;
        }
        entry_ok = true;
      }
      const int row = mt * TP_BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (p.mode == 2 && p.tma_red) {
        // 64-column slices of the tile go through a swizzled shared-memory staging tile and are added into the owner's
        // bf16 buffer by the copy engine: full-width packets on NVLink instead of 16-byte reductions per thread
        const int et = threadIdx.x - 64;                    // 0..127 among the epilogue threads
        const int owner = (mt * TP_BM) / p.rows_per_rank;
        const int y0 = mt * TP_BM - owner * p.rows_per_rank;
        const uint32_t rr = static_cast<uint32_t>(q * 32 + lane);
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 64; ++c2) {
          uint8_t* buf = stg + (stg_it & 1u) * TP2_STG_BYTES;
          if (et == 0) tma_store_wait_read<1>();            // the reduction that last read this buffer has drained it
          asm volatile("bar.sync 1, 128;" ::: "memory");
          uint32_t r[64];
          tmem_ld_32x32b_x32(t_row + c2 * 64, r);
          tmem_ld_32x32b_x32(t_row + c2 * 64 + 32, r + 32);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(buf + sw128_offset(rr, static_cast<uint32_t>(j))) = v;
          }
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0 && n0 + c2 * 64 < p.N) {
            tma_reduce_add_2d(&maps.m[owner], buf, n0 + c2 * 64, y0);
            tma_store_commit();
          }
          ++stg_it;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(&tempty_bar[acc], 0);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (row >= p.M || col0 >= p.N) continue;
        if (p.mode == 2) {
          tp_reduce_chunk(p, peers, r, row, col0);
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
          if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(dst + 8 * j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&tempty_bar[acc], 0);
    }
    if (p.mode == 2 && p.tma_red && threadIdx.x == 64) tma_store_wait<0>();   // every bulk reduction of this CTA is done
    __threadfence_system();
  } else {
    // ------------------------------ copiers (warps 6..9): identical protocol to the single-CTA kernel ------------------------------
    const int ct = threadIdx.x - 192;
    if (blockIdx.x == 0) {
      if (ct < p.world) {
        __threadfence_system();
        st_release_sys(peers.pad[ct] + p.slot0 + p.rank, p.epoch);
        if (!flag_wait_geq_sys(peers.pad[p.rank] + p.slot0 + ct, p.epoch, p.wait_cycles, 1130) && p.status)
          atomicExch(p.status, 1u);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ct == 0) {
        const unsigned int bad = p.status ? atomicAdd(p.status, 0u) : 0u;
        if (!bad) st_release_gpu(p.flags, p.epoch);
      }
    }
    if (p.mode == 1 || p.mode == 3) {
      if (!flag_wait_geq_gpu(p.flags, p.epoch, p.wait_cycles, 1131)) {
        if (ct == 0 && p.status) atomicExch(p.status, 1u);
      } else {
        // GATHER stages rows of A ([M][K]), GATHER_B rows of the weight ([N][K]); same walk, other extents
        const int total_blocks = (p.mode == 1 ? p.M : p.N) / TP_BM;
        const int m_blocks_per_rank = total_blocks / p.world;
        const int remote_blocks = total_blocks - m_blocks_per_rank;
        const int items = remote_blocks * TP_SUB;
        const int vec_per_row = (p.K / TP_SUB) >> 3;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
          const int jb = item / TP_SUB, sub = item - jb * TP_SUB;
          const int mt = (jb + (p.rank + 1) * m_blocks_per_rank) % total_blocks;
          const int owner = mt / m_blocks_per_rank;
          const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(peers.src[owner]) +
                                     static_cast<size_t>(mt - owner * m_blocks_per_rank) * TP_BM * p.K + sub * (p.K / TP_SUB);
          __nv_bfloat16* dst = p.a_full + static_cast<size_t>(mt) * TP_BM * p.K + sub * (p.K / TP_SUB);
          // eight independent 16-byte peer loads per thread are in flight before the first store: a remote load
          // takes microseconds, and one-at-a-time copies would leave the link idle
          const int nvec = TP_BM * vec_per_row;
          for (int v0 = ct; v0 < nvec; v0 += 128 * 8) {
            uint4 val[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int v = v0 + u * 128;
              if (v < nvec) {
                const int rr = v / vec_per_row, cc = v - rr * vec_per_row;
                val[u] = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(rr) * p.K + cc * 8);
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int v = v0 + u * 128;
              if (v < nvec) {
                const int rr = v / vec_per_row, cc = v - rr * vec_per_row;
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rr) * p.K + cc * 8) = val[u];
              }
            }
          }
          __threadfence();
          asm volatile("bar.sync 2, 128;" ::: "memory");
          if (ct == 0) atom_add_release_gpu(p.flags + 2 + mt, 1u);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
  if (warp == 6) {
    unsigned int last = 0;
    if (lane == 0) {
      __threadfence_system();
      last = (atomicAdd(p.flags + 1, 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      bool ok = true;
      if (lane < p.world) {
        __threadfence_system();
        st_release_sys(peers.pad[lane] + p.slot0 + TP_MAX_WORLD + p.rank, p.epoch);
        ok = flag_wait_geq_sys(peers.pad[p.rank] + p.slot0 + TP_MAX_WORLD + lane, p.epoch, p.wait_cycles, 1140);
      }
      if (!ok && p.status) atomicExch(p.status, 1u);
      __syncwarp();
      if (lane == 0) p.flags[1] = 0u;
    }
  }
}

static int launch_tp_2cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const TpParams& p, const TpPeers& peers,
                          const TpMaps& maps, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tp_gemm_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TP2_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = (p.M / 256) * ((p.N + 255) / 256);
  int clusters = sm_count() / 2;
  if (tiles < clusters) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * 2);      // all CTAs resident at once: at most one per SM
  cfg.blockDim = dim3(TP_THREADS);
  cfg.dynamicSmemBytes = TP2_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, tp_gemm_2cta_kernel, tmA, tmB, p, peers, maps);
}

// out[i] = own[i] + acc[i]; acc[i] = 0  (bf16: the rank's own partial sums plus what the peers reduced into the shared
// buffer, which is re-armed for the next call)
__global__ void add_and_clear_kernel(const __nv_bfloat16* __restrict__ own, __nv_bfloat16* __restrict__ acc,
                                     __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    const uint4 a = *reinterpret_cast<const uint4*>(own + i);
    const uint4 b = *reinterpret_cast<const uint4*>(acc + i);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    uint4 o;
    o.x = pack_bf16x2(a0.x + b0.x, a0.y + b0.y);
    o.y = pack_bf16x2(a1.x + b1.x, a1.y + b1.y);
    o.z = pack_bf16x2(a2.x + b2.x, a2.y + b2.y);
    o.w = pack_bf16x2(a3.x + b3.x, a3.y + b3.y);
    *reinterpret_cast<uint4*>(out + i) = o;
    *reinterpret_cast<uint4*>(acc + i) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// dst[i] = bf16(src[i]); src[i] = 0  (turns a finished fp32 reduction buffer into the layer output and re-arms it)
__global__ void cast_and_clear_kernel(float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(src + i);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + i) = o;
    *reinterpret_cast<float4*>(src + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <int BN>
static int launch_tp(const CUtensorMap& tmA, const CUtensorMap& tmB, const TpParams& p, const TpPeers& peers,
                     cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tp_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, TpSmem<BN>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  // every CTA must be resident at once (CTA 0 publishes the entry barrier, the last CTA runs the exit barrier,
  // copiers feed other CTAs' tiles): never launch more CTAs than SMs
  const int grid = tiles < sm_count() ? tiles : sm_count();
  tp_gemm_kernel<BN><<<grid, TP_THREADS, TpSmem<BN>::TOTAL, st>>>(tmA, tmB, p, peers);
  return (int)cudaGetLastError();
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_tp_gemm)

using namespace ts;

// mode 1 (all-gather -> GEMM):  C[M,N] = gather_rows(A_shards)[M,K] . B^T.  `a_full` is a local [M][K] bf16 buffer
//   whose own block (rows rank*rows_per_rank ...) already holds this rank's shard; src_ptrs[r] = rank r's shard.
// mode 2 (GEMM -> reduce-scatter): dst_ptrs[owner][row - owner*rows_per_rank][:] += A[M,K] . B^T rows, fp32.
// mode 5: as mode 3 (shared bf16 accumulation buffers), but every 128 x 64 slice of an output tile is staged in shared
//   memory and added by one bulk tensor reduction (`cp.reduce.async.bulk.tensor ... add`) into the owner's buffer;
//   needs the paired-CTA kernel (rows_per_rank % 256 == 0, N >= 256, N % 8 == 0), else returns -13.
// mode 4: no atomics.  dst_ptrs[owner] is a [W][rows_per_rank][N] bf16 staging buffer; this rank stores its partial sums
//   of the owner's rows into slot `rank` with plain 16-byte stores and its own rows into C ([rows_per_rank][N]); the
//   caller then adds the W - 1 foreign slots to C (ts_sum_slots).
// mode 3: as mode 2 with bf16 accumulation buffers (8 elements per 16-byte red; the sum of W partials is rounded to
//   bf16 after every addition, like a bf16 ring reduce-scatter).
// B: b_mn == 0 -> [N][ldb] K-major, b_mn == 1 -> [K][ldb] N-major.  flags: device u32[2 + M/128], zero-initialised once
// and reused across calls with a growing `epoch`.  pad_ptrs / slot0: signal pads (2*16 slots from slot0 are used).
extern "C" int ts_tp_gemm(int mode, const void* A, const void* B, void* C, void* a_full, int M, int N, int K, int lda,
                          int ldb, int ldc, int b_mn, const unsigned long long* src_ptrs,
                          const unsigned long long* dst_ptrs, const unsigned long long* pad_ptrs, int rank, int world,
                          unsigned int* flags, unsigned int epoch, unsigned int slot0, long long wait_cycles,
                          unsigned int* status, void* stream) {
  if (world > TP_MAX_WORLD || M % (TP_BM * world) != 0 || K % (8 * TP_SUB) != 0) return -10;
  const int acc_bf16 = (mode == 3);     // mode 3: GEMM -> reduce-scatter with packed-bf16 accumulation buffers
  const int push = (mode == 4);         // mode 4: GEMM -> reduce-scatter by plain stores into per-source staging slots
  const int tma_red = (mode == 5);      // mode 5: as mode 3, tiles added by bulk tensor reductions (paired-CTA kernel only)
  if (mode == 3 || mode == 4 || mode == 5) mode = 2;
  if (mode != 1 && mode != 2) return -11;
  // paired-CTA kernel: every rank's rows split into 256-row super-blocks and enough 256 x 256 tiles for every CTA pair
  const bool two_cta = (M / world) % 256 == 0 && N >= 256 && (M / 256) * ((N + 255) / 256) >= sm_count() / 2 &&
                       getenv("TS_TP_GEMM_1CTA") == nullptr;
  const int bn = two_cta ? 128 : ((N >= 256) ? 256 : 128);     // B box rows (the paired kernel loads half tiles)
  const void* a_base = (mode == 1) ? a_full : A;
  const int a_ld = (mode == 1) ? K : lda;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, a_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)a_ld, TP_BM, 64);
  if (rc) return rc * 100 - 1;
  if (!b_mn)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)bn, 64);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
  if (rc) return rc * 100 - 2;
  TpParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.b_mn = b_mn; p.mode = mode; p.rank = rank; p.world = world;
  p.acc_bf16 = acc_bf16;
  p.push = push;
  p.tma_red = tma_red;
  p.acc_bf16 = acc_bf16 || tma_red;
  p.rows_per_rank = M / world; p.C = C; p.a_full = (__nv_bfloat16*)a_full;
  p.num_m_tiles = M / TP_BM; p.num_n_tiles = (N + bn - 1) / bn; p.k_blocks = (K + TP_BK - 1) / TP_BK;
  p.flags = flags; p.epoch = epoch; p.slot0 = slot0; p.wait_cycles = wait_cycles; p.status = status;
  TpPeers peers{};
  for (int r = 0; r < world; ++r) {
    peers.src[r] = src_ptrs ? reinterpret_cast<const void*>(src_ptrs[r]) : nullptr;
    peers.dst[r] = dst_ptrs ? reinterpret_cast<void*>(dst_ptrs[r]) : nullptr;
    peers.pad[r] = reinterpret_cast<unsigned int*>(pad_ptrs[r]);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tma_red && (!two_cta || N % 8 != 0)) return -13;   // the caller falls back to mode 3 for such shapes
  if (two_cta) {
    TpMaps maps{};
    if (tma_red) {
      for (int r = 0; r < world; ++r) {
        rc = make_tmap_2d(&maps.m[r], peers.dst[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)(M / world),
                          (uint64_t)N, (uint64_t)N, 128, 64);
        if (rc) return rc * 100 - 3;
      }
    }
    return launch_tp_2cta(tmA, tmB, p, peers, maps, st);
  }
  return bn == 256 ? launch_tp<256>(tmA, tmB, p, peers, st) : launch_tp<128>(tmA, tmB, p, peers, st);
}

extern "C" int ts_cast_and_clear(float* src, void* dst, long long n, void* stream) {
  if (n <= 0 || n % 4 != 0) return n == 0 ? 0 : -10;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > (long long)sm_count() * 8) blocks = (long long)sm_count() * 8;
  cast_and_clear_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(src, (__nv_bfloat16*)dst, n);
  return (int)cudaGetLastError();
}

// out = own + acc (bf16), acc = 0.  In place when out == own.
extern "C" int ts_add_and_clear(const void* own, void* acc, void* out, long long n, void* stream) {
  if (n <= 0 || n % 8 != 0) return n == 0 ? 0 : -10;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > (long long)sm_count() * 8) blocks = (long long)sm_count() * 8;
  add_and_clear_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)own, (__nv_bfloat16*)acc, (__nv_bfloat16*)out, n);
  return (int)cudaGetLastError();
}

// out[i] = own[i] + sum over s != rank of staging[s][i]  (bf16, fp32 accumulation).  In place when out == own.
__global__ void sum_slots_kernel(const __nv_bfloat16* __restrict__ own, const __nv_bfloat16* __restrict__ staging,
                                 __nv_bfloat16* __restrict__ out, long long n, int world, int rank) {
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    float acc[8];
    {
      const uint4 a = *reinterpret_cast<const uint4*>(own + i);
      const float2 a0 = ts::unpack_bf16x2(a.x), a1 = ts::unpack_bf16x2(a.y), a2 = ts::unpack_bf16x2(a.z),
                   a3 = ts::unpack_bf16x2(a.w);
      acc[0] = a0.x; acc[1] = a0.y; acc[2] = a1.x; acc[3] = a1.y; acc[4] = a2.x; acc[5] = a2.y; acc[6] = a3.x; acc[7] = a3.y;
    }
    for (int s = 0; s < world; ++s) {
      if (s == rank) continue;
      const uint4 b = *reinterpret_cast<const uint4*>(staging + static_cast<size_t>(s) * n + i);
      const float2 b0 = ts::unpack_bf16x2(b.x), b1 = ts::unpack_bf16x2(b.y), b2 = ts::unpack_bf16x2(b.z),
                   b3 = ts::unpack_bf16x2(b.w);
      acc[0] += b0.x; acc[1] += b0.y; acc[2] += b1.x; acc[3] += b1.y; acc[4] += b2.x; acc[5] += b2.y; acc[6] += b3.x; acc[7] += b3.y;
    }
    uint4 o;
    o.x = ts::pack_bf16x2(acc[0], acc[1]);
    o.y = ts::pack_bf16x2(acc[2], acc[3]);
    o.z = ts::pack_bf16x2(acc[4], acc[5]);
    o.w = ts::pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i) = o;
  }
}

extern "C" int ts_sum_slots(const void* own, const void* staging, void* out, long long n, int world, int rank,
                            void* stream) {
  if (n <= 0 || n % 8 != 0) return n == 0 ? 0 : -10;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > (long long)sm_count() * 8) blocks = (long long)sm_count() * 8;
  sum_slots_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)own, (const __nv_bfloat16*)staging, (__nv_bfloat16*)out, n, world, rank);
  return (int)cudaGetLastError();
}

// Weight-gather GEMM (the ZeRO-3 / FSDP forward in one kernel): C[M][N] = A[M][K] . gather_rows(W_shards)[N][K]^T.
// Every rank owns N / world consecutive rows of the weight; `w_full` is a local [N][K] bf16 buffer whose own block
// already holds this rank's shard, src_ptrs[r] = rank r's shard.  Copier warps of the persistent paired-CTA GEMM pull
// the remote row blocks in the order the tiles need them (the own N tiles are computed first) and the TMA producer of
// a CTA waits on the counter of the 128-row block it loads.  Requires (N / world) % 256 == 0, M % 256 == 0.
// flags: device u32[2 + N/128].
extern "C" int ts_weight_gather_gemm(const void* A, void* C, void* w_full, int M, int N, int K, int lda, int ldc,
                                     const unsigned long long* src_ptrs, const unsigned long long* pad_ptrs, int rank,
                                     int world, unsigned int* flags, unsigned int epoch, unsigned int slot0,
                                     long long wait_cycles, unsigned int* status, void* stream) {
  if (world > TP_MAX_WORLD || world <= 0 || N % (256 * world) != 0 || M % 256 != 0 || K % (8 * TP_SUB) != 0) return -10;
  if ((M / 256) * (N / 256) < sm_count() / 2) return -13;       // too small for the paired-CTA kernel
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TP_BM, 64);
  if (rc) return rc * 100 - 1;
  rc = make_tmap_2d(&tmB, w_full, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128, 64);
  if (rc) return rc * 100 - 2;
  TpParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.b_mn = 0; p.mode = 3; p.rank = rank; p.world = world;
  p.rows_per_rank = M;        // A is not sharded
  p.C = C; p.a_full = (__nv_bfloat16*)w_full;                  // staging target of the copiers
  p.num_m_tiles = M / TP_BM; p.num_n_tiles = N / 128; p.k_blocks = (K + TP_BK - 1) / TP_BK;
  p.flags = flags; p.epoch = epoch; p.slot0 = slot0; p.wait_cycles = wait_cycles; p.status = status;
  TpPeers peers{};
  for (int r = 0; r < world; ++r) {
    peers.src[r] = reinterpret_cast<const void*>(src_ptrs[r]);
    peers.pad[r] = reinterpret_cast<unsigned int*>(pad_ptrs[r]);
  }
  TpMaps maps{};
  return launch_tp_2cta(tmA, tmB, p, peers, maps, reinterpret_cast<cudaStream_t>(stream));
}
