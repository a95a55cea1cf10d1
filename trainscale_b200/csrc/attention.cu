// Flash attention for sm_100a on tcgen05 / TMEM / TMA: causal or full, GQA, packed documents (cu_seqlens).
//
// Forward, per CTA (one 256-row query block of one head = two 128-row tiles that ping-pong):
//   warp 0        TMA loader: Q tiles once, then a 2-deep ring of 128-row K and V tiles (128-byte swizzle)
//   warp 1        MMA issuer (one thread): S_t = Q_t K^T into TMEM, later O_t += P_t V with P_t read from TMEM
//   warps 2..5    softmax for tile 0, warps 6..9 for tile 1: one thread per query row (its own TMEM lane), so row
//                 max / sum need no shuffles; P is written back over S as packed bf16, O is rescaled in TMEM
//                 only when the running max moved by more than 2^8 (exact: O and the row sum share the stale max)
// While one tile's rows are in softmax the tensor core works on the other tile.
// Backward is two kernels that recompute S and dP: one owns a K/V tile and accumulates dK, dV over the query
// tiles of its head group; one owns a Q tile and accumulates dQ over the K/V tiles.  No atomics, deterministic.
//
// Replaces data_pipeline/trainer/kernels/flash_attention.py:147-560 (Triton forward, dq and dk/dv kernels).
#include <type_traits>
#include "common.cuh"
#include "host_common.h"

namespace ts {

struct AttnParams {
  // strides are in elements; q/k/v/o/do/dq/dk/dv rows are tokens, heads are laid out along the row
  int q_col0, k_col0, v_col0;   // column of head 0 inside the q / k / v tensor maps
  int Hq, Hkv, group;           // group = Hq / Hkv
  int B, S;                     // uniform batch (ignored when cu_seqlens != nullptr)
  const int* cu_seqlens;        // [B + 1] or nullptr
  int causal;
  float scale_log2;             // softmax scale * log2(e)
  __nv_bfloat16* o;             // [rows][o_stride], head h at column h*D
  int o_stride;
  float* lse;                   // [Hq][total_rows]
  long long total_rows;
  // backward
  const __nv_bfloat16* dout;    // [rows][o_stride]
  const float* delta;           // [Hq][total_rows] rowsum(dO * O)
  __nv_bfloat16* dq;            // written at column q_col0 + h*D of rows with stride dqkv_stride
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int dqkv_stride;
  float scale;                  // softmax scale (natural units)
  int window;                   // > 0: key j is visible to query i only if j > i - window (sliding window)
  float cap_inv, cap_log2;      // logit soft-cap c: s' = c * tanh(s * scale / c); cap_inv = scale / c, cap_log2 = c * log2(e)
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void seq_bounds(const AttnParams& p, int b, int& start, int& len) {
  if (p.cu_seqlens) {
    start = p.cu_seqlens[b];
    len = p.cu_seqlens[b + 1] - start;
  } else {
    start = b * p.S;
    len = p.S;
  }
}

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
template <int D>
struct FwdSmem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int KV_STAGES = 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = 2 * TILE;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

constexpr int FWD_THREADS = 320;

template <int D, bool EXT>   // EXT: sliding window / logit soft-cap code paths compiled in
__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, AttnParams p) {
  using SM = FwdSmem<D>;
  constexpr int DCH = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL0 = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars;          // [2]
  uint64_t* k_full = bars + 2;      // [2]
  uint64_t* k_empty = bars + 4;     // [2]
  uint64_t* v_full = bars + 6;      // [2]
  uint64_t* v_empty = bars + 8;     // [2]
  uint64_t* s_full = bars + 10;     // [2]
  uint64_t* p_full = bars + 12;     // [2]
  uint64_t* o_full = bars + 14;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid: x = head + heads * batch (fastest), y = tile: the whole grid is dispatched longest-tile-first
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int hk = h / p.group;
  int q_start, Lq, k_start, Lk;
  seq_bounds(p, b, q_start, Lq);
  k_start = q_start;
  Lk = Lq;
  const int n_qblocks = (Lq + 255) / 256;
  if ((int)blockIdx.y >= n_qblocks) return;
  const int qb = n_qblocks - 1 - blockIdx.y;   // heaviest (latest) causal blocks first
  const int off = Lk - Lq;
  int r0[2], nkv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    r0[t] = qb * 256 + t * 128;
    if (r0[t] >= Lq) {
      nkv[t] = 0;
    } else {
      const int kv_end = p.causal ? min(Lk, r0[t] + 128 + off) : Lk;
      nkv[t] = (kv_end + 127) / 128;
    }
  }
  // sliding window: key blocks entirely left of the first row's window are never loaded
  const int kb_lo = (EXT && p.window > 0) ? max(0, qb * 256 + off - p.window + 1) / 128 : 0;
#pragma unroll
  for (int t = 0; t < 2; ++t) nkv[t] = max(0, nkv[t] - kb_lo);
  const int n = max(nkv[0], nkv[1]);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    for (int i = 0; i < 16; ++i) mbar_init(&bars[i], (i == 12 || i == 13) ? 4 : 1);
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
  bool alive = true;

  if (warp == 0) {
    if (elect_one_sync()) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (nkv[t] == 0) continue;
        mbar_expect_tx(&q_full[t], SM::TILE);
#pragma unroll
        for (int j = 0; j < DCH; ++j)
          tma_load_2d(smem + SM::Q_OFF + t * SM::TILE + j * 16384, &tmQ, &q_full[t], p.q_col0 + h * D + j * 64,
                      q_start + r0[t]);
      }
      for (int i = 0; i < n && alive; ++i) {
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1u;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, alive, 400)) break;
        mbar_expect_tx(&k_full[s], SM::TILE);
#pragma unroll
        for (int j = 0; j < DCH; ++j)
          tma_load_2d(smem + SM::K_OFF + s * SM::TILE + j * 16384, &tmK, &k_full[s], p.k_col0 + hk * D + j * 64,
                      k_start + (kb_lo + i) * 128);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, alive, 401)) break;
        mbar_expect_tx(&v_full[s], SM::TILE);
#pragma unroll
        for (int j = 0; j < DCH; ++j)
          tma_load_2d(smem + SM::V_OFF + s * SM::TILE + j * 16384, &tmV, &v_full[s], p.v_col0 + hk * D + j * 64,
                      k_start + (kb_lo + i) * 128);
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      const uint32_t idesc_s = make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t idesc_o = make_idesc(128, D, 1, 1, 0, 1);
      auto issue_s = [&](int t, int stage) {
        const uint32_t qa = smem_u32(smem + SM::Q_OFF + t * SM::TILE);
        const uint32_t ka = smem_u32(smem + SM::K_OFF + stage * SM::TILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t o = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16_ss(tmem_base + t * 128, make_smem_desc_sw128(qa + o, 16, 1024),
                      make_smem_desc_sw128(ka + o, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(&s_full[t]);
      };
      for (int t = 0; t < 2; ++t)
        if (nkv[t] > 0) mbar_wait(&q_full[t], 0, alive, 500);
      if (n > 0 && mbar_wait(&k_full[0], 0, alive, 501)) {
        tc_fence_after_sync();
        for (int t = 0; t < 2; ++t)
          if (nkv[t] > 0) issue_s(t, 0);
        umma_commit(&k_empty[0]);
      }
      for (int i = 0; i < n && alive; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&v_full[s], (i >> 1) & 1u, alive, 502)) break;
        bool k_waited = false;
        for (int t = 0; t < 2 && alive; ++t) {
          if (i < nkv[t]) {
            if (!mbar_wait(&p_full[t], i & 1u, alive, 503)) break;
            tc_fence_after_sync();
            const uint32_t va = smem_u32(smem + SM::V_OFF + s * SM::TILE);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_f16_ts(tmem_base + O_COL0 + t * D, tmem_base + t * 128 + kk * 8,
                          make_smem_desc_sw128(va + kk * 2048, 16384, 1024), idesc_o, (i | kk) != 0);
            if (i == nkv[t] - 1) umma_commit(&o_full[t]);
          }
          if (i + 1 < nkv[t]) {
            if (!k_waited) {
              if (!mbar_wait(&k_full[(i + 1) & 1], ((i + 1) >> 1) & 1u, alive, 504)) break;
              tc_fence_after_sync();
              k_waited = true;
            }
            issue_s(t, (i + 1) & 1);
          }
        }
        if (!alive) break;
        if (i + 1 < n) umma_commit(&k_empty[(i + 1) & 1]);
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int t = (warp - 2) >> 2;
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const int row = r0[t] + r;                  // row inside the sequence
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16);
    const uint32_t t_s = t_lane + t * 128;
    const uint32_t t_o = t_lane + O_COL0 + t * D;
    float m_used = -INFINITY, l = 0.f;
    const int nt = nkv[t];
    for (int i = 0; i < nt && alive; ++i) {
      if (!mbar_wait(&s_full[t], i & 1u, alive, 600)) break;
      tc_fence_after_sync();
      const int c0 = (kb_lo + i) * 128;
      const bool need_mask = (p.causal && (c0 + 127 > r0[t] + off)) || (c0 + 128 > Lk) ||
                             (EXT && p.window > 0 && c0 <= r0[t] + 127 + off - p.window);
      const int limit = p.causal ? min(Lk - 1, row + off) : Lk - 1;   // last visible column
      const int lo = (EXT && p.window > 0) ? row + off - p.window + 1 : 0;  // first visible column
      // the thread's whole row of S (128 columns) comes into registers once
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, v + c * 32);
      tc_wait_ld();
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      float sc = p.scale_log2;
      if (EXT && p.cap_log2 > 0.f) {   // soft-capped logits, already in log2 units
#pragma unroll
        for (int j = 0; j < 128; ++j) v[j] = __float_as_uint(p.cap_log2 * fast_tanh(__uint_as_float(v[j]) * p.cap_inv));
        sc = 1.f;
      }
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < 128; ++j)
          if (c0 + j > limit || c0 + j < lo) v[j] = 0xff800000u;   // -inf: drops out of the max, exp2 gives 0
      }
#pragma unroll
      for (int j = 0; j < 128; j += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(v[j]));
        mx1 = fmaxf(mx1, __uint_as_float(v[j + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(v[j + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(v[j + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m_used, mx * sc);
      const bool grow = (m_new - m_used > 8.0f);   // also true on the first block (m_used = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = (m_used == -INFINITY) ? 0.f : fast_ex2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
        if (i > 0) {
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x32b_x16(t_o + c * 16, o);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st_32x32b_x16(t_o + c * 16, o);
          }
        }
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      // P = exp2(S*scale - m), packed bf16 written over the first 64 columns of S
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = fast_ex2(fmaf(__uint_as_float(v[c * 32 + j]), sc, -m_sub));
          const float p1 = fast_ex2(fmaf(__uint_as_float(v[c * 32 + j + 1]), sc, -m_sub));
          l0 += p0;
          l1 += p1;
          pk[j >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32b_x16(t_s + c * 16, pk);
      }
      l += l0 + l1;
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (nt > 0 && alive && mbar_wait(&o_full[t], 0, alive, 601)) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool valid = row < Lq;
      __nv_bfloat16* dst = p.o + static_cast<size_t>(q_start + row) * p.o_stride + h * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_o + c * 32, v);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * j]) * inv, __uint_as_float(v[8 * j + 1]) * inv);
            o4.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]) * inv, __uint_as_float(v[8 * j + 3]) * inv);
            o4.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]) * inv, __uint_as_float(v[8 * j + 5]) * inv);
            o4.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]) * inv, __uint_as_float(v[8 * j + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = o4;
          }
        }
      }
      if (valid && p.lse)
        p.lse[static_cast<size_t>(h) * p.total_rows + q_start + row] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// delta[h][row] = sum_d dO[row][h*D + d] * O[row][h*D + d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, long long total_rows, int Hq, int D, int o_stride) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= total_rows * Hq) return;
  const long long row = gw / Hq;
  const int h = static_cast<int>(gw - row * Hq);
  const __nv_bfloat16* a = o + row * o_stride + h * D;
  const __nv_bfloat16* g = dout + row * o_stride + h * D;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 x = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + d));
    const float2 y = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(g + d));
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<size_t>(h) * total_rows + row] = s;
}


// ------------------------------------------------------------------------------------------------
// backward, kernel 1: dK / dV.  One CTA owns a 128-row K/V tile of one kv head and walks the 64-row query
// sub-tiles of every query head in its group.  TMEM: two (S^T | dP^T) buffers of 64+64 columns, dV and dK
// accumulators.  P^T and dS^T are written back over S^T / dP^T as packed bf16 and fed to the MMA from TMEM.
// ------------------------------------------------------------------------------------------------
template <int D>
struct BwdSmem {
  static constexpr int BIG = 128 * D * 2;     // resident 128-row tile
  static constexpr int SMALL = 64 * D * 2;    // streamed 64-row tile
  static constexpr int STAGES = 4;
  static constexpr int A_OFF = 0;             // resident tile 0 (K or Q)
  static constexpr int B_OFF = BIG;           // resident tile 1 (V or dO)
  static constexpr int S0_OFF = 2 * BIG;      // streamed tile 0 ring (Q or K)
  static constexpr int S1_OFF = S0_OFF + STAGES * SMALL;   // streamed tile 1 ring (dO or V)
  static constexpr int VEC_OFF = S1_OFF + STAGES * SMALL;  // per stage: 64 x (lse * log2e, delta) float pairs
  static constexpr int BAR_OFF = VEC_OFF + STAGES * 512;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

constexpr int BWD_THREADS = 320;   // warp 0 TMA, warp 1 MMA, warps 2..5 and 6..9: two compute warpgroups (32 columns each)

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <int D, bool EXT>   // EXT: sliding window / logit soft-cap code paths compiled in
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmK128,
                      const __grid_constant__ CUtensorMap tmV128, const __grid_constant__ CUtensorMap tmdO64,
                      AttnParams p) {
  using SM = BwdSmem<D>;
  constexpr int DCH = D / 64;
  constexpr int STAGES = SM::STAGES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t DV_COL = 256, DK_COL = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* vec = reinterpret_cast<float*>(smem + SM::VEC_OFF);   // [STAGES][64] (lse * log2e, delta) pairs
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* kv_full = bars;            // [1]
  uint64_t* s_full = bars + 1;         // [2]
  uint64_t* p_full = bars + 3;         // [2]
  uint64_t* acc_full = bars + 5;       // [1]
  uint64_t* qd_full = bars + 6;        // [STAGES]
  uint64_t* qd_empty = bars + 6 + SM::STAGES;   // [STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6 + 2 * SM::STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid: x = kv head + kv heads * batch (fastest), y = kv tile; low tiles see the most queries and go first
  const int j = blockIdx.y, hk = blockIdx.x % p.Hkv, b = blockIdx.x / p.Hkv;
  int q_start, Lq;
  seq_bounds(p, b, q_start, Lq);
  const int k_start = q_start, Lk = Lq;
  if (j * 128 >= Lk) return;
  const int off = Lk - Lq;
  const int n_u = (Lq + 63) / 64;
  const int u_start = p.causal ? max(0, (j * 128 - off) / 64) : 0;
  // sliding window: the last query row that sees any key of this tile is (j*128 + 127) - off + window - 1
  const int u_end = (EXT && p.window > 0) ? min(n_u, (j * 128 + 127 - off + p.window - 1) / 64 + 1) : n_u;
  const int per_head = u_end - u_start;
  const int total = per_head * p.group;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ64);
    tma_prefetch_desc(&tmK128);
    tma_prefetch_desc(&tmV128);
    tma_prefetch_desc(&tmdO64);
    for (int i = 0; i < 6 + 2 * SM::STAGES; ++i)
      mbar_init(&bars[i], (i == 3 || i == 4) ? 8 : ((i >= 6 && i < 6 + SM::STAGES) ? 2 : 1));
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
  bool alive = true;

  if (warp == 0) {
    // the whole warp runs the producer loop: lane 0 issues the tiled loads, every lane brings two columns'
    // (lse * log2e, delta) pairs of the sub-tile into the stage's vector buffer (fetched one stage ahead)
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * SM::BIG);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_2d(smem + SM::A_OFF + c * 16384, &tmK128, kv_full, p.k_col0 + hk * D + c * 64, k_start + j * 128);
        tma_load_2d(smem + SM::B_OFF + c * 16384, &tmV128, kv_full, p.v_col0 + hk * D + c * 64, k_start + j * 128);
      }
    }
    auto fetch_vec = [&](int it, int col) -> float2 {
      const int g = it / per_head, u = u_start + it % per_head;
      const int h = hk * p.group + g;
      const int qrow = u * 64 + col;
      if (it >= total || qrow >= Lq) return make_float2(0.f, 0.f);
      const size_t idx = static_cast<size_t>(h) * p.total_rows + q_start + qrow;
      return make_float2(p.lse[idx] * 1.4426950408889634f, p.delta[idx]);
    };
    float2 n0 = fetch_vec(0, lane), n1 = fetch_vec(0, lane + 32);
    for (int it = 0; it < total && alive; ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1u;
      const int g = it / per_head, u = u_start + it % per_head;
      const int h = hk * p.group + g;
      if (!mbar_wait(&qd_empty[s], ph ^ 1u, alive, 700)) break;
      if (lane == 0) {
        mbar_expect_tx(&qd_full[s], 2 * SM::SMALL);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_2d(smem + SM::S0_OFF + s * SM::SMALL + c * 8192, &tmQ64, &qd_full[s], p.q_col0 + h * D + c * 64,
                      q_start + u * 64);
          tma_load_2d(smem + SM::S1_OFF + s * SM::SMALL + c * 8192, &tmdO64, &qd_full[s], h * D + c * 64,
                      q_start + u * 64);
        }
      }
      float2* vb2 = reinterpret_cast<float2*>(vec + s * 128);
      vb2[lane] = n0;
      vb2[lane + 32] = n1;
      n0 = fetch_vec(it + 1, lane);
      n1 = fetch_vec(it + 1, lane + 32);
      __syncwarp();
      if (lane == 0) mbar_arrive(&qd_full[s]);   // second arrival of the phase: the vectors are in place
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      const uint32_t idesc_s = make_idesc(128, 64, 1, 1, 0, 0);
      const uint32_t idesc_acc = make_idesc(128, D, 1, 1, 0, 1);
      const uint32_t ka = smem_u32(smem + SM::A_OFF), va = smem_u32(smem + SM::B_OFF);
      auto issue12 = [&](int it) {
        const int s = it % STAGES;
        if (!mbar_wait(&qd_full[s], (it / STAGES) & 1u, alive, 710)) return;
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(smem + SM::S0_OFF + s * SM::SMALL);
        const uint32_t da = smem_u32(smem + SM::S1_OFF + s * SM::SMALL);
        const uint32_t st = tmem_base + (it & 1) * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t oa = (k >> 2) * 16384 + (k & 3) * 32, ob = (k >> 2) * 8192 + (k & 3) * 32;
          umma_f16_ss(st, make_smem_desc_sw128(ka + oa, 16, 1024), make_smem_desc_sw128(qa + ob, 16, 1024), idesc_s,
                      k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t oa = (k >> 2) * 16384 + (k & 3) * 32, ob = (k >> 2) * 8192 + (k & 3) * 32;
          umma_f16_ss(st + 64, make_smem_desc_sw128(va + oa, 16, 1024), make_smem_desc_sw128(da + ob, 16, 1024),
                      idesc_s, k != 0);
        }
        umma_commit(&s_full[it & 1]);
      };
      if (mbar_wait(kv_full, 0, alive, 711)) {
        issue12(0);
        if (total > 1 && alive) issue12(1);
        for (int it = 0; it < total && alive; ++it) {
          const int bsel = it & 1, s = it % STAGES;
          if (!mbar_wait(&p_full[bsel], (it >> 1) & 1u, alive, 712)) break;
          tc_fence_after_sync();
          const uint32_t qa = smem_u32(smem + SM::S0_OFF + s * SM::SMALL);
          const uint32_t da = smem_u32(smem + SM::S1_OFF + s * SM::SMALL);
          const uint32_t st = tmem_base + bsel * 128;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ts(tmem_base + DV_COL, st + (kk >> 1) * 32 + (kk & 1) * 8,
                        make_smem_desc_sw128(da + kk * 2048, 8192, 1024), idesc_acc, (it | kk) != 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ts(tmem_base + DK_COL, st + 64 + (kk >> 1) * 32 + (kk & 1) * 8,
                        make_smem_desc_sw128(qa + kk * 2048, 8192, 1024), idesc_acc, (it | kk) != 0);
          umma_commit(&qd_empty[s]);
          if (it + 2 < total) issue12(it + 2);
        }
        if (alive) umma_commit(acc_full);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int wg = (warp - 2) >> 2;          // compute warpgroup: owns query columns [wg*32, wg*32+32) of the sub-tile
    const int r = q4 * 32 + lane;            // kv row inside the tile
    const int kv_row = j * 128 + r;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16);
    for (int it = 0; it < total && alive; ++it) {
      const int u = u_start + it % per_head;
      // written by the producer warp before its arrival on qd_full, which the MMA thread observed before s_full
      const float* vb = vec + (it % STAGES) * 128;
      if (!mbar_wait(&s_full[it & 1], (it >> 1) & 1u, alive, 720)) break;
      tc_fence_after_sync();
      const uint32_t t_s = t_lane + (it & 1) * 128;
      const bool need_mask = (p.causal && (j * 128 + 127 > u * 64 + off)) || (u * 64 + 64 > Lq) ||
                             (j * 128 + 128 > Lk) || (EXT && p.window > 0 && j * 128 <= u * 64 + 63 + off - p.window);
      {
        const int cc = wg;
        uint32_t sv[32], dv[32], pp[16], ds[16];
        tmem_ld_32x32b_x32(t_s + cc * 32, sv);
        tmem_ld_32x32b_x32(t_s + 64 + cc * 32, dv);
        tc_wait_ld();
        // the masked and the unmasked tile bodies are separate straight-line code: a per-element branch would
        // serialise the 32 independent exp chains
        auto body = [&](auto masked, auto capped) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float4 ld4 = *reinterpret_cast<const float4*>(vb + 2 * (cc * 32 + e));   // warp-wide broadcast
            float p0, p1, g0 = 1.f, g1 = 1.f;   // g = d(capped logit) / d(scaled logit)
            if constexpr (decltype(capped)::value) {
              const float t0 = fast_tanh(__uint_as_float(sv[e]) * p.cap_inv);
              const float t1 = fast_tanh(__uint_as_float(sv[e + 1]) * p.cap_inv);
              p0 = fast_ex2(fmaf(t0, p.cap_log2, -ld4.x));
              p1 = fast_ex2(fmaf(t1, p.cap_log2, -ld4.z));
              g0 = 1.f - t0 * t0;
              g1 = 1.f - t1 * t1;
            } else {
              p0 = fast_ex2(fmaf(__uint_as_float(sv[e]), p.scale_log2, -ld4.x));
              p1 = fast_ex2(fmaf(__uint_as_float(sv[e + 1]), p.scale_log2, -ld4.z));
            }
            if constexpr (decltype(masked)::value) {
              const int qrow = u * 64 + cc * 32 + e;
              const bool rok = kv_row < Lk;
              p0 = (rok && qrow < Lq && (!p.causal || kv_row <= qrow + off)) ? p0 : 0.f;
              p1 = (rok && qrow + 1 < Lq && (!p.causal || kv_row <= qrow + 1 + off)) ? p1 : 0.f;
              if constexpr (EXT) {   // sliding window: visible iff kv_row > qrow + off - window
                if (p.window > 0) {
                  p0 = (kv_row > qrow + off - p.window) ? p0 : 0.f;
                  p1 = (kv_row > qrow + 1 + off - p.window) ? p1 : 0.f;
                }
              }
            }
            pp[e >> 1] = pack_bf16x2(p0, p1);
            if constexpr (decltype(capped)::value)
              ds[e >> 1] = pack_bf16x2(p0 * g0 * (__uint_as_float(dv[e]) - ld4.y),
                                       p1 * g1 * (__uint_as_float(dv[e + 1]) - ld4.w));
            else
              ds[e >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[e]) - ld4.y), p1 * (__uint_as_float(dv[e + 1]) - ld4.w));
          }
        };
        if (EXT && p.cap_log2 > 0.f) body(std::true_type{}, std::true_type{});   // soft-cap: one (masked) variant only
        else if (need_mask) body(std::true_type{}, std::false_type{});
        else body(std::false_type{}, std::false_type{});
        // each warpgroup overwrites only columns of its own (already consumed) chunk
        tmem_st_32x32b_x16(t_s + cc * 32, pp);
        tmem_st_32x32b_x16(t_s + 64 + cc * 32, ds);
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[it & 1]);
    }
    if (alive && mbar_wait(acc_full, 0, alive, 721)) {
      tc_fence_after_sync();
      const bool valid = kv_row < Lk;
      __nv_bfloat16* dvp = p.dv + static_cast<size_t>(k_start + kv_row) * p.dqkv_stride + p.v_col0 + hk * D;
      __nv_bfloat16* dkp = p.dk + static_cast<size_t>(k_start + kv_row) * p.dqkv_stride + p.k_col0 + hk * D;
#pragma unroll 1
      for (int c = wg; c < D / 32; c += 2) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_lane + DV_COL + c * 32, v);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * x]), __uint_as_float(v[8 * x + 1]));
            o4.y = pack_bf16x2(__uint_as_float(v[8 * x + 2]), __uint_as_float(v[8 * x + 3]));
            o4.z = pack_bf16x2(__uint_as_float(v[8 * x + 4]), __uint_as_float(v[8 * x + 5]));
            o4.w = pack_bf16x2(__uint_as_float(v[8 * x + 6]), __uint_as_float(v[8 * x + 7]));
            *reinterpret_cast<uint4*>(dvp + c * 32 + x * 8) = o4;
          }
        }
        tmem_ld_32x32b_x32(t_lane + DK_COL + c * 32, v);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * x]) * p.scale, __uint_as_float(v[8 * x + 1]) * p.scale);
            o4.y = pack_bf16x2(__uint_as_float(v[8 * x + 2]) * p.scale, __uint_as_float(v[8 * x + 3]) * p.scale);
            o4.z = pack_bf16x2(__uint_as_float(v[8 * x + 4]) * p.scale, __uint_as_float(v[8 * x + 5]) * p.scale);
            o4.w = pack_bf16x2(__uint_as_float(v[8 * x + 6]) * p.scale, __uint_as_float(v[8 * x + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dkp + c * 32 + x * 8) = o4;
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

// ------------------------------------------------------------------------------------------------
// backward, kernel 2: dQ.  One CTA owns a 128-row query tile of one head (Q and dO resident) and walks the
// 64-row K/V sub-tiles it can see.  TMEM: two (S | dP) buffers of 64+64 columns and the dQ accumulator.
// ------------------------------------------------------------------------------------------------
template <int D, bool EXT>   // EXT: sliding window / logit soft-cap code paths compiled in
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ128, const __grid_constant__ CUtensorMap tmK64,
                    const __grid_constant__ CUtensorMap tmV64, const __grid_constant__ CUtensorMap tmdO128,
                    AttnParams p) {
  using SM = BwdSmem<D>;
  constexpr int DCH = D / 64;
  constexpr int STAGES = SM::STAGES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t DQ_COL = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars;             // [1]
  uint64_t* s_full = bars + 1;         // [2]
  uint64_t* p_full = bars + 3;         // [2]
  uint64_t* acc_full = bars + 5;       // [1]
  uint64_t* kv_full = bars + 6;        // [STAGES]
  uint64_t* kv_empty = bars + 6 + SM::STAGES;   // [STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6 + 2 * SM::STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid: x = head + heads * batch (fastest), y = tile: the whole grid is dispatched longest-tile-first
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int hk = h / p.group;
  int q_start, Lq;
  seq_bounds(p, b, q_start, Lq);
  const int k_start = q_start, Lk = Lq;
  const int n_qt = (Lq + 127) / 128;
  if ((int)blockIdx.y >= n_qt) return;
  const int i = n_qt - 1 - blockIdx.y;
  const int off = Lk - Lq;
  const int kv_end = p.causal ? min(Lk, i * 128 + 128 + off) : Lk;
  // sliding window: 64-key sub-tiles entirely left of the first row's window are skipped
  const int sub0 = (EXT && p.window > 0) ? max(0, i * 128 + off - p.window + 1) / 64 : 0;
  const int total = (kv_end + 63) / 64 - sub0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ128);
    tma_prefetch_desc(&tmK64);
    tma_prefetch_desc(&tmV64);
    tma_prefetch_desc(&tmdO128);
    for (int x = 0; x < 6 + 2 * SM::STAGES; ++x) mbar_init(&bars[x], (x == 3 || x == 4) ? 8 : 1);
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
  bool alive = true;

  if (warp == 0) {
    if (elect_one_sync()) {
      mbar_expect_tx(q_full, 2 * SM::BIG);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_2d(smem + SM::A_OFF + c * 16384, &tmQ128, q_full, p.q_col0 + h * D + c * 64, q_start + i * 128);
        tma_load_2d(smem + SM::B_OFF + c * 16384, &tmdO128, q_full, h * D + c * 64, q_start + i * 128);
      }
      for (int it = 0; it < total && alive; ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&kv_empty[s], ((it / STAGES) & 1u) ^ 1u, alive, 800)) break;
        mbar_expect_tx(&kv_full[s], 2 * SM::SMALL);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_2d(smem + SM::S0_OFF + s * SM::SMALL + c * 8192, &tmK64, &kv_full[s], p.k_col0 + hk * D + c * 64,
                      k_start + (sub0 + it) * 64);
          tma_load_2d(smem + SM::S1_OFF + s * SM::SMALL + c * 8192, &tmV64, &kv_full[s], p.v_col0 + hk * D + c * 64,
                      k_start + (sub0 + it) * 64);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      const uint32_t idesc_s = make_idesc(128, 64, 1, 1, 0, 0);
      const uint32_t idesc_acc = make_idesc(128, D, 1, 1, 0, 1);
      const uint32_t qa = smem_u32(smem + SM::A_OFF), da = smem_u32(smem + SM::B_OFF);
      auto issue12 = [&](int it) {
        const int s = it % STAGES;
        if (!mbar_wait(&kv_full[s], (it / STAGES) & 1u, alive, 810)) return;
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(smem + SM::S0_OFF + s * SM::SMALL);
        const uint32_t va = smem_u32(smem + SM::S1_OFF + s * SM::SMALL);
        const uint32_t st = tmem_base + (it & 1) * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t oa = (k >> 2) * 16384 + (k & 3) * 32, ob = (k >> 2) * 8192 + (k & 3) * 32;
          umma_f16_ss(st, make_smem_desc_sw128(qa + oa, 16, 1024), make_smem_desc_sw128(ka + ob, 16, 1024), idesc_s,
                      k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t oa = (k >> 2) * 16384 + (k & 3) * 32, ob = (k >> 2) * 8192 + (k & 3) * 32;
          umma_f16_ss(st + 64, make_smem_desc_sw128(da + oa, 16, 1024), make_smem_desc_sw128(va + ob, 16, 1024),
                      idesc_s, k != 0);
        }
        umma_commit(&s_full[it & 1]);
      };
      if (mbar_wait(q_full, 0, alive, 811)) {
        issue12(0);
        if (total > 1 && alive) issue12(1);
        for (int it = 0; it < total && alive; ++it) {
          const int bsel = it & 1, s = it % STAGES;
          if (!mbar_wait(&p_full[bsel], (it >> 1) & 1u, alive, 812)) break;
          tc_fence_after_sync();
          const uint32_t ka = smem_u32(smem + SM::S0_OFF + s * SM::SMALL);
          const uint32_t st = tmem_base + bsel * 128;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ts(tmem_base + DQ_COL, st + 64 + (kk >> 1) * 32 + (kk & 1) * 8,
                        make_smem_desc_sw128(ka + kk * 2048, 8192, 1024), idesc_acc, (it | kk) != 0);
          umma_commit(&kv_empty[s]);
          if (it + 2 < total) issue12(it + 2);
        }
        if (alive) umma_commit(acc_full);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int r = q4 * 32 + lane;
    const int qrow = i * 128 + r;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16);
    float lse2 = 0.f, delta = 0.f;
    if (qrow < Lq) {
      const size_t idx = static_cast<size_t>(h) * p.total_rows + q_start + qrow;
      lse2 = p.lse[idx] * 1.4426950408889634f;
      delta = p.delta[idx];
    }
    const int limit = (qrow < Lq) ? (p.causal ? min(Lk - 1, qrow + off) : Lk - 1) : -1;
    const int lo = (EXT && p.window > 0) ? qrow + off - p.window + 1 : 0;
    for (int it = 0; it < total && alive; ++it) {
      if (!mbar_wait(&s_full[it & 1], (it >> 1) & 1u, alive, 820)) break;
      tc_fence_after_sync();
      const uint32_t t_s = t_lane + (it & 1) * 128;
      const int col0 = (sub0 + it) * 64;
      const bool need_mask = (col0 + 63 > i * 128 + off && p.causal) || (col0 + 64 > Lk) || (i * 128 + 128 > Lq) ||
                             (EXT && p.window > 0 && col0 <= i * 128 + 127 + off - p.window);
      {
        const int cc = wg;
        uint32_t sv[32], dv[32], ds[16];
        tmem_ld_32x32b_x32(t_s + cc * 32, sv);
        tmem_ld_32x32b_x32(t_s + 64 + cc * 32, dv);
        tc_wait_ld();
        auto body = [&](auto masked, auto capped) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float p0, p1, g0 = 1.f, g1 = 1.f;
            if constexpr (decltype(capped)::value) {
              const float t0 = fast_tanh(__uint_as_float(sv[e]) * p.cap_inv);
              const float t1 = fast_tanh(__uint_as_float(sv[e + 1]) * p.cap_inv);
              p0 = fast_ex2(fmaf(t0, p.cap_log2, -lse2));
              p1 = fast_ex2(fmaf(t1, p.cap_log2, -lse2));
              g0 = 1.f - t0 * t0;
              g1 = 1.f - t1 * t1;
            } else {
              p0 = fast_ex2(fmaf(__uint_as_float(sv[e]), p.scale_log2, -lse2));
              p1 = fast_ex2(fmaf(__uint_as_float(sv[e + 1]), p.scale_log2, -lse2));
            }
            if constexpr (decltype(masked)::value) {
              const int col = col0 + cc * 32 + e;
              p0 = (col <= limit) ? p0 : 0.f;
              p1 = (col + 1 <= limit) ? p1 : 0.f;
              if constexpr (EXT) {
                p0 = (col >= lo) ? p0 : 0.f;
                p1 = (col + 1 >= lo) ? p1 : 0.f;
              }
            }
            if constexpr (decltype(capped)::value)
              ds[e >> 1] = pack_bf16x2(p0 * g0 * (__uint_as_float(dv[e]) - delta),
                                       p1 * g1 * (__uint_as_float(dv[e + 1]) - delta));
            else
              ds[e >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[e]) - delta), p1 * (__uint_as_float(dv[e + 1]) - delta));
          }
        };
        if (EXT && p.cap_log2 > 0.f) body(std::true_type{}, std::true_type{});
        else if (need_mask) body(std::true_type{}, std::false_type{});
        else body(std::false_type{}, std::false_type{});
        tmem_st_32x32b_x16(t_s + 64 + cc * 32, ds);
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[it & 1]);
    }
    if (alive && mbar_wait(acc_full, 0, alive, 821)) {
      tc_fence_after_sync();
      const bool valid = qrow < Lq;
      __nv_bfloat16* dqp = p.dq + static_cast<size_t>(q_start + qrow) * p.dqkv_stride + p.q_col0 + h * D;
#pragma unroll 1
      for (int c = wg; c < D / 32; c += 2) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_lane + DQ_COL + c * 32, v);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * x]) * p.scale, __uint_as_float(v[8 * x + 1]) * p.scale);
            o4.y = pack_bf16x2(__uint_as_float(v[8 * x + 2]) * p.scale, __uint_as_float(v[8 * x + 3]) * p.scale);
            o4.z = pack_bf16x2(__uint_as_float(v[8 * x + 4]) * p.scale, __uint_as_float(v[8 * x + 5]) * p.scale);
            o4.w = pack_bf16x2(__uint_as_float(v[8 * x + 6]) * p.scale, __uint_as_float(v[8 * x + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dqp + c * 32 + x * 8) = o4;
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

template <int D, bool EXT>
static int launch_bwd(const CUtensorMap* m, const AttnParams& p, int max_len, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_dkdv_kernel<D, EXT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         BwdSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(flash_bwd_dq_kernel<D, EXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // m: [0]=q64 [1]=k128 [2]=v128 [3]=do64 [4]=q128 [5]=k64 [6]=v64 [7]=do128
  dim3 g1(p.Hkv * p.B, (max_len + 127) / 128, 1);
  flash_bwd_dkdv_kernel<D, EXT><<<g1, BWD_THREADS, BwdSmem<D>::TOTAL, st>>>(m[0], m[1], m[2], m[3], p);
  dim3 g2(p.Hq * p.B, (max_len + 127) / 128, 1);
  flash_bwd_dq_kernel<D, EXT><<<g2, BWD_THREADS, BwdSmem<D>::TOTAL, st>>>(m[4], m[5], m[6], m[7], p);
  return (int)cudaGetLastError();
}

template <int D, bool EXT>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                      int max_len, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<D, EXT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FwdSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.Hq * p.B, (max_len + 255) / 256, 1);
  flash_fwd_kernel<D, EXT><<<grid, FWD_THREADS, FwdSmem<D>::TOTAL, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_attention)

using namespace ts;

// q, k, v: bf16 row-major token matrices [total_rows][*_stride]; head h of q starts at column h*D (+ col0).
// They may alias one fused qkv buffer (pass the same base with different col0).
// cu_seqlens: device int32 [B+1] for packed documents or nullptr for B sequences of S tokens.
// max_len: longest sequence (host knowledge; S for the uniform case).
// window > 0 restricts every query to the last `window` keys; softcap > 0 applies c * tanh(s / c) to the scaled logits.
extern "C" int ts_flash_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, long long total_rows,
                               int q_stride, int k_stride, int v_stride, int o_stride, int q_col0, int k_col0,
                               int v_col0, int Hq, int Hkv, int D, int B, int S, const int* cu_seqlens, int max_len,
                               int causal, float scale, int window, float softcap, void* stream) {
  if ((D != 64 && D != 128) || Hq % Hkv != 0 || total_rows <= 0) return -10;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows, (uint64_t)q_stride,
                        (uint64_t)q_stride, 128, 64);
  if (rc) return rc * 100 - 1;
  rc = make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows, (uint64_t)k_stride,
                    (uint64_t)k_stride, 128, 64);
  if (rc) return rc * 100 - 2;
  rc = make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows, (uint64_t)v_stride,
                    (uint64_t)v_stride, 128, 64);
  if (rc) return rc * 100 - 3;
  AttnParams p{};
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.Hq = Hq; p.Hkv = Hkv; p.group = Hq / Hkv; p.B = B; p.S = S; p.cu_seqlens = cu_seqlens; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window > 0 ? window : 0;
  p.cap_inv = softcap > 0.f ? scale / softcap : 0.f;
  p.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  p.o = (__nv_bfloat16*)o; p.o_stride = o_stride; p.lse = lse; p.total_rows = total_rows;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool ext = p.window > 0 || p.cap_log2 > 0.f;
  if (D == 128) return ext ? launch_fwd<128, true>(tq, tk, tv, p, max_len, st) : launch_fwd<128, false>(tq, tk, tv, p, max_len, st);
  return ext ? launch_fwd<64, true>(tq, tk, tv, p, max_len, st) : launch_fwd<64, false>(tq, tk, tv, p, max_len, st);
}

extern "C" int ts_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, long long total_rows,
                            int q_stride, int k_stride, int v_stride, int o_stride, int q_col0, int k_col0,
                            int v_col0, int Hq, int Hkv, int D, int B, int S, const int* cu_seqlens, int max_len,
                            int causal, float scale, void* stream) {
  return ts_flash_fwd_ex(q, k, v, o, lse, total_rows, q_stride, k_stride, v_stride, o_stride, q_col0, k_col0, v_col0, Hq,
                         Hkv, D, B, S, cu_seqlens, max_len, causal, scale, 0, 0.f, stream);
}

extern "C" int ts_attn_delta(const void* o, const void* dout, float* delta, long long total_rows, int Hq, int D,
                             int o_stride, void* stream) {
  const long long warps = total_rows * Hq;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  attn_delta_kernel<<<(unsigned)blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, total_rows, Hq, D, o_stride);
  return (int)cudaGetLastError();
}

// Gradient of ts_flash_fwd. dq/dk/dv are written into `dqkv` (same row layout and column offsets as q/k/v inside
// a fused buffer of row stride `qkv_stride`); every element of the q|k|v column range is written.
extern "C" int ts_flash_bwd_ex(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                               const float* delta, void* dqkv, long long total_rows, int qkv_stride, int o_stride,
                               int q_col0, int k_col0, int v_col0, int Hq, int Hkv, int D, int B, int S,
                               const int* cu_seqlens, int max_len, int causal, float scale, int window, float softcap,
                               void* stream) {
  if ((D != 64 && D != 128) || Hq % Hkv != 0 || total_rows <= 0) return -10;
  CUtensorMap m[8];
  const void* bases[4] = {q, k, v, dout};
  const int strides[4] = {qkv_stride, qkv_stride, qkv_stride, o_stride};
  const int small_first[4] = {1, 0, 0, 1};   // q, dO are streamed (64 rows) in the dK/dV kernel; k, v in the dQ kernel
  for (int t = 0; t < 4; ++t) {
    int rc = make_tmap_2d(&m[t], bases[t], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows,
                          (uint64_t)strides[t], (uint64_t)strides[t], small_first[t] ? 64 : 128, 64);
    if (rc) return rc * 100 - 10 - t;
    rc = make_tmap_2d(&m[4 + t], bases[t], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows,
                      (uint64_t)strides[t], (uint64_t)strides[t], small_first[t] ? 128 : 64, 64);
    if (rc) return rc * 100 - 20 - t;
  }
  AttnParams p{};
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.Hq = Hq; p.Hkv = Hkv; p.group = Hq / Hkv; p.B = B; p.S = S; p.cu_seqlens = cu_seqlens; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window > 0 ? window : 0;
  p.cap_inv = softcap > 0.f ? scale / softcap : 0.f;
  p.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  p.o_stride = o_stride; p.lse = const_cast<float*>(lse); p.delta = delta; p.total_rows = total_rows;
  p.dout = (const __nv_bfloat16*)dout;
  p.dq = p.dk = p.dv = (__nv_bfloat16*)dqkv;
  p.dqkv_stride = qkv_stride;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool ext = p.window > 0 || p.cap_log2 > 0.f;
  if (D == 128) return ext ? launch_bwd<128, true>(m, p, max_len, st) : launch_bwd<128, false>(m, p, max_len, st);
  return ext ? launch_bwd<64, true>(m, p, max_len, st) : launch_bwd<64, false>(m, p, max_len, st);
}

extern "C" int ts_flash_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                            const float* delta, void* dqkv, long long total_rows, int qkv_stride, int o_stride,
                            int q_col0, int k_col0, int v_col0, int Hq, int Hkv, int D, int B, int S,
                            const int* cu_seqlens, int max_len, int causal, float scale, void* stream) {
  return ts_flash_bwd_ex(q, k, v, dout, lse, delta, dqkv, total_rows, qkv_stride, o_stride, q_col0, k_col0, v_col0, Hq,
                         Hkv, D, B, S, cu_seqlens, max_len, causal, scale, 0, 0.f, stream);
}
