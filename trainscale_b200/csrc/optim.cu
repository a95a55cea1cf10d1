// Optimizer step kernels beyond flat AdamW / Lion (those live in elementwise.cu next to the engine's fused paths):
//   ts_adam8bit        AdamW on block-wise int8 moments: dequantise, update, requantise in one pass
//   ts_lamb_moments / ts_lamb_apply      LAMB; the trust ratio is formed on the device from two norms
//   ts_sophia_step / ts_sophia_hessian   Sophia-G clipped step and the Gauss-Newton-Bartlett EMA
//   ts_schedule_free   schedule-free AdamW (y / z iterates)
//   ts_adopt_step      ADOPT
//   ts_adafactor_stats / ts_adafactor_update / ts_adafactor_apply   factored second moments, RMS clip, update
// Every scalar that depends on the data (norms, RMS, clip factors) stays on the device: no step reads anything
// back to the host.  Parameters and gradients may be bf16 or fp32 (kind bits: 1 = parameter is bf16, 2 = gradient
// is bf16); moments are fp32 unless stated.
// Cover the Triton kernels of data_pipeline/trainer/optimizers/sota_optimizers.py:174-480 (fused AdamW / Lion,
// block-wise 8-bit codec, Sophia, schedule-free), lamb.py:46 and adafactor.py:210-540.
#include "common.cuh"
#include "host_common.h"

namespace ts {

typedef __nv_bfloat16 bf16;
#define ST(s) reinterpret_cast<cudaStream_t>(s)
constexpr int OPT_THREADS = 256;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long j) {
  if constexpr (sizeof(T) == 2) return __bfloat162float(p[j]); else return p[j];
}
template <typename T>
__device__ __forceinline__ void stf(T* p, long long j, float v) {
  if constexpr (sizeof(T) == 2) p[j] = __float2bfloat16(v); else p[j] = v;
}

static inline int opt_grid(long long n, int per_sm = 8) {
  long long g = (n + OPT_THREADS - 1) / OPT_THREADS;
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

#define GRID_STRIDE(j, n)                                                                          \
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < (n);      \
       j += static_cast<long long>(gridDim.x) * blockDim.x)

// Dispatch on the two dtype bits: CALL is compiled once per (PT, GT) pair.
#define DISPATCH_PG(kind, CALL)                                                                    \
  switch ((kind) & 3) {                                                                            \
    case 0: { typedef float PT; typedef float GT; CALL; } break;                                   \
    case 1: { typedef bf16 PT; typedef float GT; CALL; } break;                                    \
    case 2: { typedef float PT; typedef bf16 GT; CALL; } break;                                    \
    default: { typedef bf16 PT; typedef bf16 GT; CALL; } break;                                    \
  }

// ---------------------------------------------------------------------------------------------------------------
// 8-bit AdamW.  State layout: m_q / v_q int8 [nblocks][BS] (tail padded with zeros), m_s / v_s fp32 [nblocks]
// (absmax of the block, floor 1e-12); v is stored as sqrt(v) so that its range fits 8 bits.  One CTA per
// quantisation block: values live in registers between the dequantise and the requantise.
// ---------------------------------------------------------------------------------------------------------------
template <typename PT, typename GT, int ITEMS>
__global__ void __launch_bounds__(OPT_THREADS) adam8bit_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                               int8_t* __restrict__ m_q, float* __restrict__ m_s,
                                                               int8_t* __restrict__ v_q, float* __restrict__ v_s,
                                                               long long n, long long nblocks, float lr, float b1,
                                                               float b2, float eps, float wd, float bc1, float bc2) {
  constexpr int BS = ITEMS * OPT_THREADS;
  __shared__ float scratch[32];
  for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
    const float ms = m_s[blk] * (1.f / 127.f), vs = v_s[blk] * (1.f / 127.f);
    float mn[ITEMS], rn[ITEMS];
    float m_abs = 0.f, r_abs = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const long long j = blk * BS + i * OPT_THREADS + threadIdx.x;
      mn[i] = 0.f;
      rn[i] = 0.f;
      if (j < n) {
        const float gj = ldf(g, j);
        const float r = static_cast<float>(v_q[j]) * vs;
        const float m = b1 * (static_cast<float>(m_q[j]) * ms) + (1.f - b1) * gj;
        const float v = b2 * (r * r) + (1.f - b2) * gj * gj;
        const float pj = ldf(p, j) * (1.f - lr * wd) - lr * (m / bc1) / (sqrtf(v / bc2) + eps);
        stf(p, j, pj);
        mn[i] = m;
        rn[i] = sqrtf(v);
        m_abs = fmaxf(m_abs, fabsf(m));
        r_abs = fmaxf(r_abs, rn[i]);
      }
    }
    m_abs = fmaxf(block_max(m_abs, scratch), 1e-12f);
    r_abs = fmaxf(block_max(r_abs, scratch), 1e-12f);
    if (threadIdx.x == 0) {
      m_s[blk] = m_abs;
      v_s[blk] = r_abs;
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const long long j = blk * BS + i * OPT_THREADS + threadIdx.x;   // j < nblocks * BS: pad slots get zeros
      m_q[j] = static_cast<int8_t>(rintf(mn[i] / m_abs * 127.f));
      v_q[j] = static_cast<int8_t>(rintf(rn[i] / r_abs * 127.f));
    }
  }
}

// Vector form for quantisation blocks of 1024+ values: every thread owns groups of 4 CONSECUTIVE values, so parameters
// and gradients move as 16-byte (fp32) / 8-byte (bf16) accesses and the int8 state as 4-byte words instead of single
// bytes.  VEC4 = ITEMS / 4 groups per thread.
template <typename T>
__device__ __forceinline__ void ld4(const T* p, long long j, float (&o)[4]) {
  if constexpr (sizeof(T) == 2) {
    const uint2 u = *reinterpret_cast<const uint2*>(p + j);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  } else {
    const float4 f = *reinterpret_cast<const float4*>(p + j);
    o[0] = f.x; o[1] = f.y; o[2] = f.z; o[3] = f.w;
  }
}
template <typename T>
__device__ __forceinline__ void st4(T* p, long long j, const float (&v)[4]) {
  if constexpr (sizeof(T) == 2) {
    uint2 u;
    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p + j) = u;
  } else {
    *reinterpret_cast<float4*>(p + j) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

template <typename PT, typename GT, int ITEMS>
__global__ void __launch_bounds__(OPT_THREADS) adam8bit_vec_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                                   int8_t* __restrict__ m_q, float* __restrict__ m_s,
                                                                   int8_t* __restrict__ v_q, float* __restrict__ v_s,
                                                                   long long n, long long nblocks, float lr, float b1,
                                                                   float b2, float eps, float wd, float bc1, float bc2) {
  static_assert(ITEMS % 4 == 0, "vector form needs groups of 4");
  constexpr int BS = ITEMS * OPT_THREADS, VEC4 = ITEMS / 4;
  __shared__ float scratch[32];
  for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
    const float ms = m_s[blk] * (1.f / 127.f), vs = v_s[blk] * (1.f / 127.f);
    float mn[ITEMS], rn[ITEMS];
    float m_abs = 0.f, r_abs = 0.f;
#pragma unroll
    for (int i = 0; i < VEC4; ++i) {
      const long long j = blk * BS + (static_cast<long long>(i) * OPT_THREADS + threadIdx.x) * 4;
      const char4 mq = *reinterpret_cast<const char4*>(m_q + j);     // state arrays cover whole blocks: always in range
      const char4 vq = *reinterpret_cast<const char4*>(v_q + j);
      const float mqf[4] = {(float)mq.x, (float)mq.y, (float)mq.z, (float)mq.w};
      const float vqf[4] = {(float)vq.x, (float)vq.y, (float)vq.z, (float)vq.w};
      float pv[4] = {0.f, 0.f, 0.f, 0.f}, gv[4] = {0.f, 0.f, 0.f, 0.f};
      const bool full = j + 3 < n;
      if (full) {
        ld4(p, j, pv);
        ld4(g, j, gv);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (j + e < n) { pv[e] = ldf(p, j + e); gv[e] = ldf(g, j + e); }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const bool live = j + e < n;
        const float r = vqf[e] * vs;
        const float m = b1 * (mqf[e] * ms) + (1.f - b1) * gv[e];
        const float v = b2 * (r * r) + (1.f - b2) * gv[e] * gv[e];
        pv[e] = pv[e] * (1.f - lr * wd) - lr * (m / bc1) / (sqrtf(v / bc2) + eps);
        mn[i * 4 + e] = live ? m : 0.f;
        rn[i * 4 + e] = live ? sqrtf(v) : 0.f;
        m_abs = fmaxf(m_abs, fabsf(mn[i * 4 + e]));
        r_abs = fmaxf(r_abs, rn[i * 4 + e]);
      }
      if (full) {
        st4(p, j, pv);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (j + e < n) stf(p, j + e, pv[e]);
      }
    }
    m_abs = fmaxf(block_max(m_abs, scratch), 1e-12f);
    r_abs = fmaxf(block_max(r_abs, scratch), 1e-12f);
    if (threadIdx.x == 0) {
      m_s[blk] = m_abs;
      v_s[blk] = r_abs;
    }
#pragma unroll
    for (int i = 0; i < VEC4; ++i) {
      const long long j = blk * BS + (static_cast<long long>(i) * OPT_THREADS + threadIdx.x) * 4;
      char4 mq, vq;
      mq.x = static_cast<signed char>(rintf(mn[i * 4 + 0] / m_abs * 127.f));
      mq.y = static_cast<signed char>(rintf(mn[i * 4 + 1] / m_abs * 127.f));
      mq.z = static_cast<signed char>(rintf(mn[i * 4 + 2] / m_abs * 127.f));
      mq.w = static_cast<signed char>(rintf(mn[i * 4 + 3] / m_abs * 127.f));
      vq.x = static_cast<signed char>(rintf(rn[i * 4 + 0] / r_abs * 127.f));
      vq.y = static_cast<signed char>(rintf(rn[i * 4 + 1] / r_abs * 127.f));
      vq.z = static_cast<signed char>(rintf(rn[i * 4 + 2] / r_abs * 127.f));
      vq.w = static_cast<signed char>(rintf(rn[i * 4 + 3] / r_abs * 127.f));
      *reinterpret_cast<char4*>(m_q + j) = mq;
      *reinterpret_cast<char4*>(v_q + j) = vq;
    }
  }
}

// Block-wise absmax int8 codec on its own (state init, checkpoint conversion).
template <int ITEMS>
__global__ void __launch_bounds__(OPT_THREADS) quant8_kernel(const float* __restrict__ x, int8_t* __restrict__ q,
                                                             float* __restrict__ s, long long n, long long nblocks) {
  constexpr int BS = ITEMS * OPT_THREADS;
  __shared__ float scratch[32];
  for (long long blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
    float xv[ITEMS];
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const long long j = blk * BS + i * OPT_THREADS + threadIdx.x;
      xv[i] = (j < n) ? x[j] : 0.f;
      a = fmaxf(a, fabsf(xv[i]));
    }
    a = fmaxf(block_max(a, scratch), 1e-12f);
    if (threadIdx.x == 0) s[blk] = a;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
      q[blk * BS + i * OPT_THREADS + threadIdx.x] = static_cast<int8_t>(rintf(xv[i] / a * 127.f));
  }
}

__global__ void dequant8_kernel(const int8_t* __restrict__ q, const float* __restrict__ s, float* __restrict__ x,
                                long long n, int bs) {
  GRID_STRIDE(j, n) x[j] = static_cast<float>(q[j]) * (s[j / bs] * (1.f / 127.f));
}

// ---------------------------------------------------------------------------------------------------------------
// LAMB.  Pass 1 updates the moments, writes the Adam direction (+ weight decay term) to `upd` and accumulates
// norms[0] += |p|^2, norms[1] += |upd|^2 (caller zeroes norms).  Pass 2 applies lr * trust * upd with
// trust = clamp(|p| / |upd|) (1 when either norm is zero).
// ---------------------------------------------------------------------------------------------------------------
template <typename PT, typename GT>
__global__ void __launch_bounds__(OPT_THREADS) lamb_moments_kernel(const PT* __restrict__ p, const GT* __restrict__ g,
                                                                   float* __restrict__ m, float* __restrict__ v,
                                                                   float* __restrict__ upd, float* __restrict__ norms,
                                                                   long long n, float b1, float b2, float eps, float wd,
                                                                   float bc1, float bc2) {
  __shared__ float scratch[32];
  float wn = 0.f, un = 0.f;
  GRID_STRIDE(j, n) {
    const float gj = ldf(g, j), pj = ldf(p, j);
    const float mj = b1 * m[j] + (1.f - b1) * gj;
    const float vj = b2 * v[j] + (1.f - b2) * gj * gj;
    m[j] = mj;
    v[j] = vj;
    const float u = (mj / bc1) / (sqrtf(vj / bc2) + eps) + wd * pj;
    upd[j] = u;
    wn += pj * pj;
    un += u * u;
  }
  wn = block_sum(wn, scratch);
  un = block_sum(un, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(&norms[0], wn);
    atomicAdd(&norms[1], un);
  }
}

template <typename PT>
__global__ void __launch_bounds__(OPT_THREADS) lamb_apply_kernel(PT* __restrict__ p, const float* __restrict__ upd,
                                                                 const float* __restrict__ norms, long long n, float lr,
                                                                 float trust_lo, float trust_hi) {
  const float wn = sqrtf(norms[0]), un = sqrtf(norms[1]);
  float trust = (wn > 0.f && un > 0.f) ? wn / un : 1.f;
  trust = fminf(fmaxf(trust, trust_lo), trust_hi);
  const float a = lr * trust;
  GRID_STRIDE(j, n) stf(p, j, ldf(p, j) - a * upd[j]);
}

// ---------------------------------------------------------------------------------------------------------------
// Sophia-G: m <- b1 m + (1-b1) g;  p <- p (1 - lr wd) - lr sign(m) min(|m| / (rho h + eps), 1)
// Hessian EMA: h <- b2 h + (1-b2) bs g^2 (g from a backward on sampled labels).
// ---------------------------------------------------------------------------------------------------------------
template <typename PT, typename GT>
__global__ void __launch_bounds__(OPT_THREADS) sophia_step_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                                  float* __restrict__ m, const float* __restrict__ h,
                                                                  long long n, float lr, float b1, float rho, float wd,
                                                                  float eps) {
  GRID_STRIDE(j, n) {
    const float mj = b1 * m[j] + (1.f - b1) * ldf(g, j);
    m[j] = mj;
    const float ratio = fminf(fabsf(mj) / (rho * h[j] + eps), 1.f);
    const float sgn = (mj > 0.f) ? 1.f : ((mj < 0.f) ? -1.f : 0.f);
    stf(p, j, ldf(p, j) * (1.f - lr * wd) - lr * sgn * ratio);
  }
}

template <typename GT>
__global__ void __launch_bounds__(OPT_THREADS) sophia_hessian_kernel(const GT* __restrict__ g, float* __restrict__ h,
                                                                     long long n, float b2, float scale) {
  GRID_STRIDE(j, n) {
    const float gj = ldf(g, j);
    h[j] = b2 * h[j] + scale * gj * gj;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Schedule-free AdamW.  p holds the interpolated iterate y, z the base iterate:
//   v <- b2 v + (1-b2) g^2;  gn = g / (sqrt(v) + eps) + wd y;  y <- y + c (z - y) + lr (b1 (1-c) - 1) gn;  z <- z - lr gn
// (lr already carries the warm-up and the sqrt(1 - b2^k) factor; c = w_k / sum w.)
// ---------------------------------------------------------------------------------------------------------------
template <typename PT, typename GT>
__global__ void __launch_bounds__(OPT_THREADS) schedule_free_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                                    float* __restrict__ z, float* __restrict__ v,
                                                                    long long n, float lr, float b1, float b2, float eps,
                                                                    float wd, float c) {
  const float a = lr * (b1 * (1.f - c) - 1.f);
  GRID_STRIDE(j, n) {
    const float gj = ldf(g, j);
    const float vj = b2 * v[j] + (1.f - b2) * gj * gj;
    v[j] = vj;
    float y = ldf(p, j);
    const float gn = gj / (sqrtf(vj) + eps) + wd * y;
    const float zj = z[j];
    y = y + c * (zj - y) + a * gn;
    z[j] = zj - lr * gn;
    stf(p, j, y);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// ADOPT: n = clamp(g / max(sqrt(v), eps), +-clip);  m <- b1 m + (1-b1) n;  p <- p (1 - lr wd) - lr m;
//        v <- b2 v + (1-b2) g^2   (v of the previous step normalises; clip <= 0 means no clamp)
// ---------------------------------------------------------------------------------------------------------------
template <typename PT, typename GT>
__global__ void __launch_bounds__(OPT_THREADS) adopt_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                            float* __restrict__ m, float* __restrict__ v, long long n,
                                                            float lr, float b1, float b2, float eps, float wd,
                                                            float clip) {
  GRID_STRIDE(j, n) {
    const float gj = ldf(g, j), vj = v[j];
    float nj = gj / fmaxf(sqrtf(vj), eps);
    if (clip > 0.f) nj = fminf(fmaxf(nj, -clip), clip);
    const float mj = b1 * m[j] + (1.f - b1) * nj;
    m[j] = mj;
    stf(p, j, ldf(p, j) * (1.f - lr * wd) - lr * mj);
    v[j] = b2 * vj + (1.f - b2) * gj * gj;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// AdaFactor on a matrix g[R][C].
//   stats : row[r] <- b2 row[r] + (1-b2) mean_c(g^2 + eps0);  col_tmp[c] += sum_r(g^2 + eps0)  (caller zeroes col_tmp
//           and folds it into the column EMA: a C-element op)
//   update: u = g * rsqrt(row[r] / row_mean) * rsqrt(col[c])   (or, unfactored: v <- b2 v + (1-b2)(g^2+eps0), u = g rsqrt(v));
//           sums[0] += u^2, sums[1] += p^2
//   apply : u <- u / max(1, rms(u) / clip) * lr_eff, lr_eff = lr * max(eps1, rms(p)) when scale_parameter;
//           optional first moment m <- b1 m + (1-b1) u, u <- m;  p <- p (1 - wd lr_eff) - u
// ---------------------------------------------------------------------------------------------------------------
constexpr int AF_ROWS = 8;

template <typename GT>
__global__ void __launch_bounds__(OPT_THREADS) adafactor_stats_kernel(const GT* __restrict__ g, float* __restrict__ row,
                                                                      float* __restrict__ col_tmp, int R, int C, float b2,
                                                                      float eps0) {
  __shared__ float scratch[32];
  const int tiles = (R + AF_ROWS - 1) / AF_ROWS;
  for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int r0 = t * AF_ROWS;
    float racc[AF_ROWS];
#pragma unroll
    for (int i = 0; i < AF_ROWS; ++i) racc[i] = 0.f;
    for (int c = threadIdx.x; c < C; c += OPT_THREADS) {
      float cacc = 0.f;
#pragma unroll
      for (int i = 0; i < AF_ROWS; ++i) {
        if (r0 + i < R) {
          const float gj = ldf(g, static_cast<long long>(r0 + i) * C + c);
          const float val = gj * gj + eps0;
          racc[i] += val;
          cacc += val;
        }
      }
      atomicAdd(&col_tmp[c], cacc);
    }
#pragma unroll
    for (int i = 0; i < AF_ROWS; ++i) {
      const float s = block_sum(racc[i], scratch);
      if (threadIdx.x == 0 && r0 + i < R) row[r0 + i] = b2 * row[r0 + i] + (1.f - b2) * (s / C);
    }
  }
}

template <typename PT, typename GT>
__global__ void __launch_bounds__(OPT_THREADS) adafactor_update_factored_kernel(const PT* __restrict__ p,
                                                                                const GT* __restrict__ g,
                                                                                const float* __restrict__ row,
                                                                                const float* __restrict__ col,
                                                                                const float* __restrict__ row_mean,
                                                                                float* __restrict__ u,
                                                                                float* __restrict__ sums, int R, int C) {
  __shared__ float scratch[32];
  const float rm = row_mean[0];
  float su = 0.f, sp = 0.f;
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const float rf = rsqrtf(row[r] / rm);
    for (int c = threadIdx.x; c < C; c += OPT_THREADS) {
      const long long j = static_cast<long long>(r) * C + c;
      const float uj = ldf(g, j) * rf * rsqrtf(col[c]);
      const float pj = ldf(p, j);
      u[j] = uj;
      su += uj * uj;
      sp += pj * pj;
    }
  }
  su = block_sum(su, scratch);
  sp = block_sum(sp, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(&sums[0], su);
    atomicAdd(&sums[1], sp);
  }
}

template <typename PT, typename GT>
__global__ void __launch_bounds__(OPT_THREADS) adafactor_update_full_kernel(const PT* __restrict__ p,
                                                                            const GT* __restrict__ g,
                                                                            float* __restrict__ v, float* __restrict__ u,
                                                                            float* __restrict__ sums, long long n,
                                                                            float b2, float eps0) {
  __shared__ float scratch[32];
  float su = 0.f, sp = 0.f;
  GRID_STRIDE(j, n) {
    const float gj = ldf(g, j), pj = ldf(p, j);
    const float vj = b2 * v[j] + (1.f - b2) * (gj * gj + eps0);
    v[j] = vj;
    const float uj = gj * rsqrtf(vj);
    u[j] = uj;
    su += uj * uj;
    sp += pj * pj;
  }
  su = block_sum(su, scratch);
  sp = block_sum(sp, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(&sums[0], su);
    atomicAdd(&sums[1], sp);
  }
}

template <typename PT>
__global__ void __launch_bounds__(OPT_THREADS) adafactor_apply_kernel(PT* __restrict__ p, const float* __restrict__ u,
                                                                      float* __restrict__ m,
                                                                      const float* __restrict__ sums, long long n,
                                                                      float lr, float eps1, int scale_parameter,
                                                                      float clip, float b1, float wd) {
  const float inv_n = 1.f / static_cast<float>(n);
  const float rms_u = sqrtf(sums[0] * inv_n), rms_p = sqrtf(sums[1] * inv_n);
  const float lr_eff = scale_parameter ? lr * fmaxf(eps1, rms_p) : lr;
  const float a = lr_eff / fmaxf(1.f, rms_u / clip);
  const float decay = 1.f - wd * lr_eff;
  GRID_STRIDE(j, n) {
    float uj = u[j] * a;
    if (m) {
      uj = b1 * m[j] + (1.f - b1) * uj;
      m[j] = uj;
    }
    stf(p, j, ldf(p, j) * decay - uj);
  }
}

}  // namespace ts

using namespace ts;

TS_DEFINE_ERROR_API(ts_optim)

static inline int items_for(int block_size) {
  switch (block_size) {
    case 256: return 1;
    case 1024: return 4;
    case 2048: return 8;
    case 4096: return 16;
    default: return 0;
  }
}

#define DISPATCH_ITEMS(items, CALL)                                  \
  switch (items) {                                                   \
    case 1: { constexpr int IT = 1; CALL; } break;                   \
    case 4: { constexpr int IT = 4; CALL; } break;                   \
    case 8: { constexpr int IT = 8; CALL; } break;                   \
    default: { constexpr int IT = 16; CALL; } break;                 \
  }

// block_size in {256, 1024, 2048, 4096}; m_q / v_q hold ceil(n / block_size) * block_size bytes.
extern "C" int ts_adam8bit(void* p, const void* g, int kind, void* m_q, float* m_s, void* v_q, float* v_s, long long n,
                           int block_size, float lr, float b1, float b2, float eps, float wd, int step, void* stream) {
  if (n <= 0) return 0;
  const int items = items_for(block_size);
  if (!items || step < 1) return -10;
  const long long nblocks = (n + block_size - 1) / block_size;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  const long long cap = static_cast<long long>(sm_count()) * 8;
  const int grid = (int)(nblocks < cap ? nblocks : cap);
  // the vector form needs 16-byte aligned parameter / gradient / state bases (torch allocations are)
  const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                         reinterpret_cast<uintptr_t>(m_q) | reinterpret_cast<uintptr_t>(v_q)) & 15u) == 0;
  if (items == 1 || !aligned) {
    DISPATCH_PG(kind, DISPATCH_ITEMS(items, (adam8bit_kernel<PT, GT, IT><<<grid, OPT_THREADS, 0, ST(stream)>>>(
                                                (PT*)p, (const GT*)g, (int8_t*)m_q, m_s, (int8_t*)v_q, v_s, n, nblocks,
                                                lr, b1, b2, eps, wd, bc1, bc2))));
  } else {
    switch (items) {
      case 4: DISPATCH_PG(kind, (adam8bit_vec_kernel<PT, GT, 4><<<grid, OPT_THREADS, 0, ST(stream)>>>(
                                    (PT*)p, (const GT*)g, (int8_t*)m_q, m_s, (int8_t*)v_q, v_s, n, nblocks, lr, b1, b2,
                                    eps, wd, bc1, bc2))); break;
      case 8: DISPATCH_PG(kind, (adam8bit_vec_kernel<PT, GT, 8><<<grid, OPT_THREADS, 0, ST(stream)>>>(
                                    (PT*)p, (const GT*)g, (int8_t*)m_q, m_s, (int8_t*)v_q, v_s, n, nblocks, lr, b1, b2,
                                    eps, wd, bc1, bc2))); break;
      default: DISPATCH_PG(kind, (adam8bit_vec_kernel<PT, GT, 16><<<grid, OPT_THREADS, 0, ST(stream)>>>(
                                     (PT*)p, (const GT*)g, (int8_t*)m_q, m_s, (int8_t*)v_q, v_s, n, nblocks, lr, b1, b2,
                                     eps, wd, bc1, bc2))); break;
    }
  }
  return (int)cudaGetLastError();
}

extern "C" int ts_quant8(const float* x, void* q, float* s, long long n, int block_size, void* stream) {
  if (n <= 0) return 0;
  const int items = items_for(block_size);
  if (!items) return -10;
  const long long nblocks = (n + block_size - 1) / block_size;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  const int grid = (int)(nblocks < cap ? nblocks : cap);
  DISPATCH_ITEMS(items, (quant8_kernel<IT><<<grid, OPT_THREADS, 0, ST(stream)>>>(x, (int8_t*)q, s, n, nblocks)));
  return (int)cudaGetLastError();
}

extern "C" int ts_dequant8(const void* q, const float* s, float* x, long long n, int block_size, void* stream) {
  if (n <= 0) return 0;
  if (block_size <= 0) return -10;
  dequant8_kernel<<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((const int8_t*)q, s, x, n, block_size);
  return (int)cudaGetLastError();
}

extern "C" int ts_lamb_moments(const void* p, const void* g, int kind, float* m, float* v, float* upd, float* norms,
                               long long n, float b1, float b2, float eps, float wd, int step, void* stream) {
  if (n <= 0) return 0;
  if (step < 1) return -10;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  DISPATCH_PG(kind, (lamb_moments_kernel<PT, GT><<<opt_grid(n, 4), OPT_THREADS, 0, ST(stream)>>>(
                        (const PT*)p, (const GT*)g, m, v, upd, norms, n, b1, b2, eps, wd, bc1, bc2)));
  return (int)cudaGetLastError();
}

extern "C" int ts_lamb_apply(void* p, int kind, const float* upd, const float* norms, long long n, float lr,
                             float trust_lo, float trust_hi, void* stream) {
  if (n <= 0) return 0;
  if (kind & 1)
    lamb_apply_kernel<bf16><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((bf16*)p, upd, norms, n, lr, trust_lo, trust_hi);
  else
    lamb_apply_kernel<float><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((float*)p, upd, norms, n, lr, trust_lo, trust_hi);
  return (int)cudaGetLastError();
}

extern "C" int ts_sophia_step(void* p, const void* g, int kind, float* m, const float* h, long long n, float lr,
                              float b1, float rho, float wd, float eps, void* stream) {
  if (n <= 0) return 0;
  DISPATCH_PG(kind, (sophia_step_kernel<PT, GT><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>(
                        (PT*)p, (const GT*)g, m, h, n, lr, b1, rho, wd, eps)));
  return (int)cudaGetLastError();
}

extern "C" int ts_sophia_hessian(const void* g, int kind, float* h, long long n, float b2, float scale, void* stream) {
  if (n <= 0) return 0;
  if (kind & 2)
    sophia_hessian_kernel<bf16><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((const bf16*)g, h, n, b2, scale);
  else
    sophia_hessian_kernel<float><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((const float*)g, h, n, b2, scale);
  return (int)cudaGetLastError();
}

extern "C" int ts_schedule_free(void* p, const void* g, int kind, float* z, float* v, long long n, float lr, float b1,
                                float b2, float eps, float wd, float c, void* stream) {
  if (n <= 0) return 0;
  DISPATCH_PG(kind, (schedule_free_kernel<PT, GT><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>(
                        (PT*)p, (const GT*)g, z, v, n, lr, b1, b2, eps, wd, c)));
  return (int)cudaGetLastError();
}

extern "C" int ts_adopt_step(void* p, const void* g, int kind, float* m, float* v, long long n, float lr, float b1,
                             float b2, float eps, float wd, float clip, void* stream) {
  if (n <= 0) return 0;
  DISPATCH_PG(kind, (adopt_kernel<PT, GT><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((PT*)p, (const GT*)g, m, v, n,
                                                                                       lr, b1, b2, eps, wd, clip)));
  return (int)cudaGetLastError();
}

extern "C" int ts_adafactor_stats(const void* g, int kind, float* row, float* col_tmp, int R, int C, float b2,
                                  float eps0, void* stream) {
  if (R <= 0 || C <= 0) return 0;
  const int tiles = (R + AF_ROWS - 1) / AF_ROWS;
  const int cap = sm_count() * 8;
  const int grid = tiles < cap ? tiles : cap;
  if (kind & 2)
    adafactor_stats_kernel<bf16><<<grid, OPT_THREADS, 0, ST(stream)>>>((const bf16*)g, row, col_tmp, R, C, b2, eps0);
  else
    adafactor_stats_kernel<float><<<grid, OPT_THREADS, 0, ST(stream)>>>((const float*)g, row, col_tmp, R, C, b2, eps0);
  return (int)cudaGetLastError();
}

// Factored form when row/col are given (R x C matrix), otherwise the full second moment v over n = R * C values.
extern "C" int ts_adafactor_update(const void* p, const void* g, int kind, const float* row, const float* col,
                                   const float* row_mean, float* v, float* u, float* sums, int R, int C, float b2,
                                   float eps0, void* stream) {
  if (R <= 0 || C <= 0) return 0;
  if (row && col && row_mean) {
    const int cap = sm_count() * 8;
    const int grid = R < cap ? R : cap;
    DISPATCH_PG(kind, (adafactor_update_factored_kernel<PT, GT><<<grid, OPT_THREADS, 0, ST(stream)>>>(
                          (const PT*)p, (const GT*)g, row, col, row_mean, u, sums, R, C)));
  } else {
    if (!v) return -10;
    const long long n = static_cast<long long>(R) * C;
    DISPATCH_PG(kind, (adafactor_update_full_kernel<PT, GT><<<opt_grid(n, 4), OPT_THREADS, 0, ST(stream)>>>(
                          (const PT*)p, (const GT*)g, v, u, sums, n, b2, eps0)));
  }
  return (int)cudaGetLastError();
}

extern "C" int ts_adafactor_apply(void* p, int kind, const float* u, float* m, const float* sums, long long n, float lr,
                                  float eps1, int scale_parameter, float clip, float b1, float wd, void* stream) {
  if (n <= 0) return 0;
  if (kind & 1)
    adafactor_apply_kernel<bf16><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((bf16*)p, u, m, sums, n, lr, eps1,
                                                                             scale_parameter, clip, b1, wd);
  else
    adafactor_apply_kernel<float><<<opt_grid(n), OPT_THREADS, 0, ST(stream)>>>((float*)p, u, m, sums, n, lr, eps1,
                                                                              scale_parameter, clip, b1, wd);
  return (int)cudaGetLastError();
}
