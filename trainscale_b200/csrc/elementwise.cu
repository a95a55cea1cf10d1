// Bandwidth-bound sm_100a kernels: RMSNorm fwd/bwd (+ fused residual add), RoPE (rotate-half / interleaved,
// position ids), SwiGLU / GeGLU fwd/bwd, row cross-entropy with in-place gradient, flat and multi-tensor
// AdamW with a device-side clip coefficient, squared-norm reduction, Lion, and small cast / scale helpers.
// All of them move 16 bytes per thread per access and keep the row in registers between the reduction
// and the write, so that each tensor crosses HBM once.
//
// They replace the reference's Triton kernels in data_pipeline/trainer/kernels/triton_kernels.py:122-1319,
// data_pipeline/trainer/kernels/layernorm_kernels.py:143-621, data_pipeline/trainer/kernels/rope_kernels.py:385-730
// and data_pipeline/trainer/optimizers/adamw.py:182-757.
#include "common.cuh"
#include "host_common.h"

namespace ts {

struct alignas(16) bf16x8 {
  uint32_t v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void unpack8(const bf16x8& r, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = r;
}

// ---------------------------------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * w ; optional h = x + residual written to res_out.
// One CTA per row, H % 8 == 0, up to MAXV vectors per thread cached in registers.
// ---------------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;   // 256 threads * 4 vectors * 8 = rows up to 8192 wide stay in registers

__device__ __forceinline__ void unpack_u4(const uint4& r, float* f) {
  const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y), c = unpack_bf16x2(r.z), d = unpack_bf16x2(r.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack_u4(const float* f) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ residual,
                                                                   const __nv_bfloat16* __restrict__ w,
                                                                   __nv_bfloat16* __restrict__ y,
                                                                   __nv_bfloat16* __restrict__ res_out,
                                                                   float* __restrict__ rstd_out, int H, float eps,
                                                                   float w_offset) {
  // One CTA per row.  A thread's share of the row (up to NORM_MAXV 16-byte vectors: rows of up to 8192 values) stays in
  // registers as the packed words that were loaded, all loads are issued before the first use, and the second pass
  // unpacks again (see rmsnorm_fwd_warp_kernel); wider rows re-read the part that does not fit.
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + row * H) : nullptr;
  uint4* ro = residual ? reinterpret_cast<uint4*>(res_out + row * H) : nullptr;
  const int nvec = H >> 3;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 raw[NORM_MAXV], rres[NORM_MAXV];
#pragma unroll
  for (int c = 0; c < NORM_MAXV; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    raw[c] = i < nvec ? __ldcs(xr + i) : zero;
    rres[c] = (rr && i < nvec) ? __ldcs(rr + i) : zero;
  }
  float ss = 0.f;
  auto add_sq = [&](const uint4& v) {
    float a[8];
    unpack_u4(v, a);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += a[e] * a[e];
  };
  auto summed = [&](const uint4& xv, const uint4& rv) {     // residual add, rounded to bf16 as the stored stream is
    float a[8], b[8];
    unpack_u4(xv, a);
    unpack_u4(rv, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] += b[e];
    return pack_u4(a);
  };
#pragma unroll
  for (int c = 0; c < NORM_MAXV; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (rr) {
      raw[c] = summed(raw[c], rres[c]);
      if (i < nvec) ro[i] = raw[c];
    }
    add_sq(raw[c]);
  }
  for (int i = threadIdx.x + NORM_MAXV * NORM_THREADS; i < nvec; i += NORM_THREADS) {   // rows wider than 8192
    uint4 v = xr[i];
    if (rr) {
      v = summed(v, rr[i]);
      ro[i] = v;
    }
    add_sq(v);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int c = 0; c < NORM_MAXV; ++c)
    asm volatile("" : "+r"(raw[c].x), "+r"(raw[c].y), "+r"(raw[c].z), "+r"(raw[c].w));
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
  auto emit = [&](int i, const uint4& v) {
    float a[8], wv[8];
    unpack_u4(v, a);
    unpack_u4(__ldg(wr + i), wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = a[e] * rstd * (wv[e] + w_offset);
    yr[i] = pack_u4(a);
  };
#pragma unroll
  for (int c = 0; c < NORM_MAXV; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (i < nvec) emit(i, raw[c]);
  }
  const uint4* src = rr ? reinterpret_cast<const uint4*>(res_out + row * H) : xr;
  for (int i = threadIdx.x + NORM_MAXV * NORM_THREADS; i < nvec; i += NORM_THREADS) emit(i, src[i]);
}

// Warp-per-row forward for rows of up to 32 * VPL vectors (H <= 4096 with VPL = 16).  The row stays in the warp's
// registers as the PACKED bf16 words that were loaded (4 registers per 16-byte vector, not 8 floats): that leaves room
// for all VPL loads of a lane to be in flight at once, which is what the memory system needs from the few warps that
// fit on an SM.  The reduction is shuffle-only; warps walk rows with a grid stride.
template <int VPL, bool HAS_RES>
__global__ void __launch_bounds__(128) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ residual,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y,
                                                               __nv_bfloat16* __restrict__ res_out,
                                                               float* __restrict__ rstd_out, long long rows, int H,
                                                               float eps, float w_offset) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    uint4 raw[VPL];
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int i = lane + c * 32;
      raw[c] = i < nvec ? __ldcs(xr + i) : make_uint4(0u, 0u, 0u, 0u);
    }
    if constexpr (HAS_RES) {
      const uint4* rr = reinterpret_cast<const uint4*>(residual + row * H);
      uint4* ro = reinterpret_cast<uint4*>(res_out + row * H);
      uint4 rres[VPL];
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int i = lane + c * 32;
        rres[c] = i < nvec ? __ldcs(rr + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int i = lane + c * 32;
        float a[8], b[8];
        unpack_u4(raw[c], a);
        unpack_u4(rres[c], b);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += b[e];
        raw[c] = pack_u4(a);          // the sum is rounded to bf16 exactly as the stored residual stream is
        if (i < nvec) __stcs(ro + i, raw[c]);
      }
#pragma unroll
      for (int c = 0; c < VPL; ++c)
        asm volatile("" : "+r"(raw[c].x), "+r"(raw[c].y), "+r"(raw[c].z), "+r"(raw[c].w));
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      float a[8];
      unpack_u4(raw[c], a);           // out-of-range vectors are zero and add nothing
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += a[e] * a[e];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    // the second pass unpacks the words again: without this the compiler keeps all 8 * VPL floats of the first pass
    // alive, and the registers that costs are exactly the ones the in-flight loads need
#pragma unroll
    for (int c = 0; c < VPL; ++c)
      asm volatile("" : "+r"(raw[c].x), "+r"(raw[c].y), "+r"(raw[c].z), "+r"(raw[c].w));
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int i = lane + c * 32;
      if (i < nvec) {
        float a[8], wv[8];
        unpack_u4(raw[c], a);
        unpack_u4(__ldg(wr + i), wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = a[e] * rstd * (wv[e] + w_offset);
        yr[i] = pack_u4(a);          // default caching: the next kernel (a GEMM) reads y out of L2
      }
    }
  }
}

// RMSNorm backward. Each CTA walks rows blockIdx.x, +gridDim.x, ... ; dx is written per row and the
// weight gradient is accumulated in registers and written as one fp32 partial row per CTA
// (dw_partial[gridDim.x][H]); rmsnorm_dw_reduce_kernel sums the partials. `dres` (optional) is an extra
// gradient flowing into the same tensor (the residual branch) and is added into dx.
template <int MAXV>   // vectors per thread kept in registers: rows of up to 256 * MAXV * 8 elements
__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                   const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ w,
                                                                   const float* __restrict__ rstd,
                                                                   const __nv_bfloat16* __restrict__ dres,
                                                                   __nv_bfloat16* __restrict__ dx,
                                                                   float* __restrict__ dw_partial, int rows, int H,
                                                                   float w_offset) {
  __shared__ float scratch[32];
  const int nvec = H >> 3;
  float dwacc[MAXV][8];
#pragma unroll
  for (int c = 0; c < MAXV; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[c][e] = 0.f;

  // the next row's x / dy are requested before the block reduction of the current row, so the loads are in
  // flight while the CTA waits at the barrier
  bf16x8 nx[MAXV], nd[MAXV];
  auto fetch = [&](int row) {
    const size_t off = static_cast<size_t>(row) * H;
    int c = 0;
    for (int i = threadIdx.x; i < nvec && c < MAXV; i += NORM_THREADS, ++c) {
      nx[c] = *reinterpret_cast<const bf16x8*>(x + off + i * 8);
      nd[c] = *reinterpret_cast<const bf16x8*>(dy + off + i * 8);
    }
  };
  if (static_cast<int>(blockIdx.x) < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * H;
    const float rs = rstd[row];
    float xh[MAXV][8], g[MAXV][8];
    float dot = 0.f;
    int c = 0;
    for (int i = threadIdx.x; i < nvec && c < MAXV; i += NORM_THREADS, ++c) {
      float xv[8], dv[8], wv[8];
      unpack8(nx[c], xv);
      unpack8(nd[c], dv);
      load8(w + i * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xh[c][e] = xv[e] * rs;
        g[c][e] = dv[e] * (wv[e] + w_offset);
        dot += g[c][e] * xh[c][e];
        dwacc[c][e] += dv[e] * xh[c][e];
      }
    }
    if (row + static_cast<int>(gridDim.x) < rows) fetch(row + gridDim.x);
    dot = block_sum(dot, scratch) / H;
    c = 0;
    for (int i = threadIdx.x; i < nvec && c < MAXV; i += NORM_THREADS, ++c) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rs * (g[c][e] - xh[c][e] * dot);
      if (dres) {
        float r[8];
        load8(dres + off + i * 8, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += r[e];
      }
      store8(dx + off + i * 8, o);
    }
  }
  int c = 0;
  for (int i = threadIdx.x; i < nvec && c < MAXV; i += NORM_THREADS, ++c) {
    float* dst = dw_partial + static_cast<size_t>(blockIdx.x) * H + i * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(dwacc[c][0], dwacc[c][1], dwacc[c][2], dwacc[c][3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[c][4], dwacc[c][5], dwacc[c][6], dwacc[c][7]);
  }
}

__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw_f32,
                                         __nv_bfloat16* __restrict__ dw_bf16, int parts, int H, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= H) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * H + col];
  if (dw_f32) dw_f32[col] = accumulate ? dw_f32[col] + s : s;
  if (dw_bf16) dw_bf16[col] = __float2bfloat16(accumulate ? __bfloat162float(dw_bf16[col]) + s : s);
}

// ---------------------------------------------------------------------------------------------------
// LayerNorm: y = (x - mean) * rstd * w + b.  Same row-per-CTA layout as RMSNorm; mean and rstd are kept in fp32
// for the backward, which also produces per-CTA partial rows of dw and db ([parts][2][H]).
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NORM_THREADS) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                     const __nv_bfloat16* __restrict__ w,
                                                                     const __nv_bfloat16* __restrict__ b,
                                                                     __nv_bfloat16* __restrict__ y,
                                                                     float* __restrict__ mean_out,
                                                                     float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  const int nvec = H >> 3;
  float cache[NORM_MAXV][8];
  float s = 0.f;
  int c = 0;
  for (int i = threadIdx.x; i < nvec && c < NORM_MAXV; i += NORM_THREADS, ++c) {
    load8(xr + i * 8, cache[c]);
#pragma unroll
    for (int e = 0; e < 8; ++e) s += cache[c][e];
  }
  const float mean = block_sum(s, scratch) / H;
  __syncthreads();   // scratch is reused by the second reduction
  float v = 0.f;
  c = 0;
  for (int i = threadIdx.x; i < nvec && c < NORM_MAXV; i += NORM_THREADS, ++c) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      cache[c][e] -= mean;
      v += cache[c][e] * cache[c][e];
    }
  }
  const float rstd = rsqrtf(block_sum(v, scratch) / H + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  c = 0;
  for (int i = threadIdx.x; i < nvec && c < NORM_MAXV; i += NORM_THREADS, ++c) {
    float wv[8], bv[8], o[8];
    load8(w + i * 8, wv);
    if (b) load8(b + i * 8, bv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = cache[c][e] * rstd * wv[e] + (b ? bv[e] : 0.f);
    store8(y + row * H + i * 8, o);
  }
}

__global__ void __launch_bounds__(NORM_THREADS) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                     const __nv_bfloat16* __restrict__ x,
                                                                     const __nv_bfloat16* __restrict__ w,
                                                                     const float* __restrict__ mean,
                                                                     const float* __restrict__ rstd,
                                                                     __nv_bfloat16* __restrict__ dx,
                                                                     float* __restrict__ partial, int rows, int H) {
  __shared__ float scratch[32];
  const int nvec = H >> 3;
  float dwacc[NORM_MAXV][8], dbacc[NORM_MAXV][8];
#pragma unroll
  for (int c = 0; c < NORM_MAXV; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[c][e] = dbacc[c][e] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * H;
    const float mu = mean[row], rs = rstd[row];
    float xh[NORM_MAXV][8], g[NORM_MAXV][8];
    float s1 = 0.f, s2 = 0.f;
    int c = 0;
    for (int i = threadIdx.x; i < nvec && c < NORM_MAXV; i += NORM_THREADS, ++c) {
      float xv[8], dv[8], wv[8];
      load8(x + off + i * 8, xv);
      load8(dy + off + i * 8, dv);
      load8(w + i * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xh[c][e] = (xv[e] - mu) * rs;
        g[c][e] = dv[e] * wv[e];
        s1 += g[c][e];
        s2 += g[c][e] * xh[c][e];
        dwacc[c][e] += dv[e] * xh[c][e];
        dbacc[c][e] += dv[e];
      }
    }
    s1 = block_sum(s1, scratch) / H;
    __syncthreads();
    s2 = block_sum(s2, scratch) / H;
    __syncthreads();
    c = 0;
    for (int i = threadIdx.x; i < nvec && c < NORM_MAXV; i += NORM_THREADS, ++c) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rs * (g[c][e] - s1 - xh[c][e] * s2);
      store8(dx + off + i * 8, o);
    }
  }
  int c = 0;
  for (int i = threadIdx.x; i < nvec && c < NORM_MAXV; i += NORM_THREADS, ++c) {
    float* dst = partial + (static_cast<size_t>(blockIdx.x) * 2) * H + i * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dst[e] = dwacc[c][e];
      dst[H + e] = dbacc[c][e];
    }
  }
}

// partial: [parts][2][H] -> dw[H], db[H] (fp32)
__global__ void layernorm_dwdb_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                             float* __restrict__ db, int parts, int H) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= H) return;
  float sw = 0.f, sb = 0.f;
  for (int p = 0; p < parts; ++p) {
    sw += partial[(static_cast<size_t>(p) * 2) * H + col];
    sb += partial[(static_cast<size_t>(p) * 2 + 1) * H + col];
  }
  dw[col] = sw;
  if (db) db[col] = sb;
}

// ---------------------------------------------------------------------------------------------------
// RoPE applied in place to `n_heads` consecutive heads of width D at the start of every row.
// Row t of `x` starts at x + t*row_stride; position of row t is pos[t] (if given) else (t % seq) + offset.
// cos/sin tables are fp32 [max_pos][D/2]. `sign` = -1 gives the backward pass (inverse rotation).
// ---------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, long long rows,
                            int row_stride, int n_heads, int D, int seq, int offset, int interleaved, float sign) {
  const int half = D >> 1;
  const int pairs_per_row = n_heads * half;
  const long long total = rows * pairs_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / pairs_per_row;
    const int rem = static_cast<int>(idx - row * pairs_per_row);
    const int head = rem / half, i = rem - head * half;
    const int p = pos ? pos[row] : static_cast<int>(row % seq) + offset;
    const float c = cos_t[static_cast<size_t>(p) * half + i];
    const float s = sin_t[static_cast<size_t>(p) * half + i] * sign;
    __nv_bfloat16* base = x + row * row_stride + head * D;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(base[i0]), b = __bfloat162float(base[i1]);
    base[i0] = __float2bfloat16(a * c - b * s);
    base[i1] = __float2bfloat16(b * c + a * s);
  }
}

// Vectorised rotate-half variant: a thread owns 8 rotation pairs of one row (one 16-byte column slice of the first
// half of a head and its partner in the second half), loads their cos / sin once and walks ROPE_HPT heads with them.
constexpr int ROPE_HPT = 4;
__global__ void rope_half_vec_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const int* __restrict__ pos, long long rows,
                                     int row_stride, int n_heads, int D, int seq, int offset, float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;
  const int groups = (n_heads + ROPE_HPT - 1) / ROPE_HPT;
  const int items_per_row = groups * vec_per_head;
  const long long total = rows * items_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / items_per_row;
    const int rem = static_cast<int>(idx - row * items_per_row);
    const int grp = rem / vec_per_head, v = rem - grp * vec_per_head;
    const int p = pos ? pos[row] : static_cast<int>(row % seq) + offset;
    const float* cp = cos_t + static_cast<size_t>(p) * half + v * 8;
    const float* sp = sin_t + static_cast<size_t>(p) * half + v * 8;
    const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
    const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x * sign, s0.y * sign, s0.z * sign, s0.w * sign,
                         s1.x * sign, s1.y * sign, s1.z * sign, s1.w * sign};
    const int h0 = grp * ROPE_HPT;
    bf16x8 ra[ROPE_HPT], rb[ROPE_HPT];
#pragma unroll
    for (int j = 0; j < ROPE_HPT; ++j) {
      if (h0 + j < n_heads) {
        const __nv_bfloat16* base = x + row * row_stride + (h0 + j) * D + v * 8;
        ra[j] = *reinterpret_cast<const bf16x8*>(base);
        rb[j] = *reinterpret_cast<const bf16x8*>(base + half);
      }
    }
#pragma unroll
    for (int j = 0; j < ROPE_HPT; ++j) {
      if (h0 + j < n_heads) {
        __nv_bfloat16* base = x + row * row_stride + (h0 + j) * D + v * 8;
        float a[8], b[8], oa[8], ob[8];
        unpack8(ra[j], a);
        unpack8(rb[j], b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          oa[e] = a[e] * cc[e] - b[e] * sn[e];
          ob[e] = b[e] * cc[e] + a[e] * sn[e];
        }
        store8(base, oa);
        store8(base + half, ob);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Gated activations on a fused [rows][2*I] gate|up buffer. act: 0 = SiLU (SwiGLU), 1 = GELU erf, 2 = GELU tanh
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float act_fwd(float g, int act) {
  if (act == 0) return g / (1.f + __expf(-g));
  if (act == 1) return 0.5f * g * (1.f + erff(g * 0.70710678118f));
  const float u = 0.7978845608f * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.f + tanhf(u));
}
__device__ __forceinline__ float act_bwd(float g, int act) {
  if (act == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  if (act == 1) return 0.5f * (1.f + erff(g * 0.70710678118f)) + g * 0.3989422804f * __expf(-0.5f * g * g);
  const float u = 0.7978845608f * (g + 0.044715f * g * g * g);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * 0.7978845608f * (1.f + 3.f * 0.044715f * g * g);
}

__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long rows,
                               int I, int ld_in, int act) {
  const int vec_per_row = I >> 3;
  const long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / vec_per_row;
    const int v = static_cast<int>(idx - row * vec_per_row);
    float g[8], u[8], o[8];
    load8(gu + row * ld_in + v * 8, g);
    load8(gu + row * ld_in + I + v * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = act_fwd(g[e], act) * u[e];
    store8(out + row * I + v * 8, o);
  }
}

__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                               __nv_bfloat16* __restrict__ dgu, long long rows, int I, int ld, int act) {
  const int vec_per_row = I >> 3;
  const long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / vec_per_row;
    const int v = static_cast<int>(idx - row * vec_per_row);
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + row * ld + v * 8, g);
    load8(gu + row * ld + I + v * 8, u);
    load8(dout + row * I + v * 8, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dg[e] = d[e] * u[e] * act_bwd(g[e], act);
      du[e] = d[e] * act_fwd(g[e], act);
    }
    store8(dgu + row * ld + v * 8, dg);
    store8(dgu + row * ld + I + v * 8, du);
  }
}

// Plain (un-gated) activation: y = act(x); backward dx = dy * act'(x).  n is a multiple of 8.
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n, int act) {
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    float a[8], o[8];
    load8(x + i, a);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = act_fwd(a[e], act);
    store8(y + i, o);
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                               __nv_bfloat16* __restrict__ dx, long long n, int act) {
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    float a[8], d[8], o[8];
    load8(x + i, a);
    load8(dy + i, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = d[e] * act_bwd(a[e], act);
    store8(dx + i, o);
  }
}

// ---------------------------------------------------------------------------------------------------
// Row cross-entropy over materialised logits [rows][V] (a vocabulary chunk loop lives in the caller).
// Pass 1: online max / sum-exp. Pass 2 (optional): logits <- (softmax - onehot) * gscale in place.
// Supports ignore_index, label smoothing, logit soft-capping and a logit scale.
// loss[row] = lse - z[label] (smoothed); lse[row] stored for reuse.
// ---------------------------------------------------------------------------------------------------
constexpr int CE_THREADS = 512;

__device__ __forceinline__ float ce_transform(float z, float scale, float softcap) {
  z *= scale;
  if (softcap > 0.f) z = softcap * tanhf(z / softcap);
  return z;
}

__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits,
                                                                   const long long* __restrict__ labels,
                                                                   float* __restrict__ loss, float* __restrict__ lse_out,
                                                                   int V, long long ld, int ignore_index,
                                                                   float label_smoothing, float logit_scale,
                                                                   float softcap, const float* __restrict__ gscale_ptr,
                                                                   float gscale_mul,
                                                                   const float* __restrict__ row_gscale,
                                                                   int write_grad) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  __nv_bfloat16* z = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f, zsum = 0.f;
  if (!ignored || write_grad) {
    if (!ignored) {
      for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
        float f[8];
        load8(z + i * 8, f);
        float lm = m;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] = ce_transform(f[e], logit_scale, softcap);
          lm = fmaxf(lm, f[e]);
          zsum += f[e];
        }
        float add = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) add += __expf(f[e] - lm);
        s = s * __expf(m - lm) + add;
        m = lm;
      }
      for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
        const float f = ce_transform(__bfloat162float(z[i]), logit_scale, softcap);
        const float lm = fmaxf(m, f);
        s = s * __expf(m - lm) + __expf(f - lm);
        m = lm;
        zsum += f;
      }
      const float gm = block_max(m, scratch);
      s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
      s = block_sum(s, scratch);
      zsum = block_sum(zsum, scratch);
      m = gm;
    }
  }
  const float lse = ignored ? 0.f : m + __logf(s);
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignored) {
      const float zl = ce_transform(__bfloat162float(z[label]), logit_scale, softcap);
      l = (1.f - label_smoothing) * (lse - zl) + label_smoothing * (lse - zsum / V);
    }
    loss[row] = l;
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();   // z[label] was read above before any thread overwrites it
  const float gs = ignored ? 0.f : (gscale_ptr ? gscale_ptr[0] : 1.f) * gscale_mul * (row_gscale ? row_gscale[row] : 1.f);
  const float sm_u = label_smoothing / V;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    load8(z + i * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int col = i * 8 + e;
      float g = 0.f;
      if (!ignored) {
        const float raw = f[e] * logit_scale;
        const float t = softcap > 0.f ? softcap * tanhf(raw / softcap) : raw;
        g = __expf(t - lse) - sm_u - ((col == label) ? (1.f - label_smoothing) : 0.f);
        if (softcap > 0.f) {
          const float th = t / softcap;
          g *= (1.f - th * th);
        }
        g *= logit_scale * gs;
      }
      f[e] = g;
    }
    store8(z + i * 8, f);
  }
  for (int col = (nvec << 3) + threadIdx.x; col < V; col += CE_THREADS) {
    float g = 0.f;
    if (!ignored) {
      const float raw = __bfloat162float(z[col]) * logit_scale;
      const float t = softcap > 0.f ? softcap * tanhf(raw / softcap) : raw;
      g = __expf(t - lse) - sm_u - ((col == label) ? (1.f - label_smoothing) : 0.f);
      if (softcap > 0.f) {
        const float th = t / softcap;
        g *= (1.f - th * th);
      }
      g *= logit_scale * gs;
    }
    z[col] = __float2bfloat16(g);
  }
}

// Per-row log-probability of the label token (DPO / SimPO / GRPO): logp[row] = z[label] - lse, 0 if ignored.
__global__ void __launch_bounds__(CE_THREADS) token_logprob_kernel(const __nv_bfloat16* __restrict__ logits,
                                                                   const long long* __restrict__ labels,
                                                                   float* __restrict__ logp, float* __restrict__ lse_out,
                                                                   int V, long long ld, int ignore_index) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* z = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V; i += CE_THREADS) {
    const float f = __bfloat162float(z[i]);
    const float lm = fmaxf(m, f);
    s = s * __expf(m - lm) + __expf(f - lm);
    m = lm;
  }
  const float gm = block_max(m, scratch);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) {
    const float lse = gm + __logf(s);
    if (lse_out) lse_out[row] = lse;
    logp[row] = ignored ? 0.f : __bfloat162float(z[label]) - lse;
  }
}

// ---------------------------------------------------------------------------------------------------
// Optimizer kernels
// ---------------------------------------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;   // bc = 1 - beta^step
  float grad_mul;                                         // static multiplier (e.g. 1 / accumulation steps)
};

// clip coefficient from a device-side squared norm: min(1, max_norm / (sqrt(sumsq) + 1e-6))
__device__ __forceinline__ float clip_coef(const float* sumsq, float max_norm) {
  if (!sumsq || max_norm <= 0.f) return 1.f;
  const float n = sqrtf(*sumsq);
  return fminf(1.f, max_norm / (n + 1e-6f));
}

// Flat AdamW over fp32 master weights: grads are bf16 or fp32, the bf16 working copy is refreshed.
template <typename GradT>
__global__ void adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                  const GradT* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16,
                                  long long n, AdamArgs a, const float* __restrict__ sumsq, float max_norm,
                                  const float* __restrict__ skip_flag) {
  if (skip_flag && *skip_flag != 0.f) return;   // non-finite loss / grads: leave the step out
  const float gm = a.grad_mul * clip_coef(sumsq, max_norm);
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 p = *reinterpret_cast<float4*>(master + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float g[4];
      if constexpr (sizeof(GradT) == 2) {
        const uint2 gr = *reinterpret_cast<const uint2*>(grad + i);
        const float2 g0 = unpack_bf16x2(gr.x), g1 = unpack_bf16x2(gr.y);
        g[0] = g0.x; g[1] = g0.y; g[2] = g1.x; g[3] = g1.y;
      } else {
        const float4 gr = *reinterpret_cast<const float4*>(grad + i);
        g[0] = gr.x; g[1] = gr.y; g[2] = gr.z; g[3] = gr.w;
      }
      float* pp = reinterpret_cast<float*>(&p);
      float* pm = reinterpret_cast<float*>(&mm);
      float* pv = reinterpret_cast<float*>(&vv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float ge = g[e] * gm;
        pm[e] = a.beta1 * pm[e] + (1.f - a.beta1) * ge;
        pv[e] = a.beta2 * pv[e] + (1.f - a.beta2) * ge * ge;
        const float mh = pm[e] / a.bc1, vh = pv[e] / a.bc2;
        pp[e] = pp[e] * (1.f - a.lr * a.weight_decay) - a.lr * mh / (sqrtf(vh) + a.eps);
      }
      *reinterpret_cast<float4*>(master + i) = p;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (param_bf16) {
        uint2 o;
        o.x = pack_bf16x2(pp[0], pp[1]);
        o.y = pack_bf16x2(pp[2], pp[3]);
        *reinterpret_cast<uint2*>(param_bf16 + i) = o;
      }
    } else {
      for (long long j = i; j < n; ++j) {
        float ge;
        if constexpr (sizeof(GradT) == 2) ge = __bfloat162float(grad[j]) * gm; else ge = grad[j] * gm;
        const float mj = a.beta1 * m[j] + (1.f - a.beta1) * ge;
        const float vj = a.beta2 * v[j] + (1.f - a.beta2) * ge * ge;
        m[j] = mj; v[j] = vj;
        const float pj = master[j] * (1.f - a.lr * a.weight_decay) - a.lr * (mj / a.bc1) / (sqrtf(vj / a.bc2) + a.eps);
        master[j] = pj;
        if (param_bf16) param_bf16[j] = __float2bfloat16(pj);
      }
    }
  }
}

// Multi-tensor AdamW: a table of tensors, each with its own weight decay; one launch for the whole model.
struct TensorEntry {
  float* master;
  float* m;
  float* v;
  const void* grad;
  __nv_bfloat16* param_bf16;
  long long n;
  float weight_decay;
  int grad_is_bf16;
};

__global__ void adamw_multi_kernel(const TensorEntry* __restrict__ table, const int* __restrict__ block_to_tensor,
                                   const int* __restrict__ block_to_chunk, int chunk, AdamArgs a,
                                   const float* __restrict__ sumsq, float max_norm,
                                   const float* __restrict__ skip_flag) {
  if (skip_flag && *skip_flag != 0.f) return;
  const TensorEntry t = table[block_to_tensor[blockIdx.x]];
  const long long start = static_cast<long long>(block_to_chunk[blockIdx.x]) * chunk;
  const long long end = min(start + chunk, t.n);
  const float gm = a.grad_mul * clip_coef(sumsq, max_norm);
  for (long long j = start + threadIdx.x; j < end; j += blockDim.x) {
    const float ge = (t.grad_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(t.grad)[j])
                                     : reinterpret_cast<const float*>(t.grad)[j]) * gm;
    const float mj = a.beta1 * t.m[j] + (1.f - a.beta1) * ge;
    const float vj = a.beta2 * t.v[j] + (1.f - a.beta2) * ge * ge;
    t.m[j] = mj;
    t.v[j] = vj;
    const float pj = t.master[j] * (1.f - a.lr * t.weight_decay) - a.lr * (mj / a.bc1) / (sqrtf(vj / a.bc2) + a.eps);
    t.master[j] = pj;
    if (t.param_bf16) t.param_bf16[j] = __float2bfloat16(pj);
  }
}

// Lion: p <- p(1 - lr wd) - lr sign(b1 m + (1-b1) g); m <- b2 m + (1-b2) g
template <typename GradT>
__global__ void lion_flat_kernel(float* __restrict__ master, float* __restrict__ m, const GradT* __restrict__ grad,
                                 __nv_bfloat16* __restrict__ param_bf16, long long n, float lr, float b1, float b2,
                                 float wd, float grad_mul) {
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[j]) * grad_mul; else g = grad[j] * grad_mul;
    const float mj = m[j];
    const float u = b1 * mj + (1.f - b1) * g;
    const float sgn = (u > 0.f) ? 1.f : ((u < 0.f) ? -1.f : 0.f);
    const float pj = master[j] * (1.f - lr * wd) - lr * sgn;
    master[j] = pj;
    m[j] = b2 * mj + (1.f - b2) * g;
    if (param_bf16) param_bf16[j] = __float2bfloat16(pj);
  }
}

// sum of squares accumulated into out[0] (fp32 atomics; one atomic per CTA); flags non-finite values.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out,
                             float* __restrict__ nonfinite_flag, float mul) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(x[j]); else f = x[j];
    f *= mul;
    s += f * f;
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(out, s);
    if (nonfinite_flag && !isfinite(s)) *nonfinite_flag = 1.f;
  }
}

// dst (+)= src * mul with dtype conversion (gradient accumulate / cast helper)
template <typename D, typename S>
__global__ void scale_cast_kernel(D* __restrict__ dst, const S* __restrict__ src, long long n, float mul,
                                  int accumulate) {
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f;
    if constexpr (sizeof(S) == 2) f = __bfloat162float(src[j]); else f = src[j];
    f *= mul;
    if (accumulate) {
      if constexpr (sizeof(D) == 2) f += __bfloat162float(dst[j]); else f += dst[j];
    }
    if constexpr (sizeof(D) == 2) dst[j] = __float2bfloat16(f); else dst[j] = f;
  }
}

// Row softmax (fp32 math) for bf16 rows.
__global__ void __launch_bounds__(256) softmax_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                           __nv_bfloat16* __restrict__ y, int V) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, __bfloat162float(x[row * V + i]));
  m = block_max(m, scratch);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(__bfloat162float(x[row * V + i]) - m);
  s = block_sum(s, scratch);
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    y[row * V + i] = __float2bfloat16(__expf(__bfloat162float(x[row * V + i]) - m) / s);
}

static inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_elementwise)

using namespace ts;
typedef __nv_bfloat16 bf16;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int ts_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* res_out,
                              float* rstd, long long rows, int H, float eps, float w_offset, void* stream) {
  if (H % 8 != 0 || rows <= 0) return -10;
  if (H <= 4096) {
    long long blocks = (rows + 3) / 4;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
#define TS_RMS_WARP(VPL, RES)                                                                                     \
  rmsnorm_fwd_warp_kernel<VPL, RES><<<(unsigned)blocks, 128, 0, ST(stream)>>>(                                    \
      (const bf16*)x, (const bf16*)residual, (const bf16*)w, (bf16*)y, (bf16*)res_out, rstd, rows, H, eps, w_offset)
    if (H <= 2048) {
      if (residual) TS_RMS_WARP(8, true); else TS_RMS_WARP(8, false);
    } else {
      if (residual) TS_RMS_WARP(16, true); else TS_RMS_WARP(16, false);
    }
#undef TS_RMS_WARP
    return (int)cudaGetLastError();
  }
  rmsnorm_fwd_kernel<<<(unsigned)rows, NORM_THREADS, 0, ST(stream)>>>(
      (const bf16*)x, (const bf16*)residual, (const bf16*)w, (bf16*)y, (bf16*)res_out, rstd, H, eps, w_offset);
  return (int)cudaGetLastError();
}

// Number of fp32 partial rows the backward pass needs in `dw_partial` ([parts][H]).
extern "C" int ts_rmsnorm_bwd_parts(long long rows) {
  long long g = static_cast<long long>(sm_count()) * 4;
  if (g > rows) g = rows;
  return (int)g;
}

extern "C" int ts_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                              void* dx, float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate_dw,
                              long long rows, int H, float w_offset, void* stream) {
  // the kernels index rows with 32-bit integers
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAXV * 8 || rows <= 0 || rows > 2147483647LL) return -10;
  const int parts = ts_rmsnorm_bwd_parts(rows);
  if (H <= NORM_THREADS * 2 * 8)
    rmsnorm_bwd_kernel<2><<<parts, NORM_THREADS, 0, ST(stream)>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd,
                                                                  (const bf16*)dres, (bf16*)dx, dw_partial, (int)rows,
                                                                  H, w_offset);
  else
    rmsnorm_bwd_kernel<NORM_MAXV><<<parts, NORM_THREADS, 0, ST(stream)>>>((const bf16*)dy, (const bf16*)x,
                                                                          (const bf16*)w, rstd, (const bf16*)dres,
                                                                          (bf16*)dx, dw_partial, (int)rows, H, w_offset);
  rmsnorm_dw_reduce_kernel<<<(H + 255) / 256, 256, 0, ST(stream)>>>(dw_partial, dw_f32, (bf16*)dw_bf16, parts, H,
                                                                    accumulate_dw);
  return (int)cudaGetLastError();
}

extern "C" int ts_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long rows, int H, float eps, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAXV * 8 || rows <= 0) return -10;
  layernorm_fwd_kernel<<<(unsigned)rows, NORM_THREADS, 0, ST(stream)>>>((const bf16*)x, (const bf16*)w, (const bf16*)b,
                                                                         (bf16*)y, mean, rstd, H, eps);
  return (int)cudaGetLastError();
}

// partial: fp32 workspace of ts_rmsnorm_bwd_parts(rows) * 2 * H floats; dw / db: fp32 [H]
extern "C" int ts_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                void* dx, float* partial, float* dw, float* db, long long rows, int H, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAXV * 8 || rows <= 0 || rows > 2147483647LL) return -10;
  const int parts = ts_rmsnorm_bwd_parts(rows);
  layernorm_bwd_kernel<<<parts, NORM_THREADS, 0, ST(stream)>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, mean,
                                                               rstd, (bf16*)dx, partial, (int)rows, H);
  layernorm_dwdb_reduce_kernel<<<(H + 255) / 256, 256, 0, ST(stream)>>>(partial, dw, db, parts, H);
  return (int)cudaGetLastError();
}

extern "C" int ts_rope(void* x, const float* cos_t, const float* sin_t, const int* pos, long long rows,
                       int row_stride, int n_heads, int D, int seq, int offset, int interleaved, int backward,
                       void* stream) {
  if (D % 2 != 0 || rows <= 0) return -10;
  const float sign = backward ? -1.f : 1.f;
  const bool vec_ok = !interleaved && (D % 16 == 0) && (row_stride % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(cos_t) & 15u) == 0);
  if (vec_ok) {
    const long long total = rows * ((n_heads + ROPE_HPT - 1) / ROPE_HPT) * (D / 16);
    rope_half_vec_kernel<<<grid_for(total, 256, 16), 256, 0, ST(stream)>>>((bf16*)x, cos_t, sin_t, pos, rows,
                                                                           row_stride, n_heads, D, seq, offset, sign);
  } else {
    const long long total = rows * n_heads * (D / 2);
    rope_kernel<<<grid_for(total, 256, 16), 256, 0, ST(stream)>>>((bf16*)x, cos_t, sin_t, pos, rows, row_stride,
                                                                  n_heads, D, seq, offset, interleaved, sign);
  }
  return (int)cudaGetLastError();
}

extern "C" int ts_glu_fwd(const void* gate_up, void* out, long long rows, int I, int ld_in, int act, void* stream) {
  if (I % 8 != 0 || ld_in % 8 != 0) return -10;
  glu_fwd_kernel<<<grid_for(rows * (I / 8), 256, 16), 256, 0, ST(stream)>>>((const bf16*)gate_up, (bf16*)out, rows, I,
                                                                            ld_in, act);
  return (int)cudaGetLastError();
}
extern "C" int ts_glu_bwd(const void* dout, const void* gate_up, void* dgate_up, long long rows, int I, int ld,
                          int act, void* stream) {
  if (I % 8 != 0 || ld % 8 != 0) return -10;
  glu_bwd_kernel<<<grid_for(rows * (I / 8), 256, 16), 256, 0, ST(stream)>>>((const bf16*)dout, (const bf16*)gate_up,
                                                                            (bf16*)dgate_up, rows, I, ld, act);
  return (int)cudaGetLastError();
}

// act: 0 = SiLU, 1 = GELU (erf), 2 = GELU (tanh)
extern "C" int ts_act_fwd(const void* x, void* y, long long n, int act, void* stream) {
  if (n <= 0 || n % 8 != 0) return n == 0 ? 0 : -10;
  act_fwd_kernel<<<grid_for(n / 8, 256, 16), 256, 0, ST(stream)>>>((const bf16*)x, (bf16*)y, n, act);
  return (int)cudaGetLastError();
}
extern "C" int ts_act_bwd(const void* dy, const void* x, void* dx, long long n, int act, void* stream) {
  if (n <= 0 || n % 8 != 0) return n == 0 ? 0 : -10;
  act_bwd_kernel<<<grid_for(n / 8, 256, 16), 256, 0, ST(stream)>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, n, act);
  return (int)cudaGetLastError();
}

extern "C" int ts_cross_entropy(void* logits, const long long* labels, float* loss, float* lse, long long rows, int V,
                                long long ld, int ignore_index, float label_smoothing, float logit_scale,
                                float softcap, const float* gscale_ptr, float gscale_mul,
                                const float* row_gscale, int write_grad, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8 != 0 || (reinterpret_cast<uintptr_t>(logits) & 15u) != 0) return -10;
  cross_entropy_kernel<<<(unsigned)rows, CE_THREADS, 0, ST(stream)>>>((bf16*)logits, labels, loss, lse, V, ld,
                                                                      ignore_index, label_smoothing, logit_scale,
                                                                      softcap, gscale_ptr, gscale_mul, row_gscale, write_grad);
  return (int)cudaGetLastError();
}

extern "C" int ts_token_logprob(const void* logits, const long long* labels, float* logp, float* lse, long long rows,
                                int V, long long ld, int ignore_index, void* stream) {
  if (rows <= 0) return 0;
  token_logprob_kernel<<<(unsigned)rows, CE_THREADS, 0, ST(stream)>>>((const bf16*)logits, labels, logp, lse, V, ld,
                                                                      ignore_index);
  return (int)cudaGetLastError();
}

extern "C" int ts_adamw_flat(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_bf16,
                             long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                             int step, float grad_mul, const float* sumsq, float max_norm, const float* skip_flag,
                             void* stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_mul = grad_mul;
  const int grid = grid_for((n + 3) / 4, 256, 8);
  if (grad_is_bf16)
    adamw_flat_kernel<bf16><<<grid, 256, 0, ST(stream)>>>(master, m, v, (const bf16*)grad, (bf16*)param_bf16, n, a,
                                                          sumsq, max_norm, skip_flag);
  else
    adamw_flat_kernel<float><<<grid, 256, 0, ST(stream)>>>(master, m, v, (const float*)grad, (bf16*)param_bf16, n, a,
                                                           sumsq, max_norm, skip_flag);
  return (int)cudaGetLastError();
}

// `table`, `block_to_tensor`, `block_to_chunk` live in device memory (built once by the Python side).
extern "C" int ts_adamw_multi(const void* table, const int* block_to_tensor, const int* block_to_chunk, int n_blocks,
                              int chunk, float lr, float beta1, float beta2, float eps, int step, float grad_mul,
                              const float* sumsq, float max_norm, const float* skip_flag, void* stream) {
  if (n_blocks <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = 0.f;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_mul = grad_mul;
  adamw_multi_kernel<<<n_blocks, 256, 0, ST(stream)>>>((const TensorEntry*)table, block_to_tensor, block_to_chunk,
                                                       chunk, a, sumsq, max_norm, skip_flag);
  return (int)cudaGetLastError();
}
extern "C" int ts_tensor_entry_bytes() { return (int)sizeof(TensorEntry); }

extern "C" int ts_lion_flat(float* master, float* m, const void* grad, int grad_is_bf16, void* param_bf16, long long n,
                            float lr, float b1, float b2, float wd, float grad_mul, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, 256, 8);
  if (grad_is_bf16)
    lion_flat_kernel<bf16><<<grid, 256, 0, ST(stream)>>>(master, m, (const bf16*)grad, (bf16*)param_bf16, n, lr, b1,
                                                         b2, wd, grad_mul);
  else
    lion_flat_kernel<float><<<grid, 256, 0, ST(stream)>>>(master, m, (const float*)grad, (bf16*)param_bf16, n, lr, b1,
                                                          b2, wd, grad_mul);
  return (int)cudaGetLastError();
}

extern "C" int ts_sumsq(const void* x, int is_bf16, long long n, float* out, float* nonfinite_flag, float mul,
                        void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, 512, 4);
  if (is_bf16)
    sumsq_kernel<bf16><<<grid, 512, 0, ST(stream)>>>((const bf16*)x, n, out, nonfinite_flag, mul);
  else
    sumsq_kernel<float><<<grid, 512, 0, ST(stream)>>>((const float*)x, n, out, nonfinite_flag, mul);
  return (int)cudaGetLastError();
}

// kind: 0 = bf16<-bf16, 1 = fp32<-bf16, 2 = bf16<-fp32, 3 = fp32<-fp32
extern "C" int ts_scale_cast(void* dst, const void* src, long long n, float mul, int accumulate, int kind,
                             void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, 256, 16);
  switch (kind) {
    case 0: scale_cast_kernel<bf16, bf16><<<grid, 256, 0, ST(stream)>>>((bf16*)dst, (const bf16*)src, n, mul, accumulate); break;
    case 1: scale_cast_kernel<float, bf16><<<grid, 256, 0, ST(stream)>>>((float*)dst, (const bf16*)src, n, mul, accumulate); break;
    case 2: scale_cast_kernel<bf16, float><<<grid, 256, 0, ST(stream)>>>((bf16*)dst, (const float*)src, n, mul, accumulate); break;
    case 3: scale_cast_kernel<float, float><<<grid, 256, 0, ST(stream)>>>((float*)dst, (const float*)src, n, mul, accumulate); break;
    default: return -10;
  }
  return (int)cudaGetLastError();
}

extern "C" int ts_softmax_rows(const void* x, void* y, long long rows, int V, void* stream) {
  if (rows <= 0) return 0;
  softmax_rows_kernel<<<(unsigned)rows, 256, 0, ST(stream)>>>((const bf16*)x, (bf16*)y, V);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in no_alloc.h).
// ---------------------------------------------------------------------------------------------------
#include "no_alloc.h"

// Built-in workspace for the per-CTA partial sums of dw.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) float g_noalloc_dw_partial[TS_NOALLOC_MAX_PARTS * TS_NOALLOC_MAX_H];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// Device address of the workspace on the current device (looked up once per device, with that device current).
int noalloc_workspace(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -21;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dw_partial);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return -22;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int ts_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                      void* dx, float* dw_f32, void* dw_bf16, int accumulate_dw, long long rows, int H,
                                      float w_offset, void* stream) {
  if (rows <= 0 || rows > 2147483647LL || H <= 0 || H % 8 != 0 || H > TS_NOALLOC_MAX_H) {
    fprintf(stderr,
            "[trainscale_b200] ts_rmsnorm_bwd_noalloc: rows=%lld H=%d rejected (need 0 < rows < 2^31, H %% 8 == 0, "
            "H <= %d: the built-in workspace holds %d x %d floats)\n",
            rows, H, TS_NOALLOC_MAX_H, TS_NOALLOC_MAX_PARTS, TS_NOALLOC_MAX_H);
    return -20;
  }
  float* workspace = nullptr;
  const int rc = noalloc_workspace(&workspace);
  if (rc != 0) return rc;
  // one partial row per CTA, never more rows than the workspace holds
  const int parts = rows < TS_NOALLOC_MAX_PARTS ? (int)rows : TS_NOALLOC_MAX_PARTS;
  rmsnorm_bwd_kernel<NORM_MAXV><<<parts, NORM_THREADS, 0, ST(stream)>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd,
                                                             (const bf16*)dres, (bf16*)dx, workspace, (int)rows, H,
                                                             w_offset);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  // every CTA wrote its whole partial row above, so the reduction reads only values of this call
  rmsnorm_dw_reduce_kernel<<<(H + 255) / 256, 256, 0, ST(stream)>>>(workspace, dw_f32, (bf16*)dw_bf16, parts, H,
                                                                    accumulate_dw);
  return (int)cudaGetLastError();
}
