// Mixture-of-experts token plumbing around the grouped GEMM (gemm.cu, ts_gemm_grouped_bf16), all on the device and
// without a host round trip for the per-expert counts:
//   ts_moe_plan     expert ids -> stable rank inside the expert, 128-aligned segment starts, row maps, tile->expert map
//   ts_moe_permute  token rows -> expert-sorted padded buffer (pad rows zero), optionally scaled per source slot
//   ts_moe_combine  weighted gather of the k expert outputs of every token (also the backward of the permute)
//   ts_moe_combine_dw  gradient of the combine weights
// Replaces the permute / un-permute / top-k-weight kernels of data_pipeline/trainer/kernels/moe_kernels.py:219-785 and
// the host-side argsort + bincount of data_pipeline/trainer/distributed/expert_parallel.py:219.
#include "common.cuh"
#include "host_common.h"

namespace ts {

constexpr int MOE_THREADS = 256;

// grid = E.  Block e walks ids in order and gives the i-th occurrence of e rank i: a stable, deterministic order.
__global__ void __launch_bounds__(MOE_THREADS) moe_rank_kernel(const int* __restrict__ ids, int n, int* __restrict__ rank,
                                                               int* __restrict__ counts) {
  __shared__ int warp_tot[MOE_THREADS / 32];
  __shared__ int running_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) running_s = 0;
  __syncthreads();
  for (int base = 0; base < n; base += MOE_THREADS) {
    const int i = base + threadIdx.x;
    const bool hit = (i < n) && (ids[i] == e);
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    const int pre = __popc(m & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int woff = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < MOE_THREADS / 32; ++w) {
      if (w < warp) woff += warp_tot[w];
      tot += warp_tot[w];
    }
    const int run = running_s;
    if (hit) rank[i] = run + woff + pre;
    __syncthreads();
    if (threadIdx.x == 0) running_s = run + tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = running_s;
}

// one block: seg_start[e] = 128-aligned exclusive scan of counts; tile_expert[t] = expert owning rows [128t, 128t+128)
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ seg_start,
                                int* __restrict__ tile_expert, int max_tiles) {
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      seg_start[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    seg_start[E] = acc;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int t = seg_start[e] / 128; t < seg_start[e + 1] / 128 && t < max_tiles; ++t) tile_expert[t] = e;
}

__global__ void moe_dest_kernel(const int* __restrict__ ids, const int* __restrict__ rank,
                                const int* __restrict__ seg_start, int n, int* __restrict__ dest,
                                int* __restrict__ src_of_row) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = seg_start[ids[i]] + rank[i];
  dest[i] = d;
  src_of_row[d] = i;
}

// out[r] = scale * x[src / k] for rows with a source slot, zero for pad rows.  One warp per row, 16-byte vectors.
__global__ void moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_of_row,
                                   const float* __restrict__ slot_scale, __nv_bfloat16* __restrict__ out, int P, int H,
                                   int k) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < P; r += gridDim.x * warps_per_block) {
    const int src = src_of_row[r];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * H);
    if (src < 0) {
      for (int v = lane; v < H / 8; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(x + static_cast<size_t>(src / k) * H);
    if (slot_scale == nullptr) {
      for (int v = lane; v < H / 8; v += 32) dst[v] = s[v];
    } else {
      const float sc = slot_scale[src];
      for (int v = lane; v < H / 8; v += 32) {
        const uint4 a = s[v];
        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
        uint4 o;
        o.x = pack_bf16x2(a0.x * sc, a0.y * sc);
        o.y = pack_bf16x2(a1.x * sc, a1.y * sc);
        o.z = pack_bf16x2(a2.x * sc, a2.y * sc);
        o.w = pack_bf16x2(a3.x * sc, a3.y * sc);
        dst[v] = o;
      }
    }
  }
}

// out[t] = sum_j w[t*k + j] * y[dest[t*k + j]]  (w == nullptr: plain sum).  One warp per token, fp32 accumulation.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T, int H, int k) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    for (int v = lane; v < H / 8; v += 32) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int slot = t * k + j;
        const float wj = w ? w[slot] : 1.f;
        const uint4 a = reinterpret_cast<const uint4*>(y + static_cast<size_t>(dest[slot]) * H)[v];
        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
        acc[0] += wj * a0.x; acc[1] += wj * a0.y; acc[2] += wj * a1.x; acc[3] += wj * a1.y;
        acc[4] += wj * a2.x; acc[5] += wj * a2.y; acc[6] += wj * a3.x; acc[7] += wj * a3.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[v] = o;
    }
  }
}

// dw[slot] = <dout[slot / k], y[dest[slot]]>.  One warp per slot.
__global__ void moe_combine_dw_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                      const int* __restrict__ dest, float* __restrict__ dw, int n, int H, int k) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int slot = blockIdx.x * warps_per_block + (threadIdx.x >> 5); slot < n; slot += gridDim.x * warps_per_block) {
    const uint4* a = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(slot / k) * H);
    const uint4* b = reinterpret_cast<const uint4*>(y + static_cast<size_t>(dest[slot]) * H);
    float s = 0.f;
    for (int v = lane; v < H / 8; v += 32) {
      const uint4 av = a[v], bv = b[v];
      const float2 a0 = unpack_bf16x2(av.x), a1 = unpack_bf16x2(av.y), a2 = unpack_bf16x2(av.z), a3 = unpack_bf16x2(av.w);
      const float2 b0 = unpack_bf16x2(bv.x), b1 = unpack_bf16x2(bv.y), b2 = unpack_bf16x2(bv.z), b3 = unpack_bf16x2(bv.w);
      s += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
    }
    s = warp_sum(s);
    if (lane == 0) dw[slot] = s;
  }
}

// Router: softmax over E experts and top-k selection, one warp per token (E <= 1024).  probs [T][E] fp32 is written for
// the auxiliary losses and the backward; weights are the selected probabilities, optionally renormalised to sum to 1.
// Ties resolve to the lower expert index, as torch.topk does on equal values in practice for distinct logits.
constexpr int ROUTER_MAX_PER_LANE = 32;
__global__ void __launch_bounds__(128) moe_topk_softmax_kernel(const float* __restrict__ logits, float* __restrict__ probs,
                                                              float* __restrict__ weights, int* __restrict__ idx, int T,
                                                              int E, int k, int normalize) {
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) / 32;
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += gridDim.x * (blockDim.x >> 5)) {
    float v[ROUTER_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll 4
    for (int j = 0; j < per; ++j) {
      const int e = lane + j * 32;
      v[j] = e < E ? logits[static_cast<size_t>(t) * E + e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll 4
    for (int j = 0; j < per; ++j) {
      v[j] = (lane + j * 32 < E) ? __expf(v[j] - mx) : 0.f;
      sum += v[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll 4
    for (int j = 0; j < per; ++j) {
      v[j] *= inv;
      const int e = lane + j * 32;
      if (e < E) probs[static_cast<size_t>(t) * E + e] = v[j];
    }
    float wsum = 0.f;
    for (int s = 0; s < k; ++s) {
      // arg-max over what is left: (value, lowest index) reduced across the warp
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll 4
      for (int j = 0; j < per; ++j) {
        const int e = lane + j * 32;
        if (e < E && v[j] > best) {
          best = v[j];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if (lane == 0) {
        weights[static_cast<size_t>(t) * k + s] = best;
        idx[static_cast<size_t>(t) * k + s] = best_e;
      }
      wsum += best;
      if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;   // taken
    }
    if (normalize && lane < k) weights[static_cast<size_t>(t) * k + lane] /= fmaxf(wsum, 1e-9f);
  }
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_moe)
using namespace ts;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// Upper bound of padded rows for n routed slots over E experts (every segment rounded up to 128 rows).
extern "C" int ts_moe_padded_rows(int n, int E) { return ((n + E * 127) + 127) / 128 * 128; }

// ids: int32 [n].  Outputs (device int32): rank [n] (scratch), counts [E], seg_start [E + 1], tile_expert [P / 128],
// dest [n] (row of every slot in the padded buffer), src_of_row [P] (slot of every row, -1 for pad rows).
extern "C" int ts_moe_plan(const int* ids, int n, int E, int* rank, int* counts, int* seg_start, int* tile_expert,
                           int* dest, int* src_of_row, void* stream) {
  if (n <= 0 || E <= 0) return -10;
  const int P = ts_moe_padded_rows(n, E);
  cudaError_t e = cudaMemsetAsync(src_of_row, 0xff, sizeof(int) * static_cast<size_t>(P), ST(stream));
  if (e != cudaSuccess) return (int)e;
  moe_rank_kernel<<<E, MOE_THREADS, 0, ST(stream)>>>(ids, n, rank, counts);
  moe_plan_kernel<<<1, 256, 0, ST(stream)>>>(counts, E, seg_start, tile_expert, P / 128);
  moe_dest_kernel<<<(n + 255) / 256, 256, 0, ST(stream)>>>(ids, rank, seg_start, n, dest, src_of_row);
  return (int)cudaGetLastError();
}

static int row_grid(long long rows) {
  long long blocks = (rows + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return (int)(blocks < cap ? blocks : cap);
}

extern "C" int ts_moe_permute(const void* x, const int* src_of_row, const float* slot_scale, void* out, int P, int H,
                              int k, void* stream) {
  if (P <= 0 || H % 8 != 0 || k <= 0) return -10;
  moe_permute_kernel<<<row_grid(P), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, src_of_row, slot_scale,
                                                          (__nv_bfloat16*)out, P, H, k);
  return (int)cudaGetLastError();
}

extern "C" int ts_moe_combine(const void* y, const int* dest, const float* w, void* out, int T, int H, int k,
                              void* stream) {
  if (T <= 0 || H % 8 != 0 || k <= 0) return -10;
  moe_combine_kernel<<<row_grid(T), 256, 0, ST(stream)>>>((const __nv_bfloat16*)y, dest, w, (__nv_bfloat16*)out, T, H, k);
  return (int)cudaGetLastError();
}

extern "C" int ts_moe_combine_dw(const void* dout, const void* y, const int* dest, float* dw, int n, int H, int k,
                                 void* stream) {
  if (n <= 0 || H % 8 != 0 || k <= 0) return -10;
  moe_combine_dw_kernel<<<row_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, dest,
                                                             dw, n, H, k);
  return (int)cudaGetLastError();
}

// logits fp32 [T][E] -> probs fp32 [T][E], weights fp32 [T][k], idx int32 [T][k]
extern "C" int ts_moe_topk_softmax(const float* logits, float* probs, float* weights, int* idx, int T, int E, int k,
                                   int normalize, void* stream) {
  if (T <= 0 || E <= 0 || E > 32 * ROUTER_MAX_PER_LANE || k <= 0 || k > 32 || k > E) return -10;
  long long blocks = (T + 3) / 4;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  moe_topk_softmax_kernel<<<(unsigned)blocks, 128, 0, ST(stream)>>>(logits, probs, weights, idx, T, E, k, normalize);
  return (int)cudaGetLastError();
}
