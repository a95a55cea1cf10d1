// Expert-parallel token dispatch and combine over peer-mapped (symmetric) memory on NVLink 5 / NVSwitch.
//
// Rank r owns experts [r * El, (r + 1) * El).  A mixture-of-experts layer moves every routed slot (token, choice j) to
// the owner of its expert, runs the owner's grouped GEMMs there and brings the result back.  Here both moves are single
// kernels that do the data-layout work and the transfer at once, with no staging buffer, no size exchange through the
// host and no host synchronisation:
//
//   ts_ep_counts_push    every rank stores its per-expert slot counts into row `rank` of a [W][E] table on every peer
//   ts_ep_plan           from the complete table each rank derives, on the device, (a) where each of its slots lands in
//                        the owners' receive buffers - segments per local expert start on 128-row boundaries, source
//                        ranks in rank order inside a segment, so the received rows are already in the layout the
//                        grouped tcgen05 GEMM reads - and (b) its own segment starts and tile -> expert map
//   ts_ep_push_rows      permute + scale + all-to-all in one kernel: a warp reads token row x[slot / k] and stores it
//                        (optionally scaled: the backward of the weighted combine) straight into the owner's receive
//                        buffer over NVLink
//   ts_ep_finalize       the receiver copies the rows it got into a private buffer (autograd keeps it) and zeroes the
//                        pad rows of every segment
//   ts_ep_copy_used      expert outputs -> the symmetric buffer peers read from (only the rows in use)
//   ts_ep_pull_combine   all-to-all + un-permute + weighted sum in one kernel: a warp pulls the k expert outputs of a
//                        token from their owners with peer loads and accumulates them in fp32 (optionally keeping the
//                        pulled rows for the gradient of the routing weights)
//
// The rendezvous between the steps is the flag barrier of comm.cu (ts_symm_barrier), launched on the same stream.
// Replaces the all_to_all_single pair with host-side split sizes of
// data_pipeline/trainer/distributed/expert_parallel.py:219-391 (AllToAllDispatcher.dispatch / combine).
// No kernel here waits on anything, no TMA and no cluster multicast is used.
#include "common.cuh"
#include "host_common.h"

namespace ts {

typedef __nv_bfloat16 bf16;
constexpr int EP_MAX_WORLD = 16;
constexpr int EP_MAX_EXPERTS = 1024;

struct EPPeers {
  void* ptr[EP_MAX_WORLD];
};

__global__ void ep_counts_push_kernel(EPPeers cnt, const int* __restrict__ counts, int rank, int world, int E) {
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int d = i / E, e = i - d * E;
    static_cast<int*>(cnt.ptr[d])[rank * E + e] = counts[e];
  }
}

// One block.  M[s][e]: slots rank s routes to global expert e.
//   send_base[e]   row in the receive buffer of e's owner where THIS rank's first slot for e lands
//   seg_start[El + 1], seg_real[El], tile_expert[max_tiles]   this rank's receive layout (as the grouped GEMM wants it)
// A layout that does not fit `cap_rows` on some rank sets *overflow (rows beyond the capacity are then dropped by the
// push and read as zero by the pull).
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int* __restrict__ M, int rank, int W, int E, int El,
                                                       int cap_rows, int* __restrict__ send_base,
                                                       int* __restrict__ seg_start, int* __restrict__ seg_real,
                                                       int* __restrict__ tile_expert, int max_tiles,
                                                       unsigned int* overflow) {
  __shared__ int tot[EP_MAX_EXPERTS], pre[EP_MAX_EXPERTS], start[EP_MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, p = 0;
    for (int s = 0; s < W; ++s) {
      const int c = M[s * E + e];
      if (s < rank) p += c;
      t += c;
    }
    tot[e] = t;
    pre[e] = p;
  }
  __syncthreads();
  if ((int)threadIdx.x < W) {   // one thread per owner rank: 128-aligned exclusive scan over its local experts
    const int d = threadIdx.x;
    int acc = 0;
    for (int l = 0; l < El; ++l) {
      start[d * El + l] = acc;
      acc += (tot[d * El + l] + 127) / 128 * 128;
    }
    if (acc > cap_rows && overflow) atomicExch(overflow, 1u);
    if (d == rank) seg_start[El] = acc < cap_rows ? acc : cap_rows;
  }
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) send_base[e] = start[e] + pre[e];
  for (int l = threadIdx.x; l < El; l += blockDim.x) {
    const int s0 = start[rank * El + l], real = tot[rank * El + l];
    seg_start[l] = s0 < cap_rows ? s0 : cap_rows;
    seg_real[l] = real;
    const int t1 = (s0 + (real + 127) / 128 * 128) / 128;
    for (int t = s0 / 128; t < t1 && t < max_tiles; ++t) tile_expert[t] = l;
  }
}

__device__ __forceinline__ uint4 scale_u4(const uint4& a, float sc) {
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
  uint4 o;
  o.x = pack_bf16x2(a0.x * sc, a0.y * sc);
  o.y = pack_bf16x2(a1.x * sc, a1.y * sc);
  o.z = pack_bf16x2(a2.x * sc, a2.y * sc);
  o.w = pack_bf16x2(a3.x * sc, a3.y * sc);
  return o;
}

// One warp per routed slot.  dst_row (optional) records the row for the pull on the way back.
__global__ void __launch_bounds__(256) ep_push_rows_kernel(EPPeers xbuf, const bf16* __restrict__ x,
                                                           const int* __restrict__ ids,
                                                           const int* __restrict__ rank_in_expert,
                                                           const int* __restrict__ send_base,
                                                           const float* __restrict__ scale, int* __restrict__ dst_row,
                                                           int n, int H, int k, int El, int cap_rows) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31, nv = H >> 3;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n; i += gridDim.x * wpb) {
    const int e = ids[i];
    const int row = send_base[e] + rank_in_expert[i];
    if (dst_row && lane == 0) dst_row[i] = row;
    if (row < 0 || row >= cap_rows) continue;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<bf16*>(xbuf.ptr[e / El]) + static_cast<size_t>(row) * H);
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(i / k) * H);
    if (scale == nullptr) {
      for (int v = lane; v < nv; v += 32) dst[v] = src[v];
    } else {
      const float sc = scale[i];
      for (int v = lane; v < nv; v += 32) dst[v] = scale_u4(src[v], sc);
    }
  }
}

// priv[r] = xbuf[r] for received rows, zero for the pad rows of a segment; rows past seg_start[El] are left alone
// (no tile of the grouped GEMM covers them).
__global__ void __launch_bounds__(256) ep_finalize_kernel(const bf16* __restrict__ xbuf, bf16* __restrict__ priv,
                                                          const int* __restrict__ seg_start,
                                                          const int* __restrict__ seg_real,
                                                          const int* __restrict__ tile_expert, int El, int P, int H) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31, nv = H >> 3;
  int used = seg_start[El];
  if (used > P) used = P;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < used; r += gridDim.x * wpb) {
    const int l = tile_expert[r >> 7];
    const bool real = l >= 0 && l < El && (r - seg_start[l]) < seg_real[l];
    uint4* dst = reinterpret_cast<uint4*>(priv + static_cast<size_t>(r) * H);
    if (real) {
      const uint4* src = reinterpret_cast<const uint4*>(xbuf + static_cast<size_t>(r) * H);
      for (int v = lane; v < nv; v += 32) dst[v] = src[v];
    } else {
      for (int v = lane; v < nv; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

__global__ void __launch_bounds__(256) ep_copy_used_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                           const int* __restrict__ used_rows, int P, int H) {
  int used = *used_rows;
  if (used > P) used = P;
  const long long nvec = static_cast<long long>(used) * (H >> 3);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

// One warp per token: out[t] = sum_j w[t*k+j] * ybuf_owner[dst_row[t*k+j]] (w == nullptr: plain sum), fp32 accumulation.
// ys (optional, [T*k][H]) keeps the pulled rows.
__global__ void __launch_bounds__(256) ep_pull_combine_kernel(EPPeers ybuf, const int* __restrict__ ids,
                                                              const int* __restrict__ dst_row,
                                                              const float* __restrict__ w, bf16* __restrict__ out,
                                                              bf16* __restrict__ ys, int T, int H, int k, int El,
                                                              int cap_rows) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31, nv = H >> 3;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    for (int v = lane; v < nv; v += 32) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int slot = t * k + j;
        const int row = dst_row[slot];
        uint4 a = make_uint4(0u, 0u, 0u, 0u);
        if (row >= 0 && row < cap_rows)
          a = reinterpret_cast<const uint4*>(static_cast<const bf16*>(ybuf.ptr[ids[slot] / El]) +
                                             static_cast<size_t>(row) * H)[v];
        if (ys) reinterpret_cast<uint4*>(ys + static_cast<size_t>(slot) * H)[v] = a;
        const float wj = w ? w[slot] : 1.f;
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

static inline bool fill_peers(EPPeers& p, const unsigned long long* ptrs, int world) {
  if (world < 1 || world > EP_MAX_WORLD || ptrs == nullptr) return false;
  for (int i = 0; i < EP_MAX_WORLD; ++i) p.ptr[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  for (int i = 0; i < world; ++i)
    if (p.ptr[i] == nullptr) return false;
  return true;
}

static inline int warp_grid(long long items) {
  long long blocks = (items + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_ep_comm)
using namespace ts;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// Rows of a receive buffer that can hold `n_total` routed slots spread over `El` local experts in any way.
extern "C" int ts_ep_padded_rows(long long n_total, int El) {
  const long long r = ((n_total + static_cast<long long>(El) * 127) + 127) / 128 * 128;
  return r > 2147483647LL ? -1 : static_cast<int>(r);
}

// cnt_ptrs: host array of `world` device addresses of the [world][E] int32 count table on every rank.
extern "C" int ts_ep_counts_push(const unsigned long long* cnt_ptrs, const int* counts, int rank, int world, int E,
                                 void* stream) {
  EPPeers p;
  if (!fill_peers(p, cnt_ptrs, world) || E <= 0 || E > EP_MAX_EXPERTS || rank < 0 || rank >= world) return -10;
  ep_counts_push_kernel<<<1, 256, 0, ST(stream)>>>(p, counts, rank, world, E);
  return (int)cudaGetLastError();
}

// table: this rank's [world][E] count table (complete: call after the barrier that follows ts_ep_counts_push).
// Outputs (device int32): send_base [E], seg_start [El + 1], seg_real [El], tile_expert [cap_rows / 128].
extern "C" int ts_ep_plan(const int* table, int rank, int world, int E, int cap_rows, int* send_base, int* seg_start,
                          int* seg_real, int* tile_expert, unsigned int* overflow, void* stream) {
  if (world < 1 || world > EP_MAX_WORLD || E <= 0 || E > EP_MAX_EXPERTS || E % world != 0 || cap_rows <= 0 ||
      cap_rows % 128 != 0 || rank < 0 || rank >= world)
    return -10;
  ep_plan_kernel<<<1, 1024, 0, ST(stream)>>>(table, rank, world, E, E / world, cap_rows, send_base, seg_start, seg_real,
                                             tile_expert, cap_rows / 128, overflow);
  return (int)cudaGetLastError();
}

// xbuf_ptrs: the [cap_rows][H] bf16 receive buffer on every rank.  x: [n / k][H] bf16 rows of this rank; ids,
// rank_in_expert: int32 [n]; scale: fp32 [n] or null; dst_row: int32 [n] output or null.
extern "C" int ts_ep_push_rows(const unsigned long long* xbuf_ptrs, const void* x, const int* ids,
                               const int* rank_in_expert, const int* send_base, const float* scale, int* dst_row, int n,
                               int H, int k, int El, int cap_rows, int world, void* stream) {
  EPPeers p;
  if (!fill_peers(p, xbuf_ptrs, world) || n <= 0 || H <= 0 || H % 8 != 0 || k <= 0 || El <= 0 || cap_rows <= 0)
    return -10;
  ep_push_rows_kernel<<<warp_grid(n), 256, 0, ST(stream)>>>(p, (const bf16*)x, ids, rank_in_expert, send_base, scale,
                                                            dst_row, n, H, k, El, cap_rows);
  return (int)cudaGetLastError();
}

extern "C" int ts_ep_finalize(const void* xbuf, void* priv, const int* seg_start, const int* seg_real,
                              const int* tile_expert, int El, int P, int H, void* stream) {
  if (El <= 0 || P <= 0 || P % 128 != 0 || H <= 0 || H % 8 != 0) return -10;
  ep_finalize_kernel<<<warp_grid(P), 256, 0, ST(stream)>>>((const bf16*)xbuf, (bf16*)priv, seg_start, seg_real,
                                                           tile_expert, El, P, H);
  return (int)cudaGetLastError();
}

// dst[0 : *used_rows] = src[0 : *used_rows] (rows of H bf16), *used_rows read on the device and clamped to P.
extern "C" int ts_ep_copy_used(const void* src, void* dst, const int* used_rows, int P, int H, void* stream) {
  if (P <= 0 || H <= 0 || H % 8 != 0) return -10;
  const long long nvec = static_cast<long long>(P) * (H >> 3);
  long long blocks = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  ep_copy_used_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>((const uint4*)src, (uint4*)dst, used_rows, P, H);
  return (int)cudaGetLastError();
}

// ybuf_ptrs: the [cap_rows][H] bf16 buffer of expert outputs on every rank.  out: [T][H]; ys: [T * k][H] or null.
extern "C" int ts_ep_pull_combine(const unsigned long long* ybuf_ptrs, const int* ids, const int* dst_row,
                                  const float* w, void* out, void* ys, int T, int H, int k, int El, int cap_rows,
                                  int world, void* stream) {
  EPPeers p;
  if (!fill_peers(p, ybuf_ptrs, world) || T <= 0 || H <= 0 || H % 8 != 0 || k <= 0 || El <= 0 || cap_rows <= 0)
    return -10;
  ep_pull_combine_kernel<<<warp_grid(T), 256, 0, ST(stream)>>>(p, ids, dst_row, w, (bf16*)out, (bf16*)ys, T, H, k, El,
                                                               cap_rows);
  return (int)cudaGetLastError();
}
