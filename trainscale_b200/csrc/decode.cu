// Inference kernels: paged KV-cache writes and single-token (decode) attention over a paged cache with split-KV.
//
// Decode attention is bandwidth-bound (every K/V byte of the sequence is read once per step), so it runs on CUDA
// cores with 16-byte loads: one warp per cached token, lanes split the head dimension, the q heads of a GQA group
// share each K/V row.  Long sequences are split over CTAs (gridDim.z) and merged by LSE.
// Serves the role of the vLLM paged-attention kernels configured in the reference
// (data_pipeline/trainer/inference.py:786-921) and of data_pipeline/trainer/kernels/flex_attention.py:1032.
#include "common.cuh"
#include "host_common.h"

namespace ts {

// k_cache / v_cache: [num_blocks][block_size][Hkv][D] bf16.  slot = block * block_size + offset.
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride, int k_col0, int v_col0,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      const long long* __restrict__ slot_mapping, long long rows, int kv_width) {
  const int vec_per_row = kv_width >> 3;
  const long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / vec_per_row;
    const int v = static_cast<int>(idx - row * vec_per_row);
    const long long slot = slot_mapping[row];
    if (slot < 0) continue;
    const uint4 kk = *reinterpret_cast<const uint4*>(qkv + row * row_stride + k_col0 + v * 8);
    const uint4 vv = *reinterpret_cast<const uint4*>(qkv + row * row_stride + v_col0 + v * 8);
    *reinterpret_cast<uint4*>(k_cache + slot * kv_width + v * 8) = kk;
    *reinterpret_cast<uint4*>(v_cache + slot * kv_width + v * 8) = vv;
  }
}

constexpr int DEC_WARPS = 8;
constexpr int DEC_MAX_GROUP = 8;

// grid (num_seqs, Hkv, splits). Each CTA covers tokens [split*chunk, (split+1)*chunk) of one sequence for one kv head
// and all `group` q heads that share it. Writes partial out [seq][Hq][split][D] fp32 + lse [seq][Hq][split].
template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                        int max_blocks, const int* __restrict__ seq_lens, float* __restrict__ part_out,
                        float* __restrict__ part_lse, int Hq, int Hkv, int block_size, int chunk, int splits,
                        float scale) {
  constexpr int EPL = D / 32;   // elements per lane
  const int seq = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int group = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_lens[seq];
  const int t0 = split * chunk, t1 = min(len, t0 + chunk);
  __shared__ float s_acc[DEC_WARPS][DEC_MAX_GROUP][D];
  __shared__ float s_m[DEC_WARPS][DEC_MAX_GROUP], s_l[DEC_WARPS][DEC_MAX_GROUP];

  float qv[DEC_MAX_GROUP][EPL];
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) {
    if (g < group) {
      const __nv_bfloat16* qp = q + static_cast<size_t>(seq) * q_stride + (hk * group + g) * D + lane * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) qv[g][e] = __bfloat162float(qp[e]) * scale;
    }
  }
  float m[DEC_MAX_GROUP], l[DEC_MAX_GROUP], acc[DEC_MAX_GROUP][EPL];
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }
  const int kv_width = Hkv * D;
  for (int t = t0 + warp; t < t1; t += DEC_WARPS) {
    const int blk = block_table[seq * max_blocks + t / block_size];
    const size_t slot = static_cast<size_t>(blk) * block_size + (t % block_size);
    const __nv_bfloat16* kp = k_cache + slot * kv_width + hk * D + lane * EPL;
    const __nv_bfloat16* vp = v_cache + slot * kv_width + hk * D + lane * EPL;
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kf[e] = __bfloat162float(kp[e]);
      vf[e] = __bfloat162float(vp[e]);
    }
#pragma unroll
    for (int g = 0; g < DEC_MAX_GROUP; ++g) {
      if (g < group) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) s += qv[g][e] * kf[e];
        s = warp_sum(s);
        const float mn = fmaxf(m[g], s);
        const float a = __expf(m[g] - mn), p = __expf(s - mn);
        l[g] = l[g] * a + p;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * a + p * vf[e];
        m[g] = mn;
      }
    }
  }
  // merge the warps of this CTA
#pragma unroll
  for (int g = 0; g < DEC_MAX_GROUP; ++g) {
    if (g < group) {
      if (lane == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) s_acc[warp][g][lane * EPL + e] = acc[g][e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float mm = -INFINITY;
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, o = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float a = (s_m[w][g] == -INFINITY) ? 0.f : __expf(s_m[w][g] - mm);
      ll += s_l[w][g] * a;
      o += s_acc[w][g][d] * a;
    }
    const int h = hk * group + g;
    const size_t base = (static_cast<size_t>(seq) * Hq + h) * splits + split;
    part_out[base * D + d] = ll > 0.f ? o / ll : 0.f;
    if (d == 0) part_lse[base] = ll > 0.f ? mm + __logf(ll) : -INFINITY;
  }
}

template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ part_out, const float* __restrict__ part_lse,
                                    __nv_bfloat16* __restrict__ out, int out_stride, int Hq, int splits) {
  const int seq = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const size_t base = (static_cast<size_t>(seq) * Hq + h) * splits;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_lse[base + s]);
  float den = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float w = (part_lse[base + s] == -INFINITY) ? 0.f : __expf(part_lse[base + s] - mm);
    den += w;
    o += w * part_out[(base + s) * D + d];
  }
  out[static_cast<size_t>(seq) * out_stride + h * D + d] = __float2bfloat16(den > 0.f ? o / den : 0.f);
}

}  // namespace ts

TS_DEFINE_ERROR_API(ts_decode)
using namespace ts;

extern "C" int ts_kv_cache_write(const void* qkv, int row_stride, int k_col0, int v_col0, void* k_cache, void* v_cache,
                                 const long long* slot_mapping, long long rows, int kv_width, void* stream) {
  if (rows <= 0) return 0;
  if (kv_width % 8 != 0) return -10;
  long long blocks = (rows * (kv_width / 8) + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  kv_cache_write_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)qkv, row_stride, k_col0, v_col0, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
      slot_mapping, rows, kv_width);
  return (int)cudaGetLastError();
}

// part_out: fp32 [num_seqs][Hq][splits][D], part_lse: fp32 [num_seqs][Hq][splits] (caller-provided workspace);
// splits = ceil(max_len / chunk).
extern "C" int ts_decode_attention(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_table, int max_blocks, const int* seq_lens, void* out,
                                   int out_stride, float* part_out, float* part_lse, int num_seqs, int Hq, int Hkv,
                                   int D, int block_size, int chunk, int splits, float scale, void* stream) {
  if (num_seqs <= 0) return 0;
  if (Hq % Hkv != 0 || Hq / Hkv > DEC_MAX_GROUP || (D != 64 && D != 128)) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(num_seqs, Hkv, splits);
  if (D == 128) {
    decode_attention_kernel<128><<<grid, DEC_WARPS * 32, 0, st>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
        max_blocks, seq_lens, part_out, part_lse, Hq, Hkv, block_size, chunk, splits, scale);
    decode_merge_kernel<128><<<dim3(num_seqs, Hq), 128, 0, st>>>(part_out, part_lse, (__nv_bfloat16*)out, out_stride, Hq, splits);
  } else {
    decode_attention_kernel<64><<<grid, DEC_WARPS * 32, 0, st>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
        max_blocks, seq_lens, part_out, part_lse, Hq, Hkv, block_size, chunk, splits, scale);
    decode_merge_kernel<64><<<dim3(num_seqs, Hq), 64, 0, st>>>(part_out, part_lse, (__nv_bfloat16*)out, out_stride, Hq, splits);
  }
  return (int)cudaGetLastError();
}
