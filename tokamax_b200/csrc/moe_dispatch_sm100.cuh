// MoE dispatch / combine kernels around the grouped GEMM: the step either side of
// ragged_dot.  HBM-bound byte and index work (no tensor cores): coalesced 16-byte
// accesses, grids sized to cover the SMs.
//
//   sort_pairs   stable counting sort of (token, choice) pairs by expert id: for every pair
//                its position in expert-sorted order, plus the per-expert counts.
//                Deterministic (no atomics on positions), so the row order inside a group
//                -- and with it the summation order of drhs -- is reproducible.
//   gather_rows  dst[pos[p], :] = src[p / top_k, :]         (ragged_gather semantics,
//                tokamax/_src/ops/ragged_gather/base.py:26-30: x[indices])
//   combine      y[t, :] = sum_k gates[t, k] * rows[pos[t * top_k + k], :]
//                (ragged_gather_reduce, tokamax/_src/ops/ragged_gather_reduce/base.py:26-37)
//   ragged_gather / ragged_scatter   out[i, :] = x[indices[i], :], for ragged_scatter zero
//                unless start <= indices[i] < end (tokamax/_src/ops/ragged_gather/base.py:26-30,
//                tokamax/_src/ops/ragged_scatter/base.py:26-36)
//   ragged_gather_reduce   out[t, :] = sum_j mask[tR+j] ? w[tR+j] * x[indices[tR+j], :] : 0
//                (tokamax/_src/ops/ragged_gather_reduce/base.py:26-37)
//
// sort_pairs runs as three launches over fixed chunks of 1024 pairs:
//   1. per-chunk histogram            -> scratch[chunk][expert]
//   2. scan (one CTA)                 -> scratch[chunk][expert] = first position of that
//                                        chunk's pairs of that expert; counts[expert]
//   3. per-chunk ranking and scatter  -> pos[pair]
// The scratch is num_chunks * num_experts int32 of caller-provided workspace.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace tkmx {

constexpr int kSortChunk = 1024;        // pairs per CTA (one per thread)
constexpr int kSortMaxExperts = 1024;   // histogram lives in shared memory

// Rank of each thread's pair among the pairs of the same expert earlier in the chunk, and
// (in warp_hist[w][e]) how many pairs of expert e warp w holds.  Stable: lower thread index
// first.  `expert` is -1 for threads past the end.
__device__ __forceinline__ int chunk_rank(int expert, int num_experts, int* warp_hist /*[32][E]*/,
                                          int& rank_in_warp) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * num_experts; i += blockDim.x) warp_hist[i] = 0;
  __syncthreads();
  const unsigned peers = __match_any_sync(0xffffffffu, expert);
  rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (expert >= 0 && rank_in_warp == 0) warp_hist[warp * num_experts + expert] = __popc(peers);
  __syncthreads();
  return warp;
}

// 1. scratch[chunk][e] = number of pairs of expert e in the chunk.
__global__ void __launch_bounds__(kSortChunk)
moe_sort_hist_kernel(const int32_t* __restrict__ expert_ids, int num_pairs, int num_experts,
                     int32_t* __restrict__ scratch) {
  extern __shared__ int warp_hist[];
  const int p = blockIdx.x * kSortChunk + threadIdx.x;
  int e = p < num_pairs ? expert_ids[p] : -1;
  if (e >= num_experts) e = -1;  // out-of-range ids are dropped (their pos becomes -1)
  int rank_in_warp;
  chunk_rank(e, num_experts, warp_hist, rank_in_warp);
  for (int x = threadIdx.x; x < num_experts; x += blockDim.x) {
    int total = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) total += warp_hist[w * num_experts + x];
    scratch[blockIdx.x * num_experts + x] = total;
  }
}

// 2. One CTA: turn the histograms into first positions; emit per-expert counts.
__global__ void __launch_bounds__(1024)
moe_sort_scan_kernel(int32_t* __restrict__ scratch, int num_chunks, int num_experts,
                     int32_t* __restrict__ counts) {
  __shared__ int warp_sums[32];
  const int e = threadIdx.x;
  int total = 0;
  if (e < num_experts)
    for (int c = 0; c < num_chunks; ++c) total += scratch[c * num_experts + e];
  if (e < num_experts) counts[e] = total;
  // exclusive scan of `total` over experts (block-wide, 1024 threads)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = total;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += v;
    }
    warp_sums[lane] = w;  // inclusive
  }
  __syncthreads();
  const int base = incl - total + (warp > 0 ? warp_sums[warp - 1] : 0);
  if (e < num_experts) {
    int run = base;
    for (int c = 0; c < num_chunks; ++c) {
      const int h = scratch[c * num_experts + e];
      scratch[c * num_experts + e] = run;
      run += h;
    }
  }
}

// 3. pos[p] = first position of (chunk, expert) + stable rank inside the chunk; optionally also
//    sorted_pair[pos[p]] = p (which pair sits at each sorted position).
__global__ void __launch_bounds__(kSortChunk)
moe_sort_scatter_kernel(const int32_t* __restrict__ expert_ids, int num_pairs, int num_experts,
                        const int32_t* __restrict__ scratch, int32_t* __restrict__ pos,
                        int32_t* __restrict__ sorted_pair) {
  extern __shared__ int warp_hist[];
  const int p = blockIdx.x * kSortChunk + threadIdx.x;
  int e = p < num_pairs ? expert_ids[p] : -1;
  if (e >= num_experts) e = -1;
  int rank_in_warp;
  const int warp = chunk_rank(e, num_experts, warp_hist, rank_in_warp);
  // exclusive scan over warps, per expert (in place)
  for (int x = threadIdx.x; x < num_experts; x += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int h = warp_hist[w * num_experts + x];
      warp_hist[w * num_experts + x] = run;
      run += h;
    }
  }
  __syncthreads();
  if (p < num_pairs) {
    const int at = e < 0 ? -1
                         : scratch[blockIdx.x * num_experts + e] + warp_hist[warp * num_experts + e] + rank_in_warp;
    pos[p] = at;
    if (sorted_pair != nullptr && at >= 0) sorted_pair[at] = p;   // the inverse permutation
  }
}

// dst[pos[p], :] = src[p / top_k, :]; one warp per pair, 16-byte pieces.  row_bytes % 16 == 0.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ pos,
                       uint4* __restrict__ dst, int num_pairs, int top_k, int row_vec) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int p = blockIdx.x * warps_per_block + (threadIdx.x >> 5); p < num_pairs;
       p += gridDim.x * warps_per_block) {
    const int d = pos[p];
    if (d < 0) continue;
    const uint4* s = src + static_cast<size_t>(p / top_k) * row_vec;
    uint4* o = dst + static_cast<size_t>(d) * row_vec;
    for (int i = lane; i < row_vec; i += 32) o[i] = __ldg(s + i);
  }
}

// out[i, :] = x[indices[i], :] by 16-byte pieces, one warp per output row.  Indices follow
// array-indexing rules of the reference's `x[indices]`: negative values count from the end,
// anything still out of range is clamped.  With `bounds` (device int32 {start, end}) rows
// whose index is outside [start, end) are written as zeros (ragged_scatter).
__global__ void __launch_bounds__(256)
ragged_gather_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ indices,
                     const int32_t* __restrict__ start, const int32_t* __restrict__ end,
                     uint4* __restrict__ out, int in_rows, int out_rows, int row_vec) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool masked = start != nullptr;
  const int lo = masked ? __ldg(start) : 0, hi = masked ? __ldg(end) : 0;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < out_rows;
       i += gridDim.x * warps_per_block) {
    const int raw = __ldg(indices + i);
    uint4* o = out + static_cast<size_t>(i) * row_vec;
    if (masked && !(raw >= lo && raw < hi)) {
      for (int j = lane; j < row_vec; j += 32) o[j] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    int idx = raw < 0 ? raw + in_rows : raw;
    idx = min(max(idx, 0), in_rows - 1);
    const uint4* s = x + static_cast<size_t>(idx) * row_vec;
    for (int j = lane; j < row_vec; j += 32) o[j] = __ldg(s + j);
  }
}

// out[t, :] = sum_{j < R} (mask[tR + j] ? w[tR + j] * x[indices[tR + j], :] : 0), fp32
// accumulation in ascending j, bf16 rows.  One CTA per output row (grid-stride), each thread
// 8 consecutive columns.
__global__ void __launch_bounds__(256)
ragged_gather_reduce_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ indices,
                            const float* __restrict__ weights, const uint8_t* __restrict__ mask,
                            uint4* __restrict__ out, int in_rows, int out_rows, int group, int row_vec) {
  for (int t = blockIdx.x; t < out_rows; t += gridDim.x) {
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < group; ++j) {
        const int p = t * group + j;
        if (mask != nullptr && mask[p] == 0) continue;
        int idx = indices[p];
        idx = idx < 0 ? idx + in_rows : idx;
        idx = min(max(idx, 0), in_rows - 1);
        const float g = weights[p];
        const uint4 v = __ldg(x + static_cast<size_t>(idx) * row_vec + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(h[q]);
          acc[2 * q] += g * f.x;
          acc[2 * q + 1] += g * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      out[static_cast<size_t>(t) * row_vec + i] = o;
    }
  }
}

// y[t, :] = sum_k gates[t, k] * rows[pos[t * top_k + k], :] in fp32, k ascending; bf16 rows.
// One CTA per token (grid-stride), each thread 8 consecutive columns.  n % 8 == 0.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const uint4* __restrict__ rows, const int32_t* __restrict__ pos,
                   const float* __restrict__ gates, uint4* __restrict__ y, int num_tokens, int top_k,
                   int row_vec) {
  for (int t = blockIdx.x; t < num_tokens; t += gridDim.x) {
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < top_k; ++k) {
        const int d = pos[t * top_k + k];
        if (d < 0) continue;
        const float g = gates[t * top_k + k];
        const uint4 v = __ldg(rows + static_cast<size_t>(d) * row_vec + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += g * f.x;
          acc[2 * j + 1] += g * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      y[static_cast<size_t>(t) * row_vec + i] = o;
    }
  }
}

}  // namespace tkmx
