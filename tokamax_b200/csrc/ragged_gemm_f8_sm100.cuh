// Forward grouped GEMM with fp8-e4m3 weights consumed NATIVELY by the fp8 tensor cores:
//
//   out[m, n] = row_scale[m] * (sum_k (hi[m, k] + lo[m, k]) * q[g(m), k, n]) * scale[g(m), n]
//
// The weights q (e4m3, one fp32 scale per expert and output channel) go from HBM through
// TMA into shared memory and straight into tcgen05.mma.kind::f8f6f4 -- no expansion, no
// extra shared-memory traffic.  kind::f8f6f4 needs 8-bit activations as well, and one e4m3
// rounding of a bf16 activation (3 mantissa bits) would cost about 3 % relative error per
// term.  So a pre-pass splits every activation row into TWO e4m3 terms with a per-row scale,
//     a = row_scale * (hi + lo),   hi = e4m3(a / row_scale),  lo = e4m3(a / row_scale - hi),
// which keeps ~8 significant bits (the precision bf16 itself has), and the kernel issues two
// fp8 MMAs per block into the same fp32 accumulator.  fp8 MMAs run at twice the bf16 rate,
// so the tensor time equals the bf16 kernel's while weights cost half the HBM / L2 / smem
// bytes and nothing has to be converted in the main loop.
//
// Semantics: dequantise-then-dot of tokamax/_src/ops/ragged_dot/base.py:332 with the
// per-output-channel scheme of tokamax/_src/ops/experimental/gmm_v2/gmm_v2_test.py:44-105;
// the activation split is this kernel's own device (the reference's fp8 Blackwell kernel,
// pallas_mosaic_gpu_kernel_sm100_fp8_quant.py:258-1044, takes activations that are already
// fp8 QArrays).
//
// Short tiles (decode regime).  A tile holding few valid rows -- a small group, or the last
// tile of any group -- would spend a full 128-row MMA on mostly padding, and with many small
// groups that padding, not HBM, bounds the kernel.  Such a tile (valid rows <= swap_rows,
// single-CTA mode) is multiplied with the operands SWAPPED: the weights become the MMA's
// 128-row M operand (read M-major, exactly as they lie in shared memory) and the rows become
// its N operand -- the hi rows followed by the lo rows, 32 or 64 of each -- so one small MMA
// per 128 weight columns replaces two full ones and the tile turns HBM-bound on its weights.
// The accumulator then holds the tile transposed (TMEM lane = output column, hi and lo
// products side by side); the epilogue adds the two and stores column-per-lane.  Only as
// many 32-row boxes of the activation planes as the tile needs are loaded.
//
// Scratch (caller workspace): the two e4m3 planes [2][M, K] and the row scales float[M],
// written by split_rows_e4m3_kernel and read by the GEMM in the same stream.
#pragma once

#include <cuda_fp8.h>

#include "ragged_gemm_sm100.cuh"

namespace tkmx {

constexpr int kF8BlockK = 128;                          // contraction elements per ring stage
constexpr int kF8ATileBytes = kBlockM * kF8BlockK;      // one plane: 128 rows x 128 B = 16 KiB
constexpr int kF8Threads = 256;

__host__ __device__ constexpr int f8_stage_bytes(int block_n, bool pair) {
  return 2 * kF8ATileBytes + (pair ? block_n / 2 : block_n) * kF8BlockK;
}

constexpr int kF8QueueDepth = 8;  // tile numbers in flight between the producer and the other roles

struct F8SmemLayout {
  uint32_t bars, tmem_slot, abort_flag, queue, scales, row_start, tile_start, order, total;
};

__host__ __device__ inline F8SmemLayout make_f8_smem_layout(int block_n, bool pair, int num_stages,
                                                            int num_groups) {
  F8SmemLayout l;
  uint32_t off = static_cast<uint32_t>(num_stages) * f8_stage_bytes(block_n, pair);
  l.bars = off;
  off += (2u * num_stages + 4u + 2u * kF8QueueDepth) * 8u;
  l.tmem_slot = off;
  off += 4;
  l.abort_flag = off;
  off += 4;
  l.queue = off;                         // int32[kF8QueueDepth]: dynamically scheduled tile numbers
  off += 4u * kF8QueueDepth;
  off = (off + 15u) & ~15u;
  l.scales = off;                        // float[4 epilogue warps][2][block_n]: column scales, column biases
  off += 2u * 4u * block_n * 4u;
  l.row_start = off;
  off += 4u * (num_groups + 1);
  l.tile_start = off;
  off += 4u * (num_groups + 1);
  l.order = off;                         // int32[G]: visiting order of the groups
  off += 4u * (num_groups + 1);
  l.total = off;
  return l;
}

// Visiting order that mixes the two kinds of work.  Groups of at most `thr` rows are one
// short tile per column block: little tensor work, their weights streamed from HBM once
// (HBM-bound).  Larger groups reuse their weights from L2 across row tiles (tensor-bound).
// Visited in index order, a run of small groups leaves the tensor cores idle and a run of
// large ones leaves HBM idle; so the two lists are merged in proportion to their tile
// counts and the SMs hold both kinds of tile at any moment.  `large_first` instead puts all
// large groups before the small ones: with dynamic scheduling the cheap tiles then fill
// the tail and the CTAs finish together.  One warp; fills order[0..G)
// and tile_start[0..G] (prefix of row tiles by position); groups without tiles go last.
template <int kTileM>
__device__ __forceinline__ void scan_groups_mixed(const RaggedGemmParams& p, int* row_start, int* tile_start,
                                                  int* order, int lane, int thr, bool large_first) {
  scan_groups<kTileM, false>(p, row_start, tile_start, lane);
  __syncwarp();
  const int G = p.num_groups;
  auto rows_of = [&](int g) {
    return (g >= p.group_begin && g < p.group_end) ? row_start[g + 1] - row_start[g] : 0;
  };
  int big_tiles = 0, small_tiles = 0;
  for (int g = lane; g < G; g += 32) {
    const int rows = rows_of(g);
    const int tiles = (rows + kTileM - 1) / kTileM;
    if (rows > thr) big_tiles += tiles;
    else small_tiles += tiles;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    big_tiles += __shfl_xor_sync(0xffffffffu, big_tiles, d);
    small_tiles += __shfl_xor_sync(0xffffffffu, small_tiles, d);
  }
  if (lane == 0) {
    int ib = 0, is = 0, v = 0, run = 0;
    long long placed_big = 0, placed_small = 0;
    while (true) {
      while (ib < G && rows_of(ib) <= thr) ++ib;
      while (is < G && (rows_of(is) <= 0 || rows_of(is) > thr)) ++is;
      if (ib >= G && is >= G) break;
      const bool take_big =
          ib < G && (is >= G || large_first || placed_big * small_tiles <= placed_small * big_tiles);
      const int g = take_big ? ib : is;
      const int tiles = (rows_of(g) + kTileM - 1) / kTileM;
      order[v] = g;
      tile_start[v] = run;
      run += tiles;
      ++v;
      if (take_big) {
        placed_big += tiles;
        ++ib;
      } else {
        placed_small += tiles;
        ++is;
      }
    }
    for (int g = 0; g < G; ++g) {
      if (rows_of(g) <= 0) {
        order[v] = g;
        tile_start[v] = run;
        ++v;
      }
    }
    tile_start[G] = run;
  }
  __syncwarp();
}

// Smallest power of two >= amax / 448 (so that scaling is exact both ways and hi + lo is the
// plain truncation of the activation to two e4m3 terms), floored at 2^-100; 1 for a zero row.
__device__ __forceinline__ float split_row_scale(float amax) {
  if (!(amax > 0.f)) return 1.0f;
  const uint32_t u = (__float_as_uint(amax * (1.0f / 448.0f)) + 0x007FFFFFu) & 0x7F800000u;
  return fmaxf(__uint_as_float(u), 7.888609052210118e-31f);
}

// Eight bf16 -> eight hi and eight lo e4m3 bytes under the inverse row scale.
__device__ __forceinline__ void split8_e4m3(const uint4& v, float inv, uint2& out_hi, uint2& out_lo) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  uint16_t ph[4], pl[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = __bfloat1622float2(h[j]);
    f.x *= inv;
    f.y *= inv;
    const __nv_fp8x2_storage_t a8 = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
    const __half2_raw back = __nv_cvt_fp8x2_to_halfraw2(a8, __NV_E4M3);
    const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&back));
    ph[j] = a8;
    pl[j] = __nv_cvt_float2_to_fp8x2(make_float2(f.x - fb.x, f.y - fb.y), __NV_SATFINITE, __NV_E4M3);
  }
  out_hi = make_uint2(ph[0] | (uint32_t(ph[1]) << 16), ph[2] | (uint32_t(ph[3]) << 16));
  out_lo = make_uint2(pl[0] | (uint32_t(pl[1]) << 16), pl[2] | (uint32_t(pl[3]) << 16));
}

// Same split with the whole row held in registers: a lane keeps up to kVecs 16-byte pieces, so
// every load of a row is in flight at once and the row is read from memory exactly once.
// Serves k <= 256 * kVecs; one warp per row.
template <int kVecs>
__global__ void __launch_bounds__(256)
split_rows_e4m3_regs_kernel(const __nv_bfloat16* __restrict__ lhs, uint8_t* __restrict__ hi,
                            uint8_t* __restrict__ lo, float* __restrict__ row_scale,
                            int32_t* __restrict__ sched, int m, int k) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *sched = 0;  // tile counter of the GEMM that follows
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = k / 8;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < m; row += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(lhs + static_cast<size_t>(row) * k);
    uint4 v[kVecs];
#pragma unroll
    for (int i = 0; i < kVecs; ++i)
      v[i] = (i * 32 + lane < vecs) ? __ldg(src + i * 32 + lane) : make_uint4(0u, 0u, 0u, 0u);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const float s = split_row_scale(amax);
    const float inv = 1.0f / s;
    if (lane == 0) row_scale[row] = s;
    uint2* dhi = reinterpret_cast<uint2*>(hi + static_cast<size_t>(row) * k);
    uint2* dlo = reinterpret_cast<uint2*>(lo + static_cast<size_t>(row) * k);
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      if (i * 32 + lane < vecs) {
        uint2 oh, ol;
        split8_e4m3(v[i], inv, oh, ol);
        dhi[i * 32 + lane] = oh;
        dlo[i * 32 + lane] = ol;
      }
    }
  }
}

// int8 form of the split (weights stored as int8, multiplied by kind::i8 MMAs): the row scale
// is s = max|a| / 127, hi = rne(a / s), lo = rne((a / s - hi) * 254), so that
// a = s * (hi + lo / 254) to ~15 bits; both planes are int8 in [-127, 127].  One warp per row,
// kVecs 16-byte pieces per lane and pass; rows that fit one pass are read once.
constexpr float kS8LoSteps = 254.0f;
template <int kVecs>
__global__ void __launch_bounds__(256)
split_rows_s8_kernel(const __nv_bfloat16* __restrict__ lhs, uint8_t* __restrict__ hi,
                     uint8_t* __restrict__ lo, float* __restrict__ row_scale,
                     int32_t* __restrict__ sched, int m, int k) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *sched = 0;  // tile counter of the GEMM that follows
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = k / 8;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < m; row += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(lhs + static_cast<size_t>(row) * k);
    float amax = 0.f;
    uint4 v[kVecs];
    for (int base = 0; base * 32 < vecs; base += kVecs) {
#pragma unroll
      for (int i = 0; i < kVecs; ++i) {
        const int at = (base + i) * 32 + lane;
        v[i] = at < vecs ? __ldg(src + at) : make_uint4(0u, 0u, 0u, 0u);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const float s = amax > 0.f ? fmaxf(amax * (1.0f / 127.0f), 1e-30f) : 1.0f;
    const float inv = 1.0f / s;
    if (lane == 0) row_scale[row] = s;
    uint2* dhi = reinterpret_cast<uint2*>(hi + static_cast<size_t>(row) * k);
    uint2* dlo = reinterpret_cast<uint2*>(lo + static_cast<size_t>(row) * k);
    const bool single_pass = vecs <= kVecs * 32;   // the row is still in registers
    for (int base = 0; base * 32 < vecs; base += kVecs) {
#pragma unroll
      for (int i = 0; i < kVecs; ++i) {
        const int at = (base + i) * 32 + lane;
        if (at >= vecs) continue;
        const uint4 x = single_pass ? v[i] : __ldg(src + at);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
        uint32_t ph[2] = {0u, 0u}, pl[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          const float q[2] = {f.x * inv, f.y * inv};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int ih = max(-127, min(127, static_cast<int>(rintf(q[e]))));
            const int il = max(-127, min(127, static_cast<int>(rintf((q[e] - static_cast<float>(ih)) * kS8LoSteps))));
            const int byte = (2 * j + e) & 3, word = (2 * j + e) >> 2;
            ph[word] |= (static_cast<uint32_t>(ih) & 0xFFu) << (8 * byte);
            pl[word] |= (static_cast<uint32_t>(il) & 0xFFu) << (8 * byte);
          }
        }
        dhi[at] = make_uint2(ph[0], ph[1]);
        dlo[at] = make_uint2(pl[0], pl[1]);
      }
    }
  }
}

// Workspace carve-up shared by host and device code.
struct F8Workspace {
  size_t plane_bytes;  // one e4m3 plane, padded to 256 B
  size_t scales_off;   // float[M]
  size_t sched_off;    // int32 tile counter (zeroed by the split pre-pass), 256 B slot
  size_t total;
};
__host__ __device__ inline F8Workspace f8_workspace(int64_t m, int64_t k) {
  F8Workspace w;
  w.plane_bytes = (static_cast<size_t>(m) * static_cast<size_t>(k) + 255) & ~static_cast<size_t>(255);
  w.scales_off = 2 * w.plane_bytes;
  w.sched_off = (w.scales_off + static_cast<size_t>(m) * sizeof(float) + 255) & ~static_cast<size_t>(255);
  w.total = w.sched_off + 256;
  return w;
}

// One warp per row: row_scale s = max|a| / 448 rounded up to a power of two,
// hi = e4m3(a / s), lo = e4m3(a / s - hi).
// k % 16 == 0; lhs rows and planes are 16-byte aligned.
__global__ void __launch_bounds__(256)
split_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ lhs, uint8_t* __restrict__ hi,
                       uint8_t* __restrict__ lo, float* __restrict__ row_scale, int32_t* __restrict__ sched,
                       int m, int k) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *sched = 0;  // tile counter of the GEMM that follows
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < m; row += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(lhs + static_cast<size_t>(row) * k);
    const int vecs = k / 8;  // 8 bf16 per 16 bytes
    float amax = 0.f;
    for (int i = lane; i < vecs; i += 32) {
      const uint4 v = __ldg(src + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const float s = split_row_scale(amax);
    const float inv = 1.0f / s;
    if (lane == 0) row_scale[row] = s;
    uint2* dhi = reinterpret_cast<uint2*>(hi + static_cast<size_t>(row) * k);
    uint2* dlo = reinterpret_cast<uint2*>(lo + static_cast<size_t>(row) * k);
    for (int i = lane; i < vecs; i += 32) {
      const uint4 v = __ldg(src + i);  // second read of the row hits L1 / L2
      uint2 oh, ol;
      split8_e4m3(v, inv, oh, ol);
      dhi[i] = oh;
      dlo[i] = ol;
    }
  }
}

// map_a8: e4m3 planes as a 3-D tensor {K, M, 2}, box {128, 128, 1}; map_a32: the same tensor
// with 32-row boxes (short tiles).
// map_b8: weights {N, K, G}, box {128, 64, 1}.
// kInt8: the same kernel for int8 weights and int8 activation planes (kind::i8, int32
// accumulation).  The hi and lo products cannot share an integer accumulator (they carry
// different weights, 1 and 1/254), so a full tile keeps two accumulators of kBlockN columns --
// all of tensor memory at kBlockN = 256, hence no second buffer: the epilogue of a tile does not
// overlap the next tile's MMAs -- and the epilogue combines them in float.
template <int kBlockN, bool kPair, bool kInt8 = false>
__global__ void __launch_bounds__(kF8Threads, 1)
ragged_gemm_f8_kernel(const __grid_constant__ CUtensorMap map_a8, const __grid_constant__ CUtensorMap map_a32,
                      const __grid_constant__ CUtensorMap map_b8, const RaggedGemmParams p,
                      const float* __restrict__ row_scale) {
  static_assert(kBlockN == 128 || kBlockN == 256, "unsupported BLOCK_N");
  constexpr uint32_t kAccBufs = kInt8 ? 1u : 2u;           // accumulator buffers of a tile in tensor memory
  constexpr float kLoWeight = kInt8 ? 1.0f / kS8LoSteps : 1.0f;   // weight of the lo product against the hi one
  auto acc_value = [](uint32_t bits) {
    return kInt8 ? static_cast<float>(static_cast<int32_t>(bits)) : __uint_as_float(bits);
  };
  auto issue_mma = [](uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    if constexpr (kInt8) ptx::umma_i8<kPair ? 2 : 1>(d, da, db, idesc, acc);
    else ptx::umma_f8<kPair ? 2 : 1>(d, da, db, idesc, acc);
  };
  constexpr int kCtas = kPair ? 2 : 1;
  constexpr int kTileM = kBlockM * kCtas;
  constexpr int kLocalN = kBlockN / kCtas;
  static_assert(kLocalN % 128 == 0, "each CTA loads whole 128-column boxes of 8-bit weights");
  constexpr int kNChunks = kLocalN / 128;                  // 128-column chunks of B per CTA
  constexpr int kBChunkBytes = kF8BlockK * 128;            // [128 k x 128 B] = 16 KiB (two TMA boxes)
  constexpr int kStageBytes = f8_stage_bytes(kBlockN, kPair);
  constexpr uint32_t kTxBytes = kStageBytes * kCtas;
  constexpr int kTmemCols = 2 * kBlockN;
  using Walker = TileWalker<kRowsBN, kBlockN, kTileM>;
  // Short-tile decision, the same in every role: rows present in the tile, and whether it is
  // multiplied with swapped operands (never in pair mode; zero-fill tiles have no MMA).
  // At most 64 rows: hi and lo rows stacked are then <= 128 accumulator columns per 128-column
  // chunk of weights, and the chunks of a tile fit its kBlockN TMEM columns.
  const int swap_rows = kPair ? 0 : min(p.swap_rows, 64);
  auto tile_valid = [](const Tile& t) { return min(t.row_end - t.row0, kBlockM); };
  // Gate/up epilogue (p.gateup, 256-column tiles): accumulator columns [0, 128) hold gate
  // columns c0 + a, columns [128, 256) the up columns cols/2 + c0 + (a - 128), c0 = t.col0 / 2;
  // the output has cols/2 columns.  acc_src maps an accumulator column to its weight column.
  const bool gateup = kBlockN == 256 && p.gateup != 0;
  const int half_cols = p.cols / 2;
  auto acc_src = [&](const Tile& t, int a) {
    return gateup ? (t.col0 / 2 + (a < 128 ? a : half_cols + a - 128)) : t.col0 + a;
  };
  auto acc_src_ok = [&](int a, int src) { return gateup ? (a < 128 ? src < half_cols : src < p.cols) : src < p.cols; };

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const int num_stages = p.num_stages;
  const F8SmemLayout L = make_f8_smem_layout(kBlockN, kPair, num_stages, p.num_groups);
  const uint32_t bar_full = base + L.bars;
  const uint32_t bar_empty = bar_full + 8u * num_stages;
  const uint32_t bar_acc_full = bar_empty + 8u * num_stages;
  const uint32_t bar_acc_empty = bar_acc_full + 16u;
  const uint32_t bar_q_full = bar_acc_empty + 16u;
  const uint32_t bar_q_empty = bar_q_full + 8u * kF8QueueDepth;
  volatile int* tile_q = reinterpret_cast<volatile int*>(base_ptr + L.queue);
  // Dynamic scheduling (single-CTA mode with a counter): the producer draws tile numbers from
  // a global counter and hands them to the MMA and epilogue warps through a small queue, so
  // CTAs that drew cheap tiles simply draw more.  Otherwise tiles are dealt round-robin.
  const bool dynamic = !kPair && p.sched_counter != nullptr;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L.tmem_slot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L.abort_flag);
  float* s_scales = reinterpret_cast<float*>(base_ptr + L.scales);
  int* row_start = reinterpret_cast<int*>(base_ptr + L.row_start);
  int* tile_start = reinterpret_cast<int*>(base_ptr + L.tile_start);
  int* order_buf = reinterpret_cast<int*>(base_ptr + L.order);
  // Mixed visiting order goes with the short-tile path (single-CTA mode, one rhs slab per group).
  const int* order = (swap_rows > 0 && p.mixed_order && p.rhs_groups == p.num_groups) ? order_buf : nullptr;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;
  const int unit = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int num_units = kPair ? (gridDim.x >> 1) : gridDim.x;

  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&map_a8);
    ptx::prefetch_tensormap(&map_a32);
    ptx::prefetch_tensormap(&map_b8);
    for (int s = 0; s < num_stages; ++s) {
      ptx::mbar_init(bar_full + 8u * s, kCtas);
      ptx::mbar_init(bar_empty + 8u * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_acc_full + 8u * b, 1);
      ptx::mbar_init(bar_acc_empty + 8u * b, 4 * kCtas);
    }
    for (int q = 0; q < kF8QueueDepth; ++q) {
      ptx::mbar_init(bar_q_full + 8u * q, 1);
      ptx::mbar_init(bar_q_empty + 8u * q, 5);   // the MMA lane and the four epilogue warps
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc<kCtas>(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish<kCtas>();
  }
  if (warp == 3) {
    if (order != nullptr)
      scan_groups_mixed<kTileM>(p, row_start, tile_start, order_buf, lane, swap_rows, p.mixed_order == 2);
    else scan_groups<kTileM, true>(p, row_start, tile_start, lane);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if constexpr (kPair) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (p.cdim + kF8BlockK - 1) / kF8BlockK;

  if (warp == 0) {
    if (lane == 0) {
      // ===== TMA producer =====
      Walker walk(p, row_start, tile_start, unit, num_units);
      walk.order = order;
      Tile t;
      RingPos pos;
      bool ok = true;
      // L2 prefetch cursor: runs p.prefetch_blocks weight blocks ahead of the loads along this
      // CTA's own tile sequence.  The ring alone keeps too few bytes in flight to cover DRAM
      // latency when every weight byte is used by one tile only (many small groups).
      Walker pf_walk(p, row_start, tile_start, unit, num_units);
      pf_walk.order = order;
      Tile pf_t;
      int pf_kb = 0;
      bool pf_live = false;
      auto pf_next_tile = [&]() {
        do {
          pf_live = pf_walk.get(pf_t);
        } while (pf_live && pf_t.num_kb == 0);
        pf_kb = 0;
      };
      auto prefetch_one = [&]() {
        if (!pf_live) return;
        const int pcol = acc_src(pf_t, static_cast<int>(cta_rank) * kLocalN);
        const int chunk_step = gateup ? half_cols : 128;
        const int pslab = pf_t.group % p.rhs_groups;
#pragma unroll
        for (int j = 0; j < kNChunks; ++j) {
          ptx::tma_prefetch_l2_3d(&map_b8, pcol + chunk_step * j, pf_kb * kF8BlockK, pslab);
          ptx::tma_prefetch_l2_3d(&map_b8, pcol + chunk_step * j, pf_kb * kF8BlockK + 64, pslab);
        }
        if (++pf_kb == num_kb) pf_next_tile();
      };
      if (p.prefetch_blocks > 0 && !dynamic) {
        pf_next_tile();
        for (int i = 0; i < p.prefetch_blocks; ++i) prefetch_one();
      }
      RingPos qpos;
      int pending = 0;       // tile number drawn ahead
      bool primed = false;
      while (ok) {
        if (dynamic) {
          if (!bounded_wait(bar_q_empty + 8u * qpos.slot, qpos.phase ^ 1u, abort_flag, p.status,
                            kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          // The draw for this tile was issued a tile ago; the next one is issued now and read
          // after this tile's loads, so its ~1 us round trip stays off the producer's path.
          if (!primed) {
            pending = atomicAdd(p.sched_counter, 1);
            primed = true;
          }
          int lin = pending;
          if (lin >= walk.total_tiles) lin = -1;   // end of work: tell the other roles and stop
          else pending = atomicAdd(p.sched_counter, 1);
          tile_q[qpos.slot] = lin;
          ptx::mbar_arrive(bar_q_full + 8u * qpos.slot);
          qpos.advance(kF8QueueDepth);
          if (lin < 0) break;
          walk.decode(lin, t);
        } else if (!walk.get(t)) {
          break;
        }
        if (t.num_kb == 0) continue;
        const int row0 = t.row0 + static_cast<int>(cta_rank) * kBlockM;
        const int col0 = acc_src(t, static_cast<int>(cta_rank) * kLocalN);   // this CTA's first B chunk
        const int chunk_step = gateup ? half_cols : 128;                    // source distance of its next chunk
        const int slab = t.group % p.rhs_groups;
        const int valid = tile_valid(t);
        const bool swapped = valid <= swap_rows;
        const int row_boxes = (valid + 31) >> 5;  // 32-row boxes per plane of a short tile
        for (int kb = 0; kb < num_kb; ++kb, pos.advance(num_stages)) {
          const uint32_t s = pos.slot;
          if (!bounded_wait(bar_empty + 8u * s, pos.phase ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + s * kStageBytes;      // hi plane, then lo plane
          const uint32_t sb = sa + 2 * kF8ATileBytes;
          const int k0 = kb * kF8BlockK;
          if constexpr (!kPair) {
            const uint32_t full = bar_full + 8u * s;
            if (swapped) {
              // hi rows, then the lo rows directly behind them: one stacked N operand.
              ptx::mbar_arrive_expect_tx(full, kLocalN * kF8BlockK + 2u * row_boxes * 4096u);
              for (int r = 0; r < row_boxes; ++r) {
                ptx::tma_load_3d(sa + r * 4096, &map_a32, k0, row0 + 32 * r, 0, full);
                ptx::tma_load_3d(sa + (row_boxes + r) * 4096, &map_a32, k0, row0 + 32 * r, 1, full);
              }
            } else {
              ptx::mbar_arrive_expect_tx(full, kTxBytes);
              ptx::tma_load_3d(sa, &map_a8, k0, row0, 0, full);
              ptx::tma_load_3d(sa + kF8ATileBytes, &map_a8, k0, row0, 1, full);
            }
#pragma unroll
            for (int j = 0; j < kNChunks; ++j) {
              ptx::tma_load_3d(sb + j * kBChunkBytes, &map_b8, col0 + chunk_step * j, k0, slab, full);
              ptx::tma_load_3d(sb + j * kBChunkBytes + kChunkBytes, &map_b8, col0 + chunk_step * j, k0 + 64, slab, full);
            }
          } else {
            const uint32_t full = ptx::map_to_cta(bar_full + 8u * s, 0);
            if (cta_rank == 0) ptx::mbar_arrive_expect_tx(bar_full + 8u * s, kTxBytes);
            ptx::tma_load_3d_pair(sa, &map_a8, k0, row0, 0, full);
            ptx::tma_load_3d_pair(sa + kF8ATileBytes, &map_a8, k0, row0, 1, full);
#pragma unroll
            for (int j = 0; j < kNChunks; ++j) {
              ptx::tma_load_3d_pair(sb + j * kBChunkBytes, &map_b8, col0 + chunk_step * j, k0, slab, full);
              ptx::tma_load_3d_pair(sb + j * kBChunkBytes + kChunkBytes, &map_b8, col0 + chunk_step * j, k0 + 64, slab, full);
            }
            if (cta_rank != 0) ptx::mbar_arrive_remote(full);
          }
          if (!dynamic) {
            prefetch_one();
          } else if (swapped && p.prefetch_blocks > 0 && kb + p.prefetch_blocks < num_kb) {
            // Dynamic scheduling: the tile sequence is not known ahead, so only a short
            // tile's own later weight blocks are requested into L2.
            const int pk = (kb + p.prefetch_blocks) * kF8BlockK;
#pragma unroll
            for (int j = 0; j < kNChunks; ++j) {
              ptx::tma_prefetch_l2_3d(&map_b8, col0 + chunk_step * j, pk, slab);
              ptx::tma_prefetch_l2_3d(&map_b8, col0 + chunk_step * j, pk + 64, slab);
            }
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {
      // ===== UMMA issuer: two e4m3 MMAs (hi plane, lo plane) per 32-deep slice =====
      Walker walk(p, row_start, tile_start, unit, num_units);
      walk.order = order;
      Tile t;
      uint32_t acc_cnt = 0;
      RingPos pos, qpos;
      bool ok = true;
      while (ok) {
        if (dynamic) {
          if (!bounded_wait(bar_q_full + 8u * qpos.slot, qpos.phase, abort_flag, p.status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          const int lin = tile_q[qpos.slot];
          ptx::mbar_arrive(bar_q_empty + 8u * qpos.slot);
          qpos.advance(kF8QueueDepth);
          if (lin < 0) break;
          walk.decode(lin, t);
        } else if (!walk.get(t)) {
          break;
        }
        if (t.num_kb == 0) continue;
        const uint32_t b = acc_cnt % kAccBufs;
        const uint32_t acc_ph = (acc_cnt / kAccBufs) & 1u;
        ++acc_cnt;
        if (!bounded_wait<kPair>(bar_acc_empty + 8u * b, acc_ph ^ 1u, abort_flag, p.status, kDevTimeoutMma)) {
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + b * kBlockN;
        const uint32_t tmem_d_lo = kInt8 ? tmem_d + kBlockN : tmem_d;   // the lo product's accumulator
        const int valid = tile_valid(t);
        const bool swapped = valid <= swap_rows;
        // Swapped: per 128-column chunk of the weights D[128 output columns x (hi rows | lo rows)];
        // M operand = weights (M-major), N operand = the tile's hi rows followed by its lo rows
        // (contraction-major), 32 * row_boxes of each.  One MMA covers both planes, because a
        // small-N MMA costs about the same whatever N is (its time goes into fetching the
        // 128-row M operand); the epilogue adds the two halves.
        const uint32_t stacked_n = static_cast<uint32_t>(((valid + 31) >> 5) * 64);
        const uint32_t idesc_swapped = kInt8 ? ptx::make_idesc_s8(1u, 0u, 128u, stacked_n)
                                             : ptx::make_idesc(0u, 0u, 1u, 0u, 128u, stacked_n);
        for (int kb = 0; kb < num_kb; ++kb, pos.advance(num_stages)) {
          const uint32_t s = pos.slot;
          if (!bounded_wait<kPair>(bar_full + 8u * s, pos.phase, abort_flag, p.status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + 2 * kF8ATileBytes;
          const uint64_t da_hi = ptx::make_smem_desc_sw128(sa, 16u, 1024u);
          const uint64_t da_lo = ptx::make_smem_desc_sw128(sa + kF8ATileBytes, 16u, 1024u);
          // B: 128-byte lines of 128 output columns; 8-line atoms 1 KiB apart along k,
          // 128-column chunks kBChunkBytes apart.
          const uint64_t db = ptx::make_smem_desc_sw128(sb, kBChunkBytes, 1024u);
          if (swapped) {
#pragma unroll
            for (int k = 0; k < kF8BlockK / 32; ++k) {
#pragma unroll
              for (int h = 0; h < kNChunks; ++h) {
                const uint64_t dwk = db + ((h * kBChunkBytes + k * 4096u) >> 4);
                issue_mma(tmem_d + h * 128, dwk, da_hi + ((k * 32u) >> 4), idesc_swapped, (kb | k) != 0 ? 1u : 0u);
              }
            }
          } else {
#pragma unroll
            for (int k = 0; k < kF8BlockK / 32; ++k) {
              const uint64_t dbk = db + ((k * 4096u) >> 4);
              issue_mma(tmem_d, da_hi + ((k * 32u) >> 4), dbk, p.idesc, (kb | k) != 0 ? 1u : 0u);
              issue_mma(tmem_d_lo, da_lo + ((k * 32u) >> 4), dbk, p.idesc, (kInt8 && (kb | k) == 0) ? 0u : 1u);
            }
          }
          if constexpr (kPair) ptx::umma_commit_pair(bar_empty + 8u * s, 3);
          else ptx::umma_commit(bar_empty + 8u * s);
        }
        if (ok) {
          if constexpr (kPair) ptx::umma_commit_pair(bar_acc_full + 8u * b, 3);
          else ptx::umma_commit(bar_acc_full + 8u * b);
        }
      }
    }
  } else if (warp >= 4) {
    // ===== epilogue: acc * row_scale[row] * col_scale[group][col] =====
    const int ew = warp - 4;
    float* sc = s_scales + ew * 2 * kBlockN;
    Walker walk(p, row_start, tile_start, unit, num_units);
    walk.order = order;
    Tile t;
    uint32_t acc_cnt = 0;
    bool ok = true;
    const int ld_out = gateup ? half_cols : p.cols;
    float* bi = sc + kBlockN;   // this warp's column biases (zeros without rhs_bias)
    RingPos qpos;
    while (ok) {
      if (dynamic) {
        if (!bounded_wait(bar_q_full + 8u * qpos.slot, qpos.phase, abort_flag, p.status, kDevTimeoutEpilogue)) {
          ok = false;
          break;
        }
        const int lin = tile_q[qpos.slot];
        __syncwarp();   // every lane has read the slot before it is handed back
        if (lane == 0) ptx::mbar_arrive(bar_q_empty + 8u * qpos.slot);
        qpos.advance(kF8QueueDepth);
        if (lin < 0) break;
        walk.decode(lin, t);
      } else if (!walk.get(t)) {
        break;
      }
      const int row = t.row0 + static_cast<int>(cta_rank) * kBlockM + ew * 32 + lane;
      const bool row_ok = row < t.row_end;
      const size_t out_row_off = static_cast<size_t>(row) * ld_out;
      const float rs = row_ok ? __ldg(row_scale + row) : 0.f;
      __syncwarp();
      for (int i = lane; i < kBlockN; i += 32) {
        const int col = acc_src(t, i);
        const bool col_ok = t.group >= 0 && acc_src_ok(i, col);
        const size_t at = static_cast<size_t>(t.group % p.rhs_groups) * p.cols + col;
        sc[i] = col_ok ? __ldg(p.col_scale + at) : 0.f;
        bi[i] = (col_ok && p.col_bias != nullptr) ? __ldg(p.col_bias + at) : 0.f;
      }
      __syncwarp();
      uint32_t b = 0;
      const bool has_acc = t.num_kb > 0;
      if (has_acc) {
        b = acc_cnt % kAccBufs;
        const uint32_t acc_ph = (acc_cnt / kAccBufs) & 1u;
        ++acc_cnt;
        if (!bounded_wait<kPair>(bar_acc_full + 8u * b, acc_ph, abort_flag, p.status, kDevTimeoutEpilogue)) {
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
      }
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + b * kBlockN;
      const int n_chunks = min(kBlockN / 32, (p.cols - t.col0 + 31) / 32);
      uint32_t va[32], vb[32];
      const int valid = tile_valid(t);
      if (has_acc && valid <= swap_rows) {
        // Transposed accumulator: this thread owns output column n of each 128-column chunk,
        // TMEM column r is tile row r.  Per row the warp writes 32 consecutive outputs.
        const int row_chunks = (valid + 31) >> 5;
        auto store_one = [&](float val, int r, int n) {
          const size_t off = static_cast<size_t>(t.row0 + r) * ld_out + n;
          if (p.out_is_f32) reinterpret_cast<float*>(p.out)[off] = val;
          else if (p.out_is_f16) reinterpret_cast<__half*>(p.out)[off] = __float2half_rn(val);
          else reinterpret_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16_rn(val);
        };
        if (gateup) {
          // Lanes of chunk 0 hold gate columns, the same lanes of chunk 1 the matching up columns.
          const int n = t.col0 / 2 + ew * 32 + lane;
          const bool n_ok = n < half_cols;
          const float cs_g = sc[ew * 32 + lane], cs_u = sc[128 + ew * 32 + lane];
          const float bs_g = bi[ew * 32 + lane], bs_u = bi[128 + ew * 32 + lane];
#pragma unroll 1
          for (int rc = 0; rc < row_chunks; ++rc) {
            uint32_t vg[32];
            ptx::tmem_ld_32x32b_x32(tmem_row + rc * 32, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + (row_chunks + rc) * 32, vb);
            const int my_r = rc * 32 + lane;
            const float my_rs = my_r < valid ? __ldg(row_scale + t.row0 + my_r) : 0.f;
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) vg[i] = __float_as_uint(acc_value(va[i]) + kLoWeight * acc_value(vb[i]));
            ptx::tmem_ld_32x32b_x32(tmem_row + 128 + rc * 32, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + 128 + (row_chunks + rc) * 32, vb);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float rsi = __shfl_sync(0xffffffffu, my_rs, i);
              vg[i] = __float_as_uint(__uint_as_float(vg[i]) * rsi * cs_g + bs_g);
              va[i] = __float_as_uint((acc_value(va[i]) + kLoWeight * acc_value(vb[i])) * rsi * cs_u + bs_u);
            }
            gateup_act32(p.gateup, vg, va);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int r = rc * 32 + i;
              if (r < valid && n_ok) store_one(__uint_as_float(vg[i]), r, n);
            }
          }
        } else {
#pragma unroll 1
          for (int h = 0; h < kNChunks; ++h) {
            const int n = t.col0 + h * 128 + ew * 32 + lane;
            const bool n_ok = n < p.cols;
            const float cs = sc[h * 128 + ew * 32 + lane];
            const float bs = bi[h * 128 + ew * 32 + lane];
#pragma unroll 1
            for (int rc = 0; rc < row_chunks; ++rc) {
              ptx::tmem_ld_32x32b_x32(tmem_row + h * 128 + rc * 32, va);                      // hi product
              ptx::tmem_ld_32x32b_x32(tmem_row + h * 128 + (row_chunks + rc) * 32, vb);       // lo product
              const int my_r = rc * 32 + lane;
              const float my_rs = my_r < valid ? __ldg(row_scale + t.row0 + my_r) : 0.f;
              ptx::tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float rsi = __shfl_sync(0xffffffffu, my_rs, i);
                const int r = rc * 32 + i;
                if (r < valid && n_ok)
                  store_one((acc_value(va[i]) + kLoWeight * acc_value(vb[i])) * rsi * cs + bs, r, n);
              }
            }
          }
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_acc_empty + 8u * b);
        continue;
      }
      if (gateup) {
        // act(gate) * up: gate chunk c in accumulator columns [32 c, 32 c + 32), its up chunk 128
        // columns further; 32 outputs per pair of loads at column t.col0 / 2 + 32 c.
        const int out_col0 = t.col0 / 2;
        const int g_chunks = min(4, (half_cols - out_col0 + 31) / 32);   // warp-uniform
#pragma unroll 1
        for (int c = 0; c < g_chunks; ++c) {
          if (has_acc) {
            ptx::tmem_ld_32x32b_x32(tmem_row + c * 32, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + 128 + c * 32, vb);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 sg = *reinterpret_cast<const float4*>(sc + c * 32 + i);
              const float4 su = *reinterpret_cast<const float4*>(sc + 128 + c * 32 + i);
              const float4 bg = *reinterpret_cast<const float4*>(bi + c * 32 + i);
              const float4 bu = *reinterpret_cast<const float4*>(bi + 128 + c * 32 + i);
              const float sgv[4] = {sg.x, sg.y, sg.z, sg.w}, suv[4] = {su.x, su.y, su.z, su.w};
              const float bgv[4] = {bg.x, bg.y, bg.z, bg.w}, buv[4] = {bu.x, bu.y, bu.z, bu.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                va[i + j] = __float_as_uint(__uint_as_float(va[i + j]) * rs * sgv[j] + bgv[j]);
                vb[i + j] = __float_as_uint(__uint_as_float(vb[i + j]) * rs * suv[j] + buv[j]);
              }
            }
            gateup_act32(p.gateup, va, vb);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) va[i] = 0u;
          }
          store_chunk(p, va, nullptr, row_ok, out_row_off, out_col0 + c * 32, half_cols);
        }
      } else {
      if (has_acc) {
        ptx::tmem_ld_32x32b_x32(tmem_row, va);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) va[i] = vb[i] = 0u;
      }
      // Rows of no group (zero-fill tiles) have zero scales and zero biases staged: they stay 0.
      auto scaled_store = [&](uint32_t (&v)[32], int c) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 s4 = *reinterpret_cast<const float4*>(sc + c * 32 + i);
          const float4 b4 = *reinterpret_cast<const float4*>(bi + c * 32 + i);
          v[i] = __float_as_uint(__uint_as_float(v[i]) * rs * s4.x + b4.x);
          v[i + 1] = __float_as_uint(__uint_as_float(v[i + 1]) * rs * s4.y + b4.y);
          v[i + 2] = __float_as_uint(__uint_as_float(v[i + 2]) * rs * s4.z + b4.z);
          v[i + 3] = __float_as_uint(__uint_as_float(v[i + 3]) * rs * s4.w + b4.w);
        }
        store_chunk(p, v, nullptr, row_ok, out_row_off, t.col0 + c * 32, p.cols);
      };
      if constexpr (kInt8) {
        // hi product in accumulator columns [0, kBlockN), lo product kBlockN columns further.
#pragma unroll 1
        for (int c = 0; c < n_chunks; ++c) {
          if (has_acc) {
            if (c > 0) ptx::tmem_ld_32x32b_x32(tmem_row + c * 32, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + kBlockN + c * 32, vb);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) va[i] = __float_as_uint(acc_value(va[i]) + kLoWeight * acc_value(vb[i]));
          } else if (c > 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i) va[i] = 0u;
          }
          scaled_store(va, c);
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < n_chunks; c += 2) {
        if (has_acc) {
          ptx::tmem_wait_ld();
          if (c + 1 < n_chunks) ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 32, vb);
        }
        scaled_store(va, c);
        if (c + 1 < n_chunks) {
          if (has_acc) {
            ptx::tmem_wait_ld();
            if (c + 2 < n_chunks) ptx::tmem_ld_32x32b_x32(tmem_row + (c + 2) * 32, va);
          }
          scaled_store(vb, c + 1);
        }
      }
      }
      }
      if (has_acc) {
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) ptx::mbar_arrive_remote(ptx::map_to_cta(bar_acc_empty + 8u * b, 0));
          else ptx::mbar_arrive(bar_acc_empty + 8u * b);
        }
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if constexpr (kPair) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 2) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

}  // namespace tkmx
