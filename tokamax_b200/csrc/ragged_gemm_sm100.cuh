// Persistent, warp-specialised grouped GEMM for sm_100a (B200).
//
// One kernel template covers the three contractions of ragged_dot:
//
//   kRowsBN  (forward, rhs stored [G, K, N])
//       out[m, n] = sum_k lhs[m, k] * rhs[g(m), k, n]
//       A = lhs  (contraction contiguous  -> "K-major" UMMA operand)
//       B = rhs  (output-column contiguous -> "MN-major" UMMA operand, no transpose)
//   kRowsBK  (dlhs, and forward with rhs stored [G, N, K])
//       out[m, j] = sum_c a[m, c] * b[g(m), j, c]
//       both operands contraction contiguous
//   kContract (drhs / "tgmm": the ragged dimension is the contraction)
//       out[g, k, n] = sum_{m in group g} lhs[m, k] * dout[m, n]
//       both operands MN-major; rows past the end of the group are zeroed in shared
//       memory before the MMA reads them.
//
// Reference behaviour being replaced: tokamax/_src/ops/ragged_dot/
// pallas_mosaic_gpu_kernel_sm100.py:38-269 (forward / dlhs) and
// pallas_mosaic_gpu_kernel_sm90.py:184-285 + pallas_triton.py:238-333 (drhs, which has
// no Blackwell kernel upstream).  The structure here is different: tokens are the MMA
// M operand, group bookkeeping is done inside the kernel from group_sizes (no
// pre-computed task arrays), tiles start exactly at the group's first row, and stores
// are row-predicated from registers.
//
// Pair mode (kPair): two CTAs of a cluster work on one 256-row tile with
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and HALF of the B tile
// (no multicast: every load is a plain per-CTA TMA load whose bytes are credited to the
// leader CTA's full barrier), the leader issues the MMAs for both, and each CTA drains its
// own 128 x N accumulator from its own TMEM.  This halves the B traffic per SM.
//
// CTA layout (256 threads, one CTA per SM, persistent):
//   warp 0      TMA producer (one elected lane)
//   warp 1      UMMA issuer  (one elected lane)
//   warp 2      TMEM allocator; in kContract also zeroes out-of-group rows of tail blocks
//   warp 3      group_sizes prefix scan at start-up
//   warps 4-7   epilogue: TMEM -> registers -> (scale) -> bf16/f32 -> global
//
// Pipelines (all mbarriers, every wait is bounded and reports through a status word):
//   full[s]/empty[s]       smem ring, TMA -> UMMA -> TMA
//   tail[s]                kContract only: the TMA loads of a group's last, partial block
//                          complete here instead of on full[s]; the fix-up warp zeroes the
//                          rows past the group's end and then arrives on full[s] itself, so
//                          the UMMA warp sees one uniform full[s] protocol
//   acc_full[b]/acc_empty[b]  two TMEM accumulators, UMMA -> epilogue -> UMMA
//   q_empty[i] + queue words  dynamic scheduling: tile numbers drawn by the leader's producer
//                          and handed to every role of the unit (see `dynamic` in the kernel)
//
// Epilogue variants (rows modes): plain (TMA stores for blocks inside one group, predicated
// stores otherwise), per-group column bias, fused gate/up activation (`gateup`), and the
// transposed store of short tiles that were multiplied with swapped operands (`kCanSwap`).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "ep_fused_sm100.cuh"
#include "ptx_sm100.cuh"

namespace tkmx {

enum GemmMode : int { kRowsBN = 0, kRowsBK = 1, kContract = 2 };

// Device status codes written (first one wins) when a bounded wait gives up.
enum DeviceStatus : int {
  kDevOk = 0,
  kDevTimeoutProducer = 1,
  kDevTimeoutMma = 2,
  kDevTimeoutEpilogue = 3,
  kDevTimeoutFixup = 4,
  // 5-7: expert-parallel waits and overflow (ep_fused_sm100.cuh)
  kDevSchedConflict = 8,   // another launch took this launch's tile-counter word while it was drawing
};

struct RaggedGemmParams {
  const int32_t* group_sizes;  // [G] on device; negative entries count as 0
  void* out;                   // rows mode: [M, cols]; contract mode: [G, rows, cols]
  const float* col_scale;      // optional per-(group, output column) scale [G, cols], or null
  const float* col_bias;       // optional per-(group, output column) bias [G, cols] added to the product, or null
  int32_t m_total;             // number of token rows M
  int32_t rows;                // rows mode: M ; contract mode: feature dim of lhs (K)
  int32_t cols;                // output columns
  int32_t cdim;                // rows mode: contraction length ; contract mode: unused
  int32_t num_groups;
  int32_t rhs_groups;          // rows modes: groups cycle over this many rhs slabs (group g uses g % rhs_groups)
  int32_t group_begin;         // rows modes: only groups in [group_begin, group_end) are computed;
  int32_t group_end;           //   the others keep their rows (offsets still count every group)
  int32_t out_is_f32;          // 0: bf16/f16 (16-bit, see out_is_f16), 1: float
  int32_t out_is_f16;          // 16-bit output flavour: 0 bf16, 1 f16
  int32_t out_vec_ok;          // 1: every output row starts 16-byte aligned (vector stores)
  int32_t skip_zero_fill;      // 1: leave rows past sum(group_sizes) untouched (zero_initialize=False)
  int32_t tma_store;           // 1: map_out is valid: blocks that are not ragged are stored by TMA
  uint32_t idesc;              // UMMA instruction descriptor
  int32_t tile_width;          // rasterisation band width (>= 1)
  int32_t minor_is_m;          // 1: row tiles vary fastest inside a band, 0: column tiles
  int32_t num_stages;          // smem ring depth
  int32_t gateup;              // kRowsBN: 0 = plain; else GateUpAct: out[:, j] = act(acc[:, j]) * acc[:, cols/2 + j]
  int32_t activation;          // rows modes: ElementAct applied to the float32 result (after scale and bias), 0 = none
  int32_t prefetch_blocks;     // fp8 kernel: weight blocks requested into L2 ahead of the smem ring (0: none)
  unsigned long long* sched_slot;  // 16-bit kernels: (epoch << 32 | next tile) word for dynamic scheduling, or null;
                                   //   the word after it counts the units that have finished drawing
  uint32_t sched_epoch;        //   this launch's epoch (never 0, differs from the slot's previous user)
  int32_t* sched_counter;      // fp8 kernel: zeroed tile counter for dynamic scheduling, or null (static)
  int32_t mixed_order;         // fp8 kernel visiting order: 0 = by index, 1 = small and large groups merged, 2 = large groups first
  int32_t swap_rows;           // tiles with at most this many rows swap the MMA operands (0: never); see kernels
  int32_t prefetch_cold_only;  // 1: `prefetch_blocks` applies only to groups that fit one row tile
  int32_t balance_tiles;       // 1: cut multi-tile groups into equal swapped tiles where possible (see TileWalker)
  float* out_scales;           // fused output quantisation: scales [M, cols / quant_sub], else null
  int32_t quant_sub;           // columns per output scale (64, 128 or 256; divides the tile width), 0 = off
  int32_t* status;             // device status word (see DeviceStatus)
};

constexpr int kBlockM = 128;        // UMMA M (token rows, or lhs features in contract mode)
constexpr int kBlockK = 64;         // contraction elements per ring stage (one 128 B swizzle row)
constexpr int kUmmaK = 16;          // contraction elements per tcgen05.mma (16-bit inputs)
constexpr int kNumThreads = 256;
constexpr int kEpNumThreads = 384;  // expert-parallel form: four more warps that only send rows
constexpr int kEpSendWarps = 6;     // warps 2, 3 and 8-11
constexpr int kATileBytes = kBlockM * kBlockK * 2;  // 16 KiB
constexpr int kChunkBytes = 64 * 128;               // one [64 x 128 B] TMA box
constexpr int kStagingBytes = 32 * 128;             // one epilogue warp's [32 rows x 64 bf16] block
constexpr uint64_t kWaitBudgetNs = 2000000000ull;   // 2 s per wait, then give up
constexpr int kQueueDepth = 8;                      // dynamically scheduled tile numbers in flight per CTA

// Bytes of one ring stage in one CTA: its 128-row A tile plus the B columns it loads
// (all of block_n, or half of it in pair mode).
__host__ __device__ constexpr int stage_bytes(int block_n, bool pair) {
  return kATileBytes + (pair ? block_n / 2 : block_n) * kBlockK * 2;
}

// Shared-memory carve-up after the ring (offsets from the 1024-aligned base).
struct SmemLayout {
  uint32_t ring;        // num_stages * stage_bytes
  uint32_t staging;     // 4 epilogue warps x [32 rows x 128 B] output staging for TMA stores
  uint32_t bars;        // mbarriers
  uint32_t queue;       // uint64[kQueueDepth]: (sequence << 32 | tile number) handed from the producer to the other roles
  uint32_t tmem_slot;   // uint32 written by tcgen05.alloc
  uint32_t abort_flag;  // int
  uint32_t row_start;   // int32[G + 1]
  uint32_t tile_start;  // int32[G + 1]  (rows modes only)
  uint32_t ep_vstart;   // int32[ep_experts + 1]: send-order prefix sums of the expert-parallel form
  uint32_t ep_need;     // int32[G]: multiplication progress a sender waits for before it sends an expert's rows
  uint32_t total;
};

__host__ __device__ inline SmemLayout make_smem_layout(int block_n, bool pair, int num_stages,
                                                       int num_groups, bool need_tile_start,
                                                       int ep_experts = 0) {
  SmemLayout l;
  l.ring = 0;
  uint32_t off = static_cast<uint32_t>(num_stages) * stage_bytes(block_n, pair);
  l.staging = off;                     // 1024-aligned: stage sizes are multiples of 1024
  off += 4u * kStagingBytes;
  l.bars = off;
  off += (3u * num_stages + 4u + kQueueDepth) * 8u;
  l.queue = off;                         // 8-byte aligned: follows the 8-byte barriers
  off += 8u * kQueueDepth;
  l.tmem_slot = off;
  off += 4;
  l.abort_flag = off;
  off += 4;
  off = (off + 15u) & ~15u;
  l.row_start = off;
  off += 4u * (num_groups + 1);
  l.tile_start = off;
  if (need_tile_start) off += 4u * (num_groups + 1);
  l.ep_vstart = off;
  if (ep_experts > 0) off += 4u * (ep_experts + 1);
  l.ep_need = off;
  if (ep_experts > 0) off += 4u * (num_groups + 1);
  l.total = off;
  return l;
}

// Bounded mbarrier wait.  Returns false after ~2 s (or if another role already gave
// up), having recorded `code` in the status word; the caller then leaves its loop.
// kClusterScope marks waits whose arrivals may come from the peer CTA of a pair.  They use
// the same plain try_wait: operand data becomes visible through the TMA transaction
// count and the tcgen05 fences, and a cluster-scope acquire on every k-block costs about
// a microsecond each (measured: it halved throughput).
template <bool kClusterScope = false>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             int32_t* status, int code) {
#ifdef TKMX_SPIN_TEST_WAIT
  auto probe = [&]() { return ptx::mbar_test_wait(bar, parity); };
#else
  auto probe = [&]() { return ptx::mbar_try_wait(bar, parity); };
#endif
  // Fast path: a short spin without touching the (slow to read) global timer.
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (probe()) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (!probe()) {
    if ((++spins & 0xFFu) == 0) {
      if (*abort_flag) return false;
      if (ptx::globaltimer_ns() - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Tile numbers of a launch come from a shared (epoch << 32 | count) word.  claim_word makes
// the word this launch's: the first CTA that finds another launch's epoch in it resets it
// (nothing is cleaned up at the end of a kernel, so an aborted launch cannot poison the next
// user of the word).  After that every draw is one atomicAdd, whose result the caller should
// not look at before it has other work out of the way (the round trip is ~1 us).
__device__ __forceinline__ void claim_word(unsigned long long* word, uint32_t epoch) {
  // word[1] (units finished, see finish_drawing) first: every unit leaves here having seen this
  // launch's epoch in it, so finish_drawing can count with one atomicAdd each.
#pragma unroll
  for (int w = 1; w >= 0; --w) {
    unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(word + w);
    while (static_cast<uint32_t>(old >> 32) != epoch) {
      const unsigned long long seen = atomicCAS(word + w, old, static_cast<unsigned long long>(epoch) << 32);
      if (seen == old) break;
      old = seen;
    }
  }
}
// Returns the whole (epoch << 32 | tile) word: the caller checks that the epoch is still its
// own.  Another epoch means a second launch was given the same word while this one was still
// drawing (more launches in flight than there are words, or a replayed graph beside eager
// launches); the tile numbers handed out since then cannot be trusted by either launch.
__device__ __forceinline__ unsigned long long draw_tile(unsigned long long* word) {
  return atomicAdd(word, 1ull);
}
// Called by a unit once it has drawn its end-of-work mark (it never draws again).  The last
// unit puts the count back to zero under the same epoch, so that a launch repeated with
// identical parameters (same word, same epoch) starts from tile 0 again.
__device__ __forceinline__ void finish_drawing(unsigned long long* word, uint32_t epoch, int num_units) {
  // word[1] = (epoch << 32 | units finished); claim_word put this launch's epoch there.  One
  // atomicAdd per unit: a compare-and-swap loop here cost tens of microseconds when all units
  // of a small problem finished together (each success made every other unit retry).
  const unsigned long long fresh = static_cast<unsigned long long>(epoch) << 32;
  const unsigned long long mine = atomicAdd(word + 1, 1ull) + 1ull;
  if (static_cast<uint32_t>(mine) == static_cast<uint32_t>(num_units)) {
    atomicExch(word + 1, fresh);
    __threadfence();
    atomicExch(word, fresh);
  }
}

// Position in the shared-memory ring: slot index and the parity of its current use.
struct RingPos {
  uint32_t slot = 0, phase = 0;
  __device__ __forceinline__ void advance(uint32_t num_stages) {
    if (++slot == num_stages) {
      slot = 0;
      phase ^= 1u;
    }
  }
  // Jump ahead by n slots (n may exceed num_stages).
  __device__ __forceinline__ void advance_by(uint32_t n, uint32_t num_stages) {
    const uint32_t total = slot + n;
    const uint32_t wraps = total / num_stages;
    slot = total - wraps * num_stages;
    phase ^= (wraps & 1u);
  }
};

struct Tile {
  int group;     // group index, or -1 for a zero-fill tile (rows past sum(group_sizes))
  int row0;      // first output row of the tile (rows modes: token row; contract: feature row)
  int row_end;   // one past the last output row the tile owns (its group's or the matrix's end at most)
  int col0;      // first output column
  int c_begin;   // contract mode: first token row of the group
  int c_end;     // contract mode: one past the last token row of the group
  int num_kb;    // contraction blocks (0: nothing to multiply, output is zeros)
};

// Walks the tile sequence assigned to this CTA.  Every role (producer, MMA, fix-up,
// epilogue) owns one of these and sees the same sequence.
// Visiting order of groups.  When the groups cycle over fewer rhs slabs (`rhs_groups`),
// i.e. group g uses slab g % rhs_groups, tiles are visited slab-major -- every group of
// slab 0, then every group of slab 1, ... -- so that a slab's weights are streamed from
// HBM once and reused from L2 by all the groups that share it.  The rows stay where they
// are; only the order in which tiles are handed out changes.
__host__ __device__ inline int visit_cycles(int num_groups, int rhs_groups) {
  return (rhs_groups > 0 && num_groups % rhs_groups == 0) ? num_groups / rhs_groups : 1;
}
__device__ __forceinline__ int visit_to_group(int v, int cycles, int rhs_groups) {
  return cycles == 1 ? v : (v % cycles) * rhs_groups + v / cycles;
}

// One warp: exclusive prefix sums of the clamped group sizes into row_start[0..G] (by
// group index) and, if kTiles, of the row tiles per group into tile_start[0..G] (by
// position in the visiting order).
template <int kTileM, bool kTiles>
__device__ __forceinline__ void scan_groups(const RaggedGemmParams& p, int* row_start, int* tile_start,
                                            int lane) {
  // Cumulative rows saturate at the matrix height, so that a bad group_sizes can neither index
  // past the matrix nor overflow: every term is <= m_total < 2^31 and sums are formed in
  // unsigned 32-bit arithmetic before they are clamped again.
  const uint32_t cap = static_cast<uint32_t>(p.m_total);
  uint32_t carry_rows = 0;
  for (int g0 = 0; g0 < p.num_groups; g0 += 32) {
    const int g = g0 + lane;
    const uint32_t sz = (g < p.num_groups) ? min(static_cast<uint32_t>(max(p.group_sizes[g], 0)), cap) : 0u;
    uint32_t incl = sz;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl = min(incl + v, cap);
    }
    const uint32_t before = __shfl_up_sync(0xffffffffu, incl, 1);
    if (g < p.num_groups) row_start[g] = static_cast<int>(min(carry_rows + (lane == 0 ? 0u : before), cap));
    carry_rows = min(carry_rows + __shfl_sync(0xffffffffu, incl, 31), cap);
  }
  if (lane == 0) row_start[p.num_groups] = static_cast<int>(carry_rows);
  __syncwarp();
  if constexpr (kTiles) {
    const int cycles = visit_cycles(p.num_groups, p.rhs_groups);
    int carry_tiles = 0;
    for (int v0 = 0; v0 < p.num_groups; v0 += 32) {
      const int v = v0 + lane;
      int tiles = 0;
      if (v < p.num_groups) {
        const int g = visit_to_group(v, cycles, p.rhs_groups);
        if (g >= p.group_begin && g < p.group_end)
          tiles = (row_start[g + 1] - row_start[g] + kTileM - 1) / kTileM;
      }
      int incl = tiles;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += u;
      }
      if (v < p.num_groups) tile_start[v] = carry_tiles + incl - tiles;
      carry_tiles += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) tile_start[p.num_groups] = carry_tiles;
  }
}

// kTileM: output rows per tile (128, or 256 when a CTA pair shares the tile).  `unit` /
// `num_units` identify the CTA (or pair) and how many of them share the tile sequence.
template <int kMode, int kBlockN, int kTileM>
struct TileWalker {
  const int* row_start;   // smem
  const int* tile_start;  // smem (rows modes)
  int num_groups, rows, cols, cdim, m_total;
  int n_tiles, tile_width, minor_is_m;
  int total_real, total_tiles;
  int next, stride;
  int cursor;  // rows modes: current position in the visiting order
  int group_begin = 0;  // contract mode: first group of the window that is computed
  int cycles, rhs_groups;
  const int* order = nullptr;  // rows modes: explicit visiting order (smem), or null for the cyclic rule
  // Rows modes with swapped short tiles (pair mode): a group that needs several row tiles is cut
  // into EQUAL tiles (rounded up to 16 rows) when those are short enough to run swapped, since
  // a swapped tile's MMA time follows its rows while a full tile costs the same however few of
  // its rows are valid: 272 rows are two tiles of 144 instead of 256 + 16.
  int balance_rows = 0;

  __device__ TileWalker(const RaggedGemmParams& p, const int* rs, const int* ts, int unit,
                        int num_units)
      : row_start(rs), tile_start(ts) {
    num_groups = p.num_groups;
    rows = p.rows;
    cols = p.cols;
    cdim = p.cdim;
    m_total = p.m_total;
    tile_width = p.tile_width;
    minor_is_m = p.minor_is_m;
    n_tiles = (cols + kBlockN - 1) / kBlockN;
    if constexpr (kMode == kContract) {
      const int r_tiles = (rows + kTileM - 1) / kTileM;
      group_begin = p.group_begin;
      total_real = (p.group_end - p.group_begin) * r_tiles * n_tiles;   // only the window's groups
      total_tiles = total_real;
    } else {
      total_real = tile_start[num_groups] * n_tiles;
      const int covered = row_start[num_groups];
      const int zero_m = p.skip_zero_fill ? 0 : (m_total - covered + kTileM - 1) / kTileM;
      total_tiles = total_real + zero_m * n_tiles;
    }
    next = unit;
    stride = num_units;
    cursor = 0;
    rhs_groups = p.rhs_groups;
    cycles = visit_cycles(p.num_groups, p.rhs_groups);
    if (kMode != kContract && kTileM == 2 * kBlockM && kBlockN == 256 && p.balance_tiles) balance_rows = p.swap_rows;
  }

  // Band rasterisation: the minor dimension is cut into bands `tile_width` wide; inside
  // a band the major dimension is the outer loop and odd bands run it backwards.
  __device__ __forceinline__ void raster(int local, int p_minor, int q_major, int& minor,
                                         int& major) const {
    const int band_elems = tile_width * q_major;
    const int band = local / band_elems;
    const int r = local - band * band_elems;
    const int bw = min(tile_width, p_minor - band * tile_width);
    major = r / bw;
    minor = band * tile_width + (r - major * bw);
    if (band & 1) major = q_major - 1 - major;
  }

  __device__ bool get(Tile& t) {
    if (next >= total_tiles) return false;
    const int lin = next;
    next += stride;
    decode(lin, t);
    return true;
  }

  // Tile number `lin` of the sequence (0 <= lin < total_tiles).  Successive calls on one
  // walker must pass increasing numbers (the rows-mode cursor only moves forward).
  __device__ bool decode(int lin, Tile& t) {
    if constexpr (kMode == kContract) {
      const int r_tiles = (rows + kTileM - 1) / kTileM;
      const int per_group = r_tiles * n_tiles;
      const int g_local = lin / per_group;
      const int g = group_begin + g_local;
      const int local = lin - g_local * per_group;
      int mi, ni;
      if (minor_is_m) raster(local, r_tiles, n_tiles, mi, ni);
      else raster(local, n_tiles, r_tiles, ni, mi);
      t.group = g;
      t.row0 = mi * kTileM;
      t.row_end = rows;
      t.col0 = ni * kBlockN;
      t.c_begin = row_start[g];
      t.c_end = row_start[g + 1];
      t.num_kb = (t.c_end - t.c_begin + kBlockK - 1) / kBlockK;
      return true;
    } else {
      if (lin >= total_real) {
        const int z = lin - total_real;
        const int zm = z / n_tiles;
        t.group = -1;
        t.row0 = row_start[num_groups] + zm * kTileM;
        t.row_end = m_total;
        t.col0 = (z - zm * n_tiles) * kBlockN;
        t.c_begin = t.c_end = 0;
        t.num_kb = 0;
        return true;
      }
      while (lin >= tile_start[cursor + 1] * n_tiles) ++cursor;
      const int g = order != nullptr ? order[cursor] : visit_to_group(cursor, cycles, rhs_groups);
      const int m_tiles = tile_start[cursor + 1] - tile_start[cursor];
      const int local = lin - tile_start[cursor] * n_tiles;
      int mi, ni;
      if (minor_is_m) raster(local, m_tiles, n_tiles, mi, ni);
      else raster(local, n_tiles, m_tiles, ni, mi);
      int tile_rows = kTileM;
      if (balance_rows > 0 && m_tiles > 1) {
        const int rows_g = row_start[g + 1] - row_start[g];
        const int even = ((rows_g + m_tiles - 1) / m_tiles + 15) & ~15;
        if (even <= balance_rows && (m_tiles - 1) * even < rows_g) tile_rows = even;
      }
      t.group = g;
      t.row0 = row_start[g] + mi * tile_rows;
      t.row_end = min(t.row0 + tile_rows, row_start[g + 1]);   // the tile's own end
      t.col0 = ni * kBlockN;
      t.c_begin = t.c_end = 0;
      t.num_kb = (cdim + kBlockK - 1) / kBlockK;
      return true;
    }
  }
};

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Fused gate/up activations: the weights hold the gate projection in their first cols/2
// columns and the up projection in the rest, and the output is act(gate) * up
// (`fuse_gateup_activation`, tokamax/_src/ops/ragged_dot/base.py:211-217; formulas of
// tokamax/_src/ops/experimental/gmm_v2/gmm_v2.py:29-48, 92-108).
enum GateUpAct : int {
  kGateUpNone = 0,
  kGateUpSilu = 1,
  kGateUpGelu = 2,           // tanh approximation, the default of the reference's gelu
  kGateUpSwigluOai = 3,
  kGateUpSiluClamp = 4,
};

// Elementwise activations fused on the float32 accumulator (`activation=` of ragged_dot,
// tokamax/_src/ops/ragged_dot/api.py:108-113: applied in the accumulator's dtype before the
// cast to the output dtype).
enum ElementAct : int {
  kActNone = 0,
  kActRelu = 1,
  kActSilu = 2,
  kActGeluTanh = 3,
  kActGeluErf = 4,
  kActTanh = 5,
  kActSigmoid = 6,
};

// Applied to 32 accumulator values held in registers.  The switch stands outside the
// loops: inlined per element, 32 copies of all six bodies made the epilogue code so large
// that even the path that applies nothing ran from instruction-cache misses (a swapped
// 128-row tile took 27 us instead of ~5).
__device__ __forceinline__ void element_act32(int kind, uint32_t (&v)[32]) {
#define TKMX_ACT_LOOP(expr)                                             \
  _Pragma("unroll") for (int i = 0; i < 32; ++i) {                      \
    const float x = __uint_as_float(v[i]);                              \
    v[i] = __float_as_uint(expr);                                       \
  }
  switch (kind) {
    case kActRelu: TKMX_ACT_LOOP(fmaxf(x, 0.f)) break;
    case kActSilu: TKMX_ACT_LOOP(x / (1.f + expf(-x))) break;
    case kActGeluTanh: TKMX_ACT_LOOP(0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)))) break;
    case kActGeluErf: TKMX_ACT_LOOP(0.5f * x * (1.f + erff(x * 0.7071067811865476f))) break;
    case kActTanh: TKMX_ACT_LOOP(tanhf(x)) break;
    case kActSigmoid: TKMX_ACT_LOOP(1.f / (1.f + expf(-x))) break;
    default: break;
  }
#undef TKMX_ACT_LOOP
}

__device__ __forceinline__ float gateup_act(int kind, float g, float u) {
  switch (kind) {
    case kGateUpSilu:
      return __fdividef(g, 1.f + __expf(-g)) * u;   // fast reciprocal: the epilogue is one warp per scheduler
    case kGateUpGelu: {
      const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
      return 0.5f * g * (1.f + t) * u;
    }
    case kGateUpSwigluOai: {
      g = fminf(g, 7.0f);
      u = fminf(fmaxf(u, -7.0f), 7.0f);
      return (u + 1.0f) * __fdividef(g, 1.f + __expf(-1.702f * g));
    }
    case kGateUpSiluClamp: {
      g = fminf(g, 10.0f);
      u = fminf(fmaxf(u, -10.0f), 10.0f);
      return __fdividef(g, 1.f + __expf(-g)) * u;
    }
  }
  return g;
}

// gateup_act over 32 (gate, up) pairs held in registers; the result replaces the gate values.
// The switch stands outside the loops for the reason given at element_act32.
__device__ __forceinline__ void gateup_act32(int kind, uint32_t (&g)[32], const uint32_t (&u)[32]) {
  switch (kind) {
    case kGateUpSilu:
#pragma unroll
      for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(gateup_act(kGateUpSilu, __uint_as_float(g[i]), __uint_as_float(u[i])));
      break;
    case kGateUpGelu:
#pragma unroll
      for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(gateup_act(kGateUpGelu, __uint_as_float(g[i]), __uint_as_float(u[i])));
      break;
    case kGateUpSwigluOai:
#pragma unroll
      for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(gateup_act(kGateUpSwigluOai, __uint_as_float(g[i]), __uint_as_float(u[i])));
      break;
    case kGateUpSiluClamp:
#pragma unroll
      for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(gateup_act(kGateUpSiluClamp, __uint_as_float(g[i]), __uint_as_float(u[i])));
      break;
    default: break;
  }
}

// Epilogue of one 32-column chunk held by one thread (its row): optional per-column
// scale, conversion to the output dtype, row- and column-predicated stores.  `ncols` is the
// width of the output matrix (p.cols unless the epilogue narrows it).
__device__ __forceinline__ void store_chunk(const RaggedGemmParams& p, uint32_t (&v)[32],
                                            const float* scale_row, bool row_ok, size_t out_row_off,
                                            int col, int ncols, const float* bias_row = nullptr) {
  if (scale_row != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float sc = (col + i < ncols) ? __ldg(scale_row + col + i) : 0.f;
      v[i] = __float_as_uint(__uint_as_float(v[i]) * sc);
    }
  }
  if (bias_row != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float b = (col + i < ncols) ? __ldg(bias_row + col + i) : 0.f;
      v[i] = __float_as_uint(__uint_as_float(v[i]) + b);
    }
  }
  if (p.activation != 0) element_act32(p.activation, v);
  if (!row_ok) return;
  if (p.out_is_f32) {
    float* dst = reinterpret_cast<float*>(p.out) + out_row_off + col;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      if (p.out_vec_ok && col + i + 4 <= ncols) {
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (col + i + j < ncols) dst[i + j] = __uint_as_float(v[i + j]);
      }
    }
  } else {
    uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + out_row_off + col;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(v[i + 2 * j]), hi = __uint_as_float(v[i + 2 * j + 1]);
        w[j] = p.out_is_f16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
      }
      if (p.out_vec_ok && col + i + 8 <= ncols) {
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col + i + j < ncols)
            dst[i + j] = static_cast<uint16_t>((w[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu);
      }
    }
  }
}

// kEp: the expert-parallel form (rows mode, rhs [G, K, N]).  A is this rank's receive buffer;
// warps 2 and 3 push this rank's token rows into the owners' receive buffers while the other
// warps multiply what has arrived (the producer waits on per-expert arrival counters), and the
// epilogue stores finished rows straight into the source ranks' return buffers (`p.out` unused).
template <int kMode, int kBlockN, bool kPair, bool kEp = false>
__global__ void __launch_bounds__(kEp ? kEpNumThreads : kNumThreads, 1)
ragged_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_out, const RaggedGemmParams p,
                   const __grid_constant__ EpFusedParams ep) {
  static_assert(kBlockN == 64 || kBlockN == 128 || kBlockN == 256, "unsupported BLOCK_N");
  static_assert(!kEp || kMode == kRowsBN, "the expert-parallel form is a forward over [G, K, N] weights");
  static_assert(!kPair || kBlockN >= 128, "pair mode splits B into two halves of >= 64 columns");
  constexpr int kCtas = kPair ? 2 : 1;
  constexpr int kTileM = kBlockM * kCtas;            // rows of one tile (whole pair)
  constexpr int kLocalN = kBlockN / kCtas;           // B columns this CTA loads
  constexpr int kStageBytes = stage_bytes(kBlockN, kPair);
  constexpr uint32_t kTxBytes = kStageBytes * kCtas; // bytes credited to full[s] per block
  constexpr int kTmemCols = 2 * kBlockN;             // two accumulators of kBlockN fp32 columns
  constexpr bool kAMn = (kMode == kContract);
  constexpr bool kBMn = (kMode != kRowsBK);
  constexpr uint32_t kAdvA = kAMn ? 2048u : 32u;  // start-address step per 16-element k slice
  constexpr uint32_t kAdvB = kBMn ? 2048u : 32u;
  using Walker = TileWalker<kMode, kBlockN, kTileM>;
  // Short tiles (pair mode, rows modes, 256-column tiles): a tile that holds few rows -- the
  // last tile of a group -- is multiplied with the operands swapped.  The pair's 256 weight
  // columns (128 per CTA, exactly as they already lie in shared memory) become the M operand
  // and the rows the N operand (rounded up to 16 only), so the MMA costs ~118 cycles instead
  // of ~173 for a full 256 x 256 one (measured; N <= 128), and the accumulator holds the tile
  // transposed (TMEM lane = output column).  Each CTA supplies half of the N operand's rows.
  constexpr bool kCanSwap = kPair && kMode != kContract && kBlockN == 256;
  const int swap_rows = kCanSwap ? p.swap_rows : 0;
  auto tile_valid = [](const Tile& t) { return min(t.row_end - t.row0, kTileM); };
  auto swapped_n = [](int valid) { return max(32, (valid + 15) & ~15); };

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const int num_stages = p.num_stages;
  const SmemLayout L = make_smem_layout(kBlockN, kPair, num_stages, p.num_groups, kMode != kContract,
                                        kEp ? ep.num_experts : 0);
  const uint32_t bar_full = base + L.bars;
  const uint32_t bar_empty = bar_full + 8u * num_stages;
  const uint32_t bar_tail = bar_empty + 8u * num_stages;
  const uint32_t bar_acc_full = bar_tail + 8u * num_stages;
  const uint32_t bar_acc_empty = bar_acc_full + 16u;
  const uint32_t bar_q_empty = bar_acc_empty + 16u;                // leader: every role of the unit read the slot
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L.tmem_slot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L.abort_flag);
  volatile unsigned long long* tile_q = reinterpret_cast<volatile unsigned long long*>(base_ptr + L.queue);
  int* row_start = reinterpret_cast<int*>(base_ptr + L.row_start);
  int* tile_start = reinterpret_cast<int*>(base_ptr + L.tile_start);
  int* ep_vstart = reinterpret_cast<int*>(base_ptr + L.ep_vstart);
  int* ep_need = reinterpret_cast<int*>(base_ptr + L.ep_need);
  const bool ep_multiply = !kEp || (ep.phases & 2) != 0;   // false: this launch only sends rows

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;   // 0 = leader
  const int unit = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int num_units = kPair ? (gridDim.x >> 1) : gridDim.x;
  // Dynamic scheduling: the leader's producer draws tile numbers from a global counter and
  // hands each to every other role of the unit (both CTAs of a pair) through kQueueDepth
  // slots, so units that drew cheap tiles draw more and all units stay close together in the
  // tile sequence (operands shared through L2).  Without a counter: static round-robin.
  // A slot is one 64-bit word (sequence << 32 | tile) written with a single store into each
  // CTA's shared memory; readers poll their own CTA's word until the sequence is the one
  // they expect.  Data and flag being one word, no cluster-scope acquire is needed (one per
  // tile and role measured ~1 us each and cost the short-tile drhs 10 %).
  const bool dynamic = p.sched_slot != nullptr;
  // Roles that read a queue slot: MMA (leader) or producer (peer), four epilogue warps, and
  // the fix-up warp in the contraction mode -- per CTA.
  constexpr uint32_t kQueueReaders = (5u + (kMode == kContract ? 1u : 0u)) * kCtas;
  // Reader side: next tile for this role.  1 = tile, 0 = end of work, -1 = gave up.
  // `seq` counts the tiles this role has taken; q is its position in the queue.
  auto next_tile = [&](Walker& w, Tile& t, RingPos& q, uint32_t& seq, int code, bool whole_warp) -> int {
    if (!dynamic) return w.get(t) ? 1 : 0;
    const uint32_t want = ++seq;
    unsigned long long v = 0;
    bool got = true;
    if (!whole_warp || lane == 0) {
      v = tile_q[q.slot];
      if (static_cast<uint32_t>(v >> 32) != want) {
        const uint64_t t0 = ptx::globaltimer_ns();
        uint32_t spins = 0;
        while (static_cast<uint32_t>((v = tile_q[q.slot]) >> 32) != want) {
          if ((++spins & 0xFFu) == 0) {
            if (*abort_flag) {
              got = false;
              break;
            }
            if (ptx::globaltimer_ns() - t0 > kWaitBudgetNs) {
              *abort_flag = 1;
              atomicCAS(p.status, 0, code);
              got = false;
              break;
            }
          }
        }
      }
      if (got) {
        if (kPair && cta_rank != 0) ptx::mbar_arrive_remote(ptx::map_to_cta(bar_q_empty + 8u * q.slot, 0));
        else ptx::mbar_arrive(bar_q_empty + 8u * q.slot);
      }
    }
    int lin = static_cast<int>(static_cast<uint32_t>(v));
    if (whole_warp) {
      lin = __shfl_sync(0xffffffffu, lin, 0);
      got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
    }
    if (!got) return -1;
    q.advance(kQueueDepth);
    if (lin < 0) return 0;
    w.decode(lin, t);
    return 1;
  };

  // ------------------------------------------------------------------ set-up
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    if (p.tma_store) ptx::prefetch_tensormap(&map_out);
    for (int s = 0; s < num_stages; ++s) {
      // Pair mode: full[s] (used in the leader only) takes two arrivals per block, one
      // from each CTA's producer (or fix-up warp for a tail block), plus the bytes of both.
      ptx::mbar_init(bar_full + 8u * s, kCtas);
      ptx::mbar_init(bar_empty + 8u * s, 1);
      ptx::mbar_init(bar_tail + 8u * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_acc_full + 8u * b, 1);
      ptx::mbar_init(bar_acc_empty + 8u * b, 4 * kCtas);  // one arrival per epilogue warp
    }
    for (int q = 0; q < kQueueDepth; ++q) {
      ptx::mbar_init(bar_q_empty + 8u * q, kQueueReaders);
      tile_q[q] = 0ull;
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc<kCtas>(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish<kCtas>();
  }
  if (warp == 3) scan_groups<kTileM, kMode != kContract>(p, row_start, tile_start, lane);
  if constexpr (kEp) {
    const EpPlanLayout pl = ep_plan_layout(ep.num_experts, ep.world);
    for (int i = threadIdx.x; i <= ep.num_experts; i += kEpNumThreads) ep_vstart[i] = __ldg(ep.plan + pl.vstart + i);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if constexpr (kPair) {
    // Both CTAs' barriers must exist before either signals the other.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if constexpr (kEp) {
    // Pacing of the senders: rows written long before they are multiplied fall out of L2 and
    // are read back from HBM, so an expert's rows are sent only once the multiplication has
    // come within `ahead_rows` rows of it.  ep_need[e] = the progress value (1 + index of the
    // furthest expert whose tiles have been started) at which expert e may be sent.
    if (warp == 3 && lane == 0) {
      int e0 = 0;
      for (int e = 0; e < p.num_groups; ++e) {
        while (e0 < e && row_start[e] - row_start[e0] > ep.ahead_rows) ++e0;
        ep_need[e] = ep.ahead_rows > 0 ? e0 : 0;
      }
    }
    __syncthreads();
  }

  // ------------------------------------------------------------------ roles
  if (warp == 0) {
    if (lane == 0 && ep_multiply) {
      // ===== TMA producer (runs in both CTAs of a pair, each for its own operands) =====
      int ep_ready_group = -1;   // kEp: last local expert whose rows were seen complete
      Walker walk(p, row_start, tile_start, unit, num_units);
      Tile t;
      uint32_t cnt = 0;  // ring slots filled so far
      RingPos pos, qpos;
      RingPos pub;               // leader: next queue slot to publish into
      int ahead = 0;             // leader: tiles published but not yet started by this producer
      uint32_t pub_seq = 0;      // leader: tiles published so far
      unsigned long long pending = 0;   // leader: (epoch << 32 | tile number) drawn ahead, not yet published
      bool claimed = false;      // leader: the counter word carries this launch's epoch
      uint32_t seq = 0;          // peer: tiles taken so far
      bool drained = false;      // leader: the end-of-work mark has been published
      bool ok = true;
      while (ok) {
        if (dynamic && cta_rank == 0) {
          // Leader: draw the unit's tiles kDrawAhead ahead of its own loads and publish each
          // to every role of the unit, so the peer CTA's producer (which learns a tile about
          // a microsecond after the leader) never starts a tile late.
          constexpr int kDrawAhead = 3;
          if (!claimed) {
            claim_word(p.sched_slot, p.sched_epoch);
            pending = draw_tile(p.sched_slot);
            claimed = true;
          }
          while (ok && !drained && ahead < kDrawAhead) {
            if (!bounded_wait<kPair>(bar_q_empty + 8u * pub.slot, pub.phase ^ 1u, abort_flag, p.status,
                                     kDevTimeoutProducer)) {
              ok = false;
              break;
            }
            // `pending` was drawn one publication ago: its atomic has had a whole tile's worth
            // of loads to come back.  The next draw is issued now and looked at next time.
            int lin = static_cast<int>(static_cast<uint32_t>(pending));
            if (static_cast<uint32_t>(pending >> 32) != p.sched_epoch) {
              // The word was taken over: stop this unit as at the end of work and report it.
              atomicCAS(p.status, 0, kDevSchedConflict);
              lin = -1;
            } else if (lin >= walk.total_tiles) {
              lin = -1;   // end of work
              finish_drawing(p.sched_slot, p.sched_epoch, num_units);
            } else {
              pending = draw_tile(p.sched_slot);
            }
            const unsigned long long word =
                (static_cast<unsigned long long>(++pub_seq) << 32) | static_cast<uint32_t>(lin);
            tile_q[pub.slot] = word;
            if constexpr (kPair) ptx::st_shared_cluster_u64(ptx::map_to_cta(base + L.queue + 8u * pub.slot, 1), word);
            pub.advance(kQueueDepth);
            ++ahead;
            drained = lin < 0;
          }
          if (!ok) break;
          const int lin = static_cast<int>(static_cast<uint32_t>(tile_q[qpos.slot]));   // own earlier write
          qpos.advance(kQueueDepth);
          --ahead;
          if (lin < 0) break;
          walk.decode(lin, t);
        } else {
          const int r = next_tile(walk, t, qpos, seq, kDevTimeoutProducer, false);
          if (r <= 0) {
            ok = r == 0;
            break;
          }
        }
        int row0 = t.row0 + static_cast<int>(cta_rank) * kBlockM;         // this CTA's A rows
        if constexpr (kCanSwap) {
          // Swapped tile: this CTA holds its half of the N operand's rows at the top of its A tile.
          if (t.group >= 0 && tile_valid(t) <= swap_rows)
            row0 = t.row0 + static_cast<int>(cta_rank) * (swapped_n(tile_valid(t)) / 2);
        }
        int col0 = t.col0 + static_cast<int>(cta_rank) * kLocalN;         // this CTA's B columns
        if constexpr (kMode == kRowsBN) {
          if (p.gateup) {
            // Accumulator columns [0, kBlockN/2) take gate columns c0.., the other half the up
            // columns cols/2 + c0.. (c0 = t.col0 / 2); a CTA's kLocalN columns lie in one half.
            const int a = static_cast<int>(cta_rank) * kLocalN;
            col0 = t.col0 / 2 + (a < kBlockN / 2 ? a : p.cols / 2 + a - kBlockN / 2);
          }
        }
        const int gateup_jump = (kMode == kRowsBN && p.gateup && kLocalN == kBlockN)
                                    ? p.cols / 2 - kBlockN / 2 : 0;  // extra offset of the up chunks
        const int slab = (kMode != kContract && t.group >= 0) ? t.group % p.rhs_groups : 0;
        if constexpr (kEp) {
          if (cta_rank == 0 && t.group >= 0 && t.group != ep_ready_group)
            atomicMax(ep.progress, static_cast<uint32_t>(t.group) + 1u);   // what the senders pace themselves on
          // The tile's rows come from every rank: wait until the expert's arrival counter has
          // reached its row count (tiles are visited in expert order, as the rows are sent).
          if (t.group >= 0 && t.group != ep_ready_group) {
            const uint32_t expected = static_cast<uint32_t>(row_start[t.group + 1] - row_start[t.group]);
            if (!ep_wait_expert(ep, t.group, expected, abort_flag, p.status, kWaitBudgetNs)) {
              ok = false;
              break;
            }
            ep_ready_group = t.group;
          }
        }
        // L2 prefetch of the weight blocks beyond the ring; with `prefetch_cold_only`, only for
        // groups of a single row tile, whose weights nobody has pulled into L2 before.
        int prefetch_blocks = p.prefetch_blocks;
        if (p.prefetch_cold_only && kMode != kContract && t.group >= 0 &&
            row_start[t.group + 1] - row_start[t.group] > kTileM)
          prefetch_blocks = 0;
        if constexpr (kPair && kMode == kRowsBN) {
          const int ahead = min(prefetch_blocks, t.num_kb);
          for (int kb = 0; kb < ahead; ++kb) {
#pragma unroll
            for (int j = 0; j < kLocalN / 64; ++j)
              ptx::tma_prefetch_l2_3d(&map_b, col0 + 64 * j, kb * kBlockK, slab);
          }
        }
        for (int kb = 0; kb < t.num_kb; ++kb, ++cnt, pos.advance(num_stages)) {
          const uint32_t s = pos.slot;
          const uint32_t ph = pos.phase;
          if (!bounded_wait(bar_empty + 8u * s, ph ^ 1u, abort_flag, p.status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kATileBytes;
          bool tail = false;
          if constexpr (kMode == kContract)
            tail = (kb == t.num_kb - 1) && (((t.c_end - t.c_begin) % kBlockK) != 0);
          if (tail) {
            // A group's last block with rows past the group's end lands on the local
            // tail[s]; the fix-up warp completes full[s] after zeroing those rows.
            const uint32_t bar = bar_tail + 8u * s;
            ptx::mbar_arrive_expect_tx(bar, kStageBytes);
            const int m0 = t.c_begin + kb * kBlockK;
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              ptx::tma_load_2d(sa + j * kChunkBytes, &map_a, row0 + 64 * j, m0, bar);
#pragma unroll
            for (int j = 0; j < kLocalN / 64; ++j)
              ptx::tma_load_2d(sb + j * kChunkBytes, &map_b, col0 + 64 * j, m0, bar);
            continue;
          }
          if constexpr (!kPair) {
            const uint32_t full = bar_full + 8u * s;
            ptx::mbar_arrive_expect_tx(full, kTxBytes);
            if constexpr (kMode == kContract) {
              const int m0 = t.c_begin + kb * kBlockK;
#pragma unroll
              for (int j = 0; j < kBlockM / 64; ++j)
                ptx::tma_load_2d(sa + j * kChunkBytes, &map_a, row0 + 64 * j, m0, full);
#pragma unroll
              for (int j = 0; j < kLocalN / 64; ++j)
                ptx::tma_load_2d(sb + j * kChunkBytes, &map_b, col0 + 64 * j, m0, full);
            } else {
              ptx::tma_load_2d(sa, &map_a, kb * kBlockK, row0, full);
              if constexpr (kMode == kRowsBN) {
#pragma unroll
                for (int j = 0; j < kLocalN / 64; ++j)
                  ptx::tma_load_3d(sb + j * kChunkBytes, &map_b,
                                   col0 + 64 * j + (64 * j >= kBlockN / 2 ? gateup_jump : 0), kb * kBlockK, slab, full);
              } else {
                ptx::tma_load_3d(sb, &map_b, kb * kBlockK, col0, slab, full);
              }
            }
          } else {
            // The bytes of both CTAs are credited to the leader's full[s].
            const uint32_t full = ptx::map_to_cta(bar_full + 8u * s, 0);
            if (cta_rank == 0) ptx::mbar_arrive_expect_tx(bar_full + 8u * s, kTxBytes);
            if constexpr (kMode == kContract) {
              const int m0 = t.c_begin + kb * kBlockK;
#pragma unroll
              for (int j = 0; j < kBlockM / 64; ++j)
                ptx::tma_load_2d_pair(sa + j * kChunkBytes, &map_a, row0 + 64 * j, m0, full);
#pragma unroll
              for (int j = 0; j < kLocalN / 64; ++j)
                ptx::tma_load_2d_pair(sb + j * kChunkBytes, &map_b, col0 + 64 * j, m0, full);
            } else {
              ptx::tma_load_2d_pair(sa, &map_a, kb * kBlockK, row0, full);
              if constexpr (kMode == kRowsBN) {
#pragma unroll
                for (int j = 0; j < kLocalN / 64; ++j)
                  ptx::tma_load_3d_pair(sb + j * kChunkBytes, &map_b, col0 + 64 * j, kb * kBlockK, slab, full);
                // Weights that are used by one tile only come from HBM: ask L2 for the blocks
                // beyond the shared-memory ring, so more bytes are in flight than the ring holds.
                if (prefetch_blocks > 0 && kb + prefetch_blocks < t.num_kb) {
#pragma unroll
                  for (int j = 0; j < kLocalN / 64; ++j)
                    ptx::tma_prefetch_l2_3d(&map_b, col0 + 64 * j, (kb + prefetch_blocks) * kBlockK, slab);
                }
              } else {
                ptx::tma_load_3d_pair(sb, &map_b, kb * kBlockK, col0, slab, full);
              }
            }
            if (cta_rank != 0) ptx::mbar_arrive_remote(full);
          }
        }
      }
      if (!ok) {
        // Give loads already in flight a bounded chance to land before the CTA retires.
        const uint64_t t0 = ptx::globaltimer_ns();
        const uint32_t inflight = cnt < static_cast<uint32_t>(num_stages) ? cnt : num_stages;
        for (uint32_t i = 0; i < inflight && !kPair; ++i) {
          const uint32_t c = cnt - 1 - i;
          const uint32_t s = c % num_stages, ph = (c / num_stages) & 1u;
          while (!ptx::mbar_try_wait(bar_full + 8u * s, ph) &&
                 ptx::globaltimer_ns() - t0 < 100000000ull) {
          }
        }
        if constexpr (kPair) {
          while (ptx::globaltimer_ns() - t0 < 1000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0 && ep_multiply) {
      // ===== UMMA issuer (the leader CTA issues for the pair) =====
      Walker walk(p, row_start, tile_start, unit, num_units);
      Tile t;
      uint32_t acc_cnt = 0;
      RingPos pos, qpos;
      uint32_t seq = 0;
      bool ok = true;
      while (ok) {
        const int r = next_tile(walk, t, qpos, seq, kDevTimeoutMma, false);
        if (r <= 0) {
          ok = r == 0;
          break;
        }
        if (t.num_kb == 0) continue;
        const uint32_t b = acc_cnt & 1u;
        const uint32_t acc_ph = (acc_cnt >> 1) & 1u;
        ++acc_cnt;
        if (!bounded_wait<kPair>(bar_acc_empty + 8u * b, acc_ph ^ 1u, abort_flag, p.status, kDevTimeoutMma)) {
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + b * kBlockN;
        const bool swapped = kCanSwap && t.group >= 0 && tile_valid(t) <= swap_rows;
        // Same formats and accumulator type as p.idesc; M operand = weights (major as the B
        // operand normally has), N operand = rows (contraction-major), M = 256, N = rows.
        const uint32_t idesc_swapped =
            (p.idesc & 0x00007FFFu) | (kBMn ? (1u << 15) : 0u) |
            ((static_cast<uint32_t>(swapped_n(tile_valid(t))) >> 3) << 17) | ((256u >> 4) << 24);
        for (int kb = 0; kb < t.num_kb; ++kb, pos.advance(num_stages)) {
          const uint32_t s = pos.slot;
          const uint32_t ph = pos.phase;
          if (!bounded_wait<kPair>(bar_full + 8u * s, ph, abort_flag, p.status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kATileBytes;
          const uint64_t da = ptx::make_smem_desc_sw128(sa, kAMn ? kChunkBytes : 16u, 1024u);
          const uint64_t db = ptx::make_smem_desc_sw128(sb, kBMn ? kChunkBytes : 16u, 1024u);
          if (swapped) {
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              ptx::umma_f16<kCtas>(tmem_d, db + ((k * kAdvB) >> 4), da + ((k * kAdvA) >> 4), idesc_swapped,
                                   (kb | k) != 0 ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              ptx::umma_f16<kCtas>(tmem_d, da + ((k * kAdvA) >> 4), db + ((k * kAdvB) >> 4), p.idesc,
                                   (kb | k) != 0 ? 1u : 0u);
            }
          }
          // Slot reusable (in both CTAs) once these MMAs retire.
          if constexpr (kPair) ptx::umma_commit_pair(bar_empty + 8u * s, 3);
          else ptx::umma_commit(bar_empty + 8u * s);
        }
        if (ok) {
          if constexpr (kPair) ptx::umma_commit_pair(bar_acc_full + 8u * b, 3);
          else ptx::umma_commit(bar_acc_full + 8u * b);
        }
      }
    }
  } else if (warp == 2 || warp == 3 || warp >= 8) {
    if constexpr (kEp) {
      // ===== expert-parallel senders: six warps per CTA (2, 3, 8-11), all CTAs of the grid.
      // Consecutive items go to different CTAs, so every SM's links carry every expert. =====
      const int local = warp < 8 ? warp - 2 : warp - 6;
      // Once-per-rank form: kEpCopyWarps of the six put duplicate rows into place in this rank's
      // own receive buffer (all six in a launch that does not send).
      const bool copier = ep.once_per_rank && (ep.phases & 4) && (!(ep.phases & 1) || local < kEpCopyWarps);
      if (copier)
        ep_copy_rows(ep, row_start, lane, abort_flag, p.status, kWaitBudgetNs);
      else if (ep.phases & 1)
        ep_send_rows(ep, ep_vstart, (ep.phases & 2) ? ep_need : nullptr,
                     local * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x),
                     kEpSendWarps * static_cast<int>(gridDim.x), lane, p.status);
    }
    if (kMode == kContract && warp == 2) {
      // ===== tail fix-up: zero the rows of the last contraction block that lie past
      // the end of the group, in both operands, before the MMA may read the slot =====
      Walker walk(p, row_start, tile_start, unit, num_units);
      Tile t;
      uint32_t tail_phase = 0;  // one parity bit per ring slot
      RingPos pos, qpos;        // pos: slot of the NEXT tile's first block
      uint32_t seq = 0;
      bool ok = true;
      while (ok) {
        const int r = next_tile(walk, t, qpos, seq, kDevTimeoutFixup, true);
        if (r <= 0) {
          ok = r == 0;
          break;
        }
        if (t.num_kb == 0) continue;
        const int rem = (t.c_end - t.c_begin) % kBlockK;
        RingPos last = pos;
        last.advance_by(t.num_kb - 1, num_stages);
        pos.advance_by(t.num_kb, num_stages);
        if (rem == 0) continue;
        const uint32_t s = last.slot;
        // Tail blocks that use slot s are strictly ordered (the slot is not refilled
        // before the UMMA warp has consumed it), so one parity bit per slot suffices.
        const uint32_t ph = (tail_phase >> s) & 1u;
        tail_phase ^= (1u << s);
        if (!bounded_wait(bar_tail + 8u * s, ph, abort_flag, p.status, kDevTimeoutFixup)) {
          ok = false;
          break;
        }
        // Each contraction row is one 128-byte line in every [64 x 128 B] chunk, so the
        // swizzle (which permutes 16-byte pieces inside a line) does not matter here.
        uint8_t* stage_ptr = base_ptr + s * kStageBytes;
        constexpr int kChunks = kBlockM / 64 + kLocalN / 64;
        // The warp clears four lines (512 contiguous bytes) per store instruction; this sits
        // between the TMA's arrival and the MMA, so it is kept free of divisions.
        uint8_t* lane_ptr = stage_ptr + (lane & 7) * 16;
#pragma unroll
        for (int chunk = 0; chunk < kChunks; ++chunk) {
          for (int line = rem + (lane >> 3); line < kBlockK; line += 4)
            *reinterpret_cast<uint4*>(lane_ptr + chunk * kChunkBytes + line * 128) = make_uint4(0u, 0u, 0u, 0u);
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          // Completes full[s] for this block (one arrival per CTA of the pair).
          if constexpr (kPair) ptx::mbar_arrive_remote(ptx::map_to_cta(bar_full + 8u * s, 0));
          else ptx::mbar_arrive(bar_full + 8u * s);
        }
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ===== epilogue: this CTA's 128 rows of the tile =====
    const int ew = warp - 4;  // == warp % 4: the TMEM lane quarter this warp may read
    Walker walk(p, row_start, tile_start, unit, num_units);
    Tile t;
    uint32_t acc_cnt = 0;
    bool ok = true;
    const bool gateup = kMode == kRowsBN && p.gateup != 0;
    const int ld_out = gateup ? p.cols / 2 : p.cols;
    RingPos qpos;
    uint32_t seq = 0;
    EpRoute route;             // kEp: where the rows of the current expert return to
    int route_group = -1;
    while (ok && ep_multiply) {
      {
        const int r = next_tile(walk, t, qpos, seq, kDevTimeoutEpilogue, true);
        if (r <= 0) {
          ok = r == 0;
          break;
        }
      }
      const int row = t.row0 + static_cast<int>(cta_rank) * kBlockM + ew * 32 + lane;
      const bool row_ok = row < t.row_end;
      if constexpr (kEp) {
        if (t.group >= 0 && t.group != route_group) {
          route.load(ep, t.group, lane);
          route_group = t.group;
        }
      }
      size_t out_row_off;
      if constexpr (kMode == kContract)
        out_row_off = (static_cast<size_t>(t.group - p.group_begin) * p.rows + row) * ld_out;
      else
        out_row_off = static_cast<size_t>(row) * ld_out;
      const float* scale_row = nullptr;
      if (p.col_scale != nullptr && t.group >= 0)
        scale_row = p.col_scale + static_cast<size_t>(t.group % p.rhs_groups) * p.cols;
      const float* bias_row = nullptr;   // rows outside every group stay zero: no bias there
      if (kMode != kContract && p.col_bias != nullptr && t.group >= 0)
        bias_row = p.col_bias + static_cast<size_t>(t.group % p.rhs_groups) * p.cols;

      uint32_t b = 0;
      const bool has_acc = t.num_kb > 0;
      if (has_acc) {
        b = acc_cnt & 1u;
        const uint32_t acc_ph = (acc_cnt >> 1) & 1u;
        ++acc_cnt;
        if (!bounded_wait<kPair>(bar_acc_full + 8u * b, acc_ph, abort_flag, p.status, kDevTimeoutEpilogue)) {
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
      }
      // 64 columns at a time: two tcgen05.ld of 32 columns each, issued for the next chunk
      // as soon as this chunk's values have been converted, so the TMEM round trip hides
      // behind the stores.  A block of 32 rows x 64 columns that is not ragged (all 32 rows
      // belong to the tile's group; always the case in the contraction mode, where the map
      // clips at the matrix edge) is staged in swizzled shared memory and written by one TMA
      // store; ragged blocks and float32 outputs use row-predicated 16-byte stores.
      const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + b * kBlockN;
      if (kCanSwap && has_acc && tile_valid(t) <= swap_rows) {
        // Transposed accumulator: this thread owns output column `n`, TMEM column r is tile
        // row r.  Per row the warp writes 32 consecutive outputs.
        const int valid = tile_valid(t);
        const int n = t.col0 + static_cast<int>(cta_rank) * kLocalN + ew * 32 + lane;
        const bool n_ok = n < p.cols;
        const float cs = (scale_row != nullptr && n_ok) ? __ldg(scale_row + n) : 1.f;
        const float bs = (bias_row != nullptr && n_ok) ? __ldg(bias_row + n) : 0.f;
        uint32_t v[32];
#pragma unroll 1
        for (int rc = 0; rc * 32 < valid; ++rc) {
          ptx::tmem_ld_32x32b_x32(tmem_row + rc * 32, v);
          ptx::tmem_wait_ld();
          if constexpr (kEp) {
            // Lane j works out where tile row rc * 32 + j returns to; per row the warp then
            // writes its 32 consecutive 16-bit outputs there.
            const uint64_t my_addr = route.row_address(ep, t.row0 + rc * 32 + lane);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const uint64_t a = shfl64(my_addr, i);
              if (rc * 32 + i < valid && n_ok) {
                const float val = __uint_as_float(v[i]);
                uint16_t* dst = reinterpret_cast<uint16_t*>(a) + n;
                if (p.out_is_f16) *reinterpret_cast<__half*>(dst) = __float2half_rn(val);
                else *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(val);
              }
            }
            continue;
          }
          const size_t off0 = static_cast<size_t>(t.row0 + rc * 32) * ld_out + n;
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * cs + bs);
          if (p.activation != 0) element_act32(p.activation, v);
          const int nrows = n_ok ? min(32, valid - rc * 32) : 0;
          const size_t ld = static_cast<size_t>(ld_out);
          if (p.out_is_f32) {
            float* dst = reinterpret_cast<float*>(p.out) + off0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nrows) dst[i * ld] = __uint_as_float(v[i]);
          } else if (p.out_is_f16) {
            __half* dst = reinterpret_cast<__half*>(p.out) + off0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nrows) dst[i * ld] = __float2half_rn(__uint_as_float(v[i]));
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + off0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nrows) dst[i * ld] = __float2bfloat16_rn(__uint_as_float(v[i]));
          }
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) ptx::mbar_arrive_remote(ptx::map_to_cta(bar_acc_empty + 8u * b, 0));
          else ptx::mbar_arrive(bar_acc_empty + 8u * b);
        }
        continue;
      }
      if (gateup) {
        // Gate columns in the first half of the accumulator, up columns in the second:
        // 32 outputs per pair of TMEM loads, written at column t.col0 / 2 + 32 c of the
        // half-width output.
        constexpr int kHalf = kBlockN / 2;
        const int out_cols = ld_out;
        const int out_col0 = t.col0 / 2;
        const int g_chunks = min(kHalf / 32, (out_cols - out_col0 + 31) / 32);   // warp-uniform
        uint32_t vg[32], vu[32];
#pragma unroll 1
        for (int c = 0; c < g_chunks; ++c) {
          if (has_acc) {
            ptx::tmem_ld_32x32b_x32(tmem_row + c * 32, vg);
            ptx::tmem_ld_32x32b_x32(tmem_row + kHalf + c * 32, vu);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float gv = __uint_as_float(vg[i]), uv = __uint_as_float(vu[i]);
              const int j = out_col0 + c * 32 + i;
              if (bias_row != nullptr && j < out_cols) {
                gv += __ldg(bias_row + j);
                uv += __ldg(bias_row + out_cols + j);
              }
              vg[i] = __float_as_uint(gv);
              vu[i] = __float_as_uint(uv);
            }
            gateup_act32(p.gateup, vg, vu);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) vg[i] = 0u;
          }
          store_chunk(p, vg, nullptr, row_ok, out_row_off, out_col0 + c * 32, out_cols);
        }
        if (has_acc) {
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) ptx::mbar_arrive_remote(ptx::map_to_cta(bar_acc_empty + 8u * b, 0));
            else ptx::mbar_arrive(bar_acc_empty + 8u * b);
          }
        }
        continue;
      }
      if (kMode != kContract && p.quant_sub != 0) {
        // Fused output quantisation (the rule of the reference's fp8 epilogue,
        // pallas_mosaic_gpu_kernel_sm100_fp8_quant.py:800-844): per row and block of quant_sub
        // columns, scale = max|x| / 448 (1 for an all-zero block), q = e4m3(clip(x / scale)).
        // A thread owns a row: pass 1 finds the block's maximum, pass 2 reloads the
        // accumulator, divides and stores 32 bytes per chunk.
        const int sub = p.quant_sub;
        const int blocks = min(kBlockN / sub, (p.cols - t.col0 + sub - 1) / sub);   // warp-uniform
        uint8_t* qrow = reinterpret_cast<uint8_t*>(p.out) + static_cast<size_t>(row) * p.cols;
        uint32_t v[32];
#pragma unroll 1
        for (int sb = 0; sb < blocks; ++sb) {
          const int c0 = t.col0 + sb * sub;
          float amax = 0.f;
          auto load_chunk = [&](int c) {
            if (has_acc) {
              ptx::tmem_ld_32x32b_x32(tmem_row + sb * sub + c * 32, v);
              ptx::tmem_wait_ld();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float x = __uint_as_float(v[i]);
              if (bias_row != nullptr) x += __ldg(bias_row + min(c0 + c * 32 + i, p.cols - 1));
              v[i] = __float_as_uint(x);
            }
            if (p.activation != 0) element_act32(p.activation, v);
          };
#pragma unroll 1
          for (int c = 0; c < sub / 32; ++c) {
            load_chunk(c);
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c0 + c * 32 + i < p.cols) amax = fmaxf(amax, fabsf(__uint_as_float(v[i])));
          }
          const float scale = amax == 0.f ? 1.0f : amax * (1.0f / 448.0f);
          const float inv = 1.0f / scale;
          if (row_ok) p.out_scales[static_cast<size_t>(row) * (p.cols / sub) + c0 / sub] = scale;
#pragma unroll 1
          for (int c = 0; c < sub / 32; ++c) {
            load_chunk(c);
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float q[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) q[e] = fminf(fmaxf(__uint_as_float(v[4 * j + e]) * inv, -448.f), 448.f);
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), __NV_SATFINITE, __NV_E4M3);
              w[j] = lo | (hi << 16);
            }
            const int col = c0 + c * 32;
            if (row_ok && col < p.cols) {      // cols is a multiple of quant_sub, hence of 32
              *reinterpret_cast<uint4*>(qrow + col) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(qrow + col + 16) = make_uint4(w[4], w[5], w[6], w[7]);
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
        continue;
      }
      const int cols_left = p.cols - t.col0;
      const int n_chunks = min(kBlockN / 64, (cols_left + 63) / 64);        // warp-uniform
      const int warp_row0 = t.row0 + static_cast<int>(cta_rank) * kBlockM + ew * 32;
      const bool block_full = (kMode == kContract) ? (warp_row0 < t.row_end) : (warp_row0 + 32 <= t.row_end);
      const bool use_tma = p.tma_store != 0 && block_full;
      uint64_t ep_row_addr = 0;   // kEp: return address of this lane's row
      if constexpr (kEp) ep_row_addr = route.row_address(ep, row);
      uint32_t va[32], vb[32];
      if (has_acc) {
        ptx::tmem_ld_32x32b_x32(tmem_row, va);
        if constexpr (kBlockN > 32) ptx::tmem_ld_32x32b_x32(tmem_row + 32, vb);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) va[i] = vb[i] = 0u;
      }
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        const int col = t.col0 + c * 64;
        if (has_acc) {
          ptx::tmem_wait_ld();
        } else if (c > 0 && p.activation != 0) {
          // zero-fill tile: the previous chunk's activation was applied in place
#pragma unroll
          for (int i = 0; i < 32; ++i) va[i] = vb[i] = 0u;
        }
        if constexpr (kEp) {
          // 32 rows x 64 columns through the swizzled staging block, then out by rows: eight
          // lanes write one row's 128 contiguous bytes into its source rank's return buffer.
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            w[i] = p.out_is_f16 ? pack_f16x2(__uint_as_float(va[2 * i]), __uint_as_float(va[2 * i + 1]))
                                : pack_bf16x2(__uint_as_float(va[2 * i]), __uint_as_float(va[2 * i + 1]));
            w[16 + i] = p.out_is_f16 ? pack_f16x2(__uint_as_float(vb[2 * i]), __uint_as_float(vb[2 * i + 1]))
                                     : pack_bf16x2(__uint_as_float(vb[2 * i]), __uint_as_float(vb[2 * i + 1]));
          }
          if (has_acc && c + 1 < n_chunks) {
            ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 64, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 64 + 32, vb);
          }
          uint8_t* block = base_ptr + L.staging + ew * kStagingBytes;
          __syncwarp();   // the previous chunk's row reads are done
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(block + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          __syncwarp();
          const int piece = lane & 7;
          const bool col_ok = col + piece * 8 < p.cols;   // cols is a multiple of 8 in this form
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int rl = rr * 4 + (lane >> 3);
            const uint64_t a = shfl64(ep_row_addr, rl);
            const bool r_ok = __shfl_sync(0xffffffffu, row_ok ? 1 : 0, rl) != 0;
            const uint4 val = *reinterpret_cast<const uint4*>(block + rl * 128 + ((piece ^ (rl & 7)) << 4));
            if (r_ok && col_ok) *reinterpret_cast<uint4*>(a + static_cast<uint64_t>(col + piece * 8) * 2) = val;
          }
          continue;
        }
        if (use_tma) {
          uint32_t w[32];
          if (p.activation != 0) {
            element_act32(p.activation, va);
            element_act32(p.activation, vb);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            w[i] = p.out_is_f16 ? pack_f16x2(__uint_as_float(va[2 * i]), __uint_as_float(va[2 * i + 1]))
                                : pack_bf16x2(__uint_as_float(va[2 * i]), __uint_as_float(va[2 * i + 1]));
            w[16 + i] = p.out_is_f16 ? pack_f16x2(__uint_as_float(vb[2 * i]), __uint_as_float(vb[2 * i + 1]))
                                     : pack_bf16x2(__uint_as_float(vb[2 * i]), __uint_as_float(vb[2 * i + 1]));
          }
          if (has_acc && c + 1 < n_chunks) {
            ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 64, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 64 + 32, vb);
          }
          // The staging block is free once the previous store has read it.
          if (lane == 0) ptx::bulk_wait_group_read0();
          __syncwarp();
          uint8_t* line = base_ptr + L.staging + ew * kStagingBytes + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(line + ((j ^ (lane & 7)) << 4)) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const uint32_t src = base + L.staging + ew * kStagingBytes;
            if constexpr (kMode == kContract) ptx::tma_store_3d(&map_out, src, col, warp_row0, t.group - p.group_begin);
            else ptx::tma_store_2d(&map_out, src, col, warp_row0);
            ptx::bulk_commit_group();
          }
        } else {
          store_chunk(p, va, scale_row, row_ok, out_row_off, col, p.cols, bias_row);
          if (col + 32 < p.cols) store_chunk(p, vb, scale_row, row_ok, out_row_off, col + 32, p.cols, bias_row);
          if (has_acc && c + 1 < n_chunks) {
            ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 64, va);
            ptx::tmem_ld_32x32b_x32(tmem_row + (c + 1) * 64 + 32, vb);
          }
        }
      }
      if (has_acc) {
        // All of this warp's TMEM reads have completed (wait::ld above): hand the
        // accumulator back to the MMA warp (in the leader CTA).
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) ptx::mbar_arrive_remote(ptx::map_to_cta(bar_acc_empty + 8u * b, 0));
          else ptx::mbar_arrive(bar_acc_empty + 8u * b);
        }
      }
    }
  }

  // Outstanding TMA stores read this CTA's shared memory: let them finish before it retires.
  if (warp >= 4 && warp < 8 && lane == 0) ptx::bulk_wait_group0();

  // ------------------------------------------------------------------ teardown
  ptx::tcgen05_fence_before();
  __syncthreads();
  if constexpr (kPair) {
    // The leader's MMAs read the peer's shared memory and write its TMEM, and both CTAs
    // signal each other's barriers: neither may retire before both are done.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 2) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

}  // namespace tkmx
