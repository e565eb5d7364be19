// Expert-parallel pieces that run over peer-mapped memory (NVLink / NVSwitch, plain loads and
// stores; no multicast, no collective library):
//
//   ep_exchange_plan_kernel   every rank pushes its per-expert pair counts into every rank's
//                             [W, G] count matrix, passes a flag barrier, and derives from the
//                             complete matrix all the offsets of the step (where its rows go in
//                             the owners' receive buffers, where each received row's output goes
//                             back).  One CTA; replaces a chain of small index kernels and a
//                             device-to-host read.
//   cross_rank_barrier_kernel the same flag barrier alone (sequence-numbered flags, bounded
//                             wait, status word on expiry).
//   ep_send_rows              device function run by two otherwise idle warps of every CTA of
//                             the grouped-GEMM kernel: copies this rank's token rows, expert by
//                             expert, straight into the owners' receive buffers and bumps the
//                             owner's per-expert arrival counter (release at system scope).  The
//                             GEMM's TMA producer of the owning rank waits (bounded) on that
//                             counter before it loads an expert's rows, so transfer and
//                             multiplication overlap tile by tile inside ONE kernel.
//   EpRoute                   epilogue side: finished output rows are stored straight into the
//                             source rank's return buffer.
//
// The reference has no such layer (its expert-parallel affordances are `group_offset` /
// `num_actual_groups`, tokamax/_src/ops/ragged_dot/pallas_mosaic_tpu_v2.py:89-93); the data
// movement either side of ragged_dot is ragged_gather / ragged_gather_reduce
// (tokamax/_src/ops/ragged_gather/base.py:26-30, ragged_gather_reduce/base.py:26-37).
//
// Layouts.  Experts are sharded contiguously: rank r owns global experts [r * G/W, (r+1) * G/W).
// A rank's receive buffer is expert-major: (local expert, source rank), so one local expert's
// rows are ONE contiguous group of the GEMM.  A rank's return buffer holds its own pairs in
// expert-sorted order (position `pos[pair]` of the counting sort).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tkmx {

constexpr int kEpMaxWorld = 16;
constexpr int kEpItemRows = 8;     // rows a send warp moves between two arrival signals
// Rows of the peer table (device array uint64[kEpTabRows][kEpMaxWorld], entry [t][r] = address
// of buffer t on rank r as mapped into this process).
// Row kTabRefs is read only by the form that sends a token once per destination rank.
enum EpTab : int { kTabRecv = 0, kTabArrive = 1, kTabRet = 2, kTabCounts = 3, kTabFlags = 4, kTabRefs = 5, kEpTabRows = 6 };
constexpr int kEpCopyWarps = 2;    // sender warps per CTA that copy duplicate rows into place instead

// Words of a rank's arrival array (uint32), G/W = gl local experts:
//   [0, gl)            rows present per local expert, written by their senders
//   [gl]               multiplication progress      [gl + 1]  send cursor
// and, with one row per (token, destination rank) only:
//   [gl + 2, 2gl + 2)  duplicate rows announced per local expert (their reference word is written)
//   [2gl + 2, 3gl + 2) duplicate rows copied into place per local expert
//   [3gl + 2]          copy cursor
__host__ __device__ inline int ep_arrive_words(int gl, bool once_per_rank) { return once_per_rank ? 3 * gl + 3 : gl + 2; }

constexpr int kDevTimeoutBarrier = 5;    // device status codes (continuing DeviceStatus)
constexpr int kDevTimeoutArrival = 6;
constexpr int kDevEpOverflow = 7;

// int32 tables written by ep_exchange_plan_kernel (offsets in ints).
struct EpPlanLayout {
  int group_sizes;  // [G/W]        rows per local expert (sum over sources)
  int vstart;       // [G + 1]      send order v = local_expert * W + owner: first row of v among my sorted pairs' send order
  int src_off;      // [G] by v     first position, in my expert-sorted order, of my pairs of that expert
  int dst_row;      // [G] by v     first row in the owner's receive buffer for my rows of that expert
  int seg_start;    // [G/W][W + 1] first receive-buffer row of segment (local expert, source); last entry = expert's end
  int ret_off;      // [G/W][W]     first row in the source's return buffer for that segment
  int total;
};
__host__ __device__ inline EpPlanLayout ep_plan_layout(int num_experts, int world) {
  const int gl = num_experts / world;
  EpPlanLayout l;
  l.group_sizes = 0;
  l.vstart = gl;
  l.src_off = l.vstart + num_experts + 1;
  l.dst_row = l.src_off + num_experts;
  l.seg_start = l.dst_row + num_experts;
  l.ret_off = l.seg_start + gl * (world + 1);
  l.total = l.ret_off + gl * world;
  return l;
}

namespace ptx {
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_s32(int32_t* p, int32_t v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_relaxed_sys_s32(const int32_t* p) {
  int32_t v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Orders earlier generic-proxy observations before later async-proxy (TMA) accesses.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ uint64_t gtimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
}  // namespace ptx

__device__ __forceinline__ uint64_t shfl64(uint64_t v, int src_lane) {
  const uint32_t lo = __shfl_sync(0xffffffffu, static_cast<uint32_t>(v), src_lane);
  const uint32_t hi = __shfl_sync(0xffffffffu, static_cast<uint32_t>(v >> 32), src_lane);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// ------------------------------------------------------------------------------ flag barrier
// Rank r writes `seq` into slot r of every rank's flag array, then waits until every slot of
// its own array has reached `seq` (sequence numbers only grow, compared modulo 2^32).  Run by
// threads 0..W-1 of one CTA.  Returns false when the wait ran out: `code` is then in the status
// word and the caller skips what depended on the barrier.
__device__ __forceinline__ bool flag_barrier_thread(const uint64_t* __restrict__ peer_tab, uint32_t* flags,
                                                    int rank, int peer, uint32_t seq, uint64_t timeout_ns,
                                                    int32_t* status) {
  uint32_t* remote = reinterpret_cast<uint32_t*>(peer_tab[kTabFlags * kEpMaxWorld + peer]) + rank;
  ptx::st_release_sys_u32(remote, seq);
  const uint64_t t0 = ptx::gtimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ptx::ld_acquire_sys_u32(flags + peer) - seq) < 0) {
    if ((++spins & 0x3Fu) == 0 && ptx::gtimer_ns() - t0 > timeout_ns) {
      atomicCAS(status, 0, kDevTimeoutBarrier);
      return false;
    }
  }
  return true;
}

__global__ void __launch_bounds__(32)
cross_rank_barrier_kernel(const uint64_t* __restrict__ peer_tab, uint32_t* flags, int world, int rank,
                          uint32_t seq, uint64_t timeout_ns, int32_t* status) {
  __threadfence_system();
  if (static_cast<int>(threadIdx.x) < world)
    flag_barrier_thread(peer_tab, flags, rank, threadIdx.x, seq, timeout_ns, status);
}

// ------------------------------------------------------------------------------ exchange + plan
struct EpExchangeParams {
  const int32_t* my_counts;   // [G] pairs per global expert on this rank (from the counting sort)
  const uint64_t* peer_tab;   // device, see EpTab
  int32_t* counts_all;        // local [W, G]; row s is written by rank s
  uint32_t* flags;            // local [W]
  uint32_t* arrive;           // local [G/W] arrival counters, reset here
  int32_t* plan;              // local, EpPlanLayout
  int32_t num_experts, world, rank;
  uint32_t seq;
  uint64_t timeout_ns;
  int32_t* status;
  int32_t arrive_words;       // words of `arrive` to reset (ep_arrive_words)
};

// Exclusive block-wide prefix sum over 1024 threads; `total` receives the sum.
__device__ __forceinline__ int block_excl_scan_1024(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += u;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += u;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int r = (warp > 0 ? warp_sums[warp - 1] : 0) + incl - v;
  total = warp_sums[31];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(1024)
ep_exchange_plan_kernel(const EpExchangeParams x) {
  __shared__ int warp_sums[32];
  __shared__ int s_excl[1024];
  __shared__ int s_v[1024];
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  const int G = x.num_experts, W = x.world, gl = G / W;
  if (tid == 0) s_abort = 0;
  // 0. what the peers add to during this step starts at zero; they can only start adding
  //    after they have seen this rank's flag below.
  for (int i = tid; i < x.arrive_words; i += blockDim.x) x.arrive[i] = 0u;   // layout: ep_arrive_words
  // 1. this rank's counts into row `rank` of every rank's matrix
  for (int idx = tid; idx < W * G; idx += blockDim.x) {
    const int peer = idx / G, e = idx - peer * G;
    int32_t* dst = reinterpret_cast<int32_t*>(x.peer_tab[kTabCounts * kEpMaxWorld + peer]) + x.rank * G + e;
    ptx::st_relaxed_sys_s32(dst, x.my_counts[e]);
  }
  __threadfence_system();
  __syncthreads();
  // 2. barrier: every rank's counts are in place, every rank has finished its previous step
  if (tid < W && !flag_barrier_thread(x.peer_tab, x.flags, x.rank, tid, x.seq, x.timeout_ns, x.status))
    s_abort = 1;
  __syncthreads();
  if (s_abort) return;
  __threadfence_system();

  // 3. plan.  Thread e works on global expert e.
  const EpPlanLayout L = ep_plan_layout(G, W);
  const int e = tid;
  const bool live = e < G;
  int c[kEpMaxWorld], within[kEpMaxWorld];
  int tot = 0;
#pragma unroll
  for (int s = 0; s < kEpMaxWorld; ++s) {
    c[s] = (live && s < W) ? ptx::ld_relaxed_sys_s32(x.counts_all + s * G + e) : 0;
    c[s] = max(c[s], 0);
    within[s] = tot;      // rows of earlier sources in the same expert
    tot += c[s];
  }
  int total_rows;
  const int excl = block_excl_scan_1024(tot, warp_sums, total_rows);
  s_excl[tid] = excl;
  __syncthreads();
  const int owner = live ? e / gl : 0;
  const int le = e - owner * gl;
  const int expert_start = excl - s_excl[owner * gl];   // first row of the expert in its owner's receive buffer
  int my_send_off = 0;
#pragma unroll
  for (int s = 0; s < kEpMaxWorld; ++s) {
    if (s < W) {   // uniform
      int unused;
      const int so = block_excl_scan_1024(c[s], warp_sums, unused);   // source s's first sorted position of expert e
      if (live && owner == x.rank) x.plan[L.ret_off + le * W + s] = so;
      if (s == x.rank) my_send_off = so;
    }
  }
  if (live && owner == x.rank) {
    x.plan[L.group_sizes + le] = tot;
#pragma unroll
    for (int s = 0; s < kEpMaxWorld; ++s)
      if (s < W) x.plan[L.seg_start + le * (W + 1) + s] = expert_start + within[s];
    x.plan[L.seg_start + le * (W + 1) + W] = expert_start + tot;
  }
  int mine = 0, my_within = 0;
#pragma unroll
  for (int s = 0; s < kEpMaxWorld; ++s)
    if (s == x.rank) {
      mine = c[s];
      my_within = within[s];
    }
  const int v = le * W + owner;   // send order: all owners' local expert 0, then local expert 1, ...
  s_v[tid] = 0;
  __syncthreads();
  if (live) {
    s_v[v] = mine;
    x.plan[L.src_off + v] = my_send_off;
    x.plan[L.dst_row + v] = expert_start + my_within;
  }
  __syncthreads();
  int sent_total;
  const int vs = block_excl_scan_1024(tid < G ? s_v[tid] : 0, warp_sums, sent_total);
  if (tid < G) x.plan[L.vstart + tid] = vs;
  if (tid == 0) x.plan[L.vstart + G] = sent_total;
}

// ------------------------------------------------------------------------------ fused kernel side
struct EpFusedParams {
  const void* tokens;            // [T, K] this rank's token rows (16-bit elements)
  const int32_t* sorted_pair;    // [T * top_k] pair index at each expert-sorted position
  const int32_t* plan;           // EpPlanLayout tables of this step
  const uint64_t* peer_tab;      // device, see EpTab
  const uint32_t* arrive;        // local arrival counters [G/W]
  uint32_t* progress;            // local word (arrive[G/W]): 1 + furthest local expert whose tiles have been started
  uint32_t* send_cursor;         // local word (arrive[G/W + 1]): next send item to hand out
  int32_t static_items;          // 1: deal items round-robin to the sender warps instead
  int32_t ahead_rows;            // senders stay at most this many receive-buffer rows ahead of `progress` (0: no pacing)
  int32_t world, rank, top_k;
  int32_t num_experts;           // global G
  int32_t row_vec;               // 16-byte pieces per token row
  int32_t ret_row_bytes;         // bytes per output row
  int32_t capacity_rows;         // rows of every receive buffer
  int32_t phases;                // bit 0: send this rank's rows; bit 1: multiply and return; bit 2: copy duplicates
  // One row per (token, destination rank): a token routed to several experts of one rank crosses
  // the link once, for its lowest expert there; for the others the sender writes a reference
  // word and the destination copies the row inside its own memory.  All zero when off.
  int32_t once_per_rank;
  const int32_t* expert_ids;     // [T, top_k] global expert of every pair
  const int32_t* pair_pos;       // [T * top_k] expert-sorted position of every pair
};

// Reference word of a receive-buffer row: 0 = the row itself arrives; otherwise
// (local expert of the original + 1) << 24 | receive-buffer row of the original.
constexpr int kEpRefRowBits = 24;

// Sending side, one warp: rows in send order (local expert major, then owner), kEpItemRows at a
// time, so that every owner receives its first experts first.
__device__ __forceinline__ void ep_send_rows(const EpFusedParams& ep, const int* s_vstart, const int* s_need,
                                             int sender, int num_senders, int lane, int32_t* status) {
  const int G = ep.num_experts, W = ep.world;
  const EpPlanLayout L = ep_plan_layout(G, W);
  const int P = s_vstart[G];
  const int num_items = (P + kEpItemRows - 1) / kEpItemRows;
  constexpr int kU = 14;  // 16-byte pieces in flight per lane (7 KiB per warp)
  // Items are handed out through a counter, not dealt round-robin: an expert can be multiplied
  // only when ALL its rows have arrived, so one slow warp with a fixed share would hold up
  // every rank's multiplication; this way items complete in order whatever the warps' speeds.
  // (Measured on 8 GPUs the two are equal, 2.65 against 2.66 ms per step: `static_items`.)
  const int gl = G / W;
  int next_static = sender;
  while (true) {
    int item = next_static;
    if (ep.static_items && !ep.once_per_rank) {
      next_static += num_senders;
    } else {
      if (lane == 0) item = static_cast<int>(atomicAdd(ep.send_cursor, 1u));
      item = __shfl_sync(0xffffffffu, item, 0);
    }
    if (item >= num_items) break;
    const int i = item * kEpItemRows + lane;
    bool act = lane < kEpItemRows && i < P;
    int v = 0;
    uint64_t src = 0, dst = 0;
    bool dup = false;       // this row is a token's second or later row on its destination rank
    if (act) {
      int lo = 0, hi = G;            // largest v with vstart[v] <= i
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_vstart[mid] <= i) lo = mid;
        else hi = mid;
      }
      v = lo;
      const int off = i - s_vstart[v];
      const int pair = __ldg(ep.sorted_pair + __ldg(ep.plan + L.src_off + v) + off);
      const int drow = __ldg(ep.plan + L.dst_row + v) + off;
      if (drow < 0 || drow >= ep.capacity_rows || pair < 0) {
        atomicCAS(status, 0, kDevEpOverflow);
        act = false;
      } else {
        const size_t row_bytes = static_cast<size_t>(ep.row_vec) * 16;
        src = reinterpret_cast<uint64_t>(ep.tokens) + static_cast<size_t>(pair / ep.top_k) * row_bytes;
        dst = __ldg(ep.peer_tab + kTabRecv * kEpMaxWorld + (v % W)) + static_cast<size_t>(drow) * row_bytes;
        if (ep.once_per_rank) {
          // The original of a token on a rank is its pair with the lowest (expert, pair index)
          // there: the first of them in send order, so it is complete before its copies are due.
          const int owner = v % W;
          uint32_t ref = 0u;
          if (owner != ep.rank) {
            const int tok = pair / ep.top_k;
            const int e = owner * gl + v / W;
            int best_e = e, best_pair = pair;
            for (int j = 0; j < ep.top_k; ++j) {
              const int pj = tok * ep.top_k + j;
              const int ej = __ldg(ep.expert_ids + pj);
              if (ej >= owner * gl && ej < (owner + 1) * gl && (ej < best_e || (ej == best_e && pj < best_pair))) {
                best_e = ej;
                best_pair = pj;
              }
            }
            if (best_pair != pair) {
              const int le1 = best_e - owner * gl;
              const int v1 = le1 * W + owner;
              const int r1 = __ldg(ep.plan + L.dst_row + v1) + __ldg(ep.pair_pos + best_pair) - __ldg(ep.plan + L.src_off + v1);
              if (r1 < 0 || r1 >= ep.capacity_rows || r1 >= (1 << kEpRefRowBits)) {
                atomicCAS(status, 0, kDevEpOverflow);
              } else {
                dup = true;
                src = 0;    // nothing to move
                ref = (static_cast<uint32_t>(le1 + 1) << kEpRefRowBits) | static_cast<uint32_t>(r1);
              }
            }
          }
          // Every row's reference word is written (0: the row itself arrives) before the counter
          // update that tells the owner about the row.
          *(reinterpret_cast<uint32_t*>(__ldg(ep.peer_tab + kTabRefs * kEpMaxWorld + owner)) + drow) = ref;
        }
      }
    }
    const int nrows = min(kEpItemRows, P - item * kEpItemRows);
    if (s_need != nullptr) {
      // Pacing: the item's last row belongs to its furthest expert (rows are sent expert-major).
      const int le_last = __shfl_sync(0xffffffffu, v / W, nrows - 1);
      if (lane == 0) {
        const uint32_t need = static_cast<uint32_t>(s_need[le_last]);
        if (need > 0u && *reinterpret_cast<volatile uint32_t*>(ep.progress) < need) {
          const uint64_t t0 = ptx::gtimer_ns();
          uint32_t spins = 0;
          while (*reinterpret_cast<volatile uint32_t*>(ep.progress) < need) {
            __nanosleep(200);
            if ((++spins & 0xFFu) == 0 && ptx::gtimer_ns() - t0 > 2000000000ull) {
              atomicCAS(status, 0, kDevTimeoutArrival);   // give up pacing, never the rows
              break;
            }
          }
        }
      }
      __syncwarp();
    }
    for (int j = 0; j < nrows; ++j) {
      const uint4* s4 = reinterpret_cast<const uint4*>(shfl64(src, j));
      uint4* d4 = reinterpret_cast<uint4*>(shfl64(dst, j));
      if (s4 == nullptr) continue;   // warp-uniform
      for (int base = lane; base < ep.row_vec; base += 32 * kU) {
        uint4 r[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (base + 32 * u < ep.row_vec) r[u] = __ldg(s4 + base + 32 * u);
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (base + 32 * u < ep.row_vec) d4[base + 32 * u] = r[u];
      }
    }
    // Every lane's stores are ordered before the counter update the owner acquires.
    __threadfence_system();
    __syncwarp();
    const unsigned m = __ballot_sync(0xffffffffu, act && !dup);
    if (act && !dup) {
      const unsigned same = __match_any_sync(m, v);
      if (lane == __ffs(same) - 1) {
        uint32_t* ctr = reinterpret_cast<uint32_t*>(__ldg(ep.peer_tab + kTabArrive * kEpMaxWorld + (v % W))) + v / W;
        ptx::red_release_sys_add_u32(ctr, __popc(same));
      }
    }
    const unsigned md = __ballot_sync(0xffffffffu, act && dup);
    if (act && dup) {
      const unsigned same = __match_any_sync(md, v);
      if (lane == __ffs(same) - 1) {   // "announced" counters follow the arrival ones, see ep_arrive_words
        uint32_t* ctr = reinterpret_cast<uint32_t*>(__ldg(ep.peer_tab + kTabArrive * kEpMaxWorld + (v % W))) + gl + 2 + v / W;
        ptx::red_release_sys_add_u32(ctr, __popc(same));
      }
    }
  }
}

// Bounded wait of one thread until a[0] + b[0] >= expected (b may be null).
__device__ __forceinline__ bool ep_wait_sum(const uint32_t* a, const uint32_t* b, uint32_t expected,
                                            volatile int* abort_flag, int32_t* status, uint64_t budget_ns) {
  auto seen = [&]() { return ptx::ld_acquire_sys_u32(a) + (b != nullptr ? ptx::ld_acquire_sys_u32(b) : 0u); };
  if (seen() >= expected) return true;
  const uint64_t t0 = ptx::gtimer_ns();
  uint32_t spins = 0;
  while (seen() < expected) {
    if ((++spins & 0x3Fu) == 0) {
      if (*abort_flag) return false;
      if (ptx::gtimer_ns() - t0 > budget_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0, kDevTimeoutArrival);
        return false;
      }
    }
  }
  return true;
}

// Receiving side of the once-per-rank form, one warp: rows of this rank's receive buffer,
// kEpItemRows at a time in expert order.  Once every row of an expert is either present or
// announced (its reference word is written), the duplicates among them are copied from their
// originals, which lie in an earlier expert of the same buffer (or the same expert, for a token that names it twice), and counted as copied.
// `row_start` [G/W + 1]: first receive-buffer row of every local expert (shared memory).
__device__ __forceinline__ void ep_copy_rows(const EpFusedParams& ep, const int* row_start, int lane,
                                             volatile int* abort_flag, int32_t* status, uint64_t budget_ns) {
  const int gl = ep.num_experts / ep.world;
  const int R = row_start[gl];
  const int num_items = (R + kEpItemRows - 1) / kEpItemRows;
  const uint32_t* present = ep.arrive;
  const uint32_t* announced = ep.arrive + gl + 2;
  uint32_t* copied = const_cast<uint32_t*>(ep.arrive) + 2 * gl + 2;
  uint32_t* cursor = const_cast<uint32_t*>(ep.arrive) + 3 * gl + 2;
  const uint32_t* refs = reinterpret_cast<const uint32_t*>(__ldg(ep.peer_tab + kTabRefs * kEpMaxWorld + ep.rank));
  const uint64_t recv = __ldg(ep.peer_tab + kTabRecv * kEpMaxWorld + ep.rank);
  const size_t row_bytes = static_cast<size_t>(ep.row_vec) * 16;
  constexpr int kU = 14;
  while (true) {
    int item = 0;
    if (lane == 0) item = static_cast<int>(atomicAdd(cursor, 1u));
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= num_items) break;
    const int row = item * kEpItemRows + lane;
    const bool act = lane < kEpItemRows && row < R;
    int le = 0;
    bool ok = true;
    if (act) {
      int lo = 0, hi = gl;            // largest le with row_start[le] <= row (empty experts share a start: the last one holds the row)
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (row_start[mid] <= row) lo = mid;
        else hi = mid;
      }
      le = lo;
      ok = ep_wait_sum(present + le, announced + le, static_cast<uint32_t>(row_start[le + 1] - row_start[le]),
                       abort_flag, status, budget_ns);
    }
    uint64_t src = 0, dst = 0;
    bool dup = false;
    if (act && ok) {
      const uint32_t ref = static_cast<uint32_t>(ptx::ld_relaxed_sys_s32(reinterpret_cast<const int32_t*>(refs + row)));
      if (ref != 0u) {
        const int le1 = static_cast<int>(ref >> kEpRefRowBits) - 1;
        const int r1 = static_cast<int>(ref & ((1u << kEpRefRowBits) - 1u));
        // the original lies in an earlier expert, or in this one when a token names an expert twice
        if (le1 < 0 || le1 > le || r1 == row || r1 < row_start[le1] || r1 >= row_start[le1 + 1]) {
          atomicCAS(status, 0, kDevEpOverflow);
        } else if (ep_wait_sum(present + le1, announced + le1, static_cast<uint32_t>(row_start[le1 + 1] - row_start[le1]),
                               abort_flag, status, budget_ns)) {
          dup = true;
          src = recv + static_cast<size_t>(r1) * row_bytes;
          dst = recv + static_cast<size_t>(row) * row_bytes;
        }
      }
    }
    if (__any_sync(0xffffffffu, act && !ok)) break;   // a wait ran out: the status word says so
    const int nrows = min(kEpItemRows, R - item * kEpItemRows);
    for (int j = 0; j < nrows; ++j) {
      const uint4* s4 = reinterpret_cast<const uint4*>(shfl64(src, j));
      uint4* d4 = reinterpret_cast<uint4*>(shfl64(dst, j));
      if (s4 == nullptr) continue;   // warp-uniform
      for (int base = lane; base < ep.row_vec; base += 32 * kU) {
        uint4 r[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (base + 32 * u < ep.row_vec) r[u] = __ldcg(s4 + base + 32 * u);   // written by a peer during this kernel: not the read-only path
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (base + 32 * u < ep.row_vec) d4[base + 32 * u] = r[u];
      }
    }
    __threadfence();
    __syncwarp();
    const unsigned md = __ballot_sync(0xffffffffu, dup);
    if (dup) {
      const unsigned same = __match_any_sync(md, le);
      if (lane == __ffs(same) - 1) ptx::red_release_sys_add_u32(copied + le, __popc(same));
    }
  }
}

// Receiving side: wait until all `expected` rows of local expert `le` have arrived.  One thread.
__device__ __forceinline__ bool ep_wait_expert(const EpFusedParams& ep, int le, uint32_t expected,
                                               volatile int* abort_flag, int32_t* status, uint64_t budget_ns) {
  // Rows present plus, in the once-per-rank form, duplicates copied into place.
  const uint32_t* ctr = ep.arrive + le;
  const uint32_t* copied = ep.once_per_rank ? ep.arrive + 2 * (ep.num_experts / ep.world) + 2 + le : nullptr;
  if (!ep_wait_sum(ctr, copied, expected, abort_flag, status, budget_ns)) return false;
  ptx::fence_proxy_async_all();   // the rows were written by generic-proxy stores; TMA reads them next
  return true;
}

// Return route of the rows of one local expert, held across the lanes of a warp: lane j keeps
// the start of segment (expert, source j) in the receive buffer (lane W: the expert's end), the
// first row of that segment in source j's return buffer, and source j's return-buffer address.
struct EpRoute {
  int seg_lo, ret_o;
  uint64_t base;
  __device__ __forceinline__ void load(const EpFusedParams& ep, int le, int lane) {
    const int W = ep.world;
    const EpPlanLayout L = ep_plan_layout(ep.num_experts, W);
    seg_lo = lane <= W ? __ldg(ep.plan + L.seg_start + le * (W + 1) + lane) : 0x7fffffff;
    ret_o = lane < W ? __ldg(ep.plan + L.ret_off + le * W + lane) : 0;
    base = lane < W ? __ldg(ep.peer_tab + kTabRet * kEpMaxWorld + lane) : 0ull;
  }
  // Address of the output row for receive-buffer row r (all lanes call; r may differ per lane).
  __device__ __forceinline__ uint64_t row_address(const EpFusedParams& ep, int r) const {
    int src = 0;
    for (int j = 1; j < ep.world; ++j) src += (r >= __shfl_sync(0xffffffffu, seg_lo, j)) ? 1 : 0;
    const int sl = __shfl_sync(0xffffffffu, seg_lo, src);
    const int ro = __shfl_sync(0xffffffffu, ret_o, src);
    const uint64_t b = shfl64(base, src);
    return b + static_cast<uint64_t>(static_cast<uint32_t>(ro + r - sl)) * static_cast<uint64_t>(ep.ret_row_bytes);
  }
};

}  // namespace tkmx
