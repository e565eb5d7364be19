/*
 * tokamax_b200 -- C ABI of the B200 (sm_100a) ragged_dot kernels.
 *
 * Every entry point only ENQUEUES work on the given CUDA stream: it never
 * synchronises, never reads group_sizes on the host and never allocates device
 * memory.  All pointers are device pointers unless stated otherwise.  The return
 * value is a tkmx_status; tkmx_status_string() turns it into text.
 *
 * These are the symbols a binding of the reference's ragged_dot backends binds
 * (an XLA FFI handler, cgo, ctypes ...).  Each declaration names the reference
 * interface it stands in for, by file:line inside openxla/tokamax.
 */
#ifndef TOKAMAX_B200_H_
#define TOKAMAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TKMX_ABI_VERSION 1

#if defined(__GNUC__)
#define TKMX_API __attribute__((visibility("default")))
#else
#define TKMX_API
#endif

typedef enum tkmx_status {
  TKMX_OK = 0,
  TKMX_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, bad enum: reference raises ValueError */
  TKMX_ERR_UNSUPPORTED = 2,      /* legal but not implemented: reference raises NotImplementedError */
  TKMX_ERR_ALIGNMENT = 3,        /* pointer / leading dimension not 16-byte aligned (TMA rule) */
  TKMX_ERR_CUDA = 4,             /* a CUDA runtime / driver call failed; see tkmx_last_cuda_error */
  TKMX_ERR_WORKSPACE = 5,        /* workspace smaller than tkmx_ragged_dot_workspace_bytes says */
  TKMX_ERR_DEVICE_TIMEOUT = 6,   /* reported by tkmx_device_status: a bounded wait in a kernel gave up */
  TKMX_ERR_TOO_LARGE = 7,        /* size beyond a stated static limit */
  TKMX_ERR_DEVICE_STATE = 8      /* reported by tkmx_device_status: a kernel stopped early because its
                                    bookkeeping was inconsistent (tile-counter word shared by two
                                    launches in flight; expert-parallel row outside a receive buffer) */
} tkmx_status;

typedef enum tkmx_dtype {
  TKMX_BF16 = 0,
  TKMX_F16 = 1,
  TKMX_F32 = 2,
  TKMX_F8E4M3 = 3, /* weights only, with per-output-channel fp32 scales */
  TKMX_S8 = 4      /* weights only, with per-output-channel fp32 scales */
} tkmx_dtype;

/* Elementwise activations of tkmx_ragged_dot_fwd_epilogue (codes 1-4 are its gate/up forms). */
enum {
  TKMX_ACT_RELU = 16,
  TKMX_ACT_SILU = 17,
  TKMX_ACT_GELU_TANH = 18,
  TKMX_ACT_GELU_ERF = 19,
  TKMX_ACT_TANH = 20,
  TKMX_ACT_SIGMOID = 21
};

/* Storage order of the grouped right-hand side of the forward product. */
typedef enum tkmx_rhs_layout {
  TKMX_RHS_GKN = 0, /* rhs[g, k, n], n contiguous: the reference's logical layout */
  TKMX_RHS_GNK = 1  /* rhs[g, n, k], k contiguous: what the reference's Mosaic kernel is fed
                       after its `rhs.mT` (pallas_mosaic_gpu_kernel_sm100.py:259-269) */
} tkmx_rhs_layout;

/*
 * Kernel configuration.  Mirrors the fields of the reference's `Config`
 * (tokamax/_src/ops/ragged_dot/pallas_mosaic_gpu_common.py:45-73) that have a
 * meaning for these kernels.  A zero field means "library default".
 */
typedef struct tkmx_config {
  int32_t block_m;         /* output rows per tile: 128 */
  int32_t block_n;         /* output columns per tile: 64, 128 or 256 */
  int32_t block_k;         /* contraction elements per pipeline stage: 64 */
  int32_t num_stages;      /* shared-memory ring depth; 0 = as deep as fits */
  int32_t collective;      /* 1 = two CTAs of a cluster cooperate on one 256-row tile */
  int32_t grid_minor_dim;  /* 0 = M tiles vary fastest, 1 = N tiles (MatmulDimension) */
  int32_t grid_tile_width; /* rasterisation band width, >= 1 */
  int32_t max_ctas;        /* 0 = one persistent CTA per SM */
} tkmx_config;

/* Library / ABI identification (host only, no CUDA call). */
TKMX_API int tkmx_abi_version(void);
TKMX_API const char* tkmx_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
TKMX_API const char* tkmx_last_cuda_error(void);

/*
 * Scratch the caller must pass for a given problem; a pure function of shapes and
 * config (no CUDA call), so a tracing caller can size a result buffer for it.
 * `op`: 0 = fwd, 1 = dlhs, 2 = drhs.
 * Today only the forward with F8E4M3 weights has scratch (2 * m * k + 4 * m bytes plus
 * padding): the activations split into two e4m3 planes with one scale per row, which lets
 * the fp8 tensor cores read the weights as stored.  The workspace is optional: with a NULL
 * or short workspace (or k % 16 != 0) that call expands the weights to bf16 on the fly
 * instead, which is slower but needs no scratch.  256-byte alignment is required.
 */
TKMX_API size_t tkmx_ragged_dot_workspace_bytes(int op, int64_t m, int64_t k, int64_t n, int64_t g,
                                       int rhs_dtype, const tkmx_config* config);

/*
 * Forward: out[i, :] = lhs[i, :] @ rhs[group(i)] for i < sum(group_sizes), 0 for the
 * remaining rows (jax.lax.ragged_dot semantics).
 * Replaces RaggedDot._fwd with the default dimension numbers
 * (tokamax/_src/ops/ragged_dot/base.py:291-360) as served on B200 by
 * PallasMosaicGpuRaggedDot._fwd (pallas_mosaic_gpu.py:103-244) and the sm100 kernel
 * (pallas_mosaic_gpu_kernel_sm100.py:38-269).
 *   lhs          [m, k]      lhs_dtype (BF16 or F16), row-major
 *   rhs          [g, k, n] or [g, n, k] per rhs_layout; rhs_dtype = lhs_dtype, or
 *                F8E4M3 / S8 with rhs_scale
 *   group_sizes  int32[g] (uint32 values < 2^31 are the same bits)
 *   rhs_scale    float[g, n] per-output-channel scale, or NULL for unquantised rhs
 *   out          [m, n]      out_dtype (BF16, F16 or F32)
 */
TKMX_API int tkmx_ragged_dot_fwd(const void* lhs, const void* rhs, const int32_t* group_sizes,
                        const float* rhs_scale, void* out, void* workspace,
                        size_t workspace_bytes, int64_t m, int64_t k, int64_t n, int64_t g,
                        int lhs_dtype, int rhs_dtype, int out_dtype, int rhs_layout,
                        const tkmx_config* config, void* cuda_stream);

/*
 * Forward with the gate/up activation fused into the epilogue:
 *   tmp = ragged_dot(lhs, rhs);  out[:, j] = act(tmp[:, j]) * tmp[:, n/2 + j],  j < n/2
 * i.e. rhs [g, k, n] holds the gate projection in its first n/2 columns and the up
 * projection in the rest, and out is [m, n/2].  Replaces `fuse_gateup_activation` of
 * RaggedDot (tokamax/_src/ops/ragged_dot/base.py:211-217), formulas of
 * tokamax/_src/ops/experimental/gmm_v2/gmm_v2.py:29-48 and :92-108, computed in float32 on
 * the accumulator.  activation: 1 = silu, 2 = gelu (tanh form, also "gelu_tanh"),
 * 3 = swigluoai (alpha 1.702, limit 7), 4 = silu_and_mul_with_clamp (limit 10).
 * lhs / rhs in one 16-bit dtype; block_n of the config must be 128 or 256.
 */
TKMX_API int tkmx_ragged_dot_fwd_gateup(const void* lhs, const void* rhs, const int32_t* group_sizes,
                                        void* out, int64_t m, int64_t k, int64_t n, int64_t g,
                                        int in_dtype, int out_dtype, int activation,
                                        const tkmx_config* config, void* cuda_stream);

/*
 * Forward with an epilogue: tmp = ragged_dot(lhs, rhs) + rhs_bias[group] (rows of no group
 * stay zero), then either out = tmp (activation 0), or the gate/up activation of
 * tkmx_ragged_dot_fwd_gateup on tmp (activation 1-4, rhs_layout GKN only, out [m, n/2]), or an
 * elementwise activation of tmp computed in float32 before the cast to out_dtype (activation
 * TKMX_ACT_RELU ... TKMX_ACT_SIGMOID, 16-bit weights only): the `activation=` argument of
 * ragged_dot (tokamax/_src/ops/ragged_dot/api.py:84,108-113).
 *   rhs_scale  float[g, n] with F8E4M3 weights (then the workspace of
 *              tkmx_ragged_dot_workspace_bytes is required: the epilogue extras live in the
 *              native fp8 kernel; n/2 must be a multiple of 16 for the gate/up form), else NULL
 *   rhs_bias   float[g, n] or NULL
 * Replaces `rhs_bias` and `fuse_gateup_activation` of RaggedDot
 * (tokamax/_src/ops/ragged_dot/base.py:207-217; reference arithmetic gmm_v2_test.py:44-99:
 * the scale multiplies and the bias is added to the float32 product of its group).
 */
TKMX_API int tkmx_ragged_dot_fwd_epilogue(const void* lhs, const void* rhs, const int32_t* group_sizes,
                                          const float* rhs_scale, const float* rhs_bias, void* out,
                                          void* workspace, size_t workspace_bytes, int64_t m, int64_t k,
                                          int64_t n, int64_t g, int lhs_dtype, int rhs_dtype,
                                          int out_dtype, int rhs_layout, int activation,
                                          const tkmx_config* config, void* cuda_stream);

/*
 * Forward with the output quantised in the epilogue: tmp = act(ragged_dot(lhs, rhs) + rhs_bias)
 * in float32, then per row and block of `subchannel` columns (64, 128 or 256; divides n and
 * the tile width) scale = max|tmp| / 448 (1 for an all-zero block) and
 * q = e4m3(clip(tmp / scale, -448, 448)): out_q uint8 [m, n] (e4m3 bits), out_scale float
 * [m, n / subchannel].  Rows of no group give q = 0, scale = 1.  The float32 product never
 * reaches memory.  Replaces the fused epilogue quantisation of the reference's Blackwell
 * quant kernel (`epilogue_quant_qtype` / `epilogue_quant_subchannel_size`,
 * tokamax/_src/ops/ragged_dot/pallas_mosaic_gpu_common.py:63-68; rule of
 * pallas_mosaic_gpu_kernel_sm100_fp8_quant.py:800-844), here on the 16-bit kernel.
 * activation: 0 or TKMX_ACT_*.
 */
TKMX_API int tkmx_ragged_dot_fwd_quant_out(const void* lhs, const void* rhs, const int32_t* group_sizes,
                                           const float* rhs_bias, void* out_q, float* out_scale, int64_t m,
                                           int64_t k, int64_t n, int64_t g, int in_dtype, int rhs_layout,
                                           int activation, int subchannel, const tkmx_config* config,
                                           void* cuda_stream);

/*
 * dlhs[i, :] = dout[i, :] @ rhs[group(i)]^T  (contraction over n; rhs read as stored,
 * no transpose pass).  Replaces the dlhs_ragged_dot call of `vjp`
 * (tokamax/_src/ops/ragged_dot/base.py:434-446, TRANS_RHS dimension numbers
 * base.py:45-49), served upstream by the forward kernel after `rhs.mT`
 * (pallas_mosaic_gpu.py:148-150).
 *   dout [m, n], rhs [g, k, n], dlhs [m, k]; rows >= sum(group_sizes) are 0.
 */
TKMX_API int tkmx_ragged_dot_dlhs(const void* dout, const void* rhs, const int32_t* group_sizes,
                         void* dlhs, void* workspace, size_t workspace_bytes, int64_t m,
                         int64_t k, int64_t n, int64_t g, int in_dtype, int out_dtype,
                         const tkmx_config* config, void* cuda_stream);

/*
 * drhs[g] = lhs[rows of g]^T @ dout[rows of g]  (zeros for empty groups): the ragged
 * dimension is the contraction ("tgmm").  Replaces the drhs_ragged_dot call of `vjp`
 * (tokamax/_src/ops/ragged_dot/base.py:448-461, RAGGED_CONTRACTING dimension numbers
 * base.py:50-54); upstream kernels: pallas_mosaic_gpu_kernel_sm90.py:184-285 (Hopper
 * only) and pallas_triton.py:238-333.
 *   lhs [m, k], dout [m, n], drhs [g, k, n].
 */
TKMX_API int tkmx_ragged_dot_drhs(const void* lhs, const void* dout, const int32_t* group_sizes,
                         void* drhs, void* workspace, size_t workspace_bytes, int64_t m,
                         int64_t k, int64_t n, int64_t g, int in_dtype, int out_dtype,
                         const tkmx_config* config, void* cuda_stream);

/*
 * tkmx_ragged_dot_drhs for an expert-parallel shard: group_sizes counts all g groups of the
 * global problem, but only the groups [group_begin, group_begin + group_count) are contracted,
 * into drhs [group_count, k, n] (slab j = group group_begin + j).  The `num_actual_groups` /
 * `group_offset` pair of the reference's tgmm (tokamax/_src/ops/ragged_dot/pallas_mosaic_tpu_v2.py:89-93,
 * arithmetic of reference_tgmm, tokamax/_src/ops/experimental/gmm_v2/gmm_v2_test.py:109-160).
 */
TKMX_API int tkmx_ragged_dot_drhs_window(const void* lhs, const void* dout, const int32_t* group_sizes,
                                         void* drhs, int64_t m, int64_t k, int64_t n, int64_t g,
                                         int64_t group_begin, int64_t group_count, int in_dtype,
                                         int out_dtype, const tkmx_config* config, void* cuda_stream);

/*
 * Group bookkeeping as its own kernel, for callers (and tests) that need the arrays:
 * the tile table the reference computes with XLA ops before its kernel
 * (GroupInfo.create_aligned, pallas_mosaic_gpu_common.py:88-151).  All outputs are
 * int32[num_tasks] on the device.
 */
TKMX_API int tkmx_group_info_aligned(const int32_t* group_sizes, int64_t g, int32_t tile,
                            int32_t num_tasks, int32_t align_tile, int32_t* group_id,
                            int32_t* block_start, int32_t* actual_start, int32_t* actual_end,
                            int32_t* start_within_block, int32_t* actual_size,
                            void* cuda_stream);

/*
 * Forward over "cyclic" groups: group_sizes has num_segments entries and segment i is
 * multiplied by rhs[i % g_rhs].  This is the order in which an expert-parallel rank
 * receives token rows from an all-to-all -- (source rank, local expert) -- so the rows can
 * be consumed as they land, without a reorder pass.  With num_segments == g_rhs it is
 * tkmx_ragged_dot_fwd.  zero_initialize = 0 leaves the rows past sum(group_sizes) untouched
 * (the `zero_initialize=False` of tokamax/_src/ops/ragged_dot/base.py:208-209), for
 * receive buffers sized for the worst case.  Only the segments in
 * [segment_begin, segment_begin + segment_count) are computed (segment_count < 0: to the
 * end); the row offsets still count every segment, so a caller can process a buffer expert
 * chunk by expert chunk while later chunks are still arriving -- the `group_offset` idea of
 * tokamax/_src/ops/ragged_dot/pallas_mosaic_tpu_kernel.py:85-86.  The reference has no counterpart (its expert-parallel
 * affordance is `group_offset`, tokamax/_src/ops/ragged_dot/pallas_mosaic_tpu_kernel.py:85-86,
 * which every GPU backend rejects, api.py:183-184).
 * workspace / workspace_bytes: as for tkmx_ragged_dot_fwd (sized for the same m, k), or NULL / 0.
 */
TKMX_API int tkmx_ragged_dot_fwd_cyclic(const void* lhs, const void* rhs, const int32_t* group_sizes,
                                        const float* rhs_scale, void* out, int64_t m, int64_t k,
                                        int64_t n, int64_t num_segments, int64_t g_rhs, int lhs_dtype,
                                        int rhs_dtype, int out_dtype, int rhs_layout,
                                        int zero_initialize, int64_t segment_begin,
                                        int64_t segment_count, const tkmx_config* config,
                                        void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * MoE dispatch: stable counting sort of (token, choice) pairs by expert id.
 *   expert_ids     int32[num_pairs]   (pair p = token p / top_k, choice p % top_k)
 *   pos            int32[num_pairs]   position of pair p in expert-sorted order
 *                                     (-1 for ids outside [0, num_experts))
 *   expert_counts  int32[num_experts] pairs per expert (the group_sizes of the GEMM)
 *   workspace      tkmx_moe_sort_workspace_bytes(num_pairs, num_experts) bytes of scratch
 * num_experts <= 1024.  Deterministic.  Plays the role of the argsort / bincount that a
 * caller of the reference does in JAX before ragged_dot.
 */
TKMX_API size_t tkmx_moe_sort_workspace_bytes(int64_t num_pairs, int32_t num_experts);
TKMX_API int tkmx_moe_sort_pairs(const int32_t* expert_ids, int64_t num_pairs, int32_t num_experts,
                                 int32_t* pos, int32_t* expert_counts, void* workspace,
                                 size_t workspace_bytes, void* cuda_stream);

/*
 * tkmx_moe_sort_pairs for callers that have no device memory to lend: same inputs, same
 * outputs, bit for bit, but no workspace argument.  (No counterpart in the reference; it is
 * an addition of this library.)
 *
 * Who needs it: a host that handed every byte of device memory to its own arena when it
 * started (so a later cudaMalloc fails), or an XLA / framework custom-call handler that was
 * not given a scratch buffer and is not allowed to create one while it runs.  The histogram
 * matrix the sort needs is therefore a fixed 1 MiB array inside the library image; every GPU
 * that loads the library carries it until the process exits.
 *
 * Limits and rules:
 *   - ceil(num_pairs / 1024) * num_experts must not exceed 262144 (for example 1,048,576
 *     pairs over 256 experts, or 262,144 pairs over 1024); beyond that the call returns
 *     TKMX_ERR_TOO_LARGE, with the reason in tkmx_last_cuda_error(), and enqueues nothing.
 *   - The call allocates nothing (no cudaMalloc / cudaFree, no allocating library routine).
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture.  If it is also the
 *     process's first use of this library on that device, it is when the CUDA runtime loads
 *     the library image -- and with it this array and the library's other static device
 *     arrays -- into device memory: a host that is about to claim all remaining device memory
 *     for its own arena must make that first call before it does.
 *   - All calls on a device share the one array, which keeps whatever the previous call left
 *     in it.  Nothing in it has to start at zero: every entry a call reads was written by that
 *     same call first.  Two calls that may overlap on the GPU (different streams) race on it;
 *     serialise them, or give one of them tkmx_moe_sort_pairs with its own workspace.
 */
TKMX_API int tkmx_moe_sort_pairs_static(const int32_t* expert_ids, int64_t num_pairs,
                                        int32_t num_experts, int32_t* pos, int32_t* expert_counts,
                                        void* cuda_stream);

/*
 * dst[pos[p], :] = src[p / top_k, :] for every pair with pos[p] >= 0; rows of row_bytes
 * bytes (a multiple of 16).  ragged_gather (tokamax/_src/ops/ragged_gather/base.py:26-30).
 */
TKMX_API int tkmx_moe_gather_rows(const void* src, const int32_t* pos, void* dst, int64_t num_pairs,
                                  int32_t top_k, int64_t row_bytes, void* cuda_stream);

/*
 * tkmx_moe_sort_pairs that also returns the inverse permutation: sorted_pair[pos[p]] = p for
 * every pair with pos[p] >= 0 (int32[num_pairs]; entries past the number of valid pairs are
 * not written; NULL = not wanted).  The row order the expert-parallel kernel sends in.
 */
TKMX_API int tkmx_moe_sort_pairs_inverse(const int32_t* expert_ids, int64_t num_pairs, int32_t num_experts,
                                         int32_t* pos, int32_t* sorted_pair, int32_t* expert_counts,
                                         void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Expert-parallel MoE layer over peer-mapped GPU memory (one process per GPU on one NVLink /
 * NVSwitch domain).  No reference counterpart: upstream leaves sharding to the caller's
 * shard_map and only offers `group_offset` / `num_actual_groups`
 * (tokamax/_src/ops/ragged_dot/pallas_mosaic_tpu_v2.py:89-93); these entry points replace the
 * all-to-all + ragged_gather + ragged_dot + all-to-all + ragged_gather_reduce sequence such a
 * caller writes.  Experts are sharded contiguously, rank r owning [r * G/W, (r + 1) * G/W).
 *
 * Buffers every rank allocates in memory its peers can address, with the same sizes everywhere:
 *   recv     [capacity_rows, k]  token rows this rank's experts receive, (local expert, source) order
 *   arrive   uint32[G/W + 2]     rows arrived per local expert; the last two words are this rank's
 *                                multiplication progress and the cursor its senders draw work from
 *   ret      [T * top_k, n]      this rank's pairs' output rows in expert-sorted order
 *   counts   int32[W, G]         every rank's per-expert pair counts
 *   flags    uint32[W]           barrier flags, zero before the first call
 * peer_table is a DEVICE array uint64[5][16]: entry [t][r] = address of buffer t (0 recv,
 * 1 arrive, 2 ret, 3 counts, 4 flags) of rank r as mapped into this process.  W <= 16, G <= 1024.
 *
 * One step on every rank, all on one stream:
 *   tkmx_moe_sort_pairs_inverse -> tkmx_ep_exchange_plan -> tkmx_ep_moe_fused
 *   -> tkmx_cross_rank_barrier -> tkmx_moe_combine(ret, pos, gates)
 *
 * Every cross-rank wait is bounded: a flag wait gives up after timeout_ns, a wait for rows after
 * 2 s; the kernel then records a code (tkmx_device_status returns TKMX_ERR_DEVICE_TIMEOUT) and
 * returns, leaving the context usable.  `sequence` must grow by one per barrier call, the same
 * on every rank (tkmx_ep_exchange_plan contains one barrier).
 */
TKMX_API size_t tkmx_ep_plan_bytes(int32_t num_experts, int32_t world);

/* Pushes my_counts (int32[G], from the sort) into row `rank` of every rank's counts matrix,
 * zeroes this rank's arrival counters, passes the flag barrier (which also orders this step
 * after every rank's previous one), and fills `plan` (tkmx_ep_plan_bytes) from the complete
 * matrix.  One CTA. */
TKMX_API int tkmx_ep_exchange_plan(const int32_t* my_counts, const uint64_t* peer_table,
                                   int32_t* counts_all_local, uint32_t* flags_local, uint32_t* arrive_local,
                                   int32_t* plan, int32_t num_experts, int32_t world, int32_t rank,
                                   uint32_t sequence, int64_t timeout_ns, void* cuda_stream);

/* The fused kernel: while two warps of every CTA copy this rank's token rows (tokens
 * [num_tokens, k], order given by sorted_pair and plan) into the owners' recv buffers and bump
 * their arrival counters, the other warps multiply the rows that have arrived in recv_local by
 * rhs_local [G/W, k, n] (tcgen05 / TMEM / TMA pipeline of tkmx_ragged_dot_fwd) and store every
 * finished row into its source rank's ret buffer.  phases: 1 = send only, 2 = multiply and
 * return only (everything must have arrived), 3 = both (the product form).  dtype BF16 or F16;
 * k and n multiples of 8.  Only config->collective, num_stages, grid_* and max_ctas are used. */
TKMX_API int tkmx_ep_moe_fused(const void* tokens, const int32_t* sorted_pair, const void* recv_local,
                               const void* rhs_local, const int32_t* plan, const uint64_t* peer_table,
                               const uint32_t* arrive_local, int64_t num_tokens, int32_t top_k, int64_t k,
                               int64_t n, int32_t num_experts, int32_t world, int32_t rank,
                               int64_t capacity_rows, int dtype, int phases, const tkmx_config* config,
                               void* cuda_stream);

/* The same step with every token crossing the link ONCE PER DESTINATION RANK instead of once per
 * (token, expert) pair: of a token's pairs on one rank only the one with the lowest expert is
 * sent; for the others the sender writes a 4-byte reference into the owner's `refs` buffer and
 * two warps per CTA of the owner copy the row inside the owner's memory once the original is
 * complete.  With top-8 routing over 8 ranks a token has 4.6 distinct remote owners against 7
 * remote pairs, so a third of the dispatch bytes stay off the link.  Differences to the calls
 * above, on every rank alike:
 *   - one more peer-mapped buffer, refs uint32[capacity_rows], in row 5 of peer_table
 *     (uint64[6][16]);
 *   - arrive has tkmx_ep_arrive_words(G, W, 1) = 3 G/W + 3 words, and the plan call is
 *     tkmx_ep_exchange_plan_words(..., once_per_rank = 1), which resets all of them;
 *   - expert_ids [num_tokens, top_k] (the ids the pairs were sorted by) and pair_pos (the `pos`
 *     output of tkmx_moe_sort_pairs_inverse) are read by the senders;
 *   - phases: bit 2 (4) = copy duplicates; the product form is 7.
 * G/W <= 254 and capacity_rows <= 2^24, else TKMX_ERR_UNSUPPORTED.  With expert_ids and pair_pos
 * both NULL the call is tkmx_ep_moe_fused. */
TKMX_API size_t tkmx_ep_arrive_words(int32_t num_experts, int32_t world, int32_t once_per_rank);
TKMX_API int tkmx_ep_exchange_plan_words(const int32_t* my_counts, const uint64_t* peer_table,
                                         int32_t* counts_all_local, uint32_t* flags_local,
                                         uint32_t* arrive_local, int32_t* plan, int32_t num_experts,
                                         int32_t world, int32_t rank, uint32_t sequence, int64_t timeout_ns,
                                         int32_t once_per_rank, void* cuda_stream);
TKMX_API int tkmx_ep_moe_fused_once_per_rank(const void* tokens, const int32_t* sorted_pair,
                                             const int32_t* expert_ids, const int32_t* pair_pos,
                                             const void* recv_local, const void* rhs_local, const int32_t* plan,
                                             const uint64_t* peer_table, const uint32_t* arrive_local,
                                             int64_t num_tokens, int32_t top_k, int64_t k, int64_t n,
                                             int32_t num_experts, int32_t world, int32_t rank,
                                             int64_t capacity_rows, int dtype, int phases,
                                             const tkmx_config* config, void* cuda_stream);

/* Flag barrier across the ranks on the stream (one warp): all earlier work of this stream on
 * every rank is complete and visible when the kernel ends. */
TKMX_API int tkmx_cross_rank_barrier(const uint64_t* peer_table, uint32_t* flags_local, int32_t world,
                                     int32_t rank, uint32_t sequence, int64_t timeout_ns, void* cuda_stream);

/*
 * y[t, :] = sum_k gates[t, k] * rows[pos[t * top_k + k], :], accumulated in float32 in
 * ascending k, rows and y in `dtype` (BF16), n a multiple of 8.
 * ragged_gather_reduce (tokamax/_src/ops/ragged_gather_reduce/base.py:26-37).
 */
TKMX_API int tkmx_moe_combine(const void* rows, const int32_t* pos, const float* gates, void* y,
                              int64_t num_tokens, int32_t top_k, int64_t n, int dtype,
                              void* cuda_stream);

/*
 * out[i, :] = x[indices[i], :] for i < out_rows; rows are `row_bytes` long (a multiple of
 * 16, any dtype).  Negative indices count from the end, out-of-range ones are clamped
 * (array indexing of `x[indices]`).  Replaces ragged_gather
 * (tokamax/_src/ops/ragged_gather/base.py:26-30); `start` / `end`, which that function
 * ignores, are not parameters here.
 */
TKMX_API int tkmx_ragged_gather(const void* x, const int32_t* indices, void* out, int64_t in_rows,
                                int64_t out_rows, int64_t row_bytes, void* cuda_stream);

/*
 * out[i, :] = (start[0] <= indices[i] < end[0]) ? x[indices[i], :] : 0; start / end are
 * device int32 scalars.  Replaces ragged_scatter
 * (tokamax/_src/ops/ragged_scatter/base.py:26-36).
 */
TKMX_API int tkmx_ragged_scatter(const void* x, const int32_t* indices, const int32_t* start,
                                 const int32_t* end, void* out, int64_t in_rows, int64_t out_rows,
                                 int64_t row_bytes, void* cuda_stream);

/*
 * out[t, :] = sum_{j < reduce_group_size} (mask[p] ? weights[p] * x[indices[p], :] : 0) with
 * p = t * reduce_group_size + j, accumulated in float32 in ascending j; x and out in `dtype`
 * (BF16), hidden a multiple of 8; mask is one byte per row (NULL = all valid); input_size
 * must be a multiple of reduce_group_size.  Replaces ragged_gather_reduce
 * (tokamax/_src/ops/ragged_gather_reduce/base.py:26-37).
 */
TKMX_API int tkmx_ragged_gather_reduce(const void* x, const int32_t* indices, const float* weights,
                                       const uint8_t* mask, void* out, int64_t in_rows,
                                       int64_t input_size, int32_t reduce_group_size, int64_t hidden,
                                       int dtype, void* cuda_stream);

/*
 * Debug / test aid (SYNCHRONISES the current device): reads the status word kernels
 * write when a bounded wait gives up, returns it as a tkmx_status and clears it.
 */
TKMX_API int tkmx_device_status(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* TOKAMAX_B200_H_ */
