// C ABI of the B200 ragged_dot kernels (declared in include/tokamax_b200.h): argument
// checks, TMA tensor-map encoding and kernel launches.  No torch, no allocation, no
// synchronisation on the data path.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/tokamax_b200.h"
#include "group_info_sm100.cuh"
#include "moe_dispatch_sm100.cuh"
#include "ragged_gemm_sm100.cuh"
#include "ragged_gemm_f8_sm100.cuh"
#include "ragged_gemm_w8_sm100.cuh"

namespace {

using tkmx::GemmMode;
using tkmx::RaggedGemmParams;

thread_local std::string g_last_cuda_error;

int cuda_fail(cudaError_t e, const char* where) {
  g_last_cuda_error = std::string(where) + ": " + cudaGetErrorString(e);
  return TKMX_ERR_CUDA;
}

#define TKMX_CUDA_OK(expr)                                  \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) return cuda_fail(_e, #expr);     \
  } while (0)

// Device status word written by kernels whose bounded waits give up.
__device__ int32_t g_device_status;
// Tile counters for dynamically scheduled launches: (epoch << 32 | next tile) words, one per
// launch in flight, handed out round-robin by launch number.  A word is reset by the first
// CTA of a launch that finds another epoch in it, so nothing is cleaned up afterwards.
constexpr int kSchedWords = 1024;
__device__ unsigned long long g_sched_words[2 * kSchedWords];   // per launch: {counter, units finished}

constexpr int kMaxDevices = 64;
constexpr int kMaxSmemOptin = 232448;  // 227 KiB, sm_100

struct DeviceInfo {
  bool ready = false;
  int num_sms = 0;
  int smem_optin = 0;
  int32_t* status_ptr = nullptr;
  unsigned long long* sched_words = nullptr;
};
DeviceInfo g_devices[kMaxDevices];
std::mutex g_mutex;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_device_info(DeviceInfo** out) {
  int dev = 0;
  TKMX_CUDA_OK(cudaGetDevice(&dev));
  // A thread that has made no runtime call yet (an autograd worker, a thread pool) may
  // have no driver context bound, and cuTensorMapEncodeTiled needs one: bind the primary
  // context of the current device.  Cheap when it is already current.
  TKMX_CUDA_OK(cudaSetDevice(dev));
  if (dev < 0 || dev >= kMaxDevices) return TKMX_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_devices[dev];
  if (!d.ready) {
    int major = 0;
    TKMX_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) {
      g_last_cuda_error = "tokamax_b200 kernels need an sm_100 device";
      return TKMX_ERR_UNSUPPORTED;
    }
    TKMX_CUDA_OK(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev));
    TKMX_CUDA_OK(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    void* sym = nullptr;
    TKMX_CUDA_OK(cudaGetSymbolAddress(&sym, g_device_status));
    d.status_ptr = static_cast<int32_t*>(sym);
    TKMX_CUDA_OK(cudaMemset(d.status_ptr, 0, sizeof(int32_t)));
    TKMX_CUDA_OK(cudaGetSymbolAddress(&sym, g_sched_words));
    d.sched_words = static_cast<unsigned long long*>(sym);
    d.ready = true;
  }
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    TKMX_CUDA_OK(cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000,
                                                  cudaEnableDefault, &q));
    if (fn == nullptr || q != cudaDriverEntryPointSuccess) {
      g_last_cuda_error = "cuTensorMapEncodeTiled not available from the driver";
      return TKMX_ERR_CUDA;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = &d;
  return TKMX_OK;
}

// Encodes a 128B-swizzled tiled map over a row-major tensor (16-bit by default); dims / box are
// innermost first, strides (bytes) are for dims 1..rank-1.
int encode_map(CUtensorMap* map, const void* ptr, int rank, const uint64_t* dims,
               const uint64_t* strides, const uint32_t* box,
               CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
               CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_256B) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return TKMX_ERR_ALIGNMENT;
  for (int i = 0; i + 1 < rank; ++i)
    if (strides[i] % 16 != 0) return TKMX_ERR_ALIGNMENT;
  cuuint64_t gdim[3];
  cuuint64_t gstr[2];
  cuuint32_t gbox[3];
  cuuint32_t estr[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides[i];
  CUresult r = g_encode(map, dtype, rank, const_cast<void*>(ptr), gdim,
                        gstr, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r));
    return TKMX_ERR_CUDA;
  }
  return TKMX_OK;
}

// Tuning knobs with an environment override for experiments
// (read on every call; a handful of getenv calls per launch is noise next to the launch).
int env_int(const char* name, int fallback, int lo, int hi) {
  int v = fallback;
  if (const char* e = std::getenv(name)) v = std::atoi(e);
  return v < lo ? lo : (v > hi ? hi : v);
}
// Gives a launch its tile-counter word and epoch (see g_sched_words).  Dynamic scheduling is
// the default for the forward and dlhs (measured +0 ... +5 % on B200) and for drhs with long
// groups; TKMX_DYNAMIC=0 / 1 forces either for every contraction.
std::atomic<uint32_t> g_launch_seq{0};
void assign_sched(const DeviceInfo& dev, RaggedGemmParams* p, bool default_on) {
  p->sched_slot = nullptr;
  p->sched_epoch = 0;
  if (env_int("TKMX_DYNAMIC", default_on ? 1 : 0, 0, 1) == 0 || dev.sched_words == nullptr) return;
  uint32_t seq = ++g_launch_seq;
  if (seq == 0) seq = ++g_launch_seq;   // epoch 0 is what a fresh word holds
  // TKMX_SCHED_SLOT pins the word (tests: two launches on one word must end with an error
  // status, not with silently skipped tiles).
  const int forced = env_int("TKMX_SCHED_SLOT", -1, -1, kSchedWords - 1);
  p->sched_slot = dev.sched_words + 2 * (forced >= 0 ? uint32_t(forced) : seq % kSchedWords);
  p->sched_epoch = seq;
}

struct ResolvedConfig {
  int block_n;
  bool pair;
  int num_stages;
  int minor_is_m;
  int tile_width;
  int max_ctas;
};

int resolve_config(const tkmx_config* c, int64_t cols, int num_groups, bool need_tile_start,
                   const DeviceInfo& dev, ResolvedConfig* out) {
  tkmx_config d = {};
  if (c != nullptr) d = *c;
  if (d.block_m != 0 && d.block_m != 128) return TKMX_ERR_UNSUPPORTED;
  if (d.block_k != 0 && d.block_k != 64) return TKMX_ERR_UNSUPPORTED;
  if (d.collective != 0 && d.collective != 1) return TKMX_ERR_INVALID_ARGUMENT;
  const bool pair = d.collective == 1;
  int bn = d.block_n;
  if (bn == 0) bn = cols > 128 ? 256 : (cols > 64 || pair ? 128 : 64);
  if (bn != 64 && bn != 128 && bn != 256) return TKMX_ERR_UNSUPPORTED;
  if (pair && bn < 128) return TKMX_ERR_UNSUPPORTED;  // each CTA of a pair loads >= 64 B columns
  if (d.grid_minor_dim != 0 && d.grid_minor_dim != 1) return TKMX_ERR_INVALID_ARGUMENT;
  if (d.grid_tile_width < 0 || d.num_stages < 0 || d.max_ctas < 0) return TKMX_ERR_INVALID_ARGUMENT;
  const int smem_cap = dev.smem_optin < kMaxSmemOptin ? dev.smem_optin : kMaxSmemOptin;
  int stages = d.num_stages;
  if (stages == 0) {
    // Measured on B200: deeper rings than this do not help and cost a little (the
    // kernels saturate at 4-5 stages of 64).
    stages = pair ? 5 : 4;
    while (stages > 1 &&
           tkmx::make_smem_layout(bn, pair, stages, num_groups, need_tile_start).total + 1024 > (uint32_t)smem_cap)
      --stages;
  }
  if (stages > 16) return TKMX_ERR_UNSUPPORTED;
  if (tkmx::make_smem_layout(bn, pair, stages, num_groups, need_tile_start).total + 1024 > (uint32_t)smem_cap)
    return TKMX_ERR_TOO_LARGE;
  out->block_n = bn;
  out->pair = pair;
  out->num_stages = stages;
  out->minor_is_m = d.grid_minor_dim == 0 ? 1 : 0;
  out->tile_width = d.grid_tile_width == 0 ? 1 : d.grid_tile_width;
  out->max_ctas = d.max_ctas;
  return TKMX_OK;
}

// The opt-in shared-memory limit of a kernel is raised once per (device, kernel) to the
// device maximum, under the mutex: setting it per launch to that launch's size would let two
// host threads with different ring depths lower it under each other.
int raise_smem_limit_impl(const void* kernel) {
  static std::vector<std::pair<const void*, int>> done;   // (kernel, device) pairs already raised
  int dev = 0;
  TKMX_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TKMX_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  for (const auto& d : done)
    if (d.first == kernel && d.second == dev) return TKMX_OK;
  const int cap = g_devices[dev].smem_optin > 0 && g_devices[dev].smem_optin < kMaxSmemOptin
                      ? g_devices[dev].smem_optin : kMaxSmemOptin;
  TKMX_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
  done.emplace_back(kernel, dev);
  return TKMX_OK;
}
template <typename Kernel>
int raise_smem_limit(Kernel kernel, int /*smem_needed*/) {
  return raise_smem_limit_impl(reinterpret_cast<const void*>(kernel));
}

template <int kMode, int kBlockN, bool kPair, bool kEp = false>
int launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo,
               const RaggedGemmParams& p, int grid, cudaStream_t stream,
               const tkmx::EpFusedParams& ep = tkmx::EpFusedParams{}) {
  auto kernel = tkmx::ragged_gemm_kernel<kMode, kBlockN, kPair, kEp>;
  const bool need_ts = kMode != tkmx::kContract;
  const int smem =
      tkmx::make_smem_layout(kBlockN, kPair, p.num_stages, p.num_groups, need_ts, kEp ? ep.num_experts : 0).total + 1024;
  {
    const int st = raise_smem_limit(kernel, smem);
    if (st != TKMX_OK) return st;
  }
  cudaLaunchConfig_t cfg = {};
  constexpr int kThreads = kEp ? tkmx::kEpNumThreads : tkmx::kNumThreads;
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if constexpr (kEp) {
    // In the expert-parallel form CTAs wait for rows that other CTAs of the same grid send, so
    // the whole grid has to be resident at once: never launch more CTAs than fit together.
    int fit = 0;
    if constexpr (kPair) {
      int clusters = 0;
      TKMX_CUDA_OK(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
      fit = clusters * 2;
    } else {
      int per_sm = 0, dev = 0, sms = 0;
      TKMX_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem));
      TKMX_CUDA_OK(cudaGetDevice(&dev));
      TKMX_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      fit = per_sm * sms;
    }
    if (fit < (kPair ? 2 : 1)) {
      g_last_cuda_error = "the expert-parallel kernel does not fit on this device";
      return TKMX_ERR_CUDA;
    }
    if (grid > fit) cfg.gridDim = dim3(fit, 1, 1);
  }
  TKMX_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, p, ep));
  return TKMX_OK;
}

template <int kMode>
int launch_mode(int block_n, bool pair, const CUtensorMap& ma, const CUtensorMap& mb,
                const CUtensorMap& mo, const RaggedGemmParams& p, int grid, cudaStream_t stream) {
  if (pair) {
    switch (block_n) {
      case 128: return launch_one<kMode, 128, true>(ma, mb, mo, p, grid, stream);
      case 256: return launch_one<kMode, 256, true>(ma, mb, mo, p, grid, stream);
    }
    return TKMX_ERR_UNSUPPORTED;
  }
  switch (block_n) {
    case 64: return launch_one<kMode, 64, false>(ma, mb, mo, p, grid, stream);
    case 128: return launch_one<kMode, 128, false>(ma, mb, mo, p, grid, stream);
    case 256: return launch_one<kMode, 256, false>(ma, mb, mo, p, grid, stream);
  }
  return TKMX_ERR_UNSUPPORTED;
}

// Persistent grid: one CTA per SM (an even number of them when CTAs work in pairs),
// never more CTAs than there can be tiles.
int grid_size(const DeviceInfo& dev, const ResolvedConfig& rc, int64_t max_tiles) {
  int64_t ctas = dev.num_sms;
  if (rc.max_ctas > 0 && rc.max_ctas < ctas) ctas = rc.max_ctas;
  if (rc.pair) {
    int64_t pairs = ctas / 2;
    if (max_tiles < pairs) pairs = max_tiles;
    if (pairs < 1) pairs = 1;
    return int(pairs * 2);
  }
  if (max_tiles < ctas) ctas = max_tiles;
  if (ctas < 1) ctas = 1;
  return int(ctas);
}

int elt_size(int dtype) {
  switch (dtype) {
    case TKMX_BF16:
    case TKMX_F16: return 2;
    case TKMX_F32: return 4;
    case TKMX_F8E4M3:
    case TKMX_S8: return 1;
  }
  return 0;
}

bool fits_i32(int64_t v) { return v >= 0 && v < (int64_t(1) << 31); }

// Shared by fwd and dlhs: D[m, cols] = A[m, cdim] . B[g][cols, cdim] with B either
// stored [g, cdim, cols] (b_cols_contiguous) or [g, cols, cdim].
int run_rows(const void* a, const void* b, bool b_cols_contiguous, const int32_t* group_sizes,
             const float* col_scale, void* out, int64_t m, int64_t cdim, int64_t cols, int64_t g,
             int64_t g_rhs, int in_dtype, int b_dtype, int out_dtype, const tkmx_config* config,
             cudaStream_t stream, bool zero_initialize = true, int64_t group_begin = 0,
             int64_t group_count = -1, int gateup = 0, const float* col_bias = nullptr,
             float* out_scales = nullptr, int quant_sub = 0) {
  if (g_rhs <= 0 && g > 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (quant_sub != 0) {
    // Fused output quantisation: e4m3 values and one float scale per row and quant_sub columns.
    if (out_dtype != TKMX_F8E4M3 || out_scales == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
    if (quant_sub != 64 && quant_sub != 128 && quant_sub != 256) return TKMX_ERR_UNSUPPORTED;
    if (cols % quant_sub != 0 || (gateup > 0 && gateup < TKMX_ACT_RELU)) return TKMX_ERR_UNSUPPORTED;
    if (g == 0 || cdim == 0 || m == 0) return TKMX_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0 || (reinterpret_cast<uintptr_t>(out_scales) & 3u) != 0)
      return TKMX_ERR_ALIGNMENT;
    out_dtype = TKMX_BF16;   // for the checks below; the epilogue writes bytes
  }
  // Codes from TKMX_ACT_RELU up are elementwise activations on the float32 result; the codes
  // below them are the gate/up forms.
  int element_act = 0;
  if (gateup >= TKMX_ACT_RELU) {
    if (gateup > TKMX_ACT_SIGMOID) return TKMX_ERR_INVALID_ARGUMENT;
    element_act = gateup - TKMX_ACT_RELU + 1;
    gateup = 0;
  }
  if (gateup != 0) {
    // act(gate) * up over the two halves of the weight columns: [G, K, N] weights only, and
    // tiles whose halves are whole 64-column boxes.
    if (gateup < 0 || gateup > tkmx::kGateUpSiluClamp || !b_cols_contiguous || col_scale != nullptr)
      return TKMX_ERR_UNSUPPORTED;
    if (cols % 2 != 0) return TKMX_ERR_INVALID_ARGUMENT;
  }
  if (group_count < 0) group_count = g - group_begin;
  if (group_begin < 0 || group_begin + group_count > g) return TKMX_ERR_INVALID_ARGUMENT;
  if (m < 0 || cdim < 0 || cols < 0 || g < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (!fits_i32(m) || !fits_i32(cdim) || !fits_i32(cols) || !fits_i32(g) ||
      !fits_i32(m + 128 * (g + 1)))
    return TKMX_ERR_TOO_LARGE;
  if (in_dtype != TKMX_BF16 && in_dtype != TKMX_F16) return TKMX_ERR_UNSUPPORTED;
  // The two operands of kind::f16 must have the same format: bf16 x f16 raises an
  // illegal-instruction fault on B200 even though the descriptor has separate fields.
  if (b_dtype != in_dtype) return TKMX_ERR_UNSUPPORTED;
  if (out_dtype != TKMX_BF16 && out_dtype != TKMX_F16 && out_dtype != TKMX_F32)
    return TKMX_ERR_UNSUPPORTED;
  if (m == 0 || cols == 0) return TKMX_OK;
  if (out == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  const size_t out_bytes = size_t(m) * size_t(gateup ? cols / 2 : cols) * elt_size(out_dtype);
  if (g == 0 || cdim == 0) {
    if (element_act == tkmx::kActSigmoid) return TKMX_ERR_UNSUPPORTED;   // sigmoid(0) = 0.5: not a memset
    TKMX_CUDA_OK(cudaMemsetAsync(out, 0, out_bytes, stream));
    return TKMX_OK;
  }
  if (a == nullptr || b == nullptr || group_sizes == nullptr) return TKMX_ERR_INVALID_ARGUMENT;

  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  ResolvedConfig rc;
  st = resolve_config(config, cols, int(g), true, *dev, &rc);
  if (st != TKMX_OK) return st;
  if (gateup && rc.block_n < 128) return TKMX_ERR_UNSUPPORTED;  // each half needs whole 64-column boxes
  if (quant_sub != 0 && rc.block_n % quant_sub != 0) return TKMX_ERR_UNSUPPORTED;

  CUtensorMap ma, mb;
  {
    const uint64_t dims[2] = {uint64_t(cdim), uint64_t(m)};
    const uint64_t strides[1] = {uint64_t(cdim) * 2};
    const uint32_t box[2] = {64, 128};
    st = encode_map(&ma, a, 2, dims, strides, box);
    if (st != TKMX_OK) return st;
  }
  if (b_cols_contiguous) {
    const uint64_t dims[3] = {uint64_t(cols), uint64_t(cdim), uint64_t(g_rhs)};
    const uint64_t strides[2] = {uint64_t(cols) * 2, uint64_t(cols) * uint64_t(cdim) * 2};
    const uint32_t box[3] = {64, 64, 1};
    st = encode_map(&mb, b, 3, dims, strides, box);
  } else {
    const uint64_t dims[3] = {uint64_t(cdim), uint64_t(cols), uint64_t(g_rhs)};
    const uint64_t strides[2] = {uint64_t(cdim) * 2, uint64_t(cols) * uint64_t(cdim) * 2};
    const uint32_t box[3] = {64, uint32_t(rc.pair ? rc.block_n / 2 : rc.block_n), 1};
    st = encode_map(&mb, b, 3, dims, strides, box);
  }
  if (st != TKMX_OK) return st;

  RaggedGemmParams p = {};
  p.group_sizes = group_sizes;
  p.out = out;
  p.col_scale = col_scale;
  p.col_bias = col_bias;
  p.m_total = int32_t(m);
  p.rows = int32_t(m);
  p.cols = int32_t(cols);
  p.cdim = int32_t(cdim);
  p.num_groups = int32_t(g);
  p.rhs_groups = int32_t(g_rhs);
  p.group_begin = int32_t(group_begin);
  p.group_end = int32_t(group_begin + group_count);
  p.skip_zero_fill = zero_initialize ? 0 : 1;
  p.out_is_f32 = out_dtype == TKMX_F32;
  p.out_is_f16 = out_dtype == TKMX_F16;
  if ((reinterpret_cast<uintptr_t>(col_bias) & 3u) != 0) return TKMX_ERR_ALIGNMENT;
  const int64_t out_cols = gateup ? cols / 2 : cols;
  p.gateup = gateup;
  p.activation = element_act;
  p.out_vec_ok = ((out_cols * elt_size(out_dtype)) % 16 == 0) &&
                 ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  const uint32_t fmt_a = in_dtype == TKMX_BF16 ? 1u : 0u;
  const uint32_t fmt_b = b_dtype == TKMX_BF16 ? 1u : 0u;
  p.idesc = tkmx::ptx::make_idesc(fmt_a, fmt_b, 0u, b_cols_contiguous ? 1u : 0u,
                                  rc.pair ? 256u : 128u, uint32_t(rc.block_n));
  p.tile_width = rc.tile_width;
  p.minor_is_m = rc.minor_is_m;
  p.num_stages = rc.num_stages;
  p.status = dev->status_ptr;
  assign_sched(*dev, &p, true);
  // Pair mode, 256-column tiles: a group's last tile with at most this many rows runs with
  // swapped MMA operands (cost follows its rows).  192 = where the swapped MMA stops being
  // cheaper than the full one (measured 141 against 173 cycles).  TKMX_SWAP_ROWS overrides.
  p.swap_rows = (rc.pair && rc.block_n == 256 && !gateup && quant_sub == 0) ? env_int("TKMX_SWAP_ROWS", 192, 0, 192) : 0;
  p.out_scales = out_scales;
  p.quant_sub = quant_sub;
  p.prefetch_blocks = env_int("TKMX_PREFETCH", 0, 0, 64);
  p.prefetch_cold_only = env_int("TKMX_PREFETCH_COLD_ONLY", 1, 0, 1);
  // Equal swapped tiles instead of full + short ones: off by default.  Measured on B200 it
  // lost (cfg4 forward 0.215 against 0.209 ms, dlhs 0.243 against 0.218): a swapped tile's
  // transposed epilogue stores 2 bytes per lane and grows with the tile's rows, which outweighs
  // the MMA time saved.
  p.balance_tiles = env_int("TKMX_BALANCE_TILES", 0, 0, 1);

  // 16-bit outputs: blocks of 32 rows x 64 columns that are not ragged leave by TMA store.
  CUtensorMap mo = {};
  p.tma_store = 0;
  if (out_dtype != TKMX_F32 && p.out_vec_ok && !gateup && col_bias == nullptr && quant_sub == 0) {
    const uint64_t dims[2] = {uint64_t(cols), uint64_t(m)};
    const uint64_t strides[1] = {uint64_t(cols) * 2};
    const uint32_t box[2] = {64, 32};
    st = encode_map(&mo, out, 2, dims, strides, box);
    if (st != TKMX_OK) return st;
    p.tma_store = 1;
  }
  const int64_t tile_m = rc.pair ? 256 : 128;
  const int64_t n_tiles = (cols + rc.block_n - 1) / rc.block_n;
  const int64_t max_tiles = ((m + tile_m - 1) / tile_m + g) * n_tiles;
  const int grid = grid_size(*dev, rc, max_tiles);
  if (b_cols_contiguous)
    return launch_mode<tkmx::kRowsBN>(rc.block_n, rc.pair, ma, mb, mo, p, grid, stream);
  return launch_mode<tkmx::kRowsBK>(rc.block_n, rc.pair, ma, mb, mo, p, grid, stream);
}


template <int kBlockN, bool kPair, int kQuant>
int launch_w8(const CUtensorMap& ma, const CUtensorMap& mb, const RaggedGemmParams& p, int grid,
              cudaStream_t stream) {
  auto kernel = tkmx::ragged_gemm_w8_kernel<kBlockN, kPair, kQuant>;
  const int smem = tkmx::make_w8_smem_layout(kBlockN, kPair, p.num_stages, p.num_groups).total + 1024;
  {
    const int st = raise_smem_limit(kernel, smem);
    if (st != TKMX_OK) return st;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(tkmx::kW8Threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TKMX_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, p));
  return TKMX_OK;
}

template <int kBlockN, bool kPair, bool kInt8 = false>
int launch_f8(const CUtensorMap& ma, const CUtensorMap& ma32, const CUtensorMap& mb,
              const RaggedGemmParams& p, const float* row_scale, int grid, cudaStream_t stream) {
  auto kernel = tkmx::ragged_gemm_f8_kernel<kBlockN, kPair, kInt8>;
  const int smem = tkmx::make_f8_smem_layout(kBlockN, kPair, p.num_stages, p.num_groups).total + 1024;
  {
    const int st = raise_smem_limit(kernel, smem);
    if (st != TKMX_OK) return st;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(tkmx::kF8Threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TKMX_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, ma32, mb, p, row_scale));
  return TKMX_OK;
}

// Native fp8 route of the e4m3-weight forward: the activation rows are split into two e4m3
// planes plus a row scale in `workspace`, then both planes are multiplied with the raw
// weights by fp8 MMAs.  Needs k % 16 == 0 (row stride of the 8-bit planes).
// Row count up to which a tile runs with swapped MMA operands (tensor time proportional to
// its rows); 0 switches the short-tile path off.
int f8_swap_rows() { return env_int("TKMX_F8_SWAP_ROWS", 64, 0, 64); }
// Weight blocks (128 contraction elements each) requested into L2 ahead of the shared-memory
// ring.  Off by default: on B200 it lowered throughput (the ring already covers the latency
// and the extra lines compete for L2 with the activations).
int f8_prefetch_blocks() { return env_int("TKMX_F8_PREFETCH", 0, 0, 64); }

bool f8_native_usable(int rhs_dtype, const void* workspace, size_t workspace_bytes, int64_t m, int64_t k) {
  return (rhs_dtype == TKMX_F8E4M3 || rhs_dtype == TKMX_S8) && workspace != nullptr && k % 16 == 0 &&
         (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 &&
         workspace_bytes >= tkmx::f8_workspace(m, k).total;
}

template <int kQuant>
int launch_w8_shape(int block_n, bool pair, const CUtensorMap& ma, const CUtensorMap& mb,
                    const RaggedGemmParams& p, int grid, cudaStream_t stream) {
  if (pair && block_n == 256) return launch_w8<256, true, kQuant>(ma, mb, p, grid, stream);
  if (!pair && block_n == 256) return launch_w8<256, false, kQuant>(ma, mb, p, grid, stream);
  if (!pair && block_n == 128) return launch_w8<128, false, kQuant>(ma, mb, p, grid, stream);
  return TKMX_ERR_UNSUPPORTED;
}

// Forward with 8-bit weights rhs[g, k, n] (n contiguous) and per-channel scales.
int run_rows_w8(const void* lhs, const void* rhs8, const int32_t* group_sizes, const float* scale,
                void* out, int64_t m, int64_t k, int64_t n, int64_t g, int64_t g_rhs, int lhs_dtype,
                int rhs_dtype, int out_dtype, const tkmx_config* config, cudaStream_t stream,
                bool zero_initialize = true, int64_t group_begin = 0, int64_t group_count = -1,
                void* workspace = nullptr, size_t workspace_bytes = 0, int gateup = 0,
                const float* col_bias = nullptr) {
  if (m < 0 || k < 0 || n < 0 || g < 0 || (g > 0 && g_rhs <= 0)) return TKMX_ERR_INVALID_ARGUMENT;
  if (group_count < 0) group_count = g - group_begin;
  if (group_begin < 0 || group_begin + group_count > g) return TKMX_ERR_INVALID_ARGUMENT;
  if (!fits_i32(m) || !fits_i32(k) || !fits_i32(n) || !fits_i32(g) || !fits_i32(m + 256 * (g + 1)))
    return TKMX_ERR_TOO_LARGE;
  if (lhs_dtype != TKMX_BF16) return TKMX_ERR_UNSUPPORTED;  // weights are expanded to bf16
  if (out_dtype != TKMX_BF16 && out_dtype != TKMX_F16 && out_dtype != TKMX_F32)
    return TKMX_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return TKMX_OK;
  if (out == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  if (g == 0 || k == 0) {
    TKMX_CUDA_OK(cudaMemsetAsync(out, 0, size_t(m) * size_t(gateup ? n / 2 : n) * elt_size(out_dtype), stream));
    return TKMX_OK;
  }
  if (lhs == nullptr || rhs8 == nullptr || group_sizes == nullptr || scale == nullptr)
    return TKMX_ERR_INVALID_ARGUMENT;

  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  tkmx_config d = {};
  if (config != nullptr) d = *config;
  if (d.block_m != 0 && d.block_m != 128) return TKMX_ERR_UNSUPPORTED;
  if (d.block_k != 0 && d.block_k != 64) return TKMX_ERR_UNSUPPORTED;
  if (d.collective != 0 && d.collective != 1) return TKMX_ERR_INVALID_ARGUMENT;
  ResolvedConfig rc;
  rc.pair = d.collective == 1;
  rc.block_n = d.block_n == 0 ? 256 : d.block_n;
  if (rc.pair ? rc.block_n != 256 : (rc.block_n != 128 && rc.block_n != 256)) return TKMX_ERR_UNSUPPORTED;
  if (d.grid_minor_dim != 0 && d.grid_minor_dim != 1) return TKMX_ERR_INVALID_ARGUMENT;
  if (d.grid_tile_width < 0 || d.num_stages < 0 || d.max_ctas < 0) return TKMX_ERR_INVALID_ARGUMENT;
  const int smem_cap = dev->smem_optin < kMaxSmemOptin ? dev->smem_optin : kMaxSmemOptin;
  const bool native_f8 = f8_native_usable(rhs_dtype, workspace, workspace_bytes, m, k);
  if (gateup != 0 || col_bias != nullptr) {
    // Epilogue extras exist in the native fp8 kernel only, on 256-column tiles whose gate and
    // up halves start on 16-byte boundaries of the 8-bit rows.
    if (!native_f8 || gateup < 0 || gateup > tkmx::kGateUpSiluClamp) return TKMX_ERR_UNSUPPORTED;
    if (gateup != 0 && rhs_dtype == TKMX_S8) return TKMX_ERR_UNSUPPORTED;   // int8: plain and bias epilogues only
    if (gateup != 0 && (n % 2 != 0 || (n / 2) % 16 != 0 || rc.block_n != 256)) return TKMX_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(col_bias) & 3u) != 0) return TKMX_ERR_ALIGNMENT;
  }
  auto smem_need = [&](int st_) -> uint32_t {
    return (native_f8 ? tkmx::make_f8_smem_layout(rc.block_n, rc.pair, st_, int(g)).total
                      : tkmx::make_w8_smem_layout(rc.block_n, rc.pair, st_, int(g)).total) + 1024;
  };
  // A native-fp8 stage holds 128 contraction elements, twice a converter-path stage; its
  // default is the deepest ring that fits (3 stages of 64 KiB for a single CTA's 256 columns).
  int stages = d.num_stages == 0 ? (native_f8 ? 8 : 5) : (native_f8 ? (d.num_stages + 1) / 2 : d.num_stages);
  if (stages > 16) return TKMX_ERR_UNSUPPORTED;
  if (native_f8 && stages < 2) stages = 2;
  while (stages > 2 && smem_need(stages) > (uint32_t)smem_cap) --stages;   // deepest ring that fits
  if (smem_need(stages) > (uint32_t)smem_cap) return TKMX_ERR_TOO_LARGE;
  rc.num_stages = stages;
  rc.minor_is_m = d.grid_minor_dim == 0 ? 1 : 0;
  rc.tile_width = d.grid_tile_width == 0 ? 1 : d.grid_tile_width;
  rc.max_ctas = d.max_ctas;

  CUtensorMap ma, ma32, mb;
  const tkmx::F8Workspace ws = tkmx::f8_workspace(m, k);
  if (native_f8) {
    const uint64_t dims[3] = {uint64_t(k), uint64_t(m), 2};
    const uint64_t strides[2] = {uint64_t(k), uint64_t(ws.plane_bytes)};
    const uint32_t box[3] = {128, 128, 1};
    st = encode_map(&ma, workspace, 3, dims, strides, box, CU_TENSOR_MAP_DATA_TYPE_UINT8);
    if (st != TKMX_OK) return st;
    const uint32_t box32[3] = {128, 32, 1};
    st = encode_map(&ma32, workspace, 3, dims, strides, box32, CU_TENSOR_MAP_DATA_TYPE_UINT8);
    if (st != TKMX_OK) return st;
    if ((reinterpret_cast<uintptr_t>(lhs) & 15u) != 0) return TKMX_ERR_ALIGNMENT;
  } else {
    const uint64_t dims[2] = {uint64_t(k), uint64_t(m)};
    const uint64_t strides[1] = {uint64_t(k) * 2};
    const uint32_t box[2] = {64, 128};
    st = encode_map(&ma, lhs, 2, dims, strides, box);
    if (st != TKMX_OK) return st;
  }
  {
    const uint64_t dims[3] = {uint64_t(n), uint64_t(k), uint64_t(g_rhs)};
    const uint64_t strides[2] = {uint64_t(n), uint64_t(n) * uint64_t(k)};
    const uint32_t box[3] = {128, 64, 1};
    // Gate/up tiles fetch two 128-byte pieces per weight row that lie n/2 bytes apart: a
    // 256-byte L2 promotion would drag in the neighbouring tiles' halves as well.
    st = encode_map(&mb, rhs8, 3, dims, strides, box, CU_TENSOR_MAP_DATA_TYPE_UINT8,
                    gateup ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (st != TKMX_OK) return st;
  }
  if ((reinterpret_cast<uintptr_t>(scale) & 3u) != 0) return TKMX_ERR_ALIGNMENT;

  RaggedGemmParams p = {};
  p.group_sizes = group_sizes;
  p.out = out;
  p.col_scale = scale;
  p.m_total = int32_t(m);
  p.rows = int32_t(m);
  p.cols = int32_t(n);
  p.cdim = int32_t(k);
  p.num_groups = int32_t(g);
  p.rhs_groups = int32_t(g_rhs);
  p.group_begin = int32_t(group_begin);
  p.group_end = int32_t(group_begin + group_count);
  p.skip_zero_fill = zero_initialize ? 0 : 1;
  p.out_is_f32 = out_dtype == TKMX_F32;
  p.out_is_f16 = out_dtype == TKMX_F16;
  p.out_vec_ok = (((gateup ? n / 2 : n) * elt_size(out_dtype)) % 16 == 0) &&
                 ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  p.gateup = gateup;
  p.col_bias = col_bias;
  p.idesc = tkmx::ptx::make_idesc(1u, 1u, 0u, 1u, rc.pair ? 256u : 128u, uint32_t(rc.block_n));
  p.tile_width = rc.tile_width;
  p.minor_is_m = rc.minor_is_m;
  p.num_stages = rc.num_stages;
  p.status = dev->status_ptr;

  const int64_t tile_m = rc.pair ? 256 : 128;
  const int64_t n_tiles = (n + rc.block_n - 1) / rc.block_n;
  const int64_t max_tiles = ((m + tile_m - 1) / tile_m + g) * n_tiles;
  const int grid = grid_size(*dev, rc, max_tiles);
  if (native_f8) {
    uint8_t* planes = static_cast<uint8_t*>(workspace);
    float* row_scale = reinterpret_cast<float*>(planes + ws.scales_off);
    const int split_blocks = int(std::min<int64_t>((m + 7) / 8, int64_t(dev->num_sms) * 8));
    int32_t* sched = reinterpret_cast<int32_t*>(planes + ws.sched_off);
    const __nv_bfloat16* a16 = static_cast<const __nv_bfloat16*>(lhs);
    uint8_t* lo_plane = planes + ws.plane_bytes;
    if (rhs_dtype == TKMX_S8) {
      // int8 weights: int8 activation planes, kind::i8 MMAs, two int32 accumulators per tile.
      if (k <= 4096)
        tkmx::split_rows_s8_kernel<16><<<split_blocks, 256, 0, stream>>>(a16, planes, lo_plane, row_scale, sched, int(m), int(k));
      else
        tkmx::split_rows_s8_kernel<28><<<split_blocks, 256, 0, stream>>>(a16, planes, lo_plane, row_scale, sched, int(m), int(k));
      TKMX_CUDA_OK(cudaGetLastError());
      p.idesc = tkmx::ptx::make_idesc_s8(0u, 1u, rc.pair ? 256u : 128u, uint32_t(rc.block_n));
      p.swap_rows = rc.pair ? 0 : f8_swap_rows();
      p.prefetch_blocks = 0;
      p.mixed_order = 0;
      p.sched_counter = (!rc.pair && env_int("TKMX_F8_DYNAMIC", 1, 0, 1)) ? sched : nullptr;
      if (rc.pair) return launch_f8<256, true, true>(ma, ma32, mb, p, row_scale, grid, stream);
      if (rc.block_n == 256) return launch_f8<256, false, true>(ma, ma32, mb, p, row_scale, grid, stream);
      return launch_f8<128, false, true>(ma, ma32, mb, p, row_scale, grid, stream);
    }
    // Rows up to 8192 elements are split from registers (read once, all loads in flight);
    // longer ones by the two-pass kernel.
    if (k <= 2048)
      tkmx::split_rows_e4m3_regs_kernel<8><<<split_blocks, 256, 0, stream>>>(a16, planes, lo_plane, row_scale, sched, int(m), int(k));
    else if (k <= 4096)
      tkmx::split_rows_e4m3_regs_kernel<16><<<split_blocks, 256, 0, stream>>>(a16, planes, lo_plane, row_scale, sched, int(m), int(k));
    else if (k <= 8192)
      tkmx::split_rows_e4m3_regs_kernel<32><<<split_blocks, 256, 0, stream>>>(a16, planes, lo_plane, row_scale, sched, int(m), int(k));
    else
      tkmx::split_rows_e4m3_kernel<<<split_blocks, 256, 0, stream>>>(a16, planes, lo_plane, row_scale, sched, int(m), int(k));
    TKMX_CUDA_OK(cudaGetLastError());
    p.idesc = tkmx::ptx::make_idesc(0u, 0u, 0u, 1u, rc.pair ? 256u : 128u, uint32_t(rc.block_n));
    p.swap_rows = rc.pair ? 0 : f8_swap_rows();
    p.prefetch_blocks = f8_prefetch_blocks();
    // Visiting order: by group index.  Merging small and large groups (1) or large groups
    // first (2) measured 3-6 % slower on the Zipf-routed DeepSeek-shaped workload, whose
    // index order already interleaves the two kinds.
    p.mixed_order = env_int("TKMX_F8_MIXED_ORDER", 0, 0, 2);
    p.sched_counter = (!rc.pair && env_int("TKMX_F8_DYNAMIC", 1, 0, 1)) ? sched : nullptr;
    if (rc.pair) return launch_f8<256, true>(ma, ma32, mb, p, row_scale, grid, stream);
    if (rc.block_n == 256) return launch_f8<256, false>(ma, ma32, mb, p, row_scale, grid, stream);
    return launch_f8<128, false>(ma, ma32, mb, p, row_scale, grid, stream);
  }
  if (rhs_dtype == TKMX_F8E4M3)
    return launch_w8_shape<tkmx::kQuantE4M3>(rc.block_n, rc.pair, ma, mb, p, grid, stream);
  return launch_w8_shape<tkmx::kQuantS8>(rc.block_n, rc.pair, ma, mb, p, grid, stream);
}

}  // namespace

extern "C" {

int tkmx_abi_version(void) { return TKMX_ABI_VERSION; }

const char* tkmx_status_string(int status) {
  switch (status) {
    case TKMX_OK: return "ok";
    case TKMX_ERR_INVALID_ARGUMENT: return "invalid argument";
    case TKMX_ERR_UNSUPPORTED: return "unsupported combination (not implemented)";
    case TKMX_ERR_ALIGNMENT: return "pointer or leading dimension is not 16-byte aligned";
    case TKMX_ERR_CUDA: return "CUDA call failed";
    case TKMX_ERR_WORKSPACE: return "workspace too small";
    case TKMX_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    case TKMX_ERR_TOO_LARGE: return "size beyond a static limit";
    case TKMX_ERR_DEVICE_STATE: return "a kernel found its bookkeeping inconsistent and stopped early";
  }
  return "unknown status";
}

const char* tkmx_last_cuda_error(void) { return g_last_cuda_error.c_str(); }

size_t tkmx_ragged_dot_workspace_bytes(int op, int64_t m, int64_t k, int64_t n, int64_t g,
                                       int rhs_dtype, const tkmx_config* config) {
  (void)n; (void)g; (void)config;
  // Only the forward with e4m3 weights uses scratch: the two e4m3 planes of the split
  // activations and their row scales.  Without it the call takes the converter kernel.
  if (op == 0 && (rhs_dtype == TKMX_F8E4M3 || rhs_dtype == TKMX_S8) && m > 0 && k > 0 && k % 16 == 0)
    return tkmx::f8_workspace(m, k).total;
  return 0;
}

static int fwd_impl(const void* lhs, const void* rhs, const int32_t* group_sizes, const float* rhs_scale,
                    void* out, int64_t m, int64_t k, int64_t n, int64_t g, int64_t g_rhs, int lhs_dtype,
                    int rhs_dtype, int out_dtype, int rhs_layout, const tkmx_config* config,
                    void* cuda_stream, bool zero_initialize = true, int64_t group_begin = 0,
                    int64_t group_count = -1, void* workspace = nullptr, size_t workspace_bytes = 0) {
  if (rhs_layout != TKMX_RHS_GKN && rhs_layout != TKMX_RHS_GNK) return TKMX_ERR_INVALID_ARGUMENT;
  const bool quantised = rhs_dtype == TKMX_F8E4M3 || rhs_dtype == TKMX_S8;
  if (quantised) {
    if (rhs_scale == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
    if (rhs_layout != TKMX_RHS_GKN) return TKMX_ERR_UNSUPPORTED;
    return run_rows_w8(lhs, rhs, group_sizes, rhs_scale, out, m, k, n, g, g_rhs, lhs_dtype, rhs_dtype,
                       out_dtype, config, static_cast<cudaStream_t>(cuda_stream), zero_initialize,
                       group_begin, group_count, workspace, workspace_bytes);
  }
  if (rhs_scale != nullptr) return TKMX_ERR_UNSUPPORTED;  // scales go with 8-bit weights only
  return run_rows(lhs, rhs, rhs_layout == TKMX_RHS_GKN, group_sizes, nullptr, out, m, k, n, g, g_rhs,
                  lhs_dtype, rhs_dtype, out_dtype, config, static_cast<cudaStream_t>(cuda_stream),
                  zero_initialize, group_begin, group_count);
}

int tkmx_ragged_dot_fwd(const void* lhs, const void* rhs, const int32_t* group_sizes,
                        const float* rhs_scale, void* out, void* workspace, size_t workspace_bytes,
                        int64_t m, int64_t k, int64_t n, int64_t g, int lhs_dtype, int rhs_dtype,
                        int out_dtype, int rhs_layout, const tkmx_config* config, void* cuda_stream) {
  return fwd_impl(lhs, rhs, group_sizes, rhs_scale, out, m, k, n, g, g, lhs_dtype, rhs_dtype, out_dtype,
                  rhs_layout, config, cuda_stream, true, 0, -1, workspace, workspace_bytes);
}

int tkmx_ragged_dot_fwd_gateup(const void* lhs, const void* rhs, const int32_t* group_sizes, void* out,
                               int64_t m, int64_t k, int64_t n, int64_t g, int in_dtype, int out_dtype,
                               int activation, const tkmx_config* config, void* cuda_stream) {
  if (activation <= 0 || activation > tkmx::kGateUpSiluClamp) return TKMX_ERR_INVALID_ARGUMENT;
  return run_rows(lhs, rhs, true, group_sizes, nullptr, out, m, k, n, g, g, in_dtype, in_dtype, out_dtype,
                  config, static_cast<cudaStream_t>(cuda_stream), true, 0, -1, activation);
}

int tkmx_ragged_dot_fwd_epilogue(const void* lhs, const void* rhs, const int32_t* group_sizes,
                                 const float* rhs_scale, const float* rhs_bias, void* out, void* workspace,
                                 size_t workspace_bytes, int64_t m, int64_t k, int64_t n, int64_t g,
                                 int lhs_dtype, int rhs_dtype, int out_dtype, int rhs_layout, int activation,
                                 const tkmx_config* config, void* cuda_stream) {
  if (activation < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (rhs_layout != TKMX_RHS_GKN && rhs_layout != TKMX_RHS_GNK) return TKMX_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (rhs_dtype == TKMX_F8E4M3 || rhs_dtype == TKMX_S8) {
    if (rhs_scale == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
    if (rhs_layout != TKMX_RHS_GKN) return TKMX_ERR_UNSUPPORTED;
    return run_rows_w8(lhs, rhs, group_sizes, rhs_scale, out, m, k, n, g, g, lhs_dtype, rhs_dtype, out_dtype,
                       config, stream, true, 0, -1, workspace, workspace_bytes, activation, rhs_bias);
  }
  if (rhs_scale != nullptr) return TKMX_ERR_UNSUPPORTED;
  return run_rows(lhs, rhs, rhs_layout == TKMX_RHS_GKN, group_sizes, nullptr, out, m, k, n, g, g, lhs_dtype,
                  rhs_dtype, out_dtype, config, stream, true, 0, -1, activation, rhs_bias);
}

int tkmx_ragged_dot_fwd_quant_out(const void* lhs, const void* rhs, const int32_t* group_sizes,
                                  const float* rhs_bias, void* out_q, float* out_scale, int64_t m, int64_t k,
                                  int64_t n, int64_t g, int in_dtype, int rhs_layout, int activation,
                                  int subchannel, const tkmx_config* config, void* cuda_stream) {
  if (rhs_layout != TKMX_RHS_GKN && rhs_layout != TKMX_RHS_GNK) return TKMX_ERR_INVALID_ARGUMENT;
  if (activation != 0 && (activation < TKMX_ACT_RELU || activation > TKMX_ACT_SIGMOID)) return TKMX_ERR_INVALID_ARGUMENT;
  if (subchannel <= 0) return TKMX_ERR_INVALID_ARGUMENT;
  return run_rows(lhs, rhs, rhs_layout == TKMX_RHS_GKN, group_sizes, nullptr, out_q, m, k, n, g, g, in_dtype,
                  in_dtype, TKMX_F8E4M3, config, static_cast<cudaStream_t>(cuda_stream), true, 0, -1, activation,
                  rhs_bias, out_scale, subchannel);
}

int tkmx_ragged_dot_fwd_cyclic(const void* lhs, const void* rhs, const int32_t* group_sizes,
                               const float* rhs_scale, void* out, int64_t m, int64_t k, int64_t n,
                               int64_t num_segments, int64_t g_rhs, int lhs_dtype, int rhs_dtype,
                               int out_dtype, int rhs_layout, int zero_initialize,
                               int64_t segment_begin, int64_t segment_count,
                               const tkmx_config* config, void* workspace, size_t workspace_bytes,
                               void* cuda_stream) {
  if (g_rhs <= 0 || num_segments < 0) return TKMX_ERR_INVALID_ARGUMENT;
  return fwd_impl(lhs, rhs, group_sizes, rhs_scale, out, m, k, n, num_segments, g_rhs, lhs_dtype,
                  rhs_dtype, out_dtype, rhs_layout, config, cuda_stream, zero_initialize != 0,
                  segment_begin, segment_count, workspace, workspace_bytes);
}

int tkmx_ragged_dot_dlhs(const void* dout, const void* rhs, const int32_t* group_sizes, void* dlhs,
                         void* workspace, size_t workspace_bytes, int64_t m, int64_t k, int64_t n,
                         int64_t g, int in_dtype, int out_dtype, const tkmx_config* config,
                         void* cuda_stream) {
  (void)workspace; (void)workspace_bytes;
  // Contraction over n; rhs[g, k, n] is already "output-row major, contraction contiguous".
  return run_rows(dout, rhs, false, group_sizes, nullptr, dlhs, m, n, k, g, g, in_dtype, in_dtype,
                  out_dtype, config, static_cast<cudaStream_t>(cuda_stream));
}

int tkmx_ragged_dot_drhs(const void* lhs, const void* dout, const int32_t* group_sizes, void* drhs,
                         void* workspace, size_t workspace_bytes, int64_t m, int64_t k, int64_t n,
                         int64_t g, int in_dtype, int out_dtype, const tkmx_config* config,
                         void* cuda_stream) {
  (void)workspace; (void)workspace_bytes;
  return tkmx_ragged_dot_drhs_window(lhs, dout, group_sizes, drhs, m, k, n, g, 0, g, in_dtype, out_dtype, config,
                                     cuda_stream);
}

int tkmx_ragged_dot_drhs_window(const void* lhs, const void* dout, const int32_t* group_sizes, void* drhs,
                                int64_t m, int64_t k, int64_t n, int64_t g, int64_t group_begin,
                                int64_t group_count, int in_dtype, int out_dtype, const tkmx_config* config,
                                void* cuda_stream) {
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (m < 0 || k < 0 || n < 0 || g < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (group_begin < 0 || group_count < 0 || group_begin + group_count > g) return TKMX_ERR_INVALID_ARGUMENT;
  const int64_t g_all = g;   // groups the offsets are counted over
  g = group_count;           // slabs of the output
  if (!fits_i32(m) || !fits_i32(k) || !fits_i32(n) || !fits_i32(g_all)) return TKMX_ERR_TOO_LARGE;
  if (in_dtype != TKMX_BF16 && in_dtype != TKMX_F16) return TKMX_ERR_UNSUPPORTED;
  if (out_dtype != TKMX_BF16 && out_dtype != TKMX_F16 && out_dtype != TKMX_F32)
    return TKMX_ERR_UNSUPPORTED;
  if (g == 0 || k == 0 || n == 0) return TKMX_OK;
  if (drhs == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  const size_t out_bytes = size_t(g) * size_t(k) * size_t(n) * elt_size(out_dtype);
  if (m == 0) {
    TKMX_CUDA_OK(cudaMemsetAsync(drhs, 0, out_bytes, stream));
    return TKMX_OK;
  }
  if (lhs == nullptr || dout == nullptr || group_sizes == nullptr) return TKMX_ERR_INVALID_ARGUMENT;

  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  ResolvedConfig rc;
  st = resolve_config(config, n, int(g_all), false, *dev, &rc);
  if (st != TKMX_OK) return st;
  const int64_t tile_m = rc.pair ? 256 : 128;
  const int64_t r_tiles = (k + tile_m - 1) / tile_m;
  const int64_t n_tiles = (n + rc.block_n - 1) / rc.block_n;
  if (!fits_i32(g * r_tiles * n_tiles)) return TKMX_ERR_TOO_LARGE;

  CUtensorMap ma, mb;
  {
    const uint64_t dims[2] = {uint64_t(k), uint64_t(m)};
    const uint64_t strides[1] = {uint64_t(k) * 2};
    const uint32_t box[2] = {64, 64};
    st = encode_map(&ma, lhs, 2, dims, strides, box);
    if (st != TKMX_OK) return st;
  }
  {
    const uint64_t dims[2] = {uint64_t(n), uint64_t(m)};
    const uint64_t strides[1] = {uint64_t(n) * 2};
    const uint32_t box[2] = {64, 64};
    st = encode_map(&mb, dout, 2, dims, strides, box);
    if (st != TKMX_OK) return st;
  }

  RaggedGemmParams p = {};
  p.group_sizes = group_sizes;
  p.out = drhs;
  p.col_scale = nullptr;
  p.m_total = int32_t(m);
  p.rows = int32_t(k);
  p.cols = int32_t(n);
  p.cdim = 0;
  p.num_groups = int32_t(g_all);
  p.rhs_groups = int32_t(g_all);
  p.group_begin = int32_t(group_begin);
  p.group_end = int32_t(group_begin + group_count);
  p.out_is_f32 = out_dtype == TKMX_F32;
  p.out_is_f16 = out_dtype == TKMX_F16;
  p.out_vec_ok = ((n * elt_size(out_dtype)) % 16 == 0) &&
                 ((reinterpret_cast<uintptr_t>(drhs) & 15u) == 0);
  const uint32_t fmt = in_dtype == TKMX_BF16 ? 1u : 0u;
  p.idesc = tkmx::ptx::make_idesc(fmt, fmt, 1u, 1u, rc.pair ? 256u : 128u, uint32_t(rc.block_n));
  p.tile_width = rc.tile_width;
  p.minor_is_m = rc.minor_is_m;
  p.num_stages = rc.num_stages;
  p.status = dev->status_ptr;
  // drhs tiles are as long as their group has rows: with short ones (~512 rows, 3 us per tile)
  // the per-tile hand-off costs more than the balance gains (-3 %), with long ones it wins
  // (+2 ... +6 % at 1024-2048 rows per group).
  assign_sched(*dev, &p, g_all > 0 && m / g_all >= 768);

  CUtensorMap mo = {};
  p.tma_store = 0;
  if (out_dtype != TKMX_F32 && p.out_vec_ok) {
    const uint64_t dims[3] = {uint64_t(n), uint64_t(k), uint64_t(g)};
    const uint64_t strides[2] = {uint64_t(n) * 2, uint64_t(n) * uint64_t(k) * 2};
    const uint32_t box[3] = {64, 32, 1};
    st = encode_map(&mo, drhs, 3, dims, strides, box);
    if (st != TKMX_OK) return st;
    p.tma_store = 1;
  }
  const int grid = grid_size(*dev, rc, g * r_tiles * n_tiles);
  return launch_mode<tkmx::kContract>(rc.block_n, rc.pair, ma, mb, mo, p, grid, stream);
}

int tkmx_group_info_aligned(const int32_t* group_sizes, int64_t g, int32_t tile, int32_t num_tasks,
                            int32_t align_tile, int32_t* group_id, int32_t* block_start,
                            int32_t* actual_start, int32_t* actual_end, int32_t* start_within_block,
                            int32_t* actual_size, void* cuda_stream) {
  if (g <= 0 || tile <= 0 || align_tile <= 0 || num_tasks < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (g > tkmx::kGroupInfoMaxGroups) return TKMX_ERR_TOO_LARGE;
  if (num_tasks == 0) return TKMX_OK;
  if (group_sizes == nullptr || group_id == nullptr || block_start == nullptr ||
      actual_start == nullptr || actual_end == nullptr || start_within_block == nullptr ||
      actual_size == nullptr)
    return TKMX_ERR_INVALID_ARGUMENT;
  tkmx::GroupInfoOut o = {group_id, block_start, actual_start, actual_end, start_within_block, actual_size};
  const int blocks = (num_tasks + 255) / 256;
  tkmx::group_info_aligned_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      group_sizes, int(g), tile, num_tasks, align_tile, o);
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

size_t tkmx_moe_sort_workspace_bytes(int64_t num_pairs, int32_t num_experts) {
  if (num_pairs <= 0 || num_experts <= 0) return 0;
  const int64_t chunks = (num_pairs + tkmx::kSortChunk - 1) / tkmx::kSortChunk;
  return size_t(chunks) * size_t(num_experts) * sizeof(int32_t);
}

static int moe_sort_launch(const int32_t* expert_ids, int64_t num_pairs, int32_t num_experts,
                           int32_t* pos, int32_t* expert_counts, int32_t* scratch, cudaStream_t stream,
                           int32_t* sorted_pair = nullptr) {
  const int chunks = int((num_pairs + tkmx::kSortChunk - 1) / tkmx::kSortChunk);
  const int smem = 32 * num_experts * int(sizeof(int));
  if (smem > 48 * 1024) {
    int st = raise_smem_limit(tkmx::moe_sort_hist_kernel, smem);
    if (st == TKMX_OK) st = raise_smem_limit(tkmx::moe_sort_scatter_kernel, smem);
    if (st != TKMX_OK) return st;
  }
  tkmx::moe_sort_hist_kernel<<<chunks, tkmx::kSortChunk, smem, stream>>>(expert_ids, int(num_pairs), num_experts, scratch);
  tkmx::moe_sort_scan_kernel<<<1, 1024, 0, stream>>>(scratch, chunks, num_experts, expert_counts);
  tkmx::moe_sort_scatter_kernel<<<chunks, tkmx::kSortChunk, smem, stream>>>(expert_ids, int(num_pairs), num_experts, scratch, pos, sorted_pair);
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

int tkmx_moe_sort_pairs(const int32_t* expert_ids, int64_t num_pairs, int32_t num_experts, int32_t* pos,
                        int32_t* expert_counts, void* workspace, size_t workspace_bytes,
                        void* cuda_stream) {
  return tkmx_moe_sort_pairs_inverse(expert_ids, num_pairs, num_experts, pos, nullptr, expert_counts, workspace,
                                     workspace_bytes, cuda_stream);
}

int tkmx_moe_sort_pairs_inverse(const int32_t* expert_ids, int64_t num_pairs, int32_t num_experts, int32_t* pos,
                                int32_t* sorted_pair, int32_t* expert_counts, void* workspace,
                                size_t workspace_bytes, void* cuda_stream) {
  if (num_pairs < 0 || num_experts <= 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (num_experts > tkmx::kSortMaxExperts || !fits_i32(num_pairs)) return TKMX_ERR_TOO_LARGE;
  if (expert_counts == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (num_pairs == 0) {
    TKMX_CUDA_OK(cudaMemsetAsync(expert_counts, 0, size_t(num_experts) * sizeof(int32_t), stream));
    return TKMX_OK;
  }
  if (expert_ids == nullptr || pos == nullptr || workspace == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  if (workspace_bytes < tkmx_moe_sort_workspace_bytes(num_pairs, num_experts)) return TKMX_ERR_WORKSPACE;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  return moe_sort_launch(expert_ids, num_pairs, num_experts, pos, expert_counts,
                         static_cast<int32_t*>(workspace), stream, sorted_pair);
}

// ---------------------------------------------------------------------------------------
// Sorting without caller scratch: the histogram matrix of tkmx_moe_sort_pairs lives in a
// fixed array inside the library image instead of a workspace argument.
constexpr int64_t kStaticSortScratchInts = 256 * 1024;  // 1 MiB per device
static __device__ __align__(256) int32_t g_static_sort_scratch[kStaticSortScratchInts];
// Device address of the array above, looked up once per device.  In host code the symbol's
// name is only a handle for cudaGetSymbolAddress, never something to hand to a kernel.
static int32_t* g_static_sort_scratch_ptr[kMaxDevices] = {};

int tkmx_moe_sort_pairs_static(const int32_t* expert_ids, int64_t num_pairs, int32_t num_experts,
                               int32_t* pos, int32_t* expert_counts, void* cuda_stream) {
  if (num_pairs < 0 || num_experts <= 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (num_experts > tkmx::kSortMaxExperts || !fits_i32(num_pairs)) return TKMX_ERR_TOO_LARGE;
  if (expert_counts == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  const int64_t chunks = (num_pairs + tkmx::kSortChunk - 1) / tkmx::kSortChunk;
  if (chunks * num_experts > kStaticSortScratchInts) {
    g_last_cuda_error = "tkmx_moe_sort_pairs_static: ceil(num_pairs / 1024) * num_experts exceeds the "
                        "built-in scratch of 262144 entries; use tkmx_moe_sort_pairs with a workspace";
    return TKMX_ERR_TOO_LARGE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (num_pairs == 0) {
    TKMX_CUDA_OK(cudaMemsetAsync(expert_counts, 0, size_t(num_experts) * sizeof(int32_t), stream));
    return TKMX_OK;
  }
  if (expert_ids == nullptr || pos == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);  // binds the current device's context; allocates nothing
  if (st != TKMX_OK) return st;
  int device = 0;
  TKMX_CUDA_OK(cudaGetDevice(&device));
  int32_t* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_static_sort_scratch_ptr[device] == nullptr) {
      void* addr = nullptr;
      TKMX_CUDA_OK(cudaGetSymbolAddress(&addr, g_static_sort_scratch));
      g_static_sort_scratch_ptr[device] = static_cast<int32_t*>(addr);
    }
    scratch = g_static_sort_scratch_ptr[device];
  }
  return moe_sort_launch(expert_ids, num_pairs, num_experts, pos, expert_counts, scratch, stream);
}

int tkmx_moe_gather_rows(const void* src, const int32_t* pos, void* dst, int64_t num_pairs, int32_t top_k,
                         int64_t row_bytes, void* cuda_stream) {
  if (num_pairs < 0 || top_k <= 0 || row_bytes < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (num_pairs == 0 || row_bytes == 0) return TKMX_OK;
  if (src == nullptr || pos == nullptr || dst == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  if (row_bytes % 16 != 0 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u))
    return TKMX_ERR_ALIGNMENT;
  if (!fits_i32(num_pairs) || !fits_i32(row_bytes / 16)) return TKMX_ERR_TOO_LARGE;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  const int grid = dev->num_sms * 8;
  tkmx::moe_gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(src), pos, static_cast<uint4*>(dst), int(num_pairs), top_k, int(row_bytes / 16));
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

int tkmx_moe_combine(const void* rows, const int32_t* pos, const float* gates, void* y, int64_t num_tokens,
                     int32_t top_k, int64_t n, int dtype, void* cuda_stream) {
  if (num_tokens < 0 || top_k <= 0 || n < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (dtype != TKMX_BF16) return TKMX_ERR_UNSUPPORTED;
  if (num_tokens == 0 || n == 0) return TKMX_OK;
  if (rows == nullptr || pos == nullptr || gates == nullptr || y == nullptr) return TKMX_ERR_INVALID_ARGUMENT;
  if (n % 8 != 0 || ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(y)) & 15u))
    return TKMX_ERR_ALIGNMENT;
  if (!fits_i32(num_tokens * top_k) || !fits_i32(n)) return TKMX_ERR_TOO_LARGE;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  int64_t grid = dev->num_sms * 8;
  if (num_tokens < grid) grid = num_tokens;
  tkmx::moe_combine_kernel<<<int(grid), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(rows), pos, gates, static_cast<uint4*>(y), int(num_tokens), top_k, int(n / 8));
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

static int gather_impl(const void* x, const int32_t* indices, const int32_t* start, const int32_t* end,
                       void* out, int64_t in_rows, int64_t out_rows, int64_t row_bytes, void* cuda_stream) {
  if (in_rows < 0 || out_rows < 0 || row_bytes < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (out_rows == 0 || row_bytes == 0) return TKMX_OK;
  if (x == nullptr || indices == nullptr || out == nullptr || in_rows == 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (row_bytes % 16 != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u))
    return TKMX_ERR_ALIGNMENT;
  if (!fits_i32(in_rows) || !fits_i32(out_rows) || !fits_i32(row_bytes)) return TKMX_ERR_TOO_LARGE;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  int64_t grid = dev->num_sms * 8;
  if ((out_rows + 7) / 8 < grid) grid = (out_rows + 7) / 8;
  tkmx::ragged_gather_kernel<<<int(grid), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(x), indices, start, end, static_cast<uint4*>(out), int(in_rows), int(out_rows),
      int(row_bytes / 16));
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

int tkmx_ragged_gather(const void* x, const int32_t* indices, void* out, int64_t in_rows, int64_t out_rows,
                       int64_t row_bytes, void* cuda_stream) {
  return gather_impl(x, indices, nullptr, nullptr, out, in_rows, out_rows, row_bytes, cuda_stream);
}

int tkmx_ragged_scatter(const void* x, const int32_t* indices, const int32_t* start, const int32_t* end,
                        void* out, int64_t in_rows, int64_t out_rows, int64_t row_bytes, void* cuda_stream) {
  if (out_rows > 0 && row_bytes > 0 && (start == nullptr || end == nullptr)) return TKMX_ERR_INVALID_ARGUMENT;
  return gather_impl(x, indices, start, end, out, in_rows, out_rows, row_bytes, cuda_stream);
}

int tkmx_ragged_gather_reduce(const void* x, const int32_t* indices, const float* weights, const uint8_t* mask,
                              void* out, int64_t in_rows, int64_t input_size, int32_t reduce_group_size,
                              int64_t hidden, int dtype, void* cuda_stream) {
  if (in_rows < 0 || input_size < 0 || reduce_group_size <= 0 || hidden < 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (input_size % reduce_group_size != 0) return TKMX_ERR_INVALID_ARGUMENT;
  if (dtype != TKMX_BF16) return TKMX_ERR_UNSUPPORTED;
  if (input_size == 0 || hidden == 0) return TKMX_OK;
  if (x == nullptr || indices == nullptr || weights == nullptr || out == nullptr || in_rows == 0)
    return TKMX_ERR_INVALID_ARGUMENT;
  if (hidden % 8 != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u))
    return TKMX_ERR_ALIGNMENT;
  if (!fits_i32(in_rows) || !fits_i32(input_size) || !fits_i32(hidden)) return TKMX_ERR_TOO_LARGE;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  const int64_t out_rows = input_size / reduce_group_size;
  int64_t grid = dev->num_sms * 8;
  if (out_rows < grid) grid = out_rows;
  tkmx::ragged_gather_reduce_kernel<<<int(grid), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(x), indices, weights, mask, static_cast<uint4*>(out), int(in_rows),
      int(out_rows), reduce_group_size, int(hidden / 8));
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

// ---------------------------------------------------------------------------------------
// Expert-parallel layer over peer-mapped memory.
size_t tkmx_ep_plan_bytes(int32_t num_experts, int32_t world) {
  if (num_experts <= 0 || world <= 0 || num_experts % world != 0) return 0;
  return size_t(tkmx::ep_plan_layout(num_experts, world).total) * sizeof(int32_t);
}

static int ep_check_world(int32_t num_experts, int32_t world, int32_t rank) {
  if (num_experts <= 0 || world <= 0 || rank < 0 || rank >= world || num_experts % world != 0)
    return TKMX_ERR_INVALID_ARGUMENT;
  if (world > tkmx::kEpMaxWorld || num_experts > 1024) return TKMX_ERR_TOO_LARGE;
  return TKMX_OK;
}

int tkmx_cross_rank_barrier(const uint64_t* peer_table, uint32_t* flags_local, int32_t world, int32_t rank,
                            uint32_t sequence, int64_t timeout_ns, void* cuda_stream) {
  if (peer_table == nullptr || flags_local == nullptr || world <= 0 || rank < 0 || rank >= world || timeout_ns <= 0)
    return TKMX_ERR_INVALID_ARGUMENT;
  if (world > tkmx::kEpMaxWorld) return TKMX_ERR_TOO_LARGE;
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  tkmx::cross_rank_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      peer_table, flags_local, world, rank, sequence, uint64_t(timeout_ns), dev->status_ptr);
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

int tkmx_ep_exchange_plan(const int32_t* my_counts, const uint64_t* peer_table, int32_t* counts_all_local,
                          uint32_t* flags_local, uint32_t* arrive_local, int32_t* plan, int32_t num_experts,
                          int32_t world, int32_t rank, uint32_t sequence, int64_t timeout_ns, void* cuda_stream) {
  return tkmx_ep_exchange_plan_words(my_counts, peer_table, counts_all_local, flags_local, arrive_local, plan,
                                     num_experts, world, rank, sequence, timeout_ns, 0, cuda_stream);
}

size_t tkmx_ep_arrive_words(int32_t num_experts, int32_t world, int32_t once_per_rank) {
  if (ep_check_world(num_experts, world, 0) != TKMX_OK) return 0;
  return size_t(tkmx::ep_arrive_words(num_experts / world, once_per_rank != 0));
}

int tkmx_ep_exchange_plan_words(const int32_t* my_counts, const uint64_t* peer_table, int32_t* counts_all_local,
                                uint32_t* flags_local, uint32_t* arrive_local, int32_t* plan, int32_t num_experts,
                                int32_t world, int32_t rank, uint32_t sequence, int64_t timeout_ns,
                                int32_t once_per_rank, void* cuda_stream) {
  int st = ep_check_world(num_experts, world, rank);
  if (st != TKMX_OK) return st;
  if (my_counts == nullptr || peer_table == nullptr || counts_all_local == nullptr || flags_local == nullptr ||
      arrive_local == nullptr || plan == nullptr || timeout_ns <= 0)
    return TKMX_ERR_INVALID_ARGUMENT;
  DeviceInfo* dev = nullptr;
  st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  tkmx::EpExchangeParams x = {};
  x.my_counts = my_counts;
  x.peer_tab = peer_table;
  x.counts_all = counts_all_local;
  x.flags = flags_local;
  x.arrive = arrive_local;
  x.plan = plan;
  x.num_experts = num_experts;
  x.world = world;
  x.rank = rank;
  x.seq = sequence;
  x.timeout_ns = uint64_t(timeout_ns);
  x.status = dev->status_ptr;
  x.arrive_words = tkmx::ep_arrive_words(num_experts / world, once_per_rank != 0);
  tkmx::ep_exchange_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(cuda_stream)>>>(x);
  TKMX_CUDA_OK(cudaGetLastError());
  return TKMX_OK;
}

int tkmx_ep_moe_fused(const void* tokens, const int32_t* sorted_pair, const void* recv_local,
                      const void* rhs_local, const int32_t* plan, const uint64_t* peer_table,
                      const uint32_t* arrive_local, int64_t num_tokens, int32_t top_k, int64_t k, int64_t n,
                      int32_t num_experts, int32_t world, int32_t rank, int64_t capacity_rows, int dtype,
                      int phases, const tkmx_config* config, void* cuda_stream) {
  return tkmx_ep_moe_fused_once_per_rank(tokens, sorted_pair, nullptr, nullptr, recv_local, rhs_local, plan,
                                         peer_table, arrive_local, num_tokens, top_k, k, n, num_experts, world,
                                         rank, capacity_rows, dtype, phases, config, cuda_stream);
}

int tkmx_ep_moe_fused_once_per_rank(const void* tokens, const int32_t* sorted_pair, const int32_t* expert_ids,
                                    const int32_t* pair_pos, const void* recv_local, const void* rhs_local,
                                    const int32_t* plan, const uint64_t* peer_table, const uint32_t* arrive_local,
                                    int64_t num_tokens, int32_t top_k, int64_t k, int64_t n, int32_t num_experts,
                                    int32_t world, int32_t rank, int64_t capacity_rows, int dtype, int phases,
                                    const tkmx_config* config, void* cuda_stream) {
  int st = ep_check_world(num_experts, world, rank);
  if (st != TKMX_OK) return st;
  // Both arrays given: a token crosses the link once per destination rank.
  const bool once = expert_ids != nullptr || pair_pos != nullptr;
  if (once && (expert_ids == nullptr || pair_pos == nullptr)) return TKMX_ERR_INVALID_ARGUMENT;
  if (num_tokens < 0 || top_k <= 0 || k <= 0 || n <= 0 || capacity_rows <= 0 || phases < 1 ||
      phases > (once ? 7 : 3))
    return TKMX_ERR_INVALID_ARGUMENT;
  // reference words hold (local expert + 1) in 8 bits and a receive-buffer row in 24
  if (once && (num_experts / world > 254 || capacity_rows > (int64_t(1) << tkmx::kEpRefRowBits)))
    return TKMX_ERR_UNSUPPORTED;
  if (dtype != TKMX_BF16 && dtype != TKMX_F16) return TKMX_ERR_UNSUPPORTED;
  if (k % 8 != 0 || n % 8 != 0) return TKMX_ERR_ALIGNMENT;   // rows move and return in 16-byte pieces
  if (!fits_i32(num_tokens * top_k) || !fits_i32(k) || !fits_i32(n) || !fits_i32(capacity_rows) ||
      !fits_i32(capacity_rows + 256 * int64_t(num_experts / world + 1)) || !fits_i32(n * 2))
    return TKMX_ERR_TOO_LARGE;
  if (num_tokens == 0) return TKMX_OK;
  if (tokens == nullptr || sorted_pair == nullptr || recv_local == nullptr || rhs_local == nullptr ||
      plan == nullptr || peer_table == nullptr || arrive_local == nullptr)
    return TKMX_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(tokens) & 15u) != 0) return TKMX_ERR_ALIGNMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const int gl = num_experts / world;

  DeviceInfo* dev = nullptr;
  st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  ResolvedConfig rc;
  tkmx_config c = {};
  if (config != nullptr) c = *config;
  c.block_n = 256;   // the only width built for this form
  st = resolve_config(&c, n, gl, true, *dev, &rc);
  if (st != TKMX_OK) return st;
  // the ring may have to give room to the send-order table
  while (rc.num_stages > 2 &&
         tkmx::make_smem_layout(rc.block_n, rc.pair, rc.num_stages, gl, true, num_experts).total + 1024 >
             uint32_t(dev->smem_optin < kMaxSmemOptin ? dev->smem_optin : kMaxSmemOptin))
    --rc.num_stages;

  CUtensorMap ma, mb, mo = {};
  {
    const uint64_t dims[2] = {uint64_t(k), uint64_t(capacity_rows)};
    const uint64_t strides[1] = {uint64_t(k) * 2};
    const uint32_t box[2] = {64, 128};
    st = encode_map(&ma, recv_local, 2, dims, strides, box);
    if (st != TKMX_OK) return st;
  }
  {
    const uint64_t dims[3] = {uint64_t(n), uint64_t(k), uint64_t(gl)};
    const uint64_t strides[2] = {uint64_t(n) * 2, uint64_t(n) * uint64_t(k) * 2};
    const uint32_t box[3] = {64, 64, 1};
    st = encode_map(&mb, rhs_local, 3, dims, strides, box);
    if (st != TKMX_OK) return st;
  }
  const tkmx::EpPlanLayout pl = tkmx::ep_plan_layout(num_experts, world);
  RaggedGemmParams p = {};
  p.group_sizes = plan + pl.group_sizes;
  p.out = nullptr;
  p.m_total = int32_t(capacity_rows);
  p.rows = int32_t(capacity_rows);
  p.cols = int32_t(n);
  p.cdim = int32_t(k);
  p.num_groups = gl;
  p.rhs_groups = gl;
  p.group_begin = 0;
  p.group_end = gl;
  p.skip_zero_fill = 1;
  p.out_is_f32 = 0;
  p.out_is_f16 = dtype == TKMX_F16;
  p.out_vec_ok = 1;
  const uint32_t fmt = dtype == TKMX_BF16 ? 1u : 0u;
  p.idesc = tkmx::ptx::make_idesc(fmt, fmt, 0u, 1u, rc.pair ? 256u : 128u, uint32_t(rc.block_n));
  p.tile_width = rc.tile_width;
  p.minor_is_m = rc.minor_is_m;
  p.num_stages = rc.num_stages;
  p.status = dev->status_ptr;
  p.tma_store = 0;
  assign_sched(*dev, &p, true);
  p.swap_rows = rc.pair ? env_int("TKMX_SWAP_ROWS", 192, 0, 192) : 0;
  p.balance_tiles = env_int("TKMX_BALANCE_TILES", 0, 0, 1);
  p.prefetch_blocks = env_int("TKMX_EP_PREFETCH", 0, 0, 64);

  tkmx::EpFusedParams ep = {};
  ep.tokens = tokens;
  ep.sorted_pair = sorted_pair;
  ep.plan = plan;
  ep.peer_tab = peer_table;
  ep.arrive = arrive_local;
  ep.world = world;
  ep.rank = rank;
  ep.top_k = top_k;
  ep.num_experts = num_experts;
  ep.row_vec = int32_t(k * 2 / 16);
  ep.ret_row_bytes = int32_t(n * 2);
  ep.capacity_rows = int32_t(capacity_rows);
  ep.phases = phases;
  ep.progress = const_cast<uint32_t*>(arrive_local) + gl;
  ep.send_cursor = const_cast<uint32_t*>(arrive_local) + gl + 1;
  ep.static_items = env_int("TKMX_EP_STATIC_ITEMS", 0, 0, 1);
  ep.once_per_rank = once ? 1 : 0;
  ep.expert_ids = expert_ids;
  ep.pair_pos = pair_pos;
  // Senders stay at most this much of the receive buffer ahead of the multiplication (rows sent
  // earlier than that have left L2 by the time they are multiplied).  TKMX_EP_AHEAD_MB = 0: no pacing.
  ep.ahead_rows = int32_t(std::min<int64_t>(int64_t(env_int("TKMX_EP_AHEAD_MB", 0, 0, 4096)) * (1 << 20) / (k * 2),
                                            int64_t(1) << 30));

  // Every SM takes part (its two sender warps do, even when it draws no tile).
  int grid = dev->num_sms;
  if (rc.max_ctas > 0 && rc.max_ctas < grid) grid = rc.max_ctas;
  if (rc.pair) grid = std::max(2, grid / 2 * 2);
  if (rc.pair) return launch_one<tkmx::kRowsBN, 256, true, true>(ma, mb, mo, p, grid, stream, ep);
  return launch_one<tkmx::kRowsBN, 256, false, true>(ma, mb, mo, p, grid, stream, ep);
}

int tkmx_device_status(void) {
  DeviceInfo* dev = nullptr;
  int st = get_device_info(&dev);
  if (st != TKMX_OK) return st;
  TKMX_CUDA_OK(cudaDeviceSynchronize());
  int32_t v = 0;
  TKMX_CUDA_OK(cudaMemcpy(&v, dev->status_ptr, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) {
    TKMX_CUDA_OK(cudaMemset(dev->status_ptr, 0, sizeof(v)));
    g_last_cuda_error = "device status word = " + std::to_string(v);
    if (v == tkmx::kDevSchedConflict)
      g_last_cuda_error += " (two launches in flight shared one tile-counter word: more than " +
                           std::to_string(kSchedWords) + " dynamically scheduled launches overlapped, or a replayed "
                           "graph ran beside eager launches; results of both are incomplete)";
    if (v == tkmx::kDevEpOverflow)
      g_last_cuda_error += " (expert-parallel rows aimed outside a receive buffer were dropped)";
    return (v == tkmx::kDevSchedConflict || v == tkmx::kDevEpOverflow) ? TKMX_ERR_DEVICE_STATE
                                                                      : TKMX_ERR_DEVICE_TIMEOUT;
  }
  return TKMX_OK;
}

}  // extern "C"
