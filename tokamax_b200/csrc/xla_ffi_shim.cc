// XLA typed-FFI handlers over the C ABI of include/tokamax_b200.h, for JAX callers
// (`jax.ffi.register_ffi_target` / `jax.ffi.ffi_call`).  This is the binding a
// maintainer of the reference adds so that `PallasMosaicGpuRaggedDot._fwd`
// (tokamax/_src/ops/ragged_dot/pallas_mosaic_gpu.py:103-244) can call these kernels.
//
// Needs jaxlib's header tree (`xla/ffi/api/ffi.h`, found via `jax.ffi.include_dir()`);
// it is therefore NOT part of libtokamax_b200.so and is compiled only where jaxlib is
// installed:
//   g++ -std=c++17 -shared -fPIC -I<jax.ffi.include_dir()> -I/usr/local/cuda/include
//       xla_ffi_shim.cc -L../lib -ltokamax_b200 -o ../lib/libtokamax_b200_ffi.so
//
// Handler contract: buffers are XLA-owned device pointers (never retained), the stream
// comes from XLA, the handler only enqueues (no synchronisation, no host read of
// group_sizes), and errors come back as ffi::Error.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <initializer_list>
#include <string>

#include "../../include/tokamax_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int ToTkmxDtype(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::BF16: return TKMX_BF16;
    case ffi::DataType::F16: return TKMX_F16;
    case ffi::DataType::F32: return TKMX_F32;
    case ffi::DataType::F8E4M3FN: return TKMX_F8E4M3;
    case ffi::DataType::S8: return TKMX_S8;
    default: return -1;
  }
}

ffi::Error ToError(int status, const char* what) {
  if (status == TKMX_OK) return ffi::Error::Success();
  std::string msg = std::string(what) + ": " + tkmx_status_string(status);
  if (status == TKMX_ERR_CUDA) msg += std::string(" (") + tkmx_last_cuda_error() + ")";
  if (status == TKMX_ERR_INVALID_ARGUMENT) return ffi::Error::InvalidArgument(msg);
  if (status == TKMX_ERR_UNSUPPORTED || status == TKMX_ERR_ALIGNMENT || status == TKMX_ERR_TOO_LARGE)
    return ffi::Error(ffi::ErrorCode::kUnimplemented, msg);
  return ffi::Error::Internal(msg);
}

// A result (or operand) buffer must have exactly the shape the kernel is about to write:
// XLA owns the memory, and a mismatched ffi_call result spec would otherwise be overrun.
template <typename Buf>
bool HasShape(const Buf& buf, std::initializer_list<int64_t> want) {
  auto d = buf.dimensions();
  if (d.size() != want.size()) return false;
  size_t i = 0;
  for (int64_t w : want)
    if (d[i++] != w) return false;
  return true;
}

tkmx_config MakeConfig(int32_t block_n, int32_t num_stages, int32_t collective,
                       int32_t grid_minor_dim, int32_t grid_tile_width) {
  tkmx_config c = {};
  c.block_m = 128;
  c.block_n = block_n;
  c.block_k = 64;
  c.num_stages = num_stages;
  c.collective = collective;
  c.grid_minor_dim = grid_minor_dim;
  c.grid_tile_width = grid_tile_width;
  return c;
}

// out[m, n] = ragged_dot(lhs[m, k], rhs[g, k, n] | rhs[g, n, k], group_sizes[g])
ffi::Error FwdImpl(cudaStream_t stream, ffi::AnyBuffer lhs, ffi::AnyBuffer rhs,
                   ffi::Buffer<ffi::DataType::S32> group_sizes, ffi::Result<ffi::AnyBuffer> out,
                   int32_t rhs_layout, int32_t block_n, int32_t num_stages, int32_t collective,
                   int32_t grid_minor_dim, int32_t grid_tile_width) {
  auto ld = lhs.dimensions();
  auto rd = rhs.dimensions();
  if (ld.size() != 2 || rd.size() != 3 || group_sizes.dimensions().size() != 1)
    return ffi::Error::InvalidArgument("ragged_dot fwd: expected lhs[m,k], rhs[g,*,*], group_sizes[g]");
  const int64_t m = ld[0], k = ld[1], g = rd[0];
  const int64_t n = rhs_layout == TKMX_RHS_GKN ? rd[2] : rd[1];
  const int64_t rk = rhs_layout == TKMX_RHS_GKN ? rd[1] : rd[2];
  if (rk != k || group_sizes.dimensions()[0] != g)
    return ffi::Error::InvalidArgument("ragged_dot fwd: contraction / group dimensions do not match");
  if (!HasShape(*out, {m, n})) return ffi::Error::InvalidArgument("ragged_dot fwd: out must be [m, n]");
  tkmx_config cfg = MakeConfig(block_n, num_stages, collective, grid_minor_dim, grid_tile_width);
  int st = tkmx_ragged_dot_fwd(lhs.untyped_data(), rhs.untyped_data(), group_sizes.typed_data(),
                               /*rhs_scale=*/nullptr, out->untyped_data(), /*workspace=*/nullptr, 0, m,
                               k, n, g, ToTkmxDtype(lhs.element_type()), ToTkmxDtype(rhs.element_type()),
                               ToTkmxDtype(out->element_type()), rhs_layout, &cfg, stream);
  return ToError(st, "tkmx_ragged_dot_fwd");
}

// Forward with 8-bit weights rhs[g, k, n] (F8E4M3FN or S8) and rhs_scale f32[g, n].  The second
// result is the scratch buffer: the caller sizes it with tkmx_ragged_dot_workspace_bytes (a
// pure function of the shapes) and XLA allocates it.  With a scratch of the size asked for,
// e4m3 weights take the native fp8 tensor-core kernel.
ffi::Error FwdQuantImpl(cudaStream_t stream, ffi::AnyBuffer lhs, ffi::AnyBuffer rhs,
                        ffi::Buffer<ffi::DataType::S32> group_sizes,
                        ffi::Buffer<ffi::DataType::F32> rhs_scale, ffi::Result<ffi::AnyBuffer> out,
                        ffi::Result<ffi::AnyBuffer> workspace, int32_t block_n, int32_t num_stages,
                        int32_t collective, int32_t grid_minor_dim, int32_t grid_tile_width) {
  auto ld = lhs.dimensions();
  auto rd = rhs.dimensions();
  if (ld.size() != 2 || rd.size() != 3 || rd[1] != ld[1] || group_sizes.dimensions()[0] != rd[0])
    return ffi::Error::InvalidArgument("ragged_dot quantised fwd: expected lhs[m,k], rhs[g,k,n], group_sizes[g]");
  if (!HasShape(rhs_scale, {rd[0], rd[2]}) && !HasShape(rhs_scale, {rd[0], 1, rd[2]}))
    return ffi::Error::InvalidArgument("ragged_dot quantised fwd: rhs_scale must be [g, n] or [g, 1, n]");
  if (!HasShape(*out, {ld[0], rd[2]}))
    return ffi::Error::InvalidArgument("ragged_dot quantised fwd: out must be [m, n]");
  tkmx_config cfg = MakeConfig(block_n, num_stages, collective, grid_minor_dim, grid_tile_width);
  int st = tkmx_ragged_dot_fwd(lhs.untyped_data(), rhs.untyped_data(), group_sizes.typed_data(),
                               rhs_scale.typed_data(), out->untyped_data(), workspace->untyped_data(),
                               workspace->size_bytes(), ld[0], ld[1], rd[2], rd[0],
                               ToTkmxDtype(lhs.element_type()), ToTkmxDtype(rhs.element_type()),
                               ToTkmxDtype(out->element_type()), TKMX_RHS_GKN, &cfg, stream);
  return ToError(st, "tkmx_ragged_dot_fwd");
}

// out[m, n/2] = act(tmp[:, :n/2]) * tmp[:, n/2:], tmp = ragged_dot(lhs, rhs[g, k, n]).
ffi::Error FwdGateUpImpl(cudaStream_t stream, ffi::AnyBuffer lhs, ffi::AnyBuffer rhs,
                         ffi::Buffer<ffi::DataType::S32> group_sizes, ffi::Result<ffi::AnyBuffer> out,
                         int32_t activation, int32_t block_n, int32_t num_stages, int32_t collective,
                         int32_t grid_minor_dim, int32_t grid_tile_width) {
  auto ld = lhs.dimensions();
  auto rd = rhs.dimensions();
  if (ld.size() != 2 || rd.size() != 3 || rd[1] != ld[1] || group_sizes.dimensions()[0] != rd[0])
    return ffi::Error::InvalidArgument("ragged_dot gate/up fwd: expected lhs[m,k], rhs[g,k,n], group_sizes[g]");
  if (rd[2] % 2 != 0 || !HasShape(*out, {ld[0], rd[2] / 2}))
    return ffi::Error::InvalidArgument("ragged_dot gate/up fwd: out must be [m, n / 2]");
  tkmx_config cfg = MakeConfig(block_n, num_stages, collective, grid_minor_dim, grid_tile_width);
  int st = tkmx_ragged_dot_fwd_gateup(lhs.untyped_data(), rhs.untyped_data(), group_sizes.typed_data(),
                                      out->untyped_data(), ld[0], ld[1], rd[2], rd[0],
                                      ToTkmxDtype(lhs.element_type()), ToTkmxDtype(out->element_type()),
                                      activation, &cfg, stream);
  return ToError(st, "tkmx_ragged_dot_fwd_gateup");
}

// dlhs[m, k] = dout[m, n] . rhs[g, k, n]^T
ffi::Error DlhsImpl(cudaStream_t stream, ffi::AnyBuffer dout, ffi::AnyBuffer rhs,
                    ffi::Buffer<ffi::DataType::S32> group_sizes, ffi::Result<ffi::AnyBuffer> dlhs,
                    int32_t block_n, int32_t num_stages, int32_t collective, int32_t grid_minor_dim,
                    int32_t grid_tile_width) {
  auto dd = dout.dimensions();
  auto rd = rhs.dimensions();
  if (dd.size() != 2 || rd.size() != 3 || rd[2] != dd[1] || !HasShape(group_sizes, {rd[0]}))
    return ffi::Error::InvalidArgument("ragged_dot dlhs: expected dout[m,n], rhs[g,k,n], group_sizes[g]");
  if (!HasShape(*dlhs, {dd[0], rd[1]})) return ffi::Error::InvalidArgument("ragged_dot dlhs: dlhs must be [m, k]");
  tkmx_config cfg = MakeConfig(block_n, num_stages, collective, grid_minor_dim, grid_tile_width);
  int st = tkmx_ragged_dot_dlhs(dout.untyped_data(), rhs.untyped_data(), group_sizes.typed_data(),
                                dlhs->untyped_data(), nullptr, 0, dd[0], rd[1], rd[2], rd[0],
                                ToTkmxDtype(dout.element_type()), ToTkmxDtype(dlhs->element_type()), &cfg,
                                stream);
  return ToError(st, "tkmx_ragged_dot_dlhs");
}

// drhs[g, k, n] = lhs[rows of g]^T . dout[rows of g]
ffi::Error DrhsImpl(cudaStream_t stream, ffi::AnyBuffer lhs, ffi::AnyBuffer dout,
                    ffi::Buffer<ffi::DataType::S32> group_sizes, ffi::Result<ffi::AnyBuffer> drhs,
                    int32_t block_n, int32_t num_stages, int32_t collective, int32_t grid_minor_dim,
                    int32_t grid_tile_width) {
  auto ld = lhs.dimensions();
  auto dd = dout.dimensions();
  if (ld.size() != 2 || dd.size() != 2 || ld[0] != dd[0])
    return ffi::Error::InvalidArgument("ragged_dot drhs: expected lhs[m,k], dout[m,n]");
  if (group_sizes.dimensions().size() != 1)
    return ffi::Error::InvalidArgument("ragged_dot drhs: group_sizes must be [g]");
  const int64_t g = group_sizes.dimensions()[0];
  if (!HasShape(*drhs, {g, ld[1], dd[1]})) return ffi::Error::InvalidArgument("ragged_dot drhs: drhs must be [g, k, n]");
  tkmx_config cfg = MakeConfig(block_n, num_stages, collective, grid_minor_dim, grid_tile_width);
  int st = tkmx_ragged_dot_drhs(lhs.untyped_data(), dout.untyped_data(), group_sizes.typed_data(),
                                drhs->untyped_data(), nullptr, 0, ld[0], ld[1], dd[1], g,
                                ToTkmxDtype(lhs.element_type()), ToTkmxDtype(drhs->element_type()), &cfg,
                                stream);
  return ToError(st, "tkmx_ragged_dot_drhs");
}

}  // namespace

#define TKMX_CONFIG_ATTRS()                \
  .Attr<int32_t>("block_n")                \
      .Attr<int32_t>("num_stages")         \
      .Attr<int32_t>("collective")         \
      .Attr<int32_t>("grid_minor_dim")     \
      .Attr<int32_t>("grid_tile_width")

XLA_FFI_DEFINE_HANDLER_SYMBOL(TkmxRaggedDotFwd, FwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()                   // lhs
                                  .Arg<ffi::AnyBuffer>()                   // rhs
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()  // group_sizes
                                  .Ret<ffi::AnyBuffer>()                   // out
                                  .Attr<int32_t>("rhs_layout") TKMX_CONFIG_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TkmxRaggedDotFwdQuant, FwdQuantImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()                   // lhs
                                  .Arg<ffi::AnyBuffer>()                   // rhs (8-bit)
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()  // group_sizes
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()  // rhs_scale
                                  .Ret<ffi::AnyBuffer>()                   // out
                                  .Ret<ffi::AnyBuffer>()                   // workspace
                                      TKMX_CONFIG_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TkmxRaggedDotFwdGateUp, FwdGateUpImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()                   // lhs
                                  .Arg<ffi::AnyBuffer>()                   // rhs
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()  // group_sizes
                                  .Ret<ffi::AnyBuffer>()                   // out [m, n/2]
                                  .Attr<int32_t>("activation") TKMX_CONFIG_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TkmxRaggedDotDlhs, DlhsImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()                   // dout
                                  .Arg<ffi::AnyBuffer>()                   // rhs
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()  // group_sizes
                                  .Ret<ffi::AnyBuffer>()                   // dlhs
                                      TKMX_CONFIG_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TkmxRaggedDotDrhs, DrhsImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()                   // lhs
                                  .Arg<ffi::AnyBuffer>()                   // dout
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()  // group_sizes
                                  .Ret<ffi::AnyBuffer>()                   // drhs
                                      TKMX_CONFIG_ATTRS());
