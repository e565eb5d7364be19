"""The B200 (sm_100a) ragged dot backend: the single registered implementation.

Takes the place of `PallasMosaicGpuRaggedDot`
(tokamax/_src/ops/ragged_dot/pallas_mosaic_gpu.py:85-518): same `Config` schema
(pallas_mosaic_gpu_common.py:45-73), same heuristics / autotuning-space hooks, same
error convention (NotImplementedError for unsupported combinations), but `_fwd`
enqueues hand-written CUDA kernels through the C ABI of include/tokamax_b200.h
instead of lowering a Pallas program.  All three dimension-number sets are served
natively (upstream has no Blackwell kernel for the ragged-contracting one,
pallas_mosaic_gpu.py:189-192).
"""

from __future__ import annotations

import dataclasses
import enum
from functools import partial
from typing import Any, Callable, ClassVar

import pydantic
import torch

from tokamax_b200 import _capi
from tokamax_b200 import op as op_lib
from tokamax_b200.quantization import QArray
from tokamax_b200.ragged_dot import base

GroupSizes = base.GroupSizes


class MatmulDimension(enum.IntEnum):
  M = 0
  N = 1


@pydantic.dataclasses.dataclass(frozen=True, slots=True)
class Config:
  """Kernel configuration; field names and defaults of the reference `Config`.

  How the fields map onto the sm_100a kernels:
    block_m     rows per output tile.  The kernels use the 128-row UMMA shape; smaller
                values are accepted (they are part of the reference search space) and
                run with 128.
    block_n     output columns per tile: 64, 128 or 256 (the reference fixes 128).
    block_k * num_stages
                contraction elements kept in flight in shared memory; realised as a
                ring of 64-element stages, capped by the 227 KiB of shared memory.
    collective  two CTAs of a cluster share one 256-row tile (`cta_group::2`).
    grid_minor_dim / grid_tile_width
                rasterisation of tiles inside a group (band width along the minor dim).
    epilogue_quant_qtype / epilogue_quant_subchannel_size
                the forward quantises its result in the epilogue and returns a QArray of
                float8_e4m3fn values with one float32 scale per row and `subchannel_size`
                (64, 128 or 256) columns.
    split_k, split_m, persistent, post_scale
                kept for schema compatibility; only their defaults are implemented.
  """

  block_m: pydantic.PositiveInt
  block_n: pydantic.PositiveInt
  block_k: pydantic.PositiveInt
  num_stages: pydantic.PositiveInt
  split_k: pydantic.PositiveInt = 1
  split_m: pydantic.PositiveInt = 1
  persistent: bool = True
  post_scale: bool = False
  collective: bool = False
  grid_minor_dim: MatmulDimension = MatmulDimension.N
  grid_tile_width: int = 1
  epilogue_quant_qtype: Any | None = None
  epilogue_quant_subchannel_size: int | None = None

  def __post_init__(self):
    if self.block_m % 8:
      raise ValueError("block_m must be a multiple of 8")

  @property
  def output_quantisation(self) -> int:
    """Columns per output scale when the epilogue quantises the result, else 0."""
    if self.epilogue_quant_qtype is None and self.epilogue_quant_subchannel_size is None:
      return 0
    name = str(self.epilogue_quant_qtype).replace("torch.", "")
    if name not in ("float8_e4m3fn", "f8_e4m3fn") or self.epilogue_quant_subchannel_size not in (64, 128, 256):
      raise NotImplementedError("epilogue quantisation: float8_e4m3fn with 64, 128 or 256 columns per scale")
    return int(self.epilogue_quant_subchannel_size)

  def native(self, max_stages: int = 8) -> tuple:
    """The knobs the kernels actually see; configs with equal `native()` run the same code."""
    stages = max(2, min(max_stages, (self.block_k * self.num_stages) // 64))
    return (self.block_n, stages, int(self.collective), int(self.grid_minor_dim),
            self.grid_tile_width)

  def to_capi(self) -> _capi.Config:
    if self.split_k != 1 or self.split_m != 1 or self.post_scale:
      raise NotImplementedError("split_k, split_m and post_scale are not implemented by the B200 kernels")
    block_n, stages, collective, minor, width = self.native()
    # The library lowers the depth itself if the ring does not fit in shared memory.
    return _capi.Config(block_m=128, block_n=block_n, block_k=64, num_stages=stages,
                        collective=collective, grid_minor_dim=minor, grid_tile_width=width, max_ctas=0)


_SUPPORTED_PRECISIONS = (None, "default", "high", "highest", "bf16_bf16_f32", "f16_f16_f32")


def canonicalize_precision(precision):
  """Accepts the precisions under which bf16/f16 inputs accumulate in float32."""
  if precision is None:
    return None
  if isinstance(precision, (tuple, list)):
    ps = {canonicalize_precision(p) for p in precision}
    if len(ps) != 1:
      raise NotImplementedError("different precisions per operand are not supported")
    return ps.pop()
  name = getattr(precision, "name", precision)
  if not isinstance(name, str):
    raise ValueError(f"unrecognised precision {precision!r}")
  name = name.lower()
  if name not in _SUPPORTED_PRECISIONS:
    raise NotImplementedError(f"precision {precision!r} is not supported by the B200 kernels")
  return name


def fusable_activation(activation) -> str | None:
  """Name of the epilogue activation that computes `activation`, or None if the callable is not
  one of the recognised ones (it is then applied after the kernel, like upstream does for
  backends without fusion).  Recognised: the torch / torch.nn.functional functions and module
  instances for relu, silu, gelu (erf form, or approximate="tanh"), tanh and sigmoid, and the
  same names as strings."""
  import functools
  import torch.nn.functional as F
  if activation is None:
    return None
  if isinstance(activation, str):
    return activation if activation in _capi.ELEMENT_ACTIVATIONS else None
  table = {torch.relu: "relu", F.relu: "relu", F.silu: "silu", torch.tanh: "tanh", F.tanh: "tanh",
           torch.sigmoid: "sigmoid", F.sigmoid: "sigmoid", F.gelu: "gelu_erf"}
  try:
    if activation in table:
      return table[activation]
  except TypeError:
    pass
  if isinstance(activation, functools.partial) and activation.func is F.gelu and not activation.args:
    kw = dict(activation.keywords)
    approx = kw.pop("approximate", "none")
    if not kw and approx in ("none", "tanh"):
      return "gelu_tanh" if approx == "tanh" else "gelu_erf"
  if isinstance(activation, torch.nn.GELU):
    return "gelu_tanh" if activation.approximate == "tanh" else "gelu_erf"
  for cls, name in ((torch.nn.ReLU, "relu"), (torch.nn.SiLU, "silu"), (torch.nn.Tanh, "tanh"),
                    (torch.nn.Sigmoid, "sigmoid")):
    if type(activation) is cls:
      return name
  return None


def _as_int32_device(gs, device) -> torch.Tensor:
  if isinstance(gs, GroupSizes):
    gs = gs.value
  if not isinstance(gs, torch.Tensor):
    gs = torch.as_tensor(gs)
  if gs.dtype != torch.int32:
    gs = gs.to(torch.int32)  # uint32 / int64 group sizes are accepted (test_base.py:137)
  if gs.device != device:
    gs = gs.to(device, non_blocking=True)
  return gs.contiguous()


def _dequantize_rows(x: QArray) -> torch.Tensor:
  """bf16 values of a row-quantised matrix: qvalue [M, K] with scale [M, K / sub]."""
  q, s = x.qvalue, x.scale
  if q.ndim != 2 or s.ndim != 2 or s.shape[0] != q.shape[0] or q.shape[1] % max(s.shape[1], 1):
    raise NotImplementedError("quantised lhs: values [M, K] with scales [M, K / subchannel]")
  sub = q.shape[1] // s.shape[1]
  return (q.to(torch.float32).reshape(q.shape[0], s.shape[1], sub) * s.to(torch.float32)[:, :, None]
          ).reshape(q.shape).to(torch.bfloat16)


def _normalize_rhs(rhs, rhs_scale):
  """Returns (rhs values [G,K,N], per-channel scale [G,N] or None)."""
  from tokamax_b200.quantization import as_array_or_qarray
  rhs = as_array_or_qarray(rhs)     # an AsQArray is quantised here, next to the kernel call
  if isinstance(rhs, QArray):
    if rhs_scale is not None:
      raise ValueError("rhs_scale given together with a quantised rhs")
    return rhs.qvalue, rhs.channel_scale()
  if rhs_scale is not None:
    s = rhs_scale
    if s.ndim == 4:  # [G, num_blocks, 1, N] of the TPU GMM-v2 route (gmm_v2.py:1423-1470)
      if s.shape[1] != 1 or s.shape[2] != 1:
        raise NotImplementedError("only one scale block along K (per-output-channel) is supported")
      s = s[:, 0, 0, :]
    elif s.ndim == 3:
      if s.shape[1] != 1:
        raise NotImplementedError("only per-output-channel scales are supported")
      s = s[:, 0, :]
    return rhs, s.to(torch.float32).contiguous()
  return rhs, None


@dataclasses.dataclass(frozen=True, kw_only=True)
class B200RaggedDot(base.RaggedDot):
  """Ragged dot on hand-written sm_100a kernels (tcgen05 + TMEM + TMA)."""

  config_cls: ClassVar[type] = Config
  supports_symbolic_shapes: ClassVar[bool] = False
  # fp8-e4m3 weights: True multiplies them as stored on the fp8 tensor cores against the
  # activations split into two e4m3 terms (needs 2*M*K bytes of scratch per call); False
  # expands the weights to bf16 inside the kernel and multiplies in bf16 (no scratch).
  native_fp8: bool = True
  # Local weight group count of the drhs (ragged-contracting) call under expert parallelism:
  # `group_sizes` then counts the global groups and the result holds the `num_actual_groups`
  # groups starting at `group_offset` (pallas_mosaic_tpu_v2.py:89-93 upstream).
  num_actual_groups: int | None = None

  def __post_init__(self):
    if self.vjp is None:
      fn = lambda *a, **kw: B200RaggedDot()(*a, **kw)  # fresh op: its own config lookup
      object.__setattr__(self, "vjp", partial(base.vjp, dlhs_ragged_dot=fn, drhs_ragged_dot=fn))

  def bind(self, lhs, rhs, *, precision=None, **kwargs):
    return super().bind(lhs, rhs, precision=canonicalize_precision(precision), **kwargs)

  def _fwd(self, lhs, rhs, *, group_sizes, ragged_dot_dimension_numbers, precision,
           preferred_element_type, return_residuals, config, activation=None,
           manual_axis_type=None, group_offset=None, rhs_scale=None, rhs_bias=None,
           maybe_quantize_lhs=False, zero_initialize=True, fuse_gateup_activation=None,
           lhs_quantization_dtype=None, rhs_quantization_dtype=None):
    del precision, manual_axis_type
    # Of the GMM-v2 keyword arguments these are implemented: the expert-parallel pair
    # `group_offset` (global group_sizes, rhs holding the local experts only) and
    # `zero_initialize`, `fuse_gateup_activation` and `rhs_bias`.  The others are refused
    # like the reference's GPU backends do.
    base.reject_gmm_v2_kwargs(
        maybe_quantize_lhs=maybe_quantize_lhs,
        lhs_quantization_dtype=lhs_quantization_dtype,
        rhs_quantization_dtype=rhs_quantization_dtype, where="B200RaggedDot")
    if fuse_gateup_activation is not None:
      if fuse_gateup_activation not in _capi.GATEUP_ACTIVATIONS:
        raise NotImplementedError(f"Unsupported activation function: {fuse_gateup_activation}")
      if return_residuals:
        # Residuals are the pre-activation product, which the fused epilogue never writes.
        raise NotImplementedError("fuse_gateup_activation cannot return residuals")
      if (ragged_dot_dimension_numbers != base.DEFAULT_RAGGED_DOT_DIM_NUMS or group_offset is not None
          or not zero_initialize):
        raise NotImplementedError("fuse_gateup_activation: default dimension numbers, no group window")
    bias = None
    if rhs_bias is not None:
      if (ragged_dot_dimension_numbers != base.DEFAULT_RAGGED_DOT_DIM_NUMS or group_offset is not None
          or not zero_initialize):
        raise NotImplementedError("rhs_bias: default dimension numbers, no group window")
      bias = rhs_bias
      if bias.ndim == 3:   # [G, 1, N], the reference's form (gmm_v2_test.py:1203-1206)
        if bias.shape[1] != 1:
          raise ValueError("rhs_bias must have shape [G, 1, N] or [G, N]")
        bias = bias[:, 0, :]
      if bias.ndim != 2:
        raise ValueError("rhs_bias must have shape [G, 1, N] or [G, N]")
    windowed = group_offset is not None or not zero_initialize
    drhs_window = (ragged_dot_dimension_numbers == base.RAGGED_CONTRACTING_DOT_DIM_NUMS
                   and (group_offset is not None or self.num_actual_groups is not None) and zero_initialize)
    if windowed and not drhs_window and ragged_dot_dimension_numbers != base.DEFAULT_RAGGED_DOT_DIM_NUMS:
      raise NotImplementedError("group_offset / zero_initialize=False: default or ragged-contracting "
                                "dimension numbers only")
    if isinstance(lhs, QArray):
      # A quantised lhs (the QArray an epilogue-quantising ragged_dot returned: e4m3 values with
      # one scale per row and block of columns) is expanded to bf16 before the product.
      lhs = _dequantize_rows(lhs)
    rhs, scale = _normalize_rhs(rhs, rhs_scale)
    if not lhs.is_cuda:
      raise NotImplementedError("B200RaggedDot runs on CUDA tensors only (no CPU fallback)")
    gs = _as_int32_device(group_sizes, lhs.device)
    lhs = lhs.contiguous()
    rhs = rhs.contiguous()
    dims = ragged_dot_dimension_numbers
    ccfg = config.to_capi() if config is not None else None

    if scale is None:
      out_dtype = preferred_element_type or torch.promote_types(lhs.dtype, rhs.dtype)
      if lhs.dtype != rhs.dtype:
        # One float32 operand next to a 16-bit one (the cotangent of a float32 output in
        # the backward pass): the tensor cores take 16-bit inputs and accumulate in
        # float32 (the BF16_BF16_F32 algorithm), so the float32 operand is rounded to the
        # other operand's dtype.  Anything else mixed is refused.
        small = {torch.bfloat16, torch.float16}
        if lhs.dtype == torch.float32 and rhs.dtype in small:
          lhs = lhs.to(rhs.dtype)
        elif rhs.dtype == torch.float32 and lhs.dtype in small:
          rhs = rhs.to(lhs.dtype)
        else:
          raise NotImplementedError(f"mixed input dtypes {lhs.dtype} x {rhs.dtype} are not supported")
    else:
      out_dtype = preferred_element_type or lhs.dtype

    if dims == base.DEFAULT_RAGGED_DOT_DIM_NUMS:
      if lhs.ndim != 2 or rhs.ndim != 3 or lhs.shape[1] != rhs.shape[1]:
        raise ValueError(f"incompatible shapes {tuple(lhs.shape)} and {tuple(rhs.shape)}")
      quant_sub = config.output_quantisation if config is not None else 0
      if quant_sub:
        if (scale is not None or windowed or return_residuals or lhs.dtype != rhs.dtype
            or fuse_gateup_activation is not None):
          raise NotImplementedError("epilogue quantisation: plain 16-bit forward without residuals")
        n = rhs.shape[2]
        if n % quant_sub:
          raise NotImplementedError("epilogue quantisation needs N to be a multiple of the subchannel size")
        act = fusable_activation(activation)
        if activation is not None and act is None:
          raise NotImplementedError("epilogue quantisation fuses only the recognised activations")
        q = torch.empty((lhs.shape[0], n), dtype=torch.float8_e4m3fn, device=lhs.device)
        qs = torch.empty((lhs.shape[0], n // quant_sub), dtype=torch.float32, device=lhs.device)
        if ccfg.block_n % quant_sub:
          ccfg.block_n = 256
        _capi.ragged_dot_fwd_quant_out(lhs, rhs, gs, q, qs, quant_sub, element_activation=act, config=ccfg)
        return QArray(q, qs), None
      # `activation` on the float32 accumulator inside the kernel (api.py:108-113 upstream), for
      # the callables the epilogue knows; never when the residuals (the result before the
      # activation) are asked for, and only on the plain 16-bit forward.
      fused_act = None
      if (activation is not None and not return_residuals and scale is None and not windowed
          and fuse_gateup_activation is None and lhs.dtype == rhs.dtype
          and (lhs.shape[0] == 0 or rhs.shape[0] > 0)):
        fused_act = fusable_activation(activation)
        if fused_act == "sigmoid" and (rhs.shape[0] == 0 or lhs.shape[1] == 0):
          fused_act = None
      if fuse_gateup_activation is not None or bias is not None or fused_act is not None:
        # Fused epilogue: tmp = ragged_dot(lhs, rhs) [* scale] + bias[group]; with
        # fuse_gateup_activation rhs = [gate | up] and out = act(tmp[:, :n/2]) * tmp[:, n/2:], so
        # the full-width product never reaches HBM (base.py:207-217 upstream).
        n = rhs.shape[2]
        if bias is not None:
          if tuple(bias.shape) != (rhs.shape[0], n):
            raise ValueError("rhs_bias must have shape [G, 1, N] or [G, N]")
          bias = bias.to(device=lhs.device, dtype=torch.float32).contiguous()
        if fuse_gateup_activation is not None and n % 2:
          raise ValueError("fuse_gateup_activation needs an even number of rhs columns")
        workspace = None
        if scale is not None:
          # 8-bit weights: the epilogue extras live in the native fp8 kernel.
          if rhs.dtype != torch.float8_e4m3fn or not self.native_fp8 or lhs.dtype != torch.bfloat16:
            raise NotImplementedError("fused epilogues with quantised rhs: fp8-e4m3 weights, bf16 lhs, native_fp8")
          need = _capi.workspace_bytes(0, lhs.shape[0], lhs.shape[1], n, rhs.shape[0], rhs.dtype)
          if not need:
            raise NotImplementedError("fused epilogues with fp8 weights need K to be a multiple of 16")
          workspace = torch.empty(need, dtype=torch.uint8, device=lhs.device)
          if ccfg is not None and fuse_gateup_activation is not None:
            ccfg.block_n, ccfg.collective = 256, 0
        elif lhs.dtype != rhs.dtype:
          raise NotImplementedError("fused epilogues: lhs and rhs of one 16-bit dtype")
        elif ccfg is not None and fuse_gateup_activation is not None and ccfg.block_n < 128:
          ccfg.block_n = 128
        out_cols = n // 2 if fuse_gateup_activation is not None else n
        out = torch.empty((lhs.shape[0], out_cols), dtype=out_dtype, device=lhs.device)
        _capi.ragged_dot_fwd_epilogue(lhs, rhs, gs, out, rhs_scale=scale, rhs_bias=bias,
                                      activation=fuse_gateup_activation, element_activation=fused_act,
                                      config=ccfg, workspace=workspace)
        residuals = out   # with the bias, before `activation`; never requested with gate/up
        if activation is not None and fused_act is None:
          out = activation(out)
        return out, residuals if return_residuals else None
      out = torch.empty((lhs.shape[0], rhs.shape[2]), dtype=out_dtype, device=lhs.device)
      if windowed:
        return self._fwd_windowed(lhs, rhs, gs, scale, out, ccfg, group_offset, zero_initialize,
                                  activation, return_residuals)
      workspace = None
      if scale is not None and self.native_fp8:
        need = _capi.workspace_bytes(0, lhs.shape[0], lhs.shape[1], rhs.shape[2], rhs.shape[0], rhs.dtype)
        if need:
          workspace = torch.empty(need, dtype=torch.uint8, device=lhs.device)
      _capi.ragged_dot_fwd(lhs, rhs, gs, out, rhs_scale=scale, config=ccfg, workspace=workspace)
    elif dims == base.TRANS_RHS_RAGGED_DOT_DIM_NUMS:
      if scale is not None:
        raise NotImplementedError("quantised rhs with transposed dimension numbers")
      if lhs.ndim != 2 or rhs.ndim != 3 or lhs.shape[1] != rhs.shape[2]:
        raise ValueError(f"incompatible shapes {tuple(lhs.shape)} and {tuple(rhs.shape)}")
      out = torch.empty((lhs.shape[0], rhs.shape[1]), dtype=out_dtype, device=lhs.device)
      _capi.ragged_dot_dlhs(lhs, rhs, gs, out, config=ccfg)
    elif dims == base.RAGGED_CONTRACTING_DOT_DIM_NUMS:
      if scale is not None:
        raise NotImplementedError("quantised rhs with ragged-contracting dimension numbers")
      if lhs.ndim != 2 or rhs.ndim != 2 or lhs.shape[0] != rhs.shape[0]:
        raise ValueError(f"incompatible shapes {tuple(lhs.shape)} and {tuple(rhs.shape)}")
      if drhs_window:
        # Expert-parallel shard: global group_sizes, the local experts' slabs only
        # (reference_tgmm, gmm_v2_test.py:109-160).  group_offset is read on the host.
        begin = 0 if group_offset is None else int(torch.as_tensor(group_offset).reshape(-1)[0])
        count = self.num_actual_groups if self.num_actual_groups is not None else gs.shape[0] - begin
        if begin < 0 or count < 0 or begin + count > gs.shape[0]:
          raise ValueError(f"group_offset ({begin}) + num_actual_groups ({count}) exceeds the "
                           f"{gs.shape[0]} entries of group_sizes")
        out = torch.empty((count, lhs.shape[1], rhs.shape[1]), dtype=out_dtype, device=lhs.device)
        _capi.ragged_dot_drhs(lhs, rhs, gs, out, config=ccfg, group_begin=begin)
      else:
        out = torch.empty((gs.shape[0], lhs.shape[1], rhs.shape[1]), dtype=out_dtype, device=lhs.device)
        _capi.ragged_dot_drhs(lhs, rhs, gs, out, config=ccfg)
    else:
      raise NotImplementedError(f"unsupported ragged dot dimension numbers: {dims}")

    residuals = out
    if activation is not None:
      out = activation(out)
    return out, residuals if return_residuals else None

  def _fwd_windowed(self, lhs, rhs, gs, scale, out, ccfg, group_offset, zero_initialize, activation,
                    return_residuals):
    """`group_sizes` counts the groups of the whole (global) problem while `rhs` holds the
    G_local experts starting at global group `group_offset`: global group j is multiplied by
    rhs[j - group_offset] if that index exists, and its rows are zeros otherwise -- or are
    left as allocated when zero_initialize=False (the caller overwrites or ignores them).
    Semantics of the reference's expert-parallel arguments (gmm_v2_test.py:44-99,
    pallas_mosaic_tpu_v2.py:89-93).  `group_offset` is read on the host (one
    synchronisation if it is a device tensor)."""
    g_global, g_local = gs.shape[0], rhs.shape[0]
    offset = 0 if group_offset is None else int(torch.as_tensor(group_offset).reshape(-1)[0])
    if offset % max(g_local, 1) != 0:
      raise NotImplementedError("group_offset must be a multiple of the number of local groups")
    begin = max(offset, 0)
    count = max(min(offset + g_local, g_global) - begin, 0)
    if zero_initialize:
      out.zero_()
    if count > 0 and out.numel() > 0:
      workspace = None
      if scale is not None and self.native_fp8:
        need = _capi.workspace_bytes(0, lhs.shape[0], lhs.shape[1], rhs.shape[2], rhs.shape[0], rhs.dtype)
        if need:
          workspace = torch.empty(need, dtype=torch.uint8, device=lhs.device)
      _capi.ragged_dot_fwd_cyclic(lhs, rhs, gs, out, rhs_scale=scale, zero_initialize=False,
                                  segment_begin=begin, segment_count=count, config=ccfg, workspace=workspace)
    residuals = out
    if activation is not None:
      out = activation(out)
    return out, residuals if return_residuals else None

  # ------------------------------------------------------------------ configs
  def _get_autotuning_cache_key(self, ba: op_lib.BoundArguments):
    skip = ("return_residuals",)

    def key_of(k, v):
      if k == "group_sizes":
        # One form whether the caller passed an array or a GroupSizes: (groups, representative
        # sizes or total rows).  A bare array stands for "rows of lhs spread over the groups",
        # which is what `bind` makes of it for the default dimension numbers.
        if isinstance(v, GroupSizes):
          return ("group_sizes", int(v.value.shape[0]), v.repr_value_or_total_size)
        return ("group_sizes", int(v.shape[0]), int(ba.arguments["lhs"].shape[0]))
      return op_lib.abstractify(v)

    return tuple((k, key_of(k, v)) for k, v in ba.arguments.items()
                 if k not in skip and v is not None and not callable(v))

  def _get_heuristics_config(self, ba: op_lib.BoundArguments) -> Config:
    """Measured-on-B200 defaults: 256-column tiles; CTA pairs (256-row tiles, ring of 5)
    once groups are large enough to fill them, single CTAs (ring of 4) for small groups."""
    lhs, rhs = ba.args[:2]
    dims = ba.arguments["ragged_dot_dimension_numbers"]
    gs = ba.arguments["group_sizes"]
    rep = gs.representative_value if isinstance(gs, GroupSizes) else None
    if dims == base.RAGGED_CONTRACTING_DOT_DIM_NUMS:
      n_out = rhs.shape[1]
      rows_per_tile_dim = lhs.shape[1]      # output rows are lhs features: never ragged
    else:
      n_out = rhs.shape[1] if dims == base.TRANS_RHS_RAGGED_DOT_DIM_NUMS else rhs.shape[2]
      nz = [v for v in rep if v > 0] if rep else []
      rows_per_tile_dim = (sum(nz) / len(nz)) if nz else lhs.shape[0]
    block_n = 256 if n_out > 128 else (128 if n_out > 64 else 64)
    collective = block_n >= 128 and rows_per_tile_dim >= 256
    # Row tiles fastest: CTAs running side by side then share a weight tile (autotuning on
    # B200 picked this order for nearly every shape).
    if isinstance(rhs, QArray):
      # 8-bit weights: single CTAs (the native fp8 kernel schedules them dynamically and runs
      # short tiles with swapped operands) and the deepest ring (6 x 64 = three 128-deep stages).
      return Config(block_m=128, block_n=256 if n_out > 128 else 128, block_k=64, num_stages=6, split_k=1,
                    persistent=True, collective=False, grid_minor_dim=MatmulDimension.M, grid_tile_width=1)
    return Config(block_m=128, block_n=block_n, block_k=64, num_stages=5 if collective else 4,
                  split_k=1, persistent=True, collective=collective,
                  grid_minor_dim=MatmulDimension.M, grid_tile_width=1)

  def _get_autotuning_configs(self, ba: op_lib.BoundArguments) -> set[Config]:
    """The sm100 search space of the reference (pallas_mosaic_gpu.py:403-514), widened
    by block_n in {128, 256}.

    Reference enumeration for unquantised lhs: "prefill" block_m {128} and "generate"
    block_m {8, 16, 32, 64}; block_k {128, 256, 512} kept when one stage row is a whole
    number of 128-byte swizzle rows for both operands; num_stages {2, 4};
    grid_minor_dim {M, N}; grid_tile_width {1, 2, 4, 8}; split_m {1}; collective
    {True, False}; post_scale {False} (prefill) / {True, False} (generate).
    `collective=True` entries run the CTA-pair kernel.  `post_scale=True` entries are listed
    (they are part of the space) but refused by `Config.to_capi`; the autotuner records the
    refusal like any other failed config (autotuner.py:173-203 upstream).  `block_m` below 128
    has no kernel of its own (the UMMA shape is 128 or 256 rows; few-row tiles are handled by
    the swapped-operand path inside the kernels), so those entries run like block_m = 128 and
    the autotuner, which keys on `Config.native()`, times each distinct kernel once.
    """
    lhs, rhs = ba.args[:2]
    bits = lambda dt: torch.finfo(dt).bits if dt.is_floating_point else torch.iinfo(dt).bits
    lhs_bits = bits(lhs.dtype)
    rhs_bits = bits(rhs.qtype if isinstance(rhs, QArray) else rhs.dtype)
    block_k_choices = [bk for bk in (128, 256, 512)
                       if (bk * rhs_bits) % (128 * 8) == 0 and (bk * lhs_bits) % (128 * 8) == 0]
    # Finer ring depths than the reference's (block_k, num_stages) grid can express:
    # block_k = 64 with 3 / 5 / 6 stages (the measured optimum is 4-5 stages of 64).
    fine = [(64, 3), (64, 5), (64, 6)]
    configs: set[Config] = set()

    def generate(block_m_choices, num_stages_choices, collective_choices, post_scale_choices):
      for block_m in block_m_choices:
        for block_n in (128, 256):
          for block_k in block_k_choices:
            for num_stages in num_stages_choices:
              for minor in (MatmulDimension.M, MatmulDimension.N):
                for width in (1, 2, 4, 8):
                  for collective in collective_choices:
                    for post_scale in post_scale_choices:
                      configs.add(Config(block_m=block_m, block_n=block_n, block_k=block_k,
                                         num_stages=num_stages, split_k=1, persistent=False,
                                         collective=collective, post_scale=post_scale,
                                         grid_minor_dim=minor, grid_tile_width=width, split_m=1))

    generate([128], [2, 4], [True, False], [False])                  # prefill
    generate([8, 16, 32, 64], [2, 4], [True, False], [True, False])  # generate (decode)
    for block_k, num_stages in fine:
      for block_n in (128, 256):
        for minor in (MatmulDimension.M, MatmulDimension.N):
          for width in (1, 2, 4, 8):
            for collective in (True, False):
              configs.add(Config(block_m=128, block_n=block_n, block_k=block_k,
                                 num_stages=num_stages, split_k=1, persistent=False,
                                 collective=collective, grid_minor_dim=minor,
                                 grid_tile_width=width, split_m=1))
    return configs

  def supported_on(self, device) -> bool:
    if not torch.cuda.is_available():
      return False
    major, _ = torch.cuda.get_device_capability(device)
    return major == 10
