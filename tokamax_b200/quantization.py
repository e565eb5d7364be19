"""Quantised-array plumbing for weights.

`QArray` plays the role of `qwix.QArray` as used by tokamax/_src/quantization.py:39-93:
a quantised value with per-tile scales.  Only what the ragged_dot path needs exists
here: per-(expert, output-channel) fp32 scales for fp8-e4m3 / int8 weights, i.e. a
scale tile of (1, K, 1) over a [G, K, N] weight.
"""

from __future__ import annotations

import dataclasses

import torch

_QMAX = {torch.float8_e4m3fn: 448.0, torch.int8: 127.0}


@dataclasses.dataclass(frozen=True)
class QArray:
  """qvalue [G, K, N] (fp8-e4m3 or int8) with scale [G, 1, N] or [G, N] (float32)."""

  qvalue: torch.Tensor
  scale: torch.Tensor

  @property
  def shape(self):
    return self.qvalue.shape

  @property
  def dtype(self):
    """The dtype the dequantised array has (the scale's)."""
    return self.scale.dtype

  @property
  def qtype(self):
    return self.qvalue.dtype

  @property
  def ndim(self):
    return self.qvalue.ndim

  @property
  def scale_tile_shape(self) -> tuple[int, ...]:
    s = self.scale.shape if self.scale.ndim == self.qvalue.ndim else (
        self.scale.shape[0], 1, self.scale.shape[1])
    return tuple(q // t for q, t in zip(self.qvalue.shape, s))

  def abstractify(self):
    from tokamax_b200.op import ShapeDtype
    return ("QArray", ShapeDtype(tuple(self.qvalue.shape), self.qvalue.dtype),
            ShapeDtype(tuple(self.scale.shape), self.scale.dtype))

  def channel_scale(self) -> torch.Tensor:
    """Scales as a contiguous float32 [G, N] tensor (what the kernels take)."""
    s = self.scale
    if s.ndim == 3:
      if s.shape[1] != 1:
        raise NotImplementedError("only per-output-channel scales (tile (1, K, 1)) are supported")
      s = s[:, 0, :]
    return s.to(torch.float32).contiguous()


def quantize_per_channel(w: torch.Tensor, qtype: torch.dtype) -> QArray:
  """Absmax quantiser over K for w [G, K, N]: scale = max|w| / qmax (float32).

  Same scheme as `quantize_tensor(w, qtype, axis=1, block_size=K)` of
  tokamax/_src/ops/experimental/gmm_v2/util.py:28-51 (int8: the float is truncated
  toward zero by the final cast, fp8: rounded to nearest by the cast).
  """
  if qtype not in _QMAX:
    raise NotImplementedError(f"unsupported quantised dtype {qtype}")
  qmax = _QMAX[qtype]
  w32 = w.to(torch.float32)
  scale = w32.abs().amax(dim=1, keepdim=True) / qmax
  q = torch.nan_to_num(w32 / scale, nan=0.0).clamp(-qmax, qmax)
  q = q.trunc().to(torch.int8) if qtype == torch.int8 else q.to(qtype)
  return QArray(q.contiguous(), scale.to(torch.float32).contiguous())


@dataclasses.dataclass(frozen=True)
class AsQArray:
  """An array that is to be quantised before the computation, so that the quantisation can
  happen next to (or inside) the kernel (tokamax/_src/quantization.py:39-72).  Here only the
  scheme the kernels take exists: weights [G, K, N] with one scale per expert and output
  channel, i.e. channelwise axes (0, 2); `calibration_method` "absmax"."""

  value: torch.Tensor
  qtype: torch.dtype
  channelwise_axes: tuple = (0, 2)
  tiled_axes: dict | None = None
  calibration_method: str = "absmax"

  shape = property(lambda self: self.value.shape)
  dtype = property(lambda self: self.value.dtype)
  ndim = property(lambda self: self.value.ndim)

  def as_qarray(self) -> QArray:
    if tuple(sorted(self.channelwise_axes)) != (0, 2) or self.tiled_axes or self.calibration_method != "absmax":
      raise NotImplementedError("AsQArray: per-(expert, output-channel) absmax quantisation only")
    return quantize_per_channel(self.value, self.qtype)


def as_array_or_qarray(x):
  """Quantises an AsQArray now; passes tensors and QArrays through (quantization.py:81-84)."""
  return x.as_qarray() if isinstance(x, AsQArray) else x


def as_array(x):
  """Dequantises a QArray (qvalue * scale in the scale dtype); passes tensors through."""
  x = as_array_or_qarray(x)
  if isinstance(x, QArray):
    s = x.scale if x.scale.ndim == x.qvalue.ndim else x.scale[:, None, :]
    return x.qvalue.to(s.dtype) * s
  return x
