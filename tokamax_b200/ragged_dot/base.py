"""Ragged dot: argument canonicalisation, dimension numbers, group sizes and the VJP.

Host-side mirror of tokamax/_src/ops/ragged_dot/base.py: same names, same argument
meaning, same errors.  Unlike the reference's base class this one carries NO
implementation of `_fwd` (upstream it is the XLA path, base.py:291-360): the only
implementation in this package is the B200 backend in `b200.py`, and there is no
fallback.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Sequence

import numpy as np
import torch

from tokamax_b200 import op as op_lib
from tokamax_b200.quantization import QArray


@dataclasses.dataclass(frozen=True)
class RaggedDotDimensionNumbers:
  """Same fields as jax.lax.RaggedDotDimensionNumbers."""

  dot_dimension_numbers: tuple
  lhs_ragged_dimensions: tuple
  rhs_group_dimensions: tuple

  def __init__(self, dot_dimension_numbers, lhs_ragged_dimensions, rhs_group_dimensions):
    (lc, rc), (lb, rb) = dot_dimension_numbers
    object.__setattr__(self, "dot_dimension_numbers",
                       ((tuple(lc), tuple(rc)), (tuple(lb), tuple(rb))))
    object.__setattr__(self, "lhs_ragged_dimensions", tuple(lhs_ragged_dimensions))
    object.__setattr__(self, "rhs_group_dimensions", tuple(rhs_group_dimensions))


# tokamax/_src/ops/ragged_dot/base.py:40-54
DEFAULT_RAGGED_DOT_DIM_NUMS = RaggedDotDimensionNumbers((([1], [1]), ([], [])), [0], [0])
TRANS_RHS_RAGGED_DOT_DIM_NUMS = RaggedDotDimensionNumbers((([1], [2]), ([], [])), [0], [0])
RAGGED_CONTRACTING_DOT_DIM_NUMS = RaggedDotDimensionNumbers((([0], [0]), ([], [])), [0], [])


def generate_group_sizes(*, m: int, num_groups: int, p: Sequence[float] | None = None,
                         seed: int = 0) -> tuple[int, ...]:
  """`m` draws with replacement from range(num_groups); returns the histogram (base.py:171-196)."""
  rng = np.random.default_rng(seed)
  group_ids = rng.choice(num_groups, (m,), p=p, replace=True)
  return tuple(map(int, np.bincount(group_ids, minlength=num_groups)))


class GroupSizes:
  """Group sizes with a static representative value (base.py:60-168).

  `value` is the runtime array (an int32/uint32 tensor, normally on the device).  The
  representative value -- a tuple of ints, or just the total, from which a seeded
  uniform multinomial split is generated -- is what cache keys, autotuning and
  benchmarking see, because the runtime values change from step to step.  Equality and
  hashing ignore `value`.
  """

  __slots__ = ("value", "repr_value_or_total_size")

  def __init__(self, value, repr_value_or_total_size: Sequence[int] | int):
    if isinstance(value, op_lib.ShapeDtype):
      shape, dtype = value.shape, value.dtype
    else:
      shape, dtype = tuple(value.shape), value.dtype
    if dtype not in (torch.int32, torch.int64, torch.uint8, torch.int8, torch.int16,
                     getattr(torch, "uint32", torch.int32)):
      raise ValueError("Group sizes must be integers.")
    (num_groups,) = shape
    if not isinstance(repr_value_or_total_size, int):
      if len(repr_value_or_total_size) != num_groups:
        raise ValueError("Representative value must have same length as the group sizes.")
      repr_value_or_total_size = tuple(int(v) for v in repr_value_or_total_size)
    if isinstance(value, op_lib.ShapeDtype):
      if isinstance(repr_value_or_total_size, int):
        rep = generate_group_sizes(m=repr_value_or_total_size, num_groups=num_groups)
      else:
        rep = repr_value_or_total_size
      value = torch.tensor(rep, dtype=torch.int32)
    self.value = value
    self.repr_value_or_total_size = repr_value_or_total_size

  @property
  def representative_value(self) -> tuple[int, ...]:
    if isinstance(self.repr_value_or_total_size, int):
      return generate_group_sizes(m=self.repr_value_or_total_size, num_groups=self.value.shape[0])
    return self.repr_value_or_total_size

  def abstractify(self):
    return ("GroupSizes", int(self.value.shape[0]), self.repr_value_or_total_size)

  def to_json(self):
    """`{num_groups, total_size}` or the tuple of ints (base.py:139-145)."""
    if isinstance(self.repr_value_or_total_size, int):
      return dict(num_groups=int(self.value.shape[0]), total_size=self.repr_value_or_total_size)
    return list(self.repr_value_or_total_size)

  @classmethod
  def from_json(cls, x):
    if isinstance(x, dict):
      return cls(op_lib.ShapeDtype((x["num_groups"],), torch.int32), x["total_size"])
    return cls(op_lib.ShapeDtype((len(x),), torch.int32), tuple(x))

  def __eq__(self, other):
    return (isinstance(other, GroupSizes) and self.value.shape == other.value.shape
            and self.repr_value_or_total_size == other.repr_value_or_total_size)

  def __hash__(self):
    return hash((tuple(self.value.shape), self.repr_value_or_total_size))

  def __repr__(self):
    return f"GroupSizes(num_groups={self.value.shape[0]}, repr={self.repr_value_or_total_size})"


def _shape(x) -> tuple[int, ...]:
  return tuple(x.shape)


def _dtype(x):
  return x.dtype


@dataclasses.dataclass(frozen=True)
class RaggedDot(op_lib.Op):
  """Ragged dot base class (argument handling only); see module docstring."""

  _: dataclasses.KW_ONLY
  checkify_group_sizes: bool = False

  def bind(self, lhs, rhs, *, group_sizes, ragged_dot_dimension_numbers=None, precision=None,
           preferred_element_type=None, return_residuals: bool = False, group_offset=None,
           activation: Callable | None = None, manual_axis_type=None, rhs_scale=None,
           rhs_bias=None, maybe_quantize_lhs: bool = False, zero_initialize: bool = True,
           fuse_gateup_activation: str | None = None, lhs_quantization_dtype=None,
           rhs_quantization_dtype=None) -> op_lib.BoundArguments:
    """Validates and canonicalises (base.py:226-288)."""
    if ragged_dot_dimension_numbers is None:
      ragged_dot_dimension_numbers = DEFAULT_RAGGED_DOT_DIM_NUMS
    if isinstance(group_sizes, (list, tuple)):
      group_sizes = tuple(int(v) for v in group_sizes)
      dev = lhs.device if isinstance(lhs, torch.Tensor) else None
      group_sizes = GroupSizes(torch.tensor(group_sizes, dtype=torch.int32, device=dev), group_sizes)
    if ragged_dot_dimension_numbers == DEFAULT_RAGGED_DOT_DIM_NUMS:
      if not isinstance(group_sizes, GroupSizes):
        group_sizes = GroupSizes(group_sizes, int(lhs.shape[0]))
      if self.checkify_group_sizes:
        gs = group_sizes.value
        if bool((gs.to(torch.int64) < 0).any()):
          raise ValueError("Negative group size.")
        if int(gs.to(torch.int64).sum()) > lhs.shape[0]:
          raise ValueError("Group size sum > num rows.")
    if preferred_element_type is not None and not isinstance(preferred_element_type, torch.dtype):
      raise ValueError("preferred_element_type must be a torch.dtype or None")
    return super().bind(
        lhs, rhs, group_sizes=group_sizes,
        ragged_dot_dimension_numbers=ragged_dot_dimension_numbers, precision=precision,
        preferred_element_type=preferred_element_type, return_residuals=return_residuals,
        group_offset=group_offset, activation=activation, manual_axis_type=manual_axis_type,
        rhs_scale=rhs_scale, rhs_bias=rhs_bias, maybe_quantize_lhs=maybe_quantize_lhs,
        zero_initialize=zero_initialize, fuse_gateup_activation=fuse_gateup_activation,
        lhs_quantization_dtype=lhs_quantization_dtype,
        rhs_quantization_dtype=rhs_quantization_dtype)

  def _fwd(self, lhs, rhs, *, group_sizes, ragged_dot_dimension_numbers, precision,
           preferred_element_type, return_residuals, config, activation=None,
           manual_axis_type=None, group_offset=None, rhs_scale=None, rhs_bias=None,
           maybe_quantize_lhs=False, zero_initialize=True, fuse_gateup_activation=None,
           lhs_quantization_dtype=None, rhs_quantization_dtype=None):
    raise NotImplementedError(
        "RaggedDot has no generic implementation in this package; use B200RaggedDot "
        "(tokamax_b200.ragged_dot.b200), the single registered backend.")


def reject_gmm_v2_kwargs(*, group_offset=None, rhs_bias=None, maybe_quantize_lhs=False,
                         zero_initialize=True, fuse_gateup_activation=None,
                         lhs_quantization_dtype=None, rhs_quantization_dtype=None,
                         where: str = "ragged_dot") -> None:
  """The TPU GMM-v2-only keyword arguments are accepted by `bind` and refused here,
  with the error type the reference uses (base.py:315-330, 395-410)."""
  if (group_offset is not None or rhs_bias is not None or maybe_quantize_lhs
      or not zero_initialize or fuse_gateup_activation is not None
      or lhs_quantization_dtype is not None or rhs_quantization_dtype is not None):
    raise NotImplementedError(
        f"{where} does not support group_offset, rhs_bias, maybe_quantize_lhs, "
        "zero_initialize=False, fuse_gateup_activation, lhs_quantization_dtype or "
        "rhs_quantization_dtype.")


def vjp(residuals, out, dout, lhs, rhs, *, group_sizes, ragged_dot_dimension_numbers, precision,
        preferred_element_type, activation=None, dlhs_ragged_dot: Callable[..., Any] = None,
        drhs_ragged_dot: Callable[..., Any] = None, manual_axis_type=None, group_offset=None,
        rhs_scale=None, rhs_bias=None, maybe_quantize_lhs=False, zero_initialize=True,
        fuse_gateup_activation=None, lhs_quantization_dtype=None, rhs_quantization_dtype=None):
  """Ragged dot VJP: (dlhs, drhs).  Follows base.py:363-462.

  dlhs = ragged_dot(dout, rhs) with the rhs contraction moved to its kept dimension
  (TRANS_RHS for the default numbers), in lhs.dtype; drhs = ragged_dot(lhs, dout) with
  the ragged dimension contracted and no group dimension (RAGGED_CONTRACTING), in
  rhs.dtype.
  """
  del out, preferred_element_type
  if rhs_scale is not None:
    raise NotImplementedError("rhs_scale is not supported on the ragged_dot backward path.")
  reject_gmm_v2_kwargs(group_offset=group_offset, rhs_bias=rhs_bias,
                       maybe_quantize_lhs=maybe_quantize_lhs, zero_initialize=zero_initialize,
                       fuse_gateup_activation=fuse_gateup_activation,
                       lhs_quantization_dtype=lhs_quantization_dtype,
                       rhs_quantization_dtype=rhs_quantization_dtype,
                       where="the ragged_dot backward path")
  if isinstance(lhs, QArray):
    raise NotImplementedError("gradients with respect to a quantised lhs are not defined")
  rhs_is_quantised = isinstance(rhs, QArray)
  if rhs_is_quantised:
    # The reference's vjp hands the quantised rhs on to the dlhs product (base.py:434-446);
    # here it is dequantised for it.  A quantised array has no gradient of its own.
    from tokamax_b200.quantization import as_array
    rhs = as_array(rhs).to(lhs.dtype)

  if activation is not None:
    # d(activation)/d(pre-activation) applied to dout (base.py:412-414).
    with torch.enable_grad():
      pre = residuals.detach().requires_grad_(True)
      act = activation(pre)
      (dout,) = torch.autograd.grad(act, pre, dout)
    dout = dout.contiguous()

  dot_dim_nums = ragged_dot_dimension_numbers.dot_dimension_numbers
  lhs_ragged = ragged_dot_dimension_numbers.lhs_ragged_dimensions
  rhs_group = ragged_dot_dimension_numbers.rhs_group_dimensions
  (lhs_contract, rhs_contract), (lhs_batch, rhs_batch) = dot_dim_nums
  lhs_not_kept = (*lhs_batch, *lhs_contract)
  rhs_not_kept = (*rhs_batch, *rhs_contract, *rhs_group)
  lhs_kept = [i for i in range(lhs.ndim) if i not in lhs_not_kept]
  rhs_kept = [i for i in range(rhs.ndim) if i not in rhs_not_kept]
  assert len(lhs_batch) == len(rhs_batch)
  assert dout.ndim == len(lhs_batch) + len(lhs_kept) + len(rhs_kept)
  dout_batch = list(range(len(lhs_batch)))
  dout_lhs_kept = list(range(len(lhs_batch), len(lhs_batch) + len(lhs_kept)))
  dout_rhs_kept = list(range(len(lhs_batch) + len(lhs_kept), dout.ndim))

  dlhs_dims = RaggedDotDimensionNumbers(
      ((dout_rhs_kept, rhs_kept), (dout_batch, rhs_batch)),
      [(len(dout_batch) + lhs_kept.index(d)) for d in lhs_ragged], rhs_group)
  dlhs = dlhs_ragged_dot(dout, rhs, group_sizes=group_sizes,
                         ragged_dot_dimension_numbers=dlhs_dims, precision=precision,
                         preferred_element_type=lhs.dtype)
  if rhs_is_quantised:
    return dlhs, None
  drhs_dims = RaggedDotDimensionNumbers(
      ((lhs_kept, dout_lhs_kept), (lhs_batch, dout_batch)), lhs_ragged, [])
  drhs = drhs_ragged_dot(lhs, dout, group_sizes=group_sizes,
                         ragged_dot_dimension_numbers=drhs_dims, precision=precision,
                         preferred_element_type=rhs.dtype)
  return dlhs, drhs
