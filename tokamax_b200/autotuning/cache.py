"""On-disk autotuning cache: one JSON file per (device kind, op class).

Same file naming as tokamax/_src/autotuning/cache.py:81-110:
`data/autotuning/<device kind lower-cased, spaces -> '_'>/<snake_case op class>.json`,
a JSON object mapping a serialised argument spec to `{serialised config: BenchmarkData}`,
keys and values in the reference's wire format (`spec_to_json` / `config_to_json` below), so
that an entry of the reference's own cache files parses here and the files written here parse
upstream; read lazily on first access per device kind.
"""

from __future__ import annotations

import dataclasses
import json
import logging
import os
import re
from typing import Any

import torch

from tokamax_b200 import benchmarking
from tokamax_b200 import config as config_lib
from tokamax_b200 import op as op_lib
from tokamax_b200.autotuning import autotuner

log = logging.getLogger(__name__)
CACHE_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "data", "autotuning")

_DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i32": torch.int32,
           "i8": torch.int8, "f8_e4m3fn": torch.float8_e4m3fn}


def cache_file(op, device_kind: str, base_dir: str = CACHE_PATH) -> str:
  kind = device_kind.lower().replace(" ", "_")
  op_name = re.sub(r"(?!^)([A-Z])", r"_\1", type(op).__name__).lower()
  return os.path.join(base_dir, kind, f"{op_name}.json")


# Field order of a key, as the reference writes it (the order of `_fwd`'s signature).
_KEY_FIELDS = ("lhs", "rhs", "group_sizes", "ragged_dot_dimension_numbers", "precision",
               "preferred_element_type", "return_residuals", "activation")
# Field order of a serialised Config (tokamax/data/autotuning/nvidia_b200/pallas_mosaic_gpu_ragged_dot.json).
_CONFIG_FIELDS = ("block_m", "block_n", "block_k", "num_stages", "split_k", "split_m", "persistent",
                  "async_store", "post_scale", "collective", "grid_minor_dim", "grid_tile_width")
_SHORT = {v: k for k, v in _DTYPES.items()}


def _array(v) -> str:
  if isinstance(v, torch.Tensor):
    v = op_lib.ShapeDtype(tuple(v.shape), v.dtype)
  return v.short()


def _encode(name: str, v: Any, arguments: dict) -> Any:
  from tokamax_b200.ragged_dot.base import GroupSizes, RaggedDotDimensionNumbers
  if isinstance(v, (op_lib.ShapeDtype, torch.Tensor)):
    if name == "group_sizes":   # a bare array: what `bind` would make of it
      total = int(arguments["lhs"].shape[0])
      return {"num_groups": int(v.shape[0]), "total_size": total}
    return _array(v)
  if isinstance(v, GroupSizes):
    return v.to_json()
  if isinstance(v, RaggedDotDimensionNumbers):
    (lc, rc), (lb, rb) = v.dot_dimension_numbers
    return {"dot_dimension_numbers": [[list(lc), list(rc)], [list(lb), list(rb)]],
            "lhs_ragged_dimensions": list(v.lhs_ragged_dimensions),
            "rhs_group_dimensions": list(v.rhs_group_dimensions)}
  if isinstance(v, torch.dtype):
    return _SHORT.get(v, str(v).replace("torch.", ""))
  if hasattr(v, "qvalue") and hasattr(v, "scale"):
    return {"qvalue": _array(v.qvalue), "scale": _array(v.scale)}
  if name == "precision":
    p = "DEFAULT" if v is None else str(getattr(v, "name", v)).upper()
    return [p, p]
  if callable(v):
    return getattr(v, "__name__", type(v).__name__)
  return v


def spec_to_json(arguments: dict) -> str:
  """Serialises bound arguments to a cache key in the reference's wire format
  (tokamax/_src/autotuning/cache.py:37-49 with the field serialisers of
  tokamax/_src/pydantic.py:245-352 and ops/ragged_dot/base.py:139-170): arrays as `bf16[M,K]`
  strings, group sizes as `{"num_groups", "total_size"}` or the representative list, named
  dimension-number fields, `precision` as a pair of names, then the keyword arguments the
  reference's GPU backends do not have (only those that are set)."""
  d = {}
  for k in _KEY_FIELDS:
    v = arguments.get(k)
    if k == "precision":
      d[k] = _encode(k, v, arguments)
    elif k == "return_residuals":
      d[k] = False       # never part of the tuning problem
    else:
      d[k] = None if v is None else _encode(k, v, arguments)
  defaults = {"maybe_quantize_lhs": False, "zero_initialize": True}
  for k in sorted(arguments):
    v = arguments[k]
    if k in _KEY_FIELDS or v is None or defaults.get(k, object()) == v:
      continue
    d[k] = _encode(k, v, arguments)
  return json.dumps(d, separators=(",", ":"))


def _decode(name: str, v: Any) -> Any:
  from tokamax_b200.ragged_dot.base import GroupSizes, RaggedDotDimensionNumbers
  if isinstance(v, str) and (m := re.fullmatch(r"(\w+)\[([\d,]*)\]", v)) and m.group(1) in _DTYPES:
    shape = tuple(int(s) for s in m.group(2).split(",") if s)
    return op_lib.ShapeDtype(shape, _DTYPES[m.group(1)])
  if name == "group_sizes":
    return GroupSizes.from_json(v)
  if name == "ragged_dot_dimension_numbers":
    d = v["dot_dimension_numbers"]
    return RaggedDotDimensionNumbers(((d[0][0], d[0][1]), (d[1][0], d[1][1])), v["lhs_ragged_dimensions"],
                                     v["rhs_group_dimensions"])
  if name == "precision":
    ps = {str(p).upper() for p in (v if isinstance(v, list) else [v])}
    return None if ps <= {"DEFAULT", "NONE"} else ps.pop().lower()
  if name == "preferred_element_type" and isinstance(v, str):
    return _DTYPES.get(v) or getattr(torch, v)
  if isinstance(v, dict) and "qvalue" in v and "scale" in v:
    from tokamax_b200.quantization import QArray
    return QArray(_decode("", v["qvalue"]), _decode("", v["scale"]))
  return v


def spec_from_json(s: str) -> dict:
  """Keyword arguments for `op.bind` from a cache key.  `activation` names are dropped (the
  callable cannot be rebuilt; it is not part of the in-memory cache key either)."""
  out = {k: _decode(k, v) for k, v in json.loads(s).items() if v is not None}
  out.pop("activation", None)
  out.pop("return_residuals", None)
  return out


def config_to_json(config) -> str:
  d = dataclasses.asdict(config)
  d.setdefault("async_store", False)     # field of the shipped reference caches' schema
  out = {k: (int(d[k]) if hasattr(d[k], "value") else d[k]) for k in _CONFIG_FIELDS}
  for k in sorted(d):                    # fields newer than those files, only when set
    if k not in out and d[k] is not None:
      out[k] = str(d[k]).replace("torch.", "") if isinstance(d[k], torch.dtype) else d[k]
  return json.dumps(out, separators=(",", ":"))


def config_from_json(config_cls, s: str):
  """A Config from its JSON, ignoring fields this Config class does not have."""
  known = {f.name for f in dataclasses.fields(config_cls)}
  return config_cls(**{k: v for k, v in json.loads(s).items() if k in known})


class AutotuningCache(dict):
  """{device_kind: {cache key: AutotuningData}}, loaded lazily per device kind."""

  def __init__(self, op, paths=(CACHE_PATH,)):
    super().__init__()
    self.op = op
    self.cache_paths = tuple(paths)

  def __missing__(self, device_kind: str) -> dict:
    self[device_kind] = cache = self._load_cache(device_kind)
    return cache

  def _load_cache(self, device_kind: str) -> dict:
    out: dict = {}
    for base_dir in self.cache_paths:
      if config_lib.ignore_autotuning_cache.value and base_dir == CACHE_PATH:
        continue
      path = cache_file(self.op, device_kind, base_dir)
      try:
        with open(path) as f:
          raw = json.load(f)
      except FileNotFoundError:
        continue
      except Exception:  # a broken cache file must not break the op
        log.exception("Failed to parse autotuning cache file: %s", path)
        continue
      for spec_json, entries in raw.items():
        try:
          ba = self.op.bind(**spec_from_json(spec_json))
          data = autotuner.AutotuningData({
              config_from_json(self.op.config_cls, cfg): benchmarking.BenchmarkData.fromdict(bd)
              for cfg, bd in entries.items()})
          out[ba.autotuning_cache_key] = data
        except Exception:
          log.exception("Skipping unreadable autotuning cache entry in %s", path)
    return out


def dump(op, entries: dict[str, "autotuner.AutotuningData"]) -> str:
  """Serialises {spec json: AutotuningData} (errors dropped) to the cache file format."""
  out = {}
  for spec_json, data in entries.items():
    out[spec_json] = {config_to_json(c): d.asdict() for c, d in data.prune_errors().items()}
  return json.dumps(out, indent=1, sort_keys=True)
