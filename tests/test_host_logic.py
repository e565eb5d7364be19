"""CPU tests of the host side: argument handling, configs, caches, the C ABI surface."""

import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

import tokamax_b200 as tk
from tokamax_b200 import _capi, config as config_lib, op as op_lib
from tokamax_b200.autotuning import autotuner, cache
from tokamax_b200.benchmarking import BenchmarkData
from tokamax_b200.ragged_dot import api, arg_specs, b200, base

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _args(m=64, k=32, n=16, g=4):
  return torch.zeros(m, k, dtype=torch.bfloat16), torch.zeros(g, k, n, dtype=torch.bfloat16)


# ---------------------------------------------------------------- C ABI surface
def test_library_exports_every_declared_symbol():
  header = open(os.path.join(ROOT, "include", "tokamax_b200.h")).read()
  declared = set(re.findall(r"TKMX_API\s+[\w\s\*]+?\b(tkmx_\w+)\s*\(", header))
  assert declared, "no declarations found in the header"
  lib = ctypes.CDLL(_capi.library_path())
  for name in sorted(declared):
    assert hasattr(lib, name), f"{name} declared in the header but not exported"
  assert declared == set(_capi.EXPORTED_SYMBOLS)


def test_library_host_only_calls():
  lib = _capi.load()
  assert lib.tkmx_abi_version() == 1
  assert _capi.status_string(0) == "ok"
  assert "not implemented" in _capi.status_string(_capi.ERR_UNSUPPORTED)
  assert _capi.workspace_bytes(_capi.OP_FWD, 1024, 128, 256, 8, torch.bfloat16) == 0


def test_status_to_exception_mapping():
  with pytest.raises(NotImplementedError):
    _capi.check(_capi.ERR_UNSUPPORTED, "x")
  with pytest.raises(NotImplementedError):
    _capi.check(_capi.ERR_ALIGNMENT, "x")
  with pytest.raises(ValueError):
    _capi.check(_capi.ERR_INVALID_ARGUMENT, "x")
  with pytest.raises(RuntimeError):
    _capi.check(_capi.ERR_CUDA, "x")


def test_no_cpu_path():
  lhs, rhs = _args()
  with pytest.raises((NotImplementedError, ValueError)):
    tk.ragged_dot(lhs, rhs, torch.tensor([16] * 4, dtype=torch.int32))


# ---------------------------------------------------------------- bind / canonicalisation
def test_bind_canonicalises():
  op = b200.B200RaggedDot()
  lhs, rhs = _args()
  ba = op.bind(lhs, rhs, group_sizes=[16, 16, 16, 16])
  a = ba.arguments
  assert a["ragged_dot_dimension_numbers"] == base.DEFAULT_RAGGED_DOT_DIM_NUMS
  assert isinstance(a["group_sizes"], base.GroupSizes)
  assert a["group_sizes"].representative_value == (16, 16, 16, 16)
  assert a["precision"] is None and a["preferred_element_type"] is None
  # a bare tensor gets the total row count as its representative size
  ba2 = op.bind(lhs, rhs, group_sizes=torch.tensor([16] * 4, dtype=torch.int32))
  assert ba2.arguments["group_sizes"].repr_value_or_total_size == 64
  assert sum(ba2.arguments["group_sizes"].representative_value) == 64
  assert ba.positional_names == ("lhs", "rhs")
  with pytest.raises(ValueError):
    op.bind(lhs, rhs, group_sizes=torch.tensor([1.0, 2.0]))
  with pytest.raises(NotImplementedError):
    op.bind(lhs, rhs, group_sizes=[16] * 4, precision="F64_F64_F64")


def test_checkify_group_sizes():
  op = b200.B200RaggedDot(checkify_group_sizes=True)
  lhs, rhs = _args(m=1024)
  with pytest.raises(ValueError, match="Negative"):
    op.bind(lhs, rhs, group_sizes=torch.tensor([2, 3, -1, 4], dtype=torch.int32))
  with pytest.raises(ValueError, match="sum"):
    op.bind(lhs, rhs, group_sizes=torch.tensor([1022, 1, 1, 1], dtype=torch.int32))


def test_group_sizes_semantics():
  v = torch.tensor([1, 2, 3], dtype=torch.int32)
  a, b = base.GroupSizes(v, 6), base.GroupSizes(torch.tensor([3, 2, 1], dtype=torch.int32), 6)
  assert a == b and hash(a) == hash(b)          # runtime values are ignored
  assert a != base.GroupSizes(v, (1, 2, 3))
  with pytest.raises(ValueError):
    base.GroupSizes(v, (1, 2))
  assert base.GroupSizes.from_json(a.to_json()) == a
  c = base.GroupSizes(v, (1, 2, 3))
  assert base.GroupSizes.from_json(c.to_json()) == c
  gs = base.generate_group_sizes(m=512, num_groups=8)
  assert sum(gs) == 512 and gs == (70, 48, 55, 60, 68, 67, 68, 76)


def test_vjp_dimension_numbers():
  """The backward sub-calls get TRANS_RHS and RAGGED_CONTRACTING numbers and the operand dtypes."""
  calls = []

  def fake(l, r, *, group_sizes, ragged_dot_dimension_numbers, precision, preferred_element_type):
    calls.append((tuple(l.shape), tuple(r.shape), ragged_dot_dimension_numbers, preferred_element_type))
    return torch.zeros(1)

  lhs, rhs = _args()
  dout = torch.zeros(64, 16, dtype=torch.bfloat16)
  base.vjp(None, None, dout, lhs, rhs, group_sizes=[16] * 4,
           ragged_dot_dimension_numbers=base.DEFAULT_RAGGED_DOT_DIM_NUMS, precision=None,
           preferred_element_type=None, dlhs_ragged_dot=fake, drhs_ragged_dot=fake)
  assert calls[0] == ((64, 16), (4, 32, 16), base.TRANS_RHS_RAGGED_DOT_DIM_NUMS, torch.bfloat16)
  assert calls[1] == ((64, 32), (64, 16), base.RAGGED_CONTRACTING_DOT_DIM_NUMS, torch.bfloat16)
  with pytest.raises(NotImplementedError):
    base.vjp(None, None, dout, lhs, rhs, group_sizes=[16] * 4,
             ragged_dot_dimension_numbers=base.DEFAULT_RAGGED_DOT_DIM_NUMS, precision=None,
             preferred_element_type=None, dlhs_ragged_dot=fake, drhs_ragged_dot=fake, rhs_bias=dout)


# ---------------------------------------------------------------- configs
def test_config_schema_and_search_space():
  op = b200.B200RaggedDot()
  lhs, rhs = _args(m=4096, k=512, n=1024, g=8)
  ba = op.bind(lhs, rhs, group_sizes=[512] * 8)
  h = ba.heuristics_config
  assert isinstance(h, b200.Config) and h.block_n == 256
  space = op._get_autotuning_configs(ba)
  # reference space: 96 prefill + 384 generate configs per block_n; two block_n values here
  assert len(space) == 2 * (96 + 768) + 3 * 2 * 2 * 4 * 2  # reference space per block_n + finer ring depths
  assert {c.block_m for c in space} == {8, 16, 32, 64, 128}
  assert {c.block_k for c in space} == {64, 128, 256, 512}
  assert {c.grid_tile_width for c in space} == {1, 2, 4, 8}
  assert h in ba.autotuning_configs
  with pytest.raises(Exception):
    b200.Config(block_m=12, block_n=128, block_k=128, num_stages=2)
  c = b200.Config(block_m=128, block_n=128, block_k=256, num_stages=2)
  assert c.native()[1] == 8 and c.native()[2] == 0 and hash(c) == hash(b200.Config(**json.loads(cache.config_to_json(c))))


def test_config_resolution_order():
  op = b200.B200RaggedDot()
  lhs, rhs = _args()
  explicit = b200.Config(block_m=128, block_n=64, block_k=128, num_stages=2)
  assert op.replace(config=explicit).bind(lhs, rhs, group_sizes=[16] * 4).default_config == explicit
  ba = op.bind(lhs, rhs, group_sizes=[16] * 4)
  with config_lib.ignore_autotuning_cache(True):
    assert ba.default_config == ba.heuristics_config
    with config_lib.autotuning_cache_miss_fallback("error"):
      with pytest.raises(ValueError, match="No config found"):
        _ = ba.default_config
  # an overlay entry wins over heuristics
  fast = b200.Config(block_m=128, block_n=128, block_k=128, num_stages=2)
  slow = b200.Config(block_m=128, block_n=64, block_k=128, num_stages=4)
  data = autotuner.AutotuningData({fast: BenchmarkData(0, 0, (1.0, 1.1)), slow: BenchmarkData(0, 0, (2.0,)),
                                   explicit: RuntimeError("boom")})
  assert data.fastest_config == fast and set(data.prune_errors()) == {fast, slow}
  result = tk.AutotuningResult("cpu", ((ba, data),))
  with result:
    assert ba.default_config == fast
  assert ba.default_config == ba.heuristics_config
  loaded = tk.AutotuningResult.loads(result.dumps())
  assert loaded.device_kind == "cpu" and loaded.data[0][1].fastest_config == fast
  with pytest.raises(ExceptionGroup):
    _ = autotuner.AutotuningData({fast: RuntimeError("x")}).fastest_config


def test_cache_key_and_json_round_trip(tmp_path):
  op = b200.B200RaggedDot()
  for spec in arg_specs.ARG_SPECS:
    ba = op.bind(**spec.args)
    s = cache.spec_to_json(dict(ba.arguments))
    ba2 = op.bind(**cache.spec_from_json(s))
    assert ba2.autotuning_cache_key == ba.autotuning_cache_key, spec.full_name
  # file naming follows the reference: <device kind>/<snake case class>.json
  assert cache.cache_file(op, "NVIDIA B200", "x").endswith(os.path.join("x", "nvidia_b200", "b200_ragged_dot.json"))
  ba = op.bind(**arg_specs.NAMED_ARG_SPECS["compute_bound"].args)
  cfg = b200.Config(block_m=128, block_n=256, block_k=128, num_stages=4)
  data = autotuner.AutotuningData({cfg: BenchmarkData(0, 0, (0.5, 0.6, 0.55))})
  path = cache.cache_file(op, "Fake GPU", str(tmp_path))
  os.makedirs(os.path.dirname(path))
  open(path, "w").write(cache.dump(op, {cache.spec_to_json(dict(ba.arguments)): data}))
  loaded = cache.AutotuningCache(op, paths=(str(tmp_path),))["Fake GPU"]
  assert loaded[ba.autotuning_cache_key].fastest_config == cfg


def test_shipped_cache_files_parse():
  d = cache.CACHE_PATH
  if not os.path.isdir(d):
    pytest.skip("no shipped autotuning cache yet")
  op = b200.B200RaggedDot()
  for kind in os.listdir(d):
    loaded = cache.AutotuningCache(op)[kind.replace("_", " ")]
    for data in loaded.values():
      assert isinstance(data.fastest_config, b200.Config)


def test_api_errors_without_gpu():
  lhs, rhs = _args()
  with pytest.raises(ValueError, match="Unknown implementation"):
    api.ragged_dot(lhs, rhs, [16] * 4, implementation="triton")
  with pytest.raises(ValueError, match="empty"):
    api.ragged_dot(lhs, rhs, [16] * 4, implementation=())
  with pytest.raises(NotImplementedError, match="group_offset"):
    api.ragged_dot(lhs, rhs, [16] * 4, group_offset=torch.zeros(1))
  with pytest.raises(ValueError, match="reduction dimension"):
    api.ragged_dot(lhs[:, :8], rhs, [16] * 4)
  assert list(api.IMPLEMENTATIONS) == ["b200"]


def test_workloads():
  for name in ("cfg1", "cfg2", "cfg3", "cfg4"):
    w = arg_specs.workload(name)
    assert len(w.group_sizes) == w.g and sum(w.group_sizes) == w.m
    assert w == arg_specs.workload(name)  # seeded
  ids, gates = arg_specs.topk_routing(64, 8, 2, seed=3)
  assert ids.shape == (64, 2) and (ids[:, 0] != ids[:, 1]).all()
  assert (gates[:, 0] >= gates[:, 1]).all() and (gates > 0).all()
  assert len(arg_specs.ARG_SPECS) == 33


def test_host_pipeline_chunk_plan():
  """Chunks of the host-buffer pipeline are whole groups, cover every group and row once, and
  carry about `chunk_bytes` of input each (pure host logic, no CUDA)."""
  from tokamax_b200.ragged_dot.host import HostRaggedDot
  plan = HostRaggedDot.plan_chunks
  class _P:  # plan_chunks only reads chunk_bytes
    chunk_bytes = 1000
  sizes = [3, 0, 5, 1, 0, 0, 7]
  chunks = plan(_P, sizes, k=10, n=4, elt=2)      # a group costs (rows * 10 + 40) * 2 bytes
  assert chunks[0][0] == 0 and chunks[-1][1] == len(sizes)
  assert all(a[1] == b[0] and a[3] == b[2] for a, b in zip(chunks, chunks[1:]))
  assert chunks[-1][3] == sum(sizes)
  for gb, ge, rb, re in chunks:
    assert re - rb == sum(sizes[gb:ge])
  big = plan(_P, [100] * 4, k=10, n=4, elt=2)      # every group alone exceeds the budget
  assert [(c[0], c[1]) for c in big] == [(0, 1), (1, 2), (2, 3), (3, 4)]
  _P.chunk_bytes = 1 << 30
  assert plan(_P, sizes, k=10, n=4, elt=2) == [(0, 7, 0, 16)]


def test_permutation_ops_have_no_cpu_path():
  from tokamax_b200 import ragged_gather as rg
  x = torch.zeros(4, 8)
  idx = torch.zeros(2, dtype=torch.int32)
  with pytest.raises(NotImplementedError):
    rg.ragged_gather(x, idx, torch.tensor([0]), torch.tensor([4]))
  with pytest.raises(NotImplementedError):
    rg.ragged_scatter(x, idx, torch.tensor([0]), torch.tensor([4]))
  with pytest.raises(NotImplementedError):
    rg.ragged_gather_reduce(x.bfloat16(), idx, torch.ones(2), torch.ones(2, dtype=torch.bool), reduce_group_size=2)
  with pytest.raises(ValueError, match="Unknown implementation"):
    rg.ragged_gather(x, idx, torch.tensor([0]), torch.tensor([4]), implementation="xla")


def test_epilogue_keyword_validation_needs_no_gpu():
  """Argument errors of the fused-epilogue keywords are raised on the host before any CUDA
  work: unknown activation names, residuals with gate/up, windows combined with epilogues,
  malformed biases."""
  from tokamax_b200.ragged_dot import api
  op = api.IMPLEMENTATIONS["b200"]
  lhs = torch.zeros(8, 16, dtype=torch.bfloat16)
  rhs = torch.zeros(2, 16, 32, dtype=torch.bfloat16)
  gs = torch.tensor([4, 4], dtype=torch.int32)
  with pytest.raises(NotImplementedError, match="Unsupported activation"):
    op(lhs, rhs, group_sizes=gs, fuse_gateup_activation="relu")
  with pytest.raises(NotImplementedError, match="residuals"):
    op(lhs, rhs, group_sizes=gs, fuse_gateup_activation="silu", return_residuals=True)
  with pytest.raises(NotImplementedError, match="group window"):
    op(lhs, rhs, group_sizes=gs, fuse_gateup_activation="silu", group_offset=0)
  with pytest.raises(NotImplementedError, match="group window"):
    op(lhs, rhs, group_sizes=gs, rhs_bias=torch.zeros(2, 32), zero_initialize=False)
  with pytest.raises(ValueError, match="rhs_bias"):
    op(lhs, rhs, group_sizes=gs, rhs_bias=torch.zeros(2, 3, 32))
  with pytest.raises(ValueError, match="rhs_bias"):
    op(lhs, rhs, group_sizes=gs, rhs_bias=torch.zeros(32))
  # everything valid: the call then stops at the device check -- there is no CPU path
  with pytest.raises(NotImplementedError, match="CUDA tensors only"):
    op(lhs, rhs, group_sizes=gs, rhs_bias=torch.zeros(2, 1, 32), fuse_gateup_activation="silu")
  with pytest.raises(NotImplementedError):   # still refused, like the reference's GPU backends
    op(lhs, rhs, group_sizes=gs, maybe_quantize_lhs=True)


def test_cache_wire_format_is_the_references():
  """Keys and configs are written in the wire format of the reference's cache files
  (tokamax/_src/autotuning/cache.py:81-110; example keys below are of the form found in
  tokamax/data/autotuning/nvidia_b200/pallas_mosaic_gpu_ragged_dot.json): such a key parses,
  binds, and serialises back to the identical string; a config with the older `async_store`
  field parses; a caller's tensors hit the entry loaded from the file."""
  op = b200.B200RaggedDot()
  keys = [
      '{"lhs":"bf16[262144,7168]","rhs":"bf16[256,7168,2048]","group_sizes":{"num_groups":256,"total_size":262144},'
      '"ragged_dot_dimension_numbers":{"dot_dimension_numbers":[[[1],[1]],[[],[]]],"lhs_ragged_dimensions":[0],'
      '"rhs_group_dimensions":[0]},"precision":["DEFAULT","DEFAULT"],"preferred_element_type":null,'
      '"return_residuals":false,"activation":null}',
      '{"lhs":"bf16[131072,2048]","rhs":"bf16[131072,768]","group_sizes":{"num_groups":128,"total_size":131072},'
      '"ragged_dot_dimension_numbers":{"dot_dimension_numbers":[[[0],[0]],[[],[]]],"lhs_ragged_dimensions":[0],'
      '"rhs_group_dimensions":[]},"precision":["DEFAULT","DEFAULT"],"preferred_element_type":null,'
      '"return_residuals":false,"activation":null}',
      '{"lhs":"bf16[8,4096]","rhs":"bf16[8,4096,4096]","group_sizes":[1,1,1,1,1,1,1,1],'
      '"ragged_dot_dimension_numbers":{"dot_dimension_numbers":[[[1],[1]],[[],[]]],"lhs_ragged_dimensions":[0],'
      '"rhs_group_dimensions":[0]},"precision":["DEFAULT","DEFAULT"],"preferred_element_type":null,'
      '"return_residuals":false,"activation":null}',
  ]
  for key in keys:
    ba = op.bind(**cache.spec_from_json(key))
    assert cache.spec_to_json(dict(ba.arguments)) == key
  cfg_json = ('{"block_m":128,"block_n":128,"block_k":128,"num_stages":2,"split_k":1,"split_m":1,"persistent":false,'
              '"async_store":false,"post_scale":false,"collective":true,"grid_minor_dim":0,"grid_tile_width":2}')
  cfg = cache.config_from_json(b200.Config, cfg_json)
  assert cfg.collective and cfg.grid_tile_width == 2 and cfg.block_k == 128
  assert cache.config_to_json(cfg) == cfg_json
  # a call with plain tensors (bare group_sizes array) finds the entry a file key binds to
  ba_file = op.bind(**cache.spec_from_json(keys[0]))
  lhs = torch.empty(262144, 7168, dtype=torch.bfloat16, device="meta")
  rhs = torch.empty(256, 7168, 2048, dtype=torch.bfloat16, device="meta")
  gs = torch.empty(256, dtype=torch.int32, device="meta")
  assert op.bind(lhs, rhs, group_sizes=gs).autotuning_cache_key == ba_file.autotuning_cache_key
  ba_drhs = op.bind(**cache.spec_from_json(keys[1]))
  a = torch.empty(131072, 2048, dtype=torch.bfloat16, device="meta")
  d = torch.empty(131072, 768, dtype=torch.bfloat16, device="meta")
  g2 = torch.empty(128, dtype=torch.int32, device="meta")
  from tokamax_b200.ragged_dot import base as base_lib
  assert op.bind(a, d, group_sizes=g2, ragged_dot_dimension_numbers=base_lib.RAGGED_CONTRACTING_DOT_DIM_NUMS
                 ).autotuning_cache_key == ba_drhs.autotuning_cache_key


def test_xla_ffi_shim_type_checks_against_the_c_abi():
  """The JAX-facing handlers (csrc/xla_ffi_shim.cc) need jaxlib's headers to build, which do
  not exist here; a test double of `xla/ffi/api/ffi.h` (tests/ffi_stub) lets the compiler check
  every call the handlers make into include/tokamax_b200.h (argument count, order and types),
  and the attribute names are compared with the binding shown in INTEGRATION.md."""
  import re
  import subprocess
  shim = os.path.join(ROOT, "tokamax_b200", "csrc", "xla_ffi_shim.cc")
  proc = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-Werror",
                         "-I" + os.path.join(ROOT, "tests", "ffi_stub"), "-I/usr/local/cuda/include", shim],
                        capture_output=True, text=True)
  assert proc.returncode == 0, proc.stderr
  src = open(shim).read()
  attrs = set(re.findall(r'Attr<int32_t>\("(\w+)"\)', src))
  assert attrs == {"rhs_layout", "activation", "block_n", "num_stages", "collective", "grid_minor_dim",
                   "grid_tile_width"}
  doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
  for name in attrs:
    assert name in doc, f"attribute {name} of the FFI handlers is not in INTEGRATION.md's binding"
  for sym in re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\((\w+),", src):
    assert sym in doc, f"handler {sym} is not named in INTEGRATION.md"
