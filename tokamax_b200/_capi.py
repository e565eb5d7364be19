"""ctypes binding of the C ABI in include/tokamax_b200.h.

torch is used here for device memory and the current stream only: every function
passes raw device pointers and sizes to `libtokamax_b200.so`.  There is no fallback:
if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libtokamax_b200.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED = 2
ERR_ALIGNMENT = 3
ERR_CUDA = 4
ERR_WORKSPACE = 5
ERR_DEVICE_TIMEOUT = 6
ERR_TOO_LARGE = 7
ERR_DEVICE_STATE = 8

BF16, F16, F32, F8E4M3, S8 = 0, 1, 2, 3, 4
RHS_GKN, RHS_GNK = 0, 1
OP_FWD, OP_DLHS, OP_DRHS = 0, 1, 2

_DTYPE_CODE = {
    torch.bfloat16: BF16,
    torch.float16: F16,
    torch.float32: F32,
    torch.float8_e4m3fn: F8E4M3,
    torch.int8: S8,
}

EXPORTED_SYMBOLS = (
    "tkmx_abi_version",
    "tkmx_status_string",
    "tkmx_last_cuda_error",
    "tkmx_ragged_dot_workspace_bytes",
    "tkmx_ragged_dot_fwd",
    "tkmx_ragged_dot_dlhs",
    "tkmx_ragged_dot_drhs",
    "tkmx_group_info_aligned",
    "tkmx_device_status",
    "tkmx_ragged_dot_fwd_cyclic",
    "tkmx_moe_sort_workspace_bytes",
    "tkmx_moe_sort_pairs",
    "tkmx_moe_gather_rows",
    "tkmx_moe_combine",
    "tkmx_ragged_dot_fwd_gateup",
    "tkmx_ragged_dot_fwd_epilogue",
    "tkmx_ragged_gather",
    "tkmx_ragged_scatter",
    "tkmx_ragged_gather_reduce",
    "tkmx_moe_sort_pairs_static",
    "tkmx_moe_sort_pairs_inverse",
    "tkmx_ep_plan_bytes",
    "tkmx_ep_exchange_plan",
    "tkmx_ep_moe_fused",
    "tkmx_ep_arrive_words",
    "tkmx_ep_exchange_plan_words",
    "tkmx_ep_moe_fused_once_per_rank",
    "tkmx_cross_rank_barrier",
    "tkmx_ragged_dot_drhs_window",
    "tkmx_ragged_dot_fwd_quant_out",
)


class Config(ctypes.Structure):
  """`tkmx_config` of include/tokamax_b200.h."""

  _fields_ = [
      ("block_m", ctypes.c_int32),
      ("block_n", ctypes.c_int32),
      ("block_k", ctypes.c_int32),
      ("num_stages", ctypes.c_int32),
      ("collective", ctypes.c_int32),
      ("grid_minor_dim", ctypes.c_int32),
      ("grid_tile_width", ctypes.c_int32),
      ("max_ctas", ctypes.c_int32),
  ]


class LibraryNotBuiltError(RuntimeError):
  pass


_lib = None
_lock = threading.Lock()


def library_path() -> str:
  return _LIB_PATH


def load() -> ctypes.CDLL:
  """Loads the shared library (once).  Raises if it has not been built."""
  global _lib
  with _lock:
    if _lib is not None:
      return _lib
    if not os.path.exists(_LIB_PATH):
      raise LibraryNotBuiltError(
          f"{_LIB_PATH} not found: build it with `python -m tokamax_b200.build` "
          "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_size_t
    cfgp = ctypes.POINTER(Config)
    lib.tkmx_abi_version.restype = ctypes.c_int
    lib.tkmx_status_string.restype = ctypes.c_char_p
    lib.tkmx_status_string.argtypes = [ctypes.c_int]
    lib.tkmx_last_cuda_error.restype = ctypes.c_char_p
    lib.tkmx_ragged_dot_workspace_bytes.restype = sz
    lib.tkmx_ragged_dot_workspace_bytes.argtypes = [ctypes.c_int, i64, i64, i64, i64, ctypes.c_int, cfgp]
    lib.tkmx_ragged_dot_fwd.restype = ctypes.c_int
    lib.tkmx_ragged_dot_fwd.argtypes = [vp, vp, vp, vp, vp, vp, sz, i64, i64, i64, i64,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        cfgp, vp]
    for fn in (lib.tkmx_ragged_dot_dlhs, lib.tkmx_ragged_dot_drhs):
      fn.restype = ctypes.c_int
      fn.argtypes = [vp, vp, vp, vp, vp, sz, i64, i64, i64, i64, ctypes.c_int, ctypes.c_int, cfgp, vp]
    lib.tkmx_ragged_dot_fwd_quant_out.restype = ctypes.c_int
    lib.tkmx_ragged_dot_fwd_quant_out.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_int, ctypes.c_int, cfgp, vp]
    lib.tkmx_ragged_dot_drhs_window.restype = ctypes.c_int
    lib.tkmx_ragged_dot_drhs_window.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, ctypes.c_int,
                                                ctypes.c_int, cfgp, vp]
    lib.tkmx_group_info_aligned.restype = ctypes.c_int
    lib.tkmx_group_info_aligned.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]
    lib.tkmx_device_status.restype = ctypes.c_int
    lib.tkmx_ragged_dot_fwd_cyclic.restype = ctypes.c_int
    lib.tkmx_ragged_dot_fwd_cyclic.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               i64, i64, cfgp, vp, sz, vp]
    lib.tkmx_moe_sort_pairs_inverse.restype = ctypes.c_int
    lib.tkmx_moe_sort_pairs_inverse.argtypes = [vp, i64, i32, vp, vp, vp, vp, sz, vp]
    lib.tkmx_ep_plan_bytes.restype = sz
    lib.tkmx_ep_plan_bytes.argtypes = [i32, i32]
    lib.tkmx_ep_exchange_plan.restype = ctypes.c_int
    lib.tkmx_ep_exchange_plan.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, ctypes.c_uint32, i64, vp]
    lib.tkmx_ep_moe_fused.restype = ctypes.c_int
    lib.tkmx_ep_moe_fused.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i32, i64, i64, i32, i32, i32, i64,
                                      ctypes.c_int, ctypes.c_int, cfgp, vp]
    lib.tkmx_ep_arrive_words.restype = sz
    lib.tkmx_ep_arrive_words.argtypes = [i32, i32, i32]
    lib.tkmx_ep_exchange_plan_words.restype = ctypes.c_int
    lib.tkmx_ep_exchange_plan_words.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, ctypes.c_uint32, i64, i32, vp]
    lib.tkmx_ep_moe_fused_once_per_rank.restype = ctypes.c_int
    lib.tkmx_ep_moe_fused_once_per_rank.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i64, i64, i32, i32,
                                                    i32, i64, ctypes.c_int, ctypes.c_int, cfgp, vp]
    lib.tkmx_cross_rank_barrier.restype = ctypes.c_int
    lib.tkmx_cross_rank_barrier.argtypes = [vp, vp, i32, i32, ctypes.c_uint32, i64, vp]
    lib.tkmx_moe_sort_workspace_bytes.restype = sz
    lib.tkmx_moe_sort_workspace_bytes.argtypes = [i64, i32]
    lib.tkmx_moe_sort_pairs.restype = ctypes.c_int
    lib.tkmx_moe_sort_pairs.argtypes = [vp, i64, i32, vp, vp, vp, sz, vp]
    lib.tkmx_moe_sort_pairs_static.restype = ctypes.c_int
    lib.tkmx_moe_sort_pairs_static.argtypes = [vp, i64, i32, vp, vp, vp]
    lib.tkmx_moe_gather_rows.restype = ctypes.c_int
    lib.tkmx_moe_gather_rows.argtypes = [vp, vp, vp, i64, i32, i64, vp]
    lib.tkmx_moe_combine.restype = ctypes.c_int
    lib.tkmx_moe_combine.argtypes = [vp, vp, vp, vp, i64, i32, i64, ctypes.c_int, vp]
    lib.tkmx_ragged_dot_fwd_gateup.restype = ctypes.c_int
    lib.tkmx_ragged_dot_fwd_gateup.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_int, cfgp, vp]
    lib.tkmx_ragged_dot_fwd_epilogue.restype = ctypes.c_int
    lib.tkmx_ragged_dot_fwd_epilogue.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i64, i64, ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, cfgp, vp]
    lib.tkmx_ragged_gather.restype = ctypes.c_int
    lib.tkmx_ragged_gather.argtypes = [vp, vp, vp, i64, i64, i64, vp]
    lib.tkmx_ragged_scatter.restype = ctypes.c_int
    lib.tkmx_ragged_scatter.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.tkmx_ragged_gather_reduce.restype = ctypes.c_int
    lib.tkmx_ragged_gather_reduce.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, i64, ctypes.c_int, vp]
    _lib = lib
    return lib


def status_string(status: int) -> str:
  return load().tkmx_status_string(status).decode()


def check(status: int, what: str) -> None:
  """Maps a tkmx_status to the exception the reference raises in the same situation."""
  if status == OK:
    return
  lib = load()
  msg = f"{what}: {lib.tkmx_status_string(status).decode()}"
  detail = lib.tkmx_last_cuda_error().decode()
  if status in (ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_TOO_LARGE, ERR_DEVICE_STATE) and detail:
    msg += f" ({detail})"
  if status in (ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_TOO_LARGE):
    raise NotImplementedError(msg)
  if status == ERR_INVALID_ARGUMENT:
    raise ValueError(msg)
  raise RuntimeError(msg)


def dtype_code(dtype: torch.dtype) -> int:
  try:
    return _DTYPE_CODE[dtype]
  except KeyError:
    raise NotImplementedError(f"dtype {dtype} is not supported by the B200 ragged_dot kernels")


def _ptr(t: torch.Tensor | None):
  return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
  return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _cfg(config: Config | None):
  return None if config is None else ctypes.byref(config)


def _require_cuda(*tensors):
  dev = None
  for t in tensors:
    if t is None:
      continue
    if not t.is_cuda:
      raise ValueError("tokamax_b200 kernels take CUDA tensors (no CPU path exists)")
    if not t.is_contiguous():
      raise ValueError("tokamax_b200 kernels take contiguous row-major tensors")
    if dev is None:
      dev = t.device
    elif t.device != dev:
      raise ValueError("all operands must live on the same device")
  return dev


def workspace_bytes(op: int, m: int, k: int, n: int, g: int, rhs_dtype: torch.dtype,
                    config: Config | None = None) -> int:
  return int(load().tkmx_ragged_dot_workspace_bytes(op, m, k, n, g, dtype_code(rhs_dtype), _cfg(config)))


def ragged_dot_fwd(lhs, rhs, group_sizes, out, *, rhs_scale=None, rhs_layout=RHS_GKN,
                   config: Config | None = None, workspace=None) -> None:
  """Enqueues out = ragged_dot(lhs, rhs, group_sizes) on the current stream."""
  dev = _require_cuda(lhs, rhs, group_sizes, out, rhs_scale, workspace)
  m, k = lhs.shape
  g = rhs.shape[0]
  n = rhs.shape[2] if rhs_layout == RHS_GKN else rhs.shape[1]
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_fwd(
        _ptr(lhs), _ptr(rhs), _ptr(group_sizes), _ptr(rhs_scale), _ptr(out), _ptr(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(),
        m, k, n, g, dtype_code(lhs.dtype), dtype_code(rhs.dtype), dtype_code(out.dtype), rhs_layout,
        _cfg(config), _stream(dev))
  check(st, "tkmx_ragged_dot_fwd")


GATEUP_ACTIVATIONS = {"silu": 1, "gelu": 2, "gelu_tanh": 2, "swigluoai": 3, "silu_and_mul_with_clamp": 4}
# Elementwise activations the epilogue applies to the float32 result (TKMX_ACT_* of the header).
ELEMENT_ACTIVATIONS = {"relu": 16, "silu": 17, "swish": 17, "gelu_tanh": 18, "gelu": 19, "gelu_erf": 19,
                       "tanh": 20, "sigmoid": 21}


def ragged_dot_fwd_gateup(lhs, rhs, group_sizes, out, activation: str, *, config: Config | None = None) -> None:
  """out[m, n/2] = act(tmp[:, :n/2]) * tmp[:, n/2:] with tmp = ragged_dot(lhs, rhs), fused."""
  dev = _require_cuda(lhs, rhs, group_sizes, out)
  if activation not in GATEUP_ACTIVATIONS:
    raise NotImplementedError(f"Unsupported activation function: {activation}")
  m, k = lhs.shape
  g, _, n = rhs.shape
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_fwd_gateup(
        _ptr(lhs), _ptr(rhs), _ptr(group_sizes), _ptr(out), m, k, n, g, dtype_code(lhs.dtype),
        dtype_code(out.dtype), GATEUP_ACTIVATIONS[activation], _cfg(config), _stream(dev))
  check(st, "tkmx_ragged_dot_fwd_gateup")


def ragged_dot_fwd_epilogue(lhs, rhs, group_sizes, out, *, rhs_scale=None, rhs_bias=None,
                            activation: str | None = None, element_activation: str | None = None,
                            rhs_layout=RHS_GKN, config: Config | None = None, workspace=None) -> None:
  """out = ragged_dot(lhs, rhs) [* rhs_scale] + rhs_bias[group], optionally followed by the
  fused gate/up activation `activation` (out then has n/2 columns) or by the elementwise
  `element_activation` (a key of ELEMENT_ACTIVATIONS), both computed in float32.  rhs_scale /
  rhs_bias: float32 [g, n] or None; 8-bit rhs needs the workspace of `workspace_bytes`."""
  dev = _require_cuda(lhs, rhs, group_sizes, out, rhs_scale, rhs_bias, workspace)
  if activation is not None and activation not in GATEUP_ACTIVATIONS:
    raise NotImplementedError(f"Unsupported activation function: {activation}")
  if element_activation is not None:
    if activation is not None:
      raise NotImplementedError("a gate/up activation and an elementwise one cannot both be fused")
    if element_activation not in ELEMENT_ACTIVATIONS:
      raise NotImplementedError(f"Unsupported activation function: {element_activation}")
  for t, what in ((rhs_bias, "rhs_bias"), (rhs_scale, "rhs_scale")):
    if t is not None and t.dtype != torch.float32:
      raise ValueError(f"{what} must be float32")
  m, k = lhs.shape
  g = rhs.shape[0]
  n = rhs.shape[2] if rhs_layout == RHS_GKN else rhs.shape[1]
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_fwd_epilogue(
        _ptr(lhs), _ptr(rhs), _ptr(group_sizes), _ptr(rhs_scale), _ptr(rhs_bias), _ptr(out), _ptr(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(), m, k, n, g,
        dtype_code(lhs.dtype), dtype_code(rhs.dtype), dtype_code(out.dtype), rhs_layout,
        ELEMENT_ACTIVATIONS[element_activation] if element_activation is not None
        else (0 if activation is None else GATEUP_ACTIVATIONS[activation]), _cfg(config), _stream(dev))
  check(st, "tkmx_ragged_dot_fwd_epilogue")


def ragged_dot_fwd_quant_out(lhs, rhs, group_sizes, out_q, out_scale, subchannel: int, *, rhs_bias=None,
                             element_activation: str | None = None, rhs_layout=RHS_GKN,
                             config: Config | None = None) -> None:
  """Forward whose epilogue quantises the result: out_q float8_e4m3fn [m, n], out_scale float32
  [m, n / subchannel] (scale = max|x| / 448 per row and block of `subchannel` columns)."""
  dev = _require_cuda(lhs, rhs, group_sizes, out_q, out_scale, rhs_bias)
  if out_q.dtype != torch.float8_e4m3fn or out_scale.dtype != torch.float32:
    raise ValueError("out_q must be float8_e4m3fn and out_scale float32")
  if element_activation is not None and element_activation not in ELEMENT_ACTIVATIONS:
    raise NotImplementedError(f"Unsupported activation function: {element_activation}")
  m, k = lhs.shape
  g = rhs.shape[0]
  n = rhs.shape[2] if rhs_layout == RHS_GKN else rhs.shape[1]
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_fwd_quant_out(
        _ptr(lhs), _ptr(rhs), _ptr(group_sizes), _ptr(rhs_bias), _ptr(out_q), _ptr(out_scale), m, k, n, g,
        dtype_code(lhs.dtype), rhs_layout,
        0 if element_activation is None else ELEMENT_ACTIVATIONS[element_activation], subchannel,
        _cfg(config), _stream(dev))
  check(st, "tkmx_ragged_dot_fwd_quant_out")


def ragged_dot_fwd_cyclic(lhs, rhs, group_sizes, out, *, rhs_scale=None, rhs_layout=RHS_GKN,
                          zero_initialize: bool = True, segment_begin: int = 0, segment_count: int = -1,
                          config: Config | None = None, workspace=None) -> None:
  """Forward where segment i of group_sizes (any multiple of the expert count) uses rhs[i % G].
  zero_initialize=False leaves the rows past sum(group_sizes) untouched; only segments
  [segment_begin, segment_begin + segment_count) are computed (offsets count all of them)."""
  dev = _require_cuda(lhs, rhs, group_sizes, out, rhs_scale, workspace)
  m, k = lhs.shape
  g_rhs = rhs.shape[0]
  n = rhs.shape[2] if rhs_layout == RHS_GKN else rhs.shape[1]
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_fwd_cyclic(
        _ptr(lhs), _ptr(rhs), _ptr(group_sizes), _ptr(rhs_scale), _ptr(out), m, k, n,
        group_sizes.numel(), g_rhs, dtype_code(lhs.dtype), dtype_code(rhs.dtype), dtype_code(out.dtype),
        rhs_layout, 1 if zero_initialize else 0, segment_begin, segment_count, _cfg(config),
        _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(), _stream(dev))
  check(st, "tkmx_ragged_dot_fwd_cyclic")


def moe_sort_pairs_inverse(expert_ids: torch.Tensor, num_experts: int, pos, sorted_pair, counts, workspace):
  """`moe_sort_pairs` into caller-owned outputs, plus sorted_pair[pos[p]] = p (int32 [num_pairs])."""
  dev = _require_cuda(expert_ids, pos, sorted_pair, counts, workspace)
  if expert_ids.dtype != torch.int32:
    raise ValueError("expert_ids must be int32")
  with torch.cuda.device(dev):
    st = load().tkmx_moe_sort_pairs_inverse(
        _ptr(expert_ids), expert_ids.numel(), num_experts, _ptr(pos), _ptr(sorted_pair), _ptr(counts),
        _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(dev))
  check(st, "tkmx_moe_sort_pairs_inverse")


def moe_sort_workspace_bytes(num_pairs: int, num_experts: int) -> int:
  return int(load().tkmx_moe_sort_workspace_bytes(num_pairs, num_experts))


EP_MAX_WORLD = 16
EP_TAB_RECV, EP_TAB_ARRIVE, EP_TAB_RET, EP_TAB_COUNTS, EP_TAB_FLAGS, EP_TAB_REFS = range(6)
EP_TAB_ROWS = 6


def ep_arrive_words(num_experts: int, world: int, once_per_rank: bool = False) -> int:
  """uint32 words of a rank's arrival array (see include/tokamax_b200.h)."""
  return int(load().tkmx_ep_arrive_words(num_experts, world, 1 if once_per_rank else 0))


def ep_plan_ints(num_experts: int, world: int) -> int:
  return int(load().tkmx_ep_plan_bytes(num_experts, world)) // 4


def ep_exchange_plan(my_counts, peer_table, counts_all, flags, arrive, plan, num_experts: int, world: int,
                     rank: int, sequence: int, timeout_ns: int, once_per_rank: bool = False) -> None:
  """Counts all-gather through peer memory + flag barrier + the step's offset tables."""
  dev = _require_cuda(my_counts, peer_table, counts_all, flags, arrive, plan)
  if arrive.numel() < ep_arrive_words(num_experts, world, once_per_rank):
    raise ValueError("arrive is shorter than tkmx_ep_arrive_words says")
  if once_per_rank:
    with torch.cuda.device(dev):
      st = load().tkmx_ep_exchange_plan_words(_ptr(my_counts), _ptr(peer_table), _ptr(counts_all), _ptr(flags),
                                              _ptr(arrive), _ptr(plan), num_experts, world, rank,
                                              sequence & 0xFFFFFFFF, timeout_ns, 1, _stream(dev))
    check(st, "tkmx_ep_exchange_plan_words")
    return
  with torch.cuda.device(dev):
    st = load().tkmx_ep_exchange_plan(_ptr(my_counts), _ptr(peer_table), _ptr(counts_all), _ptr(flags),
                                      _ptr(arrive), _ptr(plan), num_experts, world, rank,
                                      sequence & 0xFFFFFFFF, timeout_ns, _stream(dev))
  check(st, "tkmx_ep_exchange_plan")


def ep_moe_fused(tokens, sorted_pair, recv, rhs_local, plan, peer_table, arrive, top_k: int, num_experts: int,
                 world: int, rank: int, n: int, phases: int = 3, config: Config | None = None,
                 expert_ids=None, pair_pos=None) -> None:
  """The fused dispatch + grouped GEMM + return kernel (see include/tokamax_b200.h).  With
  `expert_ids` and `pair_pos` a token crosses the link once per destination rank."""
  dev = _require_cuda(tokens, sorted_pair, recv, rhs_local, plan, peer_table, arrive, expert_ids, pair_pos)
  if expert_ids is not None or pair_pos is not None:
    if expert_ids is None or pair_pos is None or expert_ids.dtype != torch.int32 or pair_pos.dtype != torch.int32:
      raise ValueError("expert_ids and pair_pos must both be int32 tensors")
    if peer_table.shape[0] < EP_TAB_ROWS or arrive.numel() < ep_arrive_words(num_experts, world, True):
      raise ValueError("the once-per-rank form needs the six-row peer table and the longer arrival array")
    with torch.cuda.device(dev):
      st = load().tkmx_ep_moe_fused_once_per_rank(
          _ptr(tokens), _ptr(sorted_pair), _ptr(expert_ids), _ptr(pair_pos), _ptr(recv), _ptr(rhs_local),
          _ptr(plan), _ptr(peer_table), _ptr(arrive), tokens.shape[0], top_k, tokens.shape[1], n, num_experts,
          world, rank, recv.shape[0], dtype_code(tokens.dtype), phases, _cfg(config), _stream(dev))
    check(st, "tkmx_ep_moe_fused_once_per_rank")
    return
  with torch.cuda.device(dev):
    st = load().tkmx_ep_moe_fused(_ptr(tokens), _ptr(sorted_pair), _ptr(recv), _ptr(rhs_local), _ptr(plan),
                                  _ptr(peer_table), _ptr(arrive), tokens.shape[0], top_k, tokens.shape[1], n,
                                  num_experts, world, rank, recv.shape[0], dtype_code(tokens.dtype), phases,
                                  _cfg(config), _stream(dev))
  check(st, "tkmx_ep_moe_fused")


def cross_rank_barrier(peer_table, flags, world: int, rank: int, sequence: int, timeout_ns: int) -> None:
  dev = _require_cuda(peer_table, flags)
  with torch.cuda.device(dev):
    st = load().tkmx_cross_rank_barrier(_ptr(peer_table), _ptr(flags), world, rank, sequence & 0xFFFFFFFF,
                                        timeout_ns, _stream(dev))
  check(st, "tkmx_cross_rank_barrier")


def moe_sort_pairs(expert_ids: torch.Tensor, num_experts: int, workspace: torch.Tensor | None = None):
  """Returns (pos int32 [num_pairs], counts int32 [num_experts]) for int32 expert ids of any shape."""
  dev = _require_cuda(expert_ids, workspace)
  if expert_ids.dtype != torch.int32:
    raise ValueError("expert_ids must be int32")
  num_pairs = expert_ids.numel()
  lib = load()
  need = int(lib.tkmx_moe_sort_workspace_bytes(num_pairs, num_experts))
  if workspace is None:
    workspace = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
  pos = torch.empty(num_pairs, dtype=torch.int32, device=dev)
  counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
  with torch.cuda.device(dev):
    st = lib.tkmx_moe_sort_pairs(_ptr(expert_ids), num_pairs, num_experts, _ptr(pos), _ptr(counts),
                                 _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(dev))
  check(st, "tkmx_moe_sort_pairs")
  return pos, counts


def moe_sort_pairs_static(expert_ids: torch.Tensor, num_experts: int, pos: torch.Tensor,
                          counts: torch.Tensor) -> None:
  """`moe_sort_pairs` through the entry point that takes no workspace and allocates nothing:
  for hosts that cannot (or may not) obtain device memory at call time.  `pos` (int32
  [num_pairs]) and `counts` (int32 [num_experts]) are written in place; sizes beyond the
  library's built-in scratch raise NotImplementedError."""
  dev = _require_cuda(expert_ids, pos, counts)
  if expert_ids.dtype != torch.int32 or pos.dtype != torch.int32 or counts.dtype != torch.int32:
    raise ValueError("expert_ids, pos and counts must be int32")
  with torch.cuda.device(dev):
    st = load().tkmx_moe_sort_pairs_static(_ptr(expert_ids), expert_ids.numel(), num_experts, _ptr(pos),
                                           _ptr(counts), _stream(dev))
  check(st, "tkmx_moe_sort_pairs_static")


def moe_gather_rows(src: torch.Tensor, pos: torch.Tensor, top_k: int, out: torch.Tensor | None = None):
  """out[pos[p]] = src[p // top_k]; `out` defaults to a new [num_pairs, row] tensor."""
  dev = _require_cuda(src, pos, out)
  num_pairs = pos.numel()
  if out is None:
    out = torch.empty((num_pairs, src.shape[1]), dtype=src.dtype, device=dev)
  with torch.cuda.device(dev):
    st = load().tkmx_moe_gather_rows(_ptr(src), _ptr(pos), _ptr(out), num_pairs, top_k,
                                     src.shape[1] * src.element_size(), _stream(dev))
  check(st, "tkmx_moe_gather_rows")
  return out


def moe_combine(rows: torch.Tensor, pos: torch.Tensor, gates: torch.Tensor, num_tokens: int, top_k: int):
  """y[t] = sum_k gates[t, k] * rows[pos[t * top_k + k]] (float32 accumulation, bf16 rows)."""
  dev = _require_cuda(rows, pos, gates)
  if gates.dtype != torch.float32:
    raise ValueError("gates must be float32")
  y = torch.empty((num_tokens, rows.shape[1]), dtype=rows.dtype, device=dev)
  with torch.cuda.device(dev):
    st = load().tkmx_moe_combine(_ptr(rows), _ptr(pos), _ptr(gates), _ptr(y), num_tokens, top_k,
                                 rows.shape[1], dtype_code(rows.dtype), _stream(dev))
  check(st, "tkmx_moe_combine")
  return y


def ragged_gather(x: torch.Tensor, indices: torch.Tensor, start=None, end=None) -> torch.Tensor:
  """out[i] = x[indices[i]]; with start / end (device int32 scalars) rows whose index is
  outside [start, end) are zeros (ragged_scatter)."""
  dev = _require_cuda(x, indices, start, end)
  if indices.dtype != torch.int32 or (start is not None and (start.dtype != torch.int32 or end.dtype != torch.int32)):
    raise ValueError("indices, start and end must be int32")
  out = torch.empty((indices.numel(), x.shape[1]), dtype=x.dtype, device=dev)
  row_bytes = x.shape[1] * x.element_size()
  with torch.cuda.device(dev):
    if start is None:
      st = load().tkmx_ragged_gather(_ptr(x), _ptr(indices), _ptr(out), x.shape[0], indices.numel(), row_bytes,
                                     _stream(dev))
    else:
      st = load().tkmx_ragged_scatter(_ptr(x), _ptr(indices), _ptr(start), _ptr(end), _ptr(out), x.shape[0],
                                      indices.numel(), row_bytes, _stream(dev))
  check(st, "tkmx_ragged_gather" if start is None else "tkmx_ragged_scatter")
  return out


def ragged_gather_reduce(x, indices, weights, mask, reduce_group_size: int) -> torch.Tensor:
  """out[t] = sum_j mask[p] * weights[p] * x[indices[p]], p = t * reduce_group_size + j."""
  dev = _require_cuda(x, indices, weights, mask)
  if indices.dtype != torch.int32 or weights.dtype != torch.float32:
    raise ValueError("indices must be int32 and weights float32")
  if mask is not None and mask.dtype not in (torch.bool, torch.uint8):
    raise ValueError("mask must be bool or uint8")
  input_size = indices.numel()
  out = torch.empty((input_size // max(reduce_group_size, 1), x.shape[1]), dtype=x.dtype, device=dev)
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_gather_reduce(_ptr(x), _ptr(indices), _ptr(weights), _ptr(mask), _ptr(out),
                                          x.shape[0], input_size, reduce_group_size, x.shape[1],
                                          dtype_code(x.dtype), _stream(dev))
  check(st, "tkmx_ragged_gather_reduce")
  return out


def ragged_dot_dlhs(dout, rhs, group_sizes, dlhs, *, config: Config | None = None,
                    workspace=None) -> None:
  dev = _require_cuda(dout, rhs, group_sizes, dlhs, workspace)
  m, n = dout.shape
  g, k, _ = rhs.shape
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_dlhs(
        _ptr(dout), _ptr(rhs), _ptr(group_sizes), _ptr(dlhs), _ptr(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(),
        m, k, n, g, dtype_code(dout.dtype), dtype_code(dlhs.dtype), _cfg(config), _stream(dev))
  check(st, "tkmx_ragged_dot_dlhs")


def ragged_dot_drhs(lhs, dout, group_sizes, drhs, *, config: Config | None = None,
                    workspace=None, group_begin: int | None = None) -> None:
  """drhs[j] = lhs[rows of group j]^T @ dout[rows of group j].  With `group_begin` the output
  holds only the groups [group_begin, group_begin + drhs.shape[0]) of the group_sizes array."""
  dev = _require_cuda(lhs, dout, group_sizes, drhs, workspace)
  m, k = lhs.shape
  n = dout.shape[1]
  g = drhs.shape[0]
  if group_begin is not None:
    with torch.cuda.device(dev):
      st = load().tkmx_ragged_dot_drhs_window(
          _ptr(lhs), _ptr(dout), _ptr(group_sizes), _ptr(drhs), m, k, n, group_sizes.numel(), group_begin, g,
          dtype_code(lhs.dtype), dtype_code(drhs.dtype), _cfg(config), _stream(dev))
    check(st, "tkmx_ragged_dot_drhs_window")
    return
  with torch.cuda.device(dev):
    st = load().tkmx_ragged_dot_drhs(
        _ptr(lhs), _ptr(dout), _ptr(group_sizes), _ptr(drhs), _ptr(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(),
        m, k, n, g, dtype_code(lhs.dtype), dtype_code(drhs.dtype), _cfg(config), _stream(dev))
  check(st, "tkmx_ragged_dot_drhs")


def group_info_aligned(group_sizes: torch.Tensor, tile: int, num_tasks: int, align_tile: int = 8):
  """Device version of the reference's GroupInfo.create_aligned; returns six int32 tensors."""
  dev = _require_cuda(group_sizes)
  outs = [torch.empty(num_tasks, dtype=torch.int32, device=dev) for _ in range(6)]
  with torch.cuda.device(dev):
    st = load().tkmx_group_info_aligned(_ptr(group_sizes), group_sizes.numel(), tile, num_tasks,
                                        align_tile, *[_ptr(o) for o in outs], _stream(dev))
  check(st, "tkmx_group_info_aligned")
  names = ("group_id", "block_start", "actual_start", "actual_end", "start_within_block", "actual_size")
  return dict(zip(names, outs))


def device_status() -> None:
  """Synchronises and raises if a kernel recorded a timed-out wait."""
  check(load().tkmx_device_status(), "tkmx_device_status")
