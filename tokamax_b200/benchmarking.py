"""Benchmark utilities: standardised functions, CUDA-event timing, `BenchmarkData`.

Mirrors the roles of tokamax/_src/benchmarking.py:76-95 (`BenchmarkData`), :328-419
(`standardize_function`, modes forward / forward_res / vjp / forward_and_vjp) and
:480-608 (`compile_benchmark`, `benchmark`).  Timing is done on the device with CUDA
events on the current stream (the reference uses CUPTI kernel times); there is nothing
to lower or compile at call time, so `compile_time_ms` / `lower_time_ms` are 0.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Sequence

import numpy as np
import torch

from tokamax_b200 import op as op_lib

BENCHMARK_MODES = ("forward", "forward_res", "vjp", "forward_and_vjp")


@dataclasses.dataclass(frozen=True)
class BenchmarkData:
  """Time (and memory) data of one benchmarked function."""

  compile_time_ms: float
  lower_time_ms: float
  evaluation_times_ms: tuple[float, ...]
  metadata: dict = dataclasses.field(default_factory=dict)
  peak_memory_mb: float | None = None

  @property
  def median_evaluation_time_ms(self) -> float:
    return float(np.median(self.evaluation_times_ms))

  def asdict(self) -> dict:
    d = dataclasses.asdict(self)
    d["median_evaluation_time_ms"] = self.median_evaluation_time_ms
    return d

  @classmethod
  def fromdict(cls, d: dict) -> "BenchmarkData":
    return cls(compile_time_ms=float(d.get("compile_time_ms", 0.0)),
               lower_time_ms=float(d.get("lower_time_ms", 0.0)),
               evaluation_times_ms=tuple(float(t) for t in d["evaluation_times_ms"]),
               metadata=dict(d.get("metadata", {})), peak_memory_mb=d.get("peak_memory_mb"))


def random_initialize(x: Any, seed: int = 0, device=None) -> Any:
  """Materialises abstract arguments with seeded values (numerics.py:179-264 upstream):
  floats ~ N(0, 1), integers in [-128, 128), GroupSizes from their representative value.
  Concrete tensors pass through."""
  from tokamax_b200.ragged_dot.base import GroupSizes  # late import: base imports op
  gen = torch.Generator(device="cpu").manual_seed(seed)
  dev = device or ("cuda" if torch.cuda.is_available() else "cpu")

  def init(v):
    if isinstance(v, op_lib.ShapeDtype):
      if v.dtype.is_floating_point:
        return torch.randn(v.shape, generator=gen, dtype=torch.float32).to(v.dtype).to(dev)
      return torch.randint(-128, 128, v.shape, generator=gen, dtype=torch.int64).to(v.dtype).to(dev)
    if isinstance(v, GroupSizes):
      rep = torch.tensor(v.representative_value, dtype=torch.int32, device=dev)
      return GroupSizes(rep, v.repr_value_or_total_size)
    if isinstance(v, dict):
      return {k: init(w) for k, w in v.items()}
    if isinstance(v, (list, tuple)):
      return type(v)(init(w) for w in v)
    return v

  return init(x)


def standardize_function(f: Callable, *args, kwargs: dict | None = None, mode: str = "forward",
                         seed: int | None = 0):
  """Returns (g, x) with g(x) running `f` in the requested mode on the array leaves `x`.

  forward: out; forward_res: (out, residuals); vjp: gradients only, for a fixed
  cotangent; forward_and_vjp: out and gradients.
  """
  if mode not in BENCHMARK_MODES:
    raise ValueError(f"unknown benchmark mode {mode!r}")
  kwargs = dict(kwargs or {})
  if seed is not None:
    args = random_initialize(tuple(args), seed)
    kwargs = random_initialize(kwargs, seed)
  names = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor) and a.dtype.is_floating_point]
  x = [args[i] for i in names]

  def rebuild(xs):
    full = list(args)
    for i, v in zip(names, xs):
      full[i] = v
    return full

  if mode == "forward":
    def g(xs):
      with torch.no_grad():
        return f(*rebuild(xs), **kwargs)
  elif mode == "forward_res":
    def g(xs):
      with torch.no_grad():
        return f(*rebuild(xs), return_residuals=True, **kwargs)
  else:
    state: dict = {}

    def g(xs):
      leaves = [v.detach().requires_grad_(True) for v in xs]
      out = f(*rebuild(leaves), **kwargs)
      if "dout" not in state:
        state["dout"] = torch.ones_like(out)
      grads = torch.autograd.grad(out, leaves, state["dout"])
      return grads if mode == "vjp" else (out, grads)
  return g, x


def _time_cuda(fn: Callable[[], Any], iterations: int, warmup: int) -> tuple[float, ...]:
  """Per-call device time in ms.  Short functions are launched several times back to back
  inside one pair of events, so that host-side launch cost hides behind device execution
  (the role CUPTI kernel timing plays in the reference)."""
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  probe_start = torch.cuda.Event(enable_timing=True)
  probe_end = torch.cuda.Event(enable_timing=True)
  probe_start.record()
  fn()
  probe_end.record()
  probe_end.synchronize()
  inner = int(min(32, max(1, 2.0 // max(probe_start.elapsed_time(probe_end), 1e-3))))
  # Functions shorter than the host needs to issue them (a few tenths of a millisecond through
  # the op layer) would be timed at the host's pace: record the burst into a CUDA graph and
  # time its replays.  A function that cannot be captured (it synchronises) is timed eagerly.
  graph = _capture(fn, inner) if inner > 1 else None
  times = []
  for _ in range(iterations):
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    if graph is not None:
      graph.replay()
    else:
      for _ in range(inner):
        fn()
    end.record()
    end.synchronize()
    times.append(start.elapsed_time(end) / inner)
  return tuple(times)


def _capture(fn: Callable[[], Any], count: int):
  """`count` calls of `fn` as one CUDA graph, or None if `fn` cannot be captured."""
  stream = torch.cuda.Stream()
  stream.wait_stream(torch.cuda.current_stream())
  graph = torch.cuda.CUDAGraph()
  try:
    with torch.cuda.stream(stream):
      fn()
      stream.synchronize()
      with torch.cuda.graph(graph, stream=stream):
        for _ in range(count):
          fn()
    torch.cuda.current_stream().wait_stream(stream)
    graph.replay()          # once untimed: the first replay uploads the graph
    torch.cuda.synchronize()
    return graph
  except Exception:  # pylint: disable=broad-except
    torch.cuda.synchronize()
    return None


def compile_benchmark(f: Callable, x: Any) -> Callable[..., BenchmarkData]:
  """Returns a runner `(x, iterations=5, warmup=2) -> BenchmarkData` (device-timed)."""
  del x

  def runner(x, *, iterations: int = 5, warmup: int = 2) -> BenchmarkData:
    if not torch.cuda.is_available():
      raise RuntimeError("benchmarking needs a CUDA device")
    torch.cuda.reset_peak_memory_stats()
    times = _time_cuda(lambda: f(x), iterations, warmup)
    peak = torch.cuda.max_memory_allocated() / 2**20
    return BenchmarkData(0.0, 0.0, times, metadata={"timer": "cuda_events"}, peak_memory_mb=peak)

  return runner


def benchmark(f: Callable, x: Any, iterations: int = 5) -> BenchmarkData:
  return compile_benchmark(f, x)(x, iterations=iterations)
