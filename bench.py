"""Benchmark of the ragged_dot hot path on B200.

  python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Metric: ragged_dot TFLOP/s, 2 * sum(group_sizes) * K * N
per product (the reference's convention, tokamax/_src/ops/ragged_dot/bench.py:52-56).

Default workload at every N: "ep", the expert-parallel MoE layer -- 256 experts sharded over
the N ranks, per rank 8192 tokens x 7168 (bf16), top-8 routing, local rhs [256/N, 7168, 2048]:
route (counting sort) -> dispatch of the token rows to the experts' owners -> grouped GEMM ->
return of the output rows -> gate-weighted combine.  A step is one call of the layer; per-GPU
work is fixed as N grows (weak scaling), so the values of N = 1, 2, 4, 8 are the same code
path on the same per-rank inputs.  Inputs (tokens 117 MB + weights 7.5 GB / N per rank)
exceed the 126 MB L2, so every step streams its operands from HBM; no extra L2 flush is done.

After the timed region every rank checks the layer's output on sampled tokens against a
dense top-k MoE recomputed on the host by the CPU oracle, and the group sizes the layer
derived against the global histogram of all ranks' routing: `parity` in the line; a
mismatch exits non-zero.

At N = 1 the line also carries `kernels`: the grouped-GEMM kernels alone on the other named
workloads (cfg2 Mixtral-shaped forward, cfg3 DeepSeek-V3-shaped fp8 / int8 forward, cfg4
Qwen3-shaped forward / dlhs / drhs, dsv3 forward / dlhs / drhs and their aggregate), each
with its time, TFLOP/s, GB/s and the fraction of max(t_flops, t_bytes) at the measured peaks.

`value` is timed with inputs resident in HBM (CUDA events on the launching stream, max over
ranks).  `e2e` is the same step through the public API with pinned HOST buffers
(`HostPipeline.submit`): every step's tokens, routing and gates are copied host->device and
its result device->host inside the timed region, the copies of one step running beside the
computation of its neighbours; the region ends when the last result is in host memory.  `cpu_baseline` (rank 0, N = 1) times the CPU restatement of the reference path on
the host cores.  --impl reference times that CPU restatement alone (the reference is pure
Python over jax/jaxlib, which is not installable here: no oracle/_ref exists).

--workload cfg1|cfg2|cfg3|cfg4|dsv3 --op fwd|dlhs|drhs times one kernel alone (profiler runs).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "ragged_dot TFLOP/s (2*M*K*N)"
UNIT = "TFLOP/s"

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures,
# by kernel-suite entry name; None where no capture exists.
NCU_TRAFFIC_BYTES = {"cfg2.fwd": 2.643e9}
# The fused expert-parallel kernel on one rank: 2.74 GB captured on a quarter-size case (2048
# tokens, 64 experts); rows and weights both scale by 4 to the full workload, traffic with them.
NCU_TRAFFIC_EP_QUARTER = 2.74e9


# ----------------------------------------------------------------------------- utilities
def load_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  try:
    with open(path) as f:
      p = json.load(f)
    return dict(bf16=float(p["bf16_tflops"]), bf16_sustained=float(p["bf16_tflops_sustained"]),
                hbm=float(p["hbm_gbs"]), source="measured (MEASURED_PEAKS.json)")
  except Exception:
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback (earlier measurement on this pool)")


class ClockSampler:
  """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

  FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
            "clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_id: str | None):
    self.gpu_id = gpu_id          # None: sample nothing (ranks whose line is not printed)
    self.proc = None
    self.lines: list[str] = []
    self.first = 0

  def wait_ready(self, timeout_s: float = 8.0):
    """Blocks until the tool has printed its first sample (its start-up takes a second or more
    on a box with many GPUs), then drops what it saw so far: those samples are of an idle GPU."""
    t_end = time.time() + timeout_s
    while self.proc is not None and not self.lines and time.time() < t_end:
      time.sleep(0.02)
    self.first = len(self.lines)

  def __enter__(self):
    if self.gpu_id is None:
      return self
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
           "-i", self.gpu_id], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except Exception:
      self.proc = None
    return self

  def _read(self):
    for line in self.proc.stdout:
      self.lines.append(line.strip())

  def __exit__(self, *exc):
    if self.proc is not None:
      self.proc.terminate()  # this exact child only
      try:
        self.proc.wait(timeout=5)
      except Exception:
        self.proc.kill()
    return False

  def summary(self) -> dict:
    sm, mx = [], []
    reasons = set()
    names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    for line in self.lines[self.first:]:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 6:
        continue
      try:
        sm.append(float(parts[0]))
        mx.append(float(parts[1]))
      except ValueError:
        continue
      for name, val in zip(names, parts[2:6]):
        if val.lower().startswith("active"):
          reasons.add(name)
    if not sm:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
            "samples": len(sm)}


def gpu_id_for_smi(local_index: int) -> str:
  """What `nvidia-smi -i` should be given for torch's device `local_index`: its UUID (stable
  under CUDA_VISIBLE_DEVICES in any form), else the physical index."""
  try:
    uuid = str(torch.cuda.get_device_properties(local_index).uuid)
    if uuid and not uuid.startswith("GPU-"):
      uuid = "GPU-" + uuid
    if uuid:
      return uuid
  except Exception:
    pass
  vis = os.environ.get("CUDA_VISIBLE_DEVICES")
  if vis:
    try:
      return str(int(vis.split(",")[local_index]))
    except Exception:
      pass
  return str(local_index)


def make_cfg_inputs(w, device, seed=0):
  """lhs ~ N(0,1), rhs ~ N(0,1)/sqrt(K), bf16, generated on the device from a seed."""
  gen = torch.Generator(device=device).manual_seed(seed)
  lhs = torch.randn(w.m, w.k, device=device, generator=gen, dtype=torch.float32).to(torch.bfloat16)
  rhs = torch.empty(w.g, w.k, w.n, device=device, dtype=torch.bfloat16)
  for g in range(w.g):  # per expert, to bound the float32 temporary
    rhs[g] = (torch.randn(w.k, w.n, device=device, generator=gen, dtype=torch.float32) * w.k ** -0.5).to(torch.bfloat16)
  gs = torch.tensor(w.group_sizes, dtype=torch.int32, device=device)
  return lhs, rhs, gs


def time_region(step, stream, launches: int, sampler_id: str | None, min_region_ms: float = 0.0):
  """Runs `step` `launches` times between two CUDA events on `stream`; returns (ms per launch,
  launches timed, clock summary).  With `min_region_ms` the count is raised so that the region
  lasts at least that long (the 100 ms clock sampler has to see it)."""
  for _ in range(3):
    step()
  torch.cuda.synchronize()
  if min_region_ms > 0:
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(stream)
    for _ in range(3):
      step()
    e.record(stream)
    torch.cuda.synchronize()
    est = max(s.elapsed_time(e) / 3, 1e-3)
    launches = max(launches, int(np.ceil(min_region_ms / est)))
  ctx = ClockSampler(sampler_id) if sampler_id is not None else None
  if ctx is not None:
    ctx.__enter__()
  try:
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record(stream)
    for _ in range(launches):
      step()
    e.record(stream)
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / launches
  finally:
    if ctx is not None:
      ctx.__exit__(None, None, None)
  return ms, launches, (ctx.summary() if ctx is not None else None)


# ----------------------------------------------------------------------------- one kernel alone
def build_kernel_step(w, op_name: str, dev, fp8_path: str = "native"):
  """Inputs and a launch closure for one contraction of workload `w` through the C ABI.
  Returns (step, algorithmic bytes per launch, config repr, tensors to keep alive)."""
  from tokamax_b200 import _capi
  from tokamax_b200.quantization import QArray, quantize_per_channel
  from tokamax_b200.ragged_dot import b200 as b200_lib
  from tokamax_b200.ragged_dot import base as base_lib

  lhs, rhs, gs = make_cfg_inputs(w, dev)
  op = b200_lib.B200RaggedDot()
  quant = w.rhs_dtype in (torch.float8_e4m3fn, torch.int8)
  scale = None
  if quant:
    if op_name != "fwd":
      raise SystemExit("8-bit weights are a forward-only workload")
    q = torch.empty(w.g, w.k, w.n, device=dev, dtype=w.rhs_dtype)
    scale = torch.empty(w.g, w.n, device=dev, dtype=torch.float32)
    for g in range(w.g):  # per expert, to bound temporaries
      qa = quantize_per_channel(rhs[g:g + 1], w.rhs_dtype)
      q[g] = qa.qvalue[0]
      scale[g] = qa.channel_scale()[0]
    rhs = q
  if op_name == "fwd":
    out = torch.empty(w.m, w.n, device=dev, dtype=torch.bfloat16)
    bound = op.bind(lhs, QArray(rhs, scale) if quant else rhs, group_sizes=gs)
    ccfg = bound.default_config.to_capi()
    workspace = None
    if quant and fp8_path == "native":
      need = _capi.workspace_bytes(0, w.m, w.k, w.n, w.g, rhs.dtype)
      workspace = torch.empty(need, dtype=torch.uint8, device=dev) if need else None
    step = lambda: _capi.ragged_dot_fwd(lhs, rhs, gs, out, rhs_scale=scale, config=ccfg, workspace=workspace)
    nz = sum(1 for v in w.group_sizes if v > 0)
    alg_bytes = (w.m * w.k * 2 + nz * w.k * w.n * rhs.element_size() + w.m * w.n * 2
                 + (nz * w.n * 4 if quant else 0))
    keep = (lhs, rhs, gs, out, scale, workspace)
  elif op_name == "dlhs":
    gen = torch.Generator(device=dev).manual_seed(7)
    dout = torch.randn(w.m, w.n, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    out = torch.empty(w.m, w.k, device=dev, dtype=torch.bfloat16)
    bound = op.bind(dout, rhs, group_sizes=gs, ragged_dot_dimension_numbers=base_lib.TRANS_RHS_RAGGED_DOT_DIM_NUMS)
    ccfg = bound.default_config.to_capi()
    step = lambda: _capi.ragged_dot_dlhs(dout, rhs, gs, out, config=ccfg)
    alg_bytes = 2 * (w.m * w.n + w.g * w.k * w.n + w.m * w.k)
    keep = (dout, rhs, gs, out)
    del lhs
  else:
    gen = torch.Generator(device=dev).manual_seed(7)
    dout = torch.randn(w.m, w.n, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    del rhs
    out = torch.empty(w.g, w.k, w.n, device=dev, dtype=torch.bfloat16)
    bound = op.bind(lhs, dout, group_sizes=gs,
                    ragged_dot_dimension_numbers=base_lib.RAGGED_CONTRACTING_DOT_DIM_NUMS)
    ccfg = bound.default_config.to_capi()
    step = lambda: _capi.ragged_dot_drhs(lhs, dout, gs, out, config=ccfg)
    alg_bytes = 2 * (w.m * w.k + w.m * w.n + w.g * w.k * w.n)
    keep = (lhs, dout, gs, out)
  return step, float(alg_bytes), repr(bound.default_config), keep


def roofline_entry(flops: float, alg_bytes: float, ms: float, peaks, peak_tflops: float):
  """t_roof = max(t_flops, t_bytes) at the measured peaks; frac = t_roof / t_measured."""
  t_flops = flops / (peak_tflops * 1e12)
  t_bytes = alg_bytes / (peaks["hbm"] * 1e9)
  t_roof = max(t_flops, t_bytes)
  t = ms * 1e-3
  return {"bound": "tensor" if t_flops >= t_bytes else "hbm", "tflops": flops / t / 1e12,
          "gbs": alg_bytes / t / 1e9, "frac_tensor": t_flops / t, "frac_hbm": t_bytes / t,
          "t_roof_ms": t_roof * 1e3, "frac": t_roof / t}


def run_kernel_entry(name: str, workload_name: str, op_name: str, dev, peaks, sampler_id, rhs_dtype=None):
  from tokamax_b200 import _capi
  from tokamax_b200.ragged_dot import arg_specs
  w = arg_specs.workload(workload_name)
  if rhs_dtype is not None:
    w = dataclasses.replace(w, rhs_dtype=rhs_dtype)
  entry = {"name": name, "workload": workload_name, "op": op_name, "m": w.m, "k": w.k, "n": w.n, "g": w.g,
           "rhs_dtype": str(w.rhs_dtype).replace("torch.", "")}
  try:
    step, alg_bytes, cfg_repr, keep = build_kernel_step(w, op_name, dev)
    # >= 50 launches and >= 0.45 s back to back: the 100 ms clock sampler sees the region, and
    # the part runs at its sustained (power-capped) clocks, so the sustained cuBLAS figure is
    # the tensor peak to divide by; the fraction of the burst figure is given beside it.
    ms, launches, clocks = time_region(step, torch.cuda.current_stream(), 50, sampler_id, min_region_ms=450.0)
    _capi.device_status()
    rl = roofline_entry(w.flops, alg_bytes, ms, peaks, peaks["bf16_sustained"])
    rl["tensor_peak"] = "bf16 sustained"
    rl["frac_vs_burst_peak"] = roofline_entry(w.flops, alg_bytes, ms, peaks, peaks["bf16"])["frac"]
    entry.update({"ms": ms, "launches": launches, "flops": w.flops, "algorithmic_bytes": alg_bytes,
                  "tflops": rl["tflops"], "gbs": rl["gbs"], "roofline": rl, "clocks": clocks,
                  "traffic": NCU_TRAFFIC_BYTES.get(name), "kernel_config": cfg_repr})
    del step, keep
  except Exception as e:  # keep the line: one failed entry must not hide the others
    entry["error"] = f"{type(e).__name__}: {e}"
  torch.cuda.empty_cache()
  return entry


def run_kernel_suite(dev, peaks, sampler_id):
  """The grouped-GEMM kernels alone on the named workloads (N = 1 only)."""
  entries = []
  plan = [("cfg2.fwd", "cfg2", "fwd", None),
          ("cfg3.fwd.fp8", "cfg3", "fwd", torch.float8_e4m3fn),
          ("cfg3.fwd.int8", "cfg3", "fwd", torch.int8),
          ("cfg4.fwd", "cfg4", "fwd", None), ("cfg4.dlhs", "cfg4", "dlhs", None), ("cfg4.drhs", "cfg4", "drhs", None),
          ("dsv3.fwd", "dsv3", "fwd", None), ("dsv3.dlhs", "dsv3", "dlhs", None), ("dsv3.drhs", "dsv3", "drhs", None)]
  for name, wl, op_name, dt in plan:
    entries.append(run_kernel_entry(name, wl, op_name, dev, peaks, sampler_id, dt))
  by = {e["name"]: e for e in entries}
  for wl in ("cfg4", "dsv3"):
    parts = [by.get(f"{wl}.{o}") for o in ("fwd", "dlhs", "drhs")]
    if all(p is not None and "ms" in p for p in parts):
      ms = sum(p["ms"] for p in parts)
      flops = sum(p["flops"] for p in parts)
      byts = sum(p["algorithmic_bytes"] for p in parts)
      rl = roofline_entry(flops, byts, ms, peaks, peaks["bf16_sustained"])
      # the sum of the three roofs, not the roof of the sums: each kernel has its own bound
      t_roof = sum(p["roofline"]["t_roof_ms"] for p in parts)
      rl.update({"t_roof_ms": t_roof, "frac": t_roof / ms})
      entries.append({"name": f"{wl}.fwd+bwd", "workload": wl, "op": "fwd+dlhs+drhs (6*M*K*N)", "ms": ms,
                      "flops": flops, "algorithmic_bytes": byts, "tflops": rl["tflops"], "gbs": rl["gbs"],
                      "roofline": rl})
  return entries


def run_single(args, w, peaks):
  """One kernel alone on one workload (profiler runs and tuning)."""
  from tokamax_b200 import _capi
  dev = torch.device("cuda", 0)
  torch.cuda.set_device(dev)
  _capi.load()
  step, alg_bytes, cfg_repr, keep = build_kernel_step(w, args.op, dev, args.fp8_path)
  for _ in range(max(args.warmup, 3)):
    step()
  ms, launches, clocks = time_region(step, torch.cuda.current_stream(), args.steps, gpu_id_for_smi(0),
                                     min_region_ms=0.0 if args.kernel_only else 450.0)
  _capi.device_status()
  rl = roofline_entry(w.flops, alg_bytes, ms, peaks, peaks["bf16"])
  return {"metric": METRIC, "value": rl["tflops"], "unit": UNIT, "n_gpus": 1, "steps": launches,
          "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
          "data": "synthetic",
          "config": {"workload": w.name, "op": args.op, "kernel_config": cfg_repr, "m": w.m, "k": w.k, "n": w.n,
                     "g": w.g},
          "kernel_only": True, "gpu_launches": launches, "clocks": clocks, "roofline": rl}


# ----------------------------------------------------------------------------- expert parallel
EP_TOKENS, EP_K, EP_N, EP_G, EP_TOPK = 8192, 7168, 2048, 256, 8


def ep_config(world: int, exchange: str, chunks: int) -> dict:
  """The `config` object of the line: identical in the GPU arm and the reference arm."""
  return {"workload": "ep" if (EP_TOKENS, EP_G) == (8192, 256) else f"ep[{EP_TOKENS} tokens, {EP_G} experts]",
          "note": "expert-parallel MoE layer: route, dispatch rows to the experts' owners, grouped GEMM, "
                  "return rows, gate-weighted combine",
          "tokens_per_rank": EP_TOKENS, "k": EP_K, "n": EP_N, "experts": EP_G, "top_k": EP_TOPK,
          "parallelism": f"ep{world}", "l2": "inputs_exceed_l2, no flush"}


def ep_routing(rank: int):
  from tokamax_b200.ragged_dot import arg_specs
  return arg_specs.topk_routing(EP_TOKENS, EP_G, EP_TOPK, seed=10_000 + rank)


def ep_parity_check(layer, tokens, ids, gates, y, plan, rhs, world, rank, dev, samples_per_rank=4):
  """Sampled tokens of every rank against a dense top-k MoE recomputed on the host by the CPU
  oracle (each rank contributes the experts it owns), and this rank's group sizes against the
  global histogram of all ranks' routing.  Returns (checked tokens, max abs err, worst err /
  tolerance, group sizes exact)."""
  import torch.distributed as dist
  from oracle import ragged_dot_ref as ref   # the checker
  gl = EP_G // world
  # group bookkeeping: exact against the histogram of every rank's (seeded) routing
  want = np.zeros(EP_G, np.int64)
  for r in range(world):
    want += np.bincount(ep_routing(r)[0].reshape(-1), minlength=EP_G)
  got = plan.group_sizes.cpu().numpy().astype(np.int64)
  gs_exact = bool(np.array_equal(got, want[rank * gl:(rank + 1) * gl]))

  s = samples_per_rank
  pick = torch.from_numpy(np.random.default_rng(77 + rank).choice(EP_TOKENS, s, replace=False)).to(dev)
  mine = dict(tok=tokens[pick].contiguous(), ids=ids[pick].to(torch.int32).contiguous(),
              gates=gates[pick].to(torch.float32).contiguous(), y=y[pick].contiguous())
  gathered = {}
  for k_, v in mine.items():
    if world > 1:
      bufs = [torch.empty_like(v) for _ in range(world)]
      dist.all_gather(bufs, v)
      gathered[k_] = torch.cat(bufs).cpu()
    else:
      gathered[k_] = v.cpu()
  n_tok = gathered["tok"].shape[0]
  partial = torch.zeros(n_tok, EP_N, dtype=torch.float64)
  for t in range(n_tok):
    for j in range(EP_TOPK):
      e = int(gathered["ids"][t, j])
      if e // gl != rank:
        continue
      w_e = rhs[e - rank * gl].cpu()[None]                         # [1, K, N] bf16, this rank's expert
      row = ref.ragged_dot_ref(gathered["tok"][t:t + 1], w_e, np.array([1]))   # bf16 [1, N]
      partial[t] += float(gathered["gates"][t, j]) * row[0].double()
  partial = partial.to(dev)
  if world > 1:
    dist.all_reduce(partial)
  want_y = partial.cpu()
  got_y = gathered["y"].double()
  err = (got_y - want_y).abs()
  tol = 2e-2 + 2e-2 * want_y.abs()
  return n_tok, float(err.max()), float((err / tol).max()), gs_exact


def cpu_ep_layer(threads: int, target_seconds: float):
  """The layer's per-rank work on the host cores by the CPU restatement: stable sort of the
  (token, expert) pairs, row gather, per-expert float32 matmul of bf16 inputs (the oracle),
  gate-weighted combine.  Rank 0's routing and token count; eight weight slabs are cycled
  over the 256 experts so that the host needs 235 MB of weights, not 7.5 GB.  Repeated until
  `target_seconds` have passed.  Returns (TFLOP/s, description, seconds per pass)."""
  from oracle import ragged_dot_ref as ref  # the checker, used here as the timed CPU baseline
  torch.set_num_threads(threads)
  rng = np.random.default_rng(0)
  ids, gates = ep_routing(0)
  tokens = torch.from_numpy(rng.standard_normal((EP_TOKENS, EP_K), dtype=np.float32)).bfloat16()
  slabs = [torch.from_numpy(rng.standard_normal((1, EP_K, EP_N), dtype=np.float32) * EP_K ** -0.5).bfloat16()
           for _ in range(8)]
  gates_t = torch.from_numpy(gates)

  def one_pass():
    t0 = time.perf_counter()
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    counts = np.bincount(flat, minlength=EP_G)
    rows = tokens[torch.from_numpy(order // EP_TOPK)]
    out = torch.empty(rows.shape[0], EP_N, dtype=torch.bfloat16)
    off = 0
    for e in range(EP_G):
      c = int(counts[e])
      if c:
        out[off:off + c] = ref.ragged_dot_ref(rows[off:off + c], slabs[e % 8], np.array([c]))
        off += c
    y = torch.zeros(EP_TOKENS, EP_N, dtype=torch.float32)
    y.index_add_(0, torch.from_numpy(order // EP_TOPK), out.float() * gates_t.reshape(-1)[torch.from_numpy(order)][:, None])
    y = y.bfloat16()
    return time.perf_counter() - t0

  one_pass()  # warm-up
  times = []
  t_begin = time.perf_counter()
  while not times or time.perf_counter() - t_begin < target_seconds:
    times.append(one_pass())
  t = float(np.median(times))
  flops = 2.0 * EP_TOKENS * EP_TOPK * EP_K * EP_N
  desc = (f"ep: one rank's whole step ({EP_TOKENS} tokens x top-{EP_TOPK}, {EP_TOKENS * EP_TOPK} rows over "
          f"{EP_G} experts: sort, gather, per-expert float32 matmul of bf16 inputs, combine), "
          f"{len(times)} passes, {threads} threads")
  return flops / t / 1e12, desc, t


def run_reference_arm(args, world, rank):
  if rank != 0:
    return None
  threads = os.cpu_count() or 1
  vals = []
  desc = ""
  for i in range(args.warmup + args.steps):
    tf, desc, t = cpu_ep_layer(threads, 0.0)   # one pass per step
    if i >= args.warmup:
      vals.append((tf, t))
    if i >= args.warmup and sum(v[1] for v in vals) > 150.0:
      break
  tf = float(np.median([v[0] for v in vals]))
  ms = float(np.mean([v[1] for v in vals]) * 1e3)
  cfg = ep_config(world, "", 0)
  cfg["reference_path"] = "CPU restatement of implementation='xla' (jax not installable here), one rank's step"
  return {
      "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus,
      "steps": len(vals), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
      "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
      "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
      "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }


def run_expert_parallel(args, peaks, world, rank, local_rank):
  import torch.distributed as dist
  from tokamax_b200 import _capi
  from tokamax_b200.expert_parallel import ExpertParallelMoE

  dev = torch.device("cuda", local_rank)
  torch.cuda.set_device(dev)
  _capi.load()
  gl = EP_G // world
  # Expert e's weights come from seed 1000 + e, so every world size sees the same model.
  rhs = torch.empty(gl, EP_K, EP_N, device=dev, dtype=torch.bfloat16)
  for i in range(gl):
    gen = torch.Generator(device=dev).manual_seed(1000 + rank * gl + i)
    rhs[i] = (torch.randn(EP_K, EP_N, device=dev, generator=gen, dtype=torch.float32) * EP_K ** -0.5).to(torch.bfloat16)
  gen = torch.Generator(device=dev).manual_seed(rank)
  tokens = torch.randn(EP_TOKENS, EP_K, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16)
  ids_np, gates_np = ep_routing(rank)
  ids = torch.from_numpy(ids_np).to(dev)
  gates = torch.from_numpy(gates_np).to(dev)
  layer = ExpertParallelMoE(rhs, EP_G, num_chunks=args.ep_chunks if args.ep_chunks > 0 else 4,
                            exchange="fused" if args.ep_exchange in ("fused_once", "fused_pairs") else args.ep_exchange)
  if args.ep_exchange == "fused_once":
    layer.once_per_rank = True
  elif args.ep_exchange == "fused_pairs":
    layer.once_per_rank = False
  stream = torch.cuda.current_stream()
  sampler_id = gpu_id_for_smi(local_rank) if rank == 0 else None   # rank 0 prints the line

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  warmup = max(args.warmup, 3)
  for _ in range(warmup):
    y, plan = layer(tokens, ids, gates)
  barrier()
  layer.gemm_events = []          # (start, end) CUDA events around the grouped-GEMM launch of each step
  with ClockSampler(sampler_id) as clocks:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks.wait_ready()
    for _ in range(3):              # the GPU is busy again when the first kept sample is taken
      layer(tokens, ids, gates)
    barrier()
    start.record(stream)
    for _ in range(args.steps):
      y, plan = layer(tokens, ids, gates)
    end.record(stream)
    barrier()
    total_ms = start.elapsed_time(end)
    gemm_ms = [s.elapsed_time(e) for s, e in layer.gemm_events]
    layer.gemm_events = None
    launches_per_step = layer.launches_last_call
    # keep the same work running until the 100 ms clock sampler has seen it; every rank runs
    # the same number of steps (the exchange is collective), taken from the slowest rank's time
    ms_all = torch.tensor([total_ms / args.steps], device=dev)
    if world > 1:
      dist.all_reduce(ms_all, op=dist.ReduceOp.MAX)
    for _ in range(int(min(2000, max(10, 700.0 / max(ms_all.item(), 1e-3))))):
      layer(tokens, ids, gates)
    barrier()
  _capi.device_status()
  layer.check_overflow()
  rows_local = int(plan.group_sizes.sum().item())     # rows this rank multiplied per step

  # parity on the result of the last timed step
  checked, max_err, worst_ratio, gs_exact = ep_parity_check(layer, tokens, ids, gates, y, plan, rhs, world, rank, dev)

  # end to end: host tokens / routing in, combined activations out
  h_tok, h_ids, h_gates = tokens.cpu().pin_memory(), ids.cpu().pin_memory(), gates.cpu().pin_memory()
  # Every step copies its inputs from pinned host memory and its result back; the layer's
  # HostPipeline runs those copies beside the neighbouring steps' computation (two staging slots,
  # two result buffers).  The region ends when the last step's result is in host memory.
  from tokamax_b200.expert_parallel import HostPipeline
  h_outs = [torch.empty(EP_TOKENS, EP_N, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
  pipe = HostPipeline(layer, depth=2)
  last = None
  for i in range(3):
    last = pipe.submit(h_tok, h_ids, h_gates, h_outs[i % 2])
  pipe.drain()
  barrier()
  s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  s2.record(stream)
  for i in range(args.steps):
    last = pipe.submit(h_tok, h_ids, h_gates, h_outs[i % 2])
  stream.wait_event(last)          # the last result has reached the host
  e2.record(stream)
  pipe.drain()
  barrier()
  e2e_pipelined = s2.elapsed_time(e2)
  e2e_ok = bool(torch.equal(h_outs[(args.steps - 1) % 2], y.cpu())) if args.steps > 0 else True

  # The same through the layer's plain call, everything on one stream (copy in, step, copy out);
  # measured beside the pipeline because with several ranks the pipeline's gain depends on the
  # host (its ranks share the host's memory and PCIe root); the line reports the faster of the two.
  d_tok, d_ids, d_gates = torch.empty_like(tokens), torch.empty_like(ids), torch.empty_like(gates)

  def e2e_step():
    d_tok.copy_(h_tok, non_blocking=True)
    d_ids.copy_(h_ids, non_blocking=True)
    d_gates.copy_(h_gates, non_blocking=True)
    yy, _ = layer(d_tok, d_ids, d_gates)
    h_outs[0].copy_(yy, non_blocking=True)

  for _ in range(2):
    e2e_step()
  barrier()
  s3, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  s3.record(stream)
  for _ in range(args.steps):
    e2e_step()
  e3.record(stream)
  barrier()
  e2e_sequential = s3.elapsed_time(e3)

  gemm_mean = float(np.mean(gemm_ms)) if gemm_ms else 0.0
  stats = torch.tensor([total_ms, e2e_pipelined, gemm_mean, max_err, worst_ratio, 0.0 if gs_exact else 1.0,
                        e2e_sequential], device=dev, dtype=torch.float64)
  sums = torch.tensor([float(rows_local), float(checked) / world], device=dev, dtype=torch.float64)
  if world > 1:
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
  parity_ok = float(stats[4]) <= 1.0 and float(stats[5]) == 0.0
  if rank != 0:
    return None, parity_ok
  rows_step = float(sums[0])                               # all ranks, one step
  flops_step = 2.0 * rows_step * EP_K * EP_N
  ms = float(stats[0]) / args.steps
  tflops = flops_step / (ms * 1e-3) / 1e12
  e2e_by_method = {"HostPipeline.submit (depth 2)": float(stats[1]) / args.steps,
                   "ExpertParallelMoE.__call__ between copies on one stream": float(stats[6]) / args.steps}
  e2e_method = min(e2e_by_method, key=e2e_by_method.get)
  e2e_ms = e2e_by_method[e2e_method]
  # Roofline of the dominant kernel (the grouped GEMM of one rank): algorithmic bytes = received rows
  # read once + this rank's expert weights read once + output rows written once.
  rows_rank = rows_step / world
  g_flops = 2.0 * rows_rank * EP_K * EP_N
  g_bytes = rows_rank * EP_K * 2 + gl * EP_K * EP_N * 2 + rows_rank * EP_N * 2
  g_ms = float(stats[2])
  peak_tf = peaks["bf16_sustained"]                        # a kernel timed inside a long step
  rl = roofline_entry(g_flops, g_bytes, g_ms, peaks, peak_tf) if g_ms > 0 else None
  full_size = (EP_TOKENS, EP_G) == (8192, 256)
  ep_traffic = 4.0 * NCU_TRAFFIC_EP_QUARTER if world == 1 and full_size and layer.exchange == "fused" else None
  if rl is not None:
    hbm = rl["bound"] == "hbm"
    roofline = {"bound": rl["bound"], "achieved": rl["gbs"] if hbm else rl["tflops"],
                "peak": peaks["hbm"] if hbm else peak_tf, "unit": "GB/s" if hbm else UNIT,
                "frac": rl["frac"], "traffic": ep_traffic, "kernel": layer.gemm_kernel_name,
                "ms_per_launch": g_ms, "algorithmic_flops_per_launch": g_flops,
                "algorithmic_bytes_per_launch": g_bytes, "frac_tensor": rl["frac_tensor"],
                "frac_hbm": rl["frac_hbm"],
                "peak_source": peaks["source"] + (", HBM copy" if hbm else ", bf16 sustained (kernel timed inside a long step)")}
    if world > 1 and layer.exchange == "fused":
      # What one launch of the fused kernel pushes over NVLink from rank 0 (every rank's routing
      # has the same statistics): token rows to remote owners -- one per (token, remote rank) when
      # a token crosses to a rank once, else one per remote pair -- plus the output rows it returns
      # to remote sources (1/world of the rows it multiplies stay local).  Link time at the
      # measured peer-copy rate of this pool, 770 GB/s per direction.
      owner = ep_routing(0)[0] // gl
      remote = owner != 0
      if layer.exchange_name.endswith("once)"):
        sent_rows = sum(int(((owner == d).any(1)).sum()) for d in range(1, world))
      else:
        sent_rows = int(remote.sum())
      link_bytes = sent_rows * EP_K * 2 + rows_rank * (world - 1) / world * EP_N * 2
      t_link = link_bytes / 770e9
      t_target = max(g_flops / (peak_tf * 1e12), t_link)
      roofline.update({"nvlink_bytes_per_launch": float(link_bytes), "t_link_ms": t_link * 1e3,
                       "nvlink_peak": "770 GB/s per direction (measured peer copy on this pool)",
                       "frac_of_max_tensor_link": t_target / (g_ms * 1e-3)})
  else:
    roofline = None
  cfg = ep_config(world, layer.exchange, layer.num_chunks)
  cfg.update({"exchange": layer.exchange_name, "rows_per_step": rows_step})
  line = {
      "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": world, "steps": args.steps,
      "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
      "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
      "roofline": roofline,
      "parity": {"checked": int(round(float(sums[1]) * world)) if world > 1 else checked,
                 "max_abs_err": float(stats[3]), "worst_err_over_tolerance": float(stats[4]),
                 "tolerance": "2e-2 + 2e-2*|x| against the CPU oracle (dense top-k MoE on sampled tokens)",
                 "group_sizes_exact": float(stats[5]) == 0.0, "ok": parity_ok},
      "e2e": {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
              "h2d_bytes_per_step": world * (h_tok.numel() * 2 + h_ids.numel() * 4 + h_gates.numel() * 4),
              "d2h_bytes_per_step": world * h_outs[0].numel() * 2, "ms_per_step": e2e_ms,
              "api": "tokamax_b200.expert_parallel: " + e2e_method + " (pinned host tensors in and out)",
              "ms_per_step_by_api": e2e_by_method,
              "note": "both calls copy every step's inputs from and its result to pinned host memory "
                      "inside the timed region; the pipeline runs a step's copies beside the neighbouring "
                      "steps' computation and is timed until the last result is in host memory",
              "result_equals_device_run": e2e_ok},
      "gpu_launches": args.steps * launches_per_step,
      "gpu_launches_per_step": launches_per_step,
      "clocks": clocks.summary(),
  }
  return line, parity_ok


def _claim_stdout():
  """Keeps stdout for the one JSON line: file descriptor 1 is pointed at stderr for the rest
  of the process (libraries such as NCCL print banners to it from C code) and the original
  stdout is returned as a file object."""
  sys.stdout.flush()
  saved = os.dup(1)
  os.dup2(2, 1)
  sys.stdout = os.fdopen(os.dup(2), "w", buffering=1)
  return os.fdopen(saved, "w", buffering=1)


def main():
  json_out = _claim_stdout()
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
  ap.add_argument("--fp8-path", default="native", choices=["native", "convert"],
                  help="e4m3 weights: fp8 tensor cores on split activations, or in-kernel expansion to bf16")
  ap.add_argument("--workload", default=None, choices=[None, "cfg1", "cfg2", "cfg3", "cfg4", "dsv3", "ep"])
  ap.add_argument("--op", default="fwd", choices=["fwd", "dlhs", "drhs"],
                  help="which contraction of the workload to time (single GPU)")
  ap.add_argument("--rhs-dtype", default=None, choices=[None, "fp8", "int8", "bf16"],
                  help="weight type of a single-kernel run (cfg3 defaults to fp8)")
  ap.add_argument("--groups", type=int, default=0,
                  help="keep only the first N groups of the workload (smaller profiler captures)")
  ap.add_argument("--ep-exchange", default=None, choices=[None, "fused", "fused_once", "fused_pairs", "nccl"],
                  help="row exchange of the expert-parallel layer (default: the fused kernel; fused_once / "
                       "fused_pairs force a token to cross to a rank once / once per routed pair)")
  ap.add_argument("--ep-chunks", type=int, default=0,
                  help="expert chunks of the nccl exchange whose transfers overlap the neighbouring GEMMs")
  ap.add_argument("--kernel-only", action="store_true",
                  help="exactly --steps launches of the timed region, no padding for the clock sampler")
  ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel suite of the N = 1 line")
  ap.add_argument("--ep-tokens", type=int, default=0, help="tokens per rank of the ep workload (profiler captures)")
  ap.add_argument("--ep-experts", type=int, default=0, help="experts of the ep workload (profiler captures)")
  args = ap.parse_args()

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  from tokamax_b200.ragged_dot import arg_specs

  workload = args.workload or "ep"
  global EP_TOKENS, EP_G
  if args.ep_tokens:
    EP_TOKENS = args.ep_tokens
  if args.ep_experts:
    EP_G = args.ep_experts
  if args.impl == "reference":
    line = run_reference_arm(args, world, rank)
    if line is not None:
      print(json.dumps(line), file=json_out, flush=True)
    return

  peaks = load_peaks()
  ok = True
  if workload == "ep":
    if world > 1:
      import torch.distributed as dist
      os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
      torch.cuda.set_device(local_rank)
      dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
      try:
        line, ok = run_expert_parallel(args, peaks, world, rank, local_rank)
      finally:
        dist.destroy_process_group()
    else:
      line, ok = run_expert_parallel(args, peaks, 1, 0, 0)
      torch.cuda.empty_cache()
      threads = os.cpu_count() or 1
      cpu_tf, cpu_desc, _ = cpu_ep_layer(threads, 2.0 if args.no_kernels else 12.0)
      line["cpu_baseline"] = {"value": cpu_tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": cpu_desc}
      if not args.no_kernels:
        line["kernels"] = run_kernel_suite(torch.device("cuda", 0), peaks, gpu_id_for_smi(0))
  else:
    w = arg_specs.workload(workload)
    if args.rhs_dtype is not None:
      w = dataclasses.replace(w, rhs_dtype={"fp8": torch.float8_e4m3fn, "int8": torch.int8,
                                            "bf16": torch.bfloat16}[args.rhs_dtype])
    if args.groups and args.groups < w.g:
      gs = tuple(w.group_sizes[:args.groups])
      w = dataclasses.replace(w, name=f"{w.name}[:{args.groups}]", g=args.groups, group_sizes=gs, m=sum(gs))
    line = run_single(args, w, peaks)
  if line is not None:
    print(json.dumps(line), file=json_out, flush=True)
  if not ok:
    sys.exit(3)


if __name__ == "__main__":
  main()
