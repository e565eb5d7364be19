"""Autotunes named ragged-dot workloads on the current GPU and writes the cache file.

  python -m tokamax_b200.autotuning.tune --workloads cfg2,cfg4,dsv3 --ops fwd,dlhs,drhs
  python -m tokamax_b200.autotuning.tune --workloads memory_bound,mixtral/8x7b --ops fwd

A workload is one of the headline configurations (cfg1 ... dsv3) or the full name of one of the
reference's benchmark specs (`arg_specs.ARG_SPECS`: "compute_bound", "memory_bound",
"mixtral/8x7b", "maxtext/deepseek-v3-...").

For every (workload, contraction) the op's search space is timed (configs that map onto the
same kernel parameters are timed once) and the best few entries are merged into
`tokamax_b200/data/autotuning/<device kind>/b200_ragged_dot.json`, the file
`BoundArguments.cached_autotuning_data` reads.  Plays the role of the reference's checked-in
`tokamax/data/autotuning/nvidia_b200/*ragged_dot.json` and of the tooling that fills them.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from tokamax_b200 import op as op_lib
from tokamax_b200.autotuning import autotuner as autotuner_lib
from tokamax_b200.autotuning import cache as cache_lib
from tokamax_b200.quantization import QArray, quantize_per_channel
from tokamax_b200.ragged_dot import arg_specs, b200, base


def bound_arguments(op: b200.B200RaggedDot, w: arg_specs.Workload, which: str, device):
  """Seeded inputs of the workload, bound the way a caller passing tensors binds them."""
  gen = torch.Generator(device=device).manual_seed(0)
  rnd = lambda *shape: torch.randn(*shape, device=device, generator=gen, dtype=torch.float32)
  gs = torch.tensor(w.group_sizes, dtype=torch.int32, device=device)
  lhs = rnd(w.m, w.k).to(torch.bfloat16)
  if which == "drhs":
    dout = rnd(w.m, w.n).to(torch.bfloat16)
    return op.bind(lhs, dout, group_sizes=gs,
                   ragged_dot_dimension_numbers=base.RAGGED_CONTRACTING_DOT_DIM_NUMS)
  rhs = torch.empty(w.g, w.k, w.n, device=device, dtype=torch.bfloat16)
  for g in range(w.g):
    rhs[g] = (rnd(w.k, w.n) * w.k ** -0.5).to(torch.bfloat16)
  if which == "dlhs":
    dout = rnd(w.m, w.n).to(torch.bfloat16)
    return op.bind(dout, rhs, group_sizes=gs, ragged_dot_dimension_numbers=base.TRANS_RHS_RAGGED_DOT_DIM_NUMS)
  if w.rhs_dtype in (torch.float8_e4m3fn, torch.int8):
    q = torch.empty(w.g, w.k, w.n, device=device, dtype=w.rhs_dtype)
    scale = torch.empty(w.g, 1, w.n, device=device, dtype=torch.float32)
    for g in range(w.g):
      qa = quantize_per_channel(rhs[g:g + 1], w.rhs_dtype)
      q[g], scale[g] = qa.qvalue[0], qa.scale[0]
    del rhs
    return op.bind(lhs, QArray(q, scale), group_sizes=gs)
  return op.bind(lhs, rhs, group_sizes=gs)


def named_workload(name: str) -> arg_specs.Workload:
  """A headline configuration, or one of the reference's benchmark specs as a Workload."""
  if name in arg_specs.NAMED_ARG_SPECS:
    a = arg_specs.NAMED_ARG_SPECS[name].args
    (m, k), (g, _, n) = a["lhs"].shape, a["rhs"].shape
    return arg_specs.Workload(name, m, k, n, g, tuple(a["group_sizes"].representative_value),
                              rhs_dtype=a["rhs"].dtype)
  return arg_specs.workload(name)


def main(argv=None):
  ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
  ap.add_argument("--workloads", default="cfg2,cfg4")
  ap.add_argument("--ops", default="fwd,dlhs,drhs")
  ap.add_argument("--keep", type=int, default=4, help="best configs kept per entry")
  ap.add_argument("--out", default=cache_lib.CACHE_PATH)
  ap.add_argument("--iterations", type=int, default=5)
  args = ap.parse_args(argv)
  if not torch.cuda.is_available():
    raise SystemExit("autotuning needs a CUDA device")
  device = torch.device("cuda", torch.cuda.current_device())
  op = b200.B200RaggedDot()
  kind = op_lib.current_device_kind()
  path = cache_lib.cache_file(op, kind, args.out)
  try:
    with open(path) as f:
      merged = json.load(f)
  except FileNotFoundError:
    merged = {}
  tuner = autotuner_lib.Autotuner(iterations=args.iterations, warmup=2)
  for name in args.workloads.split(","):
    w = named_workload(name)
    for which in args.ops.split(","):
      if which != "fwd" and w.rhs_dtype != torch.bfloat16:
        continue
      ba = bound_arguments(op, w, which, device)
      data = ba.autotune(autotuner=tuner, cache_results=False, timeout=None)
      ok = data.prune_errors()
      # best few, one per distinct set of kernel parameters (many configs share one)
      best, seen = [], set()
      for c, d in sorted(ok.items(), key=lambda cd: (cd[1].median_evaluation_time_ms, -cd[0].block_m)):
        if c.native() not in seen:
          seen.add(c.native())
          best.append((c, d))
        if len(best) == args.keep:
          break
      heur = ok.get(ba.heuristics_config)
      flops = w.flops
      print(f"{name} {which}: {len(ok)}/{len(data)} configs ran; best {best[0][1].median_evaluation_time_ms:.4f} ms "
            f"({flops / best[0][1].median_evaluation_time_ms / 1e9:.0f} TFLOP/s) native={best[0][0].native()}; "
            f"heuristics {heur.median_evaluation_time_ms if heur else float('nan'):.4f} ms", flush=True)
      merged[cache_lib.spec_to_json(dict(ba.arguments))] = {
          cache_lib.config_to_json(c): d.asdict() for c, d in best}
      del ba
      torch.cuda.empty_cache()
  os.makedirs(os.path.dirname(path), exist_ok=True)
  with open(path, "w") as f:
    json.dump(merged, f, indent=1, sort_keys=True)
  print("wrote", path, len(merged), "entries")


if __name__ == "__main__":
  main(sys.argv[1:])
