"""The fused expert-parallel path on ONE GPU, through the C ABI.

Several ranks are emulated on the one device without any kernel waiting for another launch:
every virtual rank has its own buffers, the peer table lists all of them, the barrier flags are
pre-set, and the fused kernel runs in its two phases -- every rank sends (phase 1), then every
rank multiplies and returns (phase 2) -- so each wait finds its condition already true.  The
single-rank case runs the product form (both phases in one kernel).  Expected results come from
the CPU oracle (dense top-k MoE; offset tables restated in oracle/moe_ref.py).
"""

import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import moe_ref
from oracle import ragged_dot_ref as ref
from tests import helpers
from tokamax_b200.ragged_dot import arg_specs

pytestmark = pytest.mark.gpu


def _capi():
  from tokamax_b200 import _capi
  _capi.load()
  return _capi


def _dense_moe(tok, ids, gates, rhs):
  """Per pair the oracle's bf16 expert output, gate-weighted in float32 (ascending k)."""
  t, top_k = ids.shape
  y = torch.zeros(t, rhs.shape[2], dtype=torch.float32)
  g = rhs.shape[0]
  for j in range(top_k):
    e = ids[:, j].long()
    ok = (e >= 0) & (e < g)
    for ex in torch.unique(e[ok]).tolist():
      sel = (e == ex).nonzero().reshape(-1)
      out = ref.ragged_dot_ref(tok[sel], rhs[ex:ex + 1], np.array([sel.numel()]))
      y[sel] += gates[sel, j, None].float() * out.float()
  return y.to(tok.dtype)


class VirtualRanks:
  """W ranks' buffers on one device and the peer table that lists them."""

  def __init__(self, capi, w, g, t, top_k, k, n, dtype=torch.bfloat16, once=False):
    dev = torch.device("cuda", 0)
    self.w, self.g, self.gl, self.pairs, self.cap = w, g, g // w, t * top_k, w * t * top_k
    mk = lambda shape, dt: [torch.zeros(shape, dtype=dt, device=dev) for _ in range(w)]
    self.recv = mk((self.cap, k), dtype)
    self.arrive = mk((capi.ep_arrive_words(g, w, once),), torch.int32)
    self.ret = mk((self.pairs, n), dtype)
    self.counts = mk((w, g), torch.int32)
    self.flags = mk((w,), torch.int32)
    self.refs = [torch.full((self.cap,), 0x7fffffff, dtype=torch.int32, device=dev) for _ in range(w)]   # stale garbage
    table = torch.zeros((capi.EP_TAB_ROWS, capi.EP_MAX_WORLD), dtype=torch.int64)
    for row, bufs in enumerate((self.recv, self.arrive, self.ret, self.counts, self.flags, self.refs)):
      for r in range(w):
        table[row, r] = bufs[r].data_ptr()
    self.table = table.to(dev)
    self.plan = [torch.zeros(capi.ep_plan_ints(g, w), dtype=torch.int32, device=dev) for _ in range(w)]
    self.pos = mk((self.pairs,), torch.int32)
    self.sorted_pair = mk((self.pairs,), torch.int32)
    self.my_counts = mk((g,), torch.int32)
    self.ws = torch.empty(max(capi.moe_sort_workspace_bytes(self.pairs, g), 4), dtype=torch.uint8, device=dev)

  def preset_flags(self, seq):
    for f in self.flags:
      f.fill_(seq)


def _plan_tables(capi, plan, g, w):
  gl = g // w
  p = plan.cpu().numpy()
  o = 0
  out = {}
  for name, size, shape in (("group_sizes", gl, (gl,)), ("vstart", g + 1, (g + 1,)), ("src_off", g, (g,)),
                            ("dst_row", g, (g,)), ("seg_start", gl * (w + 1), (gl, w + 1)),
                            ("ret_off", gl * w, (gl, w))):
    out[name] = p[o:o + size].reshape(shape)
    o += size
  assert o == capi.ep_plan_ints(g, w)
  return out


@pytest.mark.parametrize("w,g", [(1, 8), (2, 32), (4, 256), (8, 256), (16, 1024)])
def test_exchange_plan_tables_match_restatement(w, g):
  capi = _capi()
  rng = np.random.default_rng(w * 1000 + g)
  counts = rng.integers(0, 40, (w, g)).astype(np.int32)
  counts[rng.random((w, g)) < 0.3] = 0          # empty (source, expert) segments
  vr = VirtualRanks(capi, w, g, 8, 1, 16, 16)
  vr.preset_flags(1)
  # two rounds: after the first every rank's row is in every matrix, the second plans on all of them
  for _ in range(2):
    for r in range(w):
      vr.my_counts[r].copy_(torch.from_numpy(counts[r]))
      capi.ep_exchange_plan(vr.my_counts[r], vr.table, vr.counts[r], vr.flags[r], vr.arrive[r], vr.plan[r], g, w,
                            r, 1, 50_000_000)
  torch.cuda.synchronize()
  capi.device_status()
  for r in range(w):
    assert np.array_equal(vr.counts[r].cpu().numpy(), counts)
    got = _plan_tables(capi, vr.plan[r], g, w)
    want = moe_ref.ep_plan_ref(counts, r)
    for name in want:
      assert np.array_equal(got[name], want[name]), (r, name)


def _run_virtual(capi, w, t, k, n, g, top_k, pair, seed, bad_ids=False, dtype=torch.bfloat16, once=False):
  rng = np.random.default_rng(seed)
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).to(dtype)
  gl = g // w
  toks, idss, gatess = [], [], []
  for r in range(w):
    toks.append(torch.from_numpy(rng.normal(0, 1, (t, k)).astype(np.float32)).to(dtype))
    ids, gates = arg_specs.topk_routing(t, g, top_k, seed=seed + 10 + r)
    if bad_ids:
      ids = ids.copy()
      ids[rng.random(ids.shape) < 0.05] = g + 3      # dropped pairs
      ids[rng.random(ids.shape) < 0.03] = -1
      twice = rng.random(t) < 0.1                    # a token that names one expert twice
      ids[twice, 1] = ids[twice, 0]
    idss.append(torch.from_numpy(ids))
    gatess.append(torch.from_numpy(gates))
  vr = VirtualRanks(capi, w, g, t, top_k, k, n, dtype, once=once)
  dev = vr.table.device
  cfg = capi.Config(collective=1 if pair else 0)
  d_tok = [x.to(dev) for x in toks]
  d_ids = [x.reshape(-1).to(torch.int32).to(dev) for x in idss]
  d_rhs = [rhs[r * gl:(r + 1) * gl].contiguous().to(dev) for r in range(w)]
  for r in range(w):
    capi.moe_sort_pairs_inverse(d_ids[r], g, vr.pos[r], vr.sorted_pair[r], vr.my_counts[r], vr.ws)
  vr.preset_flags(1)
  for _ in range(2):
    for r in range(w):
      capi.ep_exchange_plan(vr.my_counts[r], vr.table, vr.counts[r], vr.flags[r], vr.arrive[r], vr.plan[r], g, w,
                            r, 1, 50_000_000, once_per_rank=once)
  # once per rank: every rank sends and announces, then every rank copies its duplicates and multiplies
  phases = ((7,) if once else (3,)) if w == 1 else ((1, 6) if once else (1, 2))
  for ph in phases:
    for r in range(w):
      capi.ep_moe_fused(d_tok[r], vr.sorted_pair[r], vr.recv[r], d_rhs[r], vr.plan[r], vr.table, vr.arrive[r],
                        top_k, g, w, r, n, phases=ph, config=cfg,
                        expert_ids=d_ids[r] if once else None, pair_pos=vr.pos[r] if once else None)
  if dtype == torch.bfloat16:
    ys = [capi.moe_combine(vr.ret[r], vr.pos[r], gatess[r].to(dev), t, top_k) for r in range(w)]
  else:   # the combine kernel takes bf16 rows: weight the returned rows with torch instead
    ys = []
    for r in range(w):
      pos = vr.pos[r].long().reshape(t, top_k)
      rows = vr.ret[r][pos.clamp(min=0)].float() * (pos >= 0)[..., None]
      ys.append((rows * gatess[r].to(dev)[..., None]).sum(1).to(dtype))
  torch.cuda.synchronize()
  capi.device_status()
  # group bookkeeping: exact
  all_ids = torch.cat([i.reshape(-1) for i in idss]).numpy()
  hist = np.bincount(all_ids[(all_ids >= 0) & (all_ids < g)], minlength=g)
  dups = 0
  for r in range(w):
    got = vr.plan[r][:gl].cpu().numpy()
    assert np.array_equal(got, hist[r * gl:(r + 1) * gl]), f"rank {r}: group sizes"
    arrive = vr.arrive[r].cpu().numpy()
    if once:
      announced, copied = arrive[gl + 2:2 * gl + 2], arrive[2 * gl + 2:3 * gl + 2]
      assert np.array_equal(announced, copied), f"rank {r}: every announced duplicate was copied"
      assert np.array_equal(arrive[:gl] + copied, got), f"rank {r}: rows present + copied"
      dups += int(copied.sum())
    else:
      assert np.array_equal(arrive[:gl], got), f"rank {r}: arrival counters"
  if once:
    # every reference word, exactly (stale words were pre-set to garbage)
    want_refs = moe_ref.ep_reference_words_ref([i.numpy() for i in idss], g)
    for r in range(w):
      got_refs = vr.refs[r][:len(want_refs[r])].cpu().numpy().astype(np.int64)
      assert np.array_equal(got_refs, want_refs[r]), f"rank {r}: reference words"
  if once and w > 1 and top_k > 1 and not bad_ids:
    # what must have stayed off the link: per source token and REMOTE rank, (its pairs there) - 1
    want_dups = 0
    for r in range(w):
      owner = idss[r].numpy() // gl
      for d in range(w):
        if d != r:
          per_tok = (owner == d).sum(1)
          want_dups += int(np.maximum(per_tok - 1, 0).sum())
    assert dups == want_dups and dups > 0, (dups, want_dups)
  for r in range(w):
    want = _dense_moe(toks[r], idss[r], gatess[r], rhs)
    helpers.assert_close(ys[r], want.to(dtype), what=f"virtual rank {r} of {w}")


@pytest.mark.parametrize("pair", [False, True])
def test_fused_single_rank_matches_dense_moe(pair):
  _run_virtual(_capi(), 1, 512, 256, 384, 8, 2, pair, seed=11)


def test_fused_single_rank_drops_out_of_range_ids():
  _run_virtual(_capi(), 1, 300, 128, 256, 8, 2, True, seed=12, bad_ids=True)


@pytest.mark.parametrize("w,pair", [(2, True), (2, False), (4, True), (8, True)])
def test_fused_virtual_ranks_match_dense_moe(w, pair):
  _run_virtual(_capi(), w, 256, 192, 320, 32, 4, pair, seed=20 + w)


@pytest.mark.parametrize("w,pair", [(2, True), (2, False), (4, True), (8, True)])
def test_fused_once_per_rank_virtual_ranks_match_dense_moe(w, pair):
  """A token crosses to a rank once; its other rows there are copied by the owner."""
  _run_virtual(_capi(), w, 256, 192, 320, 32, 4, pair, seed=40 + w, once=True)


def test_fused_once_per_rank_with_dropped_pairs_and_f16():
  _run_virtual(_capi(), 4, 300, 136, 264, 16, 4, True, seed=51, bad_ids=True, once=True)
  _run_virtual(_capi(), 2, 200, 136, 264, 16, 3, True, seed=52, dtype=torch.float16, once=True)


def test_fused_virtual_ranks_f16_and_ragged_k():
  _run_virtual(_capi(), 2, 200, 136, 264, 16, 2, True, seed=31, dtype=torch.float16)


def test_fused_layer_world1_public_call():
  """ExpertParallelMoE with the fused exchange on one rank: result, group sizes, buffer reuse."""
  capi = _capi()
  from tokamax_b200.expert_parallel import ExpertParallelMoE
  t, k, n, g, top_k = 640, 512, 512, 16, 4
  rng = np.random.default_rng(41)
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  tok = torch.from_numpy(rng.normal(0, 1, (t, k)).astype(np.float32)).bfloat16()
  ids, gates = arg_specs.topk_routing(t, g, top_k, seed=42)
  layer = ExpertParallelMoE(rhs.cuda(), g)
  assert layer.exchange == "fused"
  y, plan = layer(tok.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(gates).cuda())
  y2, _ = layer(tok.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(gates).cuda())
  torch.cuda.synchronize()
  layer.check_overflow()
  assert torch.equal(y, y2)
  assert layer.launches_last_call == 7
  assert np.array_equal(plan.group_sizes.cpu().numpy(), np.bincount(ids.reshape(-1), minlength=g))
  helpers.assert_close(y, _dense_moe(tok, torch.from_numpy(ids), torch.from_numpy(gates), rhs), what="fused layer")
  # the split form (send everything, barrier, multiply) gives the same bits
  y3, _ = layer.forward_fused(tok.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(gates).cuda(), phases=(1, 2))
  assert torch.equal(y, y3)


def test_host_pipeline_matches_device_calls_step_by_step():
  """HostPipeline: five steps with different pinned host inputs, two staging slots; every step's
  host result equals the layer called on device tensors with the same inputs."""
  _capi()
  from tokamax_b200.expert_parallel import ExpertParallelMoE, HostPipeline
  t, k, n, g, top_k = 512, 256, 384, 16, 4
  rng = np.random.default_rng(61)
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  layer = ExpertParallelMoE(rhs.cuda(), g)
  steps = []
  for i in range(5):
    tok = torch.from_numpy(rng.normal(0, 1, (t, k)).astype(np.float32)).bfloat16().pin_memory()
    ids, gates = arg_specs.topk_routing(t, g, top_k, seed=70 + i)
    steps.append((tok, torch.from_numpy(ids).pin_memory(), torch.from_numpy(gates).pin_memory(),
                  torch.empty(t, n, dtype=torch.bfloat16).pin_memory()))
  pipe = HostPipeline(layer, depth=2)
  events = [pipe.submit(*s) for s in steps]
  events[1].synchronize()
  want1, _ = layer(steps[1][0].cuda(), steps[1][1].cuda(), steps[1][2].cuda())
  assert torch.equal(steps[1][3], want1.cpu())       # readable as soon as its own event has fired
  pipe.drain()
  for tok, ids, gates, out in steps:
    want, _ = layer(tok.cuda(), ids.cuda(), gates.cuda())
    assert torch.equal(out, want.cpu())
  with pytest.raises(ValueError):
    pipe.submit(steps[0][0].clone(), steps[0][1], steps[0][2], steps[0][3])   # not pinned


def test_barrier_wait_runs_out_and_reports_status():
  """A flag that nothing sets: the barrier kernel gives up after its budget, the status word says
  so, and the device keeps working."""
  capi = _capi()
  dev = torch.device("cuda", 0)
  flags = torch.zeros(2, dtype=torch.int32, device=dev)
  sink = torch.zeros(2, dtype=torch.int32, device=dev)     # stands for the absent peer's flag array
  table = torch.zeros((5, capi.EP_MAX_WORLD), dtype=torch.int64)
  table[capi.EP_TAB_FLAGS, 0] = flags.data_ptr()
  table[capi.EP_TAB_FLAGS, 1] = sink.data_ptr()
  table = table.to(dev)
  capi.device_status()
  capi.cross_rank_barrier(table, flags, 2, 0, 1, 1_000_000)   # 1 ms budget; slot 1 is never written
  with pytest.raises(RuntimeError, match="bounded wait"):
    capi.device_status()
  assert flags.cpu().tolist() == [1, 0] and sink.cpu().tolist() == [1, 0]
  # the context is intact: a complete barrier and a GEMM still run
  capi.cross_rank_barrier(table, flags, 1, 0, 2, 1_000_000)
  capi.device_status()
  _run_virtual(capi, 1, 128, 64, 128, 4, 2, False, seed=5)
