"""World-size-2 (and 1) tests of the expert-parallel plumbing on CPU ranks over gloo.

The compute steps need a GPU; here they are replaced by the CPU oracle through the layer's
`backend` hook, so what is checked is the exchange logic: counts all-to-all, split sizes,
the (source rank, expert) segment bookkeeping and the way combine undoes dispatch.  Expected result: the single-device top-k MoE on the unsharded inputs.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_ref
from oracle import ragged_dot_ref as ref
from tokamax_b200.ragged_dot import arg_specs

T, K, N, G, TOPK = 48, 16, 24, 8, 2


def _inputs(world):
  rng = np.random.default_rng(3)
  rhs = torch.from_numpy(rng.normal(0, K ** -0.5, (G, K, N)).astype(np.float32)).bfloat16()
  per_rank = []
  for r in range(world):
    tok = torch.from_numpy(np.random.default_rng(100 + r).normal(0, 1, (T, K)).astype(np.float32)).bfloat16()
    ids, gates = arg_specs.topk_routing(T, G, TOPK, seed=200 + r)
    per_rank.append((tok, torch.from_numpy(ids), torch.from_numpy(gates)))
  return rhs, per_rank


def _dense_moe(tok, ids, gates, rhs):
  y = torch.zeros(tok.shape[0], rhs.shape[2], dtype=torch.float32)
  for j in range(ids.shape[1]):
    w = rhs[ids[:, j].long()].float()                          # [T, K, N]
    yj = torch.einsum("tk,tkn->tn", tok.float(), w).bfloat16().float()   # expert output is bf16
    y += gates[:, j, None] * yj
  return y


class OracleBackend:
  """The four compute steps of the layer on the CPU oracle."""

  def sort_pairs(self, expert_ids, num_experts):
    pos, counts = moe_ref.sort_pairs_ref(expert_ids.numpy(), num_experts)
    return torch.from_numpy(pos), torch.from_numpy(counts)

  def gather_rows(self, tokens, pos, top_k):
    return moe_ref.gather_rows_ref(tokens, pos.numpy(), top_k)

  def expert_gemm(self, rows, rhs_local, segment_sizes):
    return moe_ref.cyclic_ragged_dot_ref(rows, rhs_local, segment_sizes.numpy())

  def combine(self, rows, pos, gates, num_tokens, top_k):
    return moe_ref.combine_ref(rows, pos.numpy(), gates, num_tokens, top_k)

  def expert_gemm_dlhs(self, dout_rows, rhs_local, segment_sizes):
    return moe_ref.cyclic_ragged_dot_ref(dout_rows, rhs_local.transpose(1, 2).contiguous(), segment_sizes.numpy())

  def expert_gemm_drhs(self, rows, dout_rows, segment_sizes, local_experts):
    seg = segment_sizes.numpy().astype(np.int64)
    off = np.concatenate([[0], np.cumsum(seg)])
    out = torch.zeros((local_experts, rows.shape[1], dout_rows.shape[1]), dtype=torch.float32)
    for i in range(len(seg)):
      s0, s1 = int(off[i]), int(off[i + 1])
      if s1 > s0:
        out[i % local_experts] += rows[s0:s1].float().T @ dout_rows[s0:s1].float()
    return out


def _worker(rank, world, port, q, chunks=1):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from tokamax_b200.expert_parallel import ExpertParallelMoE
    rhs, per_rank = _inputs(world)
    gl = G // world
    layer = ExpertParallelMoE(rhs[rank * gl:(rank + 1) * gl], G, backend=OracleBackend(), num_chunks=chunks)
    tok, ids, gates = per_rank[rank]
    y, plan = layer(tok, ids, gates)
    # group bookkeeping must be exact: rows received per local expert == global histogram slice
    all_ids = torch.cat([p[1].reshape(-1) for p in per_rank])
    want_gs = torch.bincount(all_ids.long(), minlength=G)[rank * gl:(rank + 1) * gl]
    ok_gs = torch.equal(plan.group_sizes.long(), want_gs)
    want = _dense_moe(tok, ids, gates, rhs)
    err = (y.float() - want).abs().max().item()
    q.put((rank, ok_gs, err, sum(plan.recv_splits), int(want_gs.sum())))
  finally:
    dist.destroy_process_group()


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


@pytest.mark.parametrize("world,chunks", [(1, 1), (2, 1), (2, 2), (2, 4)])
def test_expert_parallel_matches_dense_moe(world, chunks):
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, q, chunks)) for r in range(world)]
  for p in procs:
    p.start()
  results = [q.get(timeout=120) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
    assert p.exitcode == 0
  for rank, ok_gs, err, recv_rows, want_rows in results:
    assert ok_gs, f"rank {rank}: received group sizes differ from the global histogram"
    assert recv_rows == want_rows
    assert err < 2e-2, f"rank {rank}: max abs err {err}"


def _bwd_worker(rank, world, port, q):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from tokamax_b200.expert_parallel import ExpertParallelMoE
    rhs, per_rank = _inputs(world)
    gl = G // world
    layer = ExpertParallelMoE(rhs[rank * gl:(rank + 1) * gl], G, backend=OracleBackend(), num_chunks=1)
    tok, ids, gates = per_rank[rank]
    y, ctx = layer.forward_with_residuals(tok, ids, gates)
    dys = [torch.from_numpy(np.random.default_rng(300 + r).normal(0, 1, (T, N)).astype(np.float32)).bfloat16()
           for r in range(world)]
    d_tok, d_rhs, d_gates = layer.backward(dys[rank], ctx)
    # dense reference by autograd over ALL ranks' tokens (the weights are shared)
    w_ref = rhs.float().requires_grad_(True)
    want_tok = want_gates = None
    for r in range(world):
      tr, ir, gr = per_rank[r]
      x = tr.float().requires_grad_(True)
      gt = gr.float().requires_grad_(True)
      yr = torch.zeros(T, N)
      for j in range(TOPK):
        yr = yr + gt[:, j, None] * torch.einsum("tk,tkn->tn", x, w_ref[ir[:, j].long()])
      (yr * dys[r].float()).sum().backward()
      if r == rank:
        want_tok, want_gates = x.grad, gt.grad
    want_rhs = w_ref.grad[rank * gl:(rank + 1) * gl]
    rel = lambda a, b: ((a.float() - b).abs().max() / (b.abs().max() + 1e-6)).item()
    q.put((rank, rel(d_tok, want_tok), rel(d_rhs, want_rhs), rel(d_gates, want_gates)))
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_expert_parallel_backward_matches_autograd(world):
  """d_tokens, d_rhs (this rank's experts) and d_gates of the sharded layer against autograd
  through a dense top-k MoE over all ranks' tokens."""
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_bwd_worker, args=(r, world, port, q)) for r in range(world)]
  for p in procs:
    p.start()
  results = [q.get(timeout=120) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
    assert p.exitcode == 0
  for rank, e_tok, e_rhs, e_gates in results:
    assert e_tok < 3e-2 and e_rhs < 3e-2 and e_gates < 3e-2, (rank, e_tok, e_rhs, e_gates)


# ---------------------------------------------------------------- host-side fault injection
class _CorruptCounts(OracleBackend):
  """A rank whose sort reports wrong per-expert counts: `phantom` announces rows it does not
  have, `dropped` forgets rows it has, `negative` reports a negative count."""

  def __init__(self, kind):
    self.kind = kind

  def sort_pairs(self, expert_ids, num_experts):
    pos, counts = super().sort_pairs(expert_ids, num_experts)
    counts = counts.clone()
    e = int(torch.nonzero(counts)[0])
    if self.kind == "phantom":
      counts[e] += 5
    elif self.kind == "dropped":
      counts[e] -= 1
    else:
      counts[e] = -counts[e]
    return pos, counts


def _fault_worker(rank, world, port, q, kind, chunks):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from tokamax_b200.expert_parallel import ExpertParallelMoE
    rhs, per_rank = _inputs(world)
    gl = G // world
    backend = _CorruptCounts(kind) if rank == 1 else OracleBackend()
    layer = ExpertParallelMoE(rhs[rank * gl:(rank + 1) * gl], G, backend=backend, num_chunks=chunks)
    tok, ids, gates = per_rank[rank]
    try:
      layer(tok, ids, gates)
      q.put((rank, "no error"))
    except RuntimeError as e:
      q.put((rank, str(e)))
    # the group is still usable: the same layer with honest counts runs afterwards
    layer2 = ExpertParallelMoE(rhs[rank * gl:(rank + 1) * gl], G, backend=OracleBackend(), num_chunks=chunks)
    y, _ = layer2(tok, ids, gates)
    q.put((rank, float((y.float() - _dense_moe(tok, ids, gates, rhs)).abs().max())))
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("kind,chunks", [("phantom", 1), ("dropped", 1), ("negative", 2)])
def test_corrupt_counts_are_refused_on_every_rank(kind, chunks):
  """Failure made on the host: one rank's counts are wrong.  Every rank raises before any row
  is exchanged (no rank is left waiting in a collective), and the next step works."""
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_fault_worker, args=(r, 2, port, q, kind, chunks)) for r in range(2)]
  for p in procs:
    p.start()
  results = [q.get(timeout=120) for _ in range(4)]
  for p in procs:
    p.join(timeout=60)
    assert p.exitcode == 0
  msgs = [r for r in results if isinstance(r[1], str)]
  errs = [r for r in results if not isinstance(r[1], str)]
  assert len(msgs) == 2 and all("inconsistent per-expert counts" in m for _, m in msgs), msgs
  assert len(errs) == 2 and all(e < 2e-2 for _, e in errs), errs
