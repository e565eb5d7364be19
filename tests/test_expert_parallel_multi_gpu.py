"""Expert-parallel layer on 2 and 4 real GPUs: result equals a dense top-k MoE, received group
sizes equal the global histogram slice.  Both exchanges: the fused kernel over peer-mapped
memory and the NCCL all-to-all form.  Skipped on boxes with fewer GPUs."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tokamax_b200.ragged_dot import arg_specs

pytestmark = pytest.mark.gpu
T, K, N, G, TOPK = 1024, 512, 384, 32, 4


def _inputs(world):
  rng = np.random.default_rng(5)
  rhs = torch.from_numpy(rng.normal(0, K ** -0.5, (G, K, N)).astype(np.float32)).bfloat16()
  per_rank = []
  for r in range(world):
    tok = torch.from_numpy(np.random.default_rng(100 + r).normal(0, 1, (T, K)).astype(np.float32)).bfloat16()
    ids, gates = arg_specs.topk_routing(T, G, TOPK, seed=300 + r)
    per_rank.append((tok, torch.from_numpy(ids), torch.from_numpy(gates)))
  return rhs, per_rank


def _worker(rank, world, port, q, chunks, exchange):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
  torch.cuda.set_device(rank)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
  try:
    from tokamax_b200 import _capi
    from tokamax_b200.expert_parallel import ExpertParallelMoE
    rhs, per_rank = _inputs(world)
    gl = G // world
    layer = ExpertParallelMoE(rhs[rank * gl:(rank + 1) * gl].cuda(), G, num_chunks=chunks,
                              exchange="fused" if exchange == "fused_once" else exchange)
    layer.once_per_rank = exchange == "fused_once"   # a token crosses to a rank once
    tok, ids, gates = per_rank[rank]
    y, plan = layer(tok.cuda(), ids.cuda(), gates.cuda())
    y = y.clone()
    gs_first = plan.group_sizes.clone()
    y2, _ = layer(tok.cuda(), ids.cuda(), gates.cuda())   # buffers are reused call after call
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    layer.check_overflow()      # no timed-out wait, no dropped row
    all_ids = torch.cat([p[1].reshape(-1) for p in per_rank])
    want_gs = torch.bincount(all_ids.long(), minlength=G)[rank * gl:(rank + 1) * gl]
    ok_gs = torch.equal(gs_first.cpu().long(), want_gs)
    want = torch.zeros(T, N)
    for j in range(TOPK):
      w = rhs[ids[:, j].long()].float()
      want += gates[:, j, None] * torch.einsum("tk,tkn->tn", tok.float(), w).bfloat16().float()
    err = ((y.float().cpu() - want).abs() / (1 + want.abs())).max().item()
    q.put((rank, ok_gs, err))
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks,exchange", [(2, 1, "nccl"), (2, 4, "nccl"), (2, 1, "fused"), (4, 1, "fused"),
                                                   (4, 2, "nccl"), (2, 1, "fused_once"), (4, 1, "fused_once")])
def test_multi_gpu_expert_parallel_matches_dense_moe(world, chunks, exchange):
  if torch.cuda.device_count() < world:
    pytest.skip(f"needs {world} GPUs")
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  procs = [ctx.Process(target=_worker, args=(r, world, port, q, chunks, exchange)) for r in range(world)]
  for p in procs:
    p.start()
  results = [q.get(timeout=300) for _ in range(world)]
  for p in procs:
    p.join(timeout=120)
    assert p.exitcode == 0
  for rank, ok_gs, err in results:
    assert ok_gs, f"rank {rank}: received group sizes differ from the global histogram"
    assert err < 2e-2, f"rank {rank}: max scaled err {err}"


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _bwd_worker(rank, world, port, q):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
  torch.cuda.set_device(rank)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
  try:
    from tokamax_b200 import _capi
    from tokamax_b200.expert_parallel import ExpertParallelMoE
    rhs, per_rank = _inputs(world)
    gl = G // world
    layer = ExpertParallelMoE(rhs[rank * gl:(rank + 1) * gl].cuda(), G, num_chunks=1, exchange="nccl")
    tok, ids, gates = per_rank[rank]
    dys = [torch.from_numpy(np.random.default_rng(400 + r).normal(0, 1, (T, N)).astype(np.float32)).bfloat16()
           for r in range(world)]
    y, ctx = layer.forward_with_residuals(tok.cuda(), ids.cuda(), gates.cuda())
    d_tok, d_rhs, d_gates = layer.backward(dys[rank].cuda(), ctx)
    torch.cuda.synchronize()
    _capi.device_status()
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
    rel = lambda a, b: ((a.float().cpu() - b).abs().max() / (b.abs().max() + 1e-6)).item()
    q.put((rank, rel(d_tok, want_tok), rel(d_rhs, want_rhs), rel(d_gates, want_gates)))
  finally:
    dist.destroy_process_group()


def test_two_gpu_expert_parallel_backward():
  """d_tokens, d_rhs (local experts) and d_gates on 2 GPUs against autograd through a dense MoE
  over both ranks' tokens."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_bwd_worker, args=(r, 2, port, q)) for r in range(2)]
  for p in procs:
    p.start()
  results = [q.get(timeout=300) for _ in range(2)]
  for p in procs:
    p.join(timeout=120)
    assert p.exitcode == 0
  for rank, e_tok, e_rhs, e_gates in results:
    assert e_tok < 3e-2 and e_rhs < 3e-2 and e_gates < 3e-2, (rank, e_tok, e_rhs, e_gates)
