"""CPU oracle for the MoE dispatch / combine steps around ragged_dot.  TEST INFRASTRUCTURE ONLY
(imported by tests/ and nothing else).

Restates, in NumPy / torch on CPU:
* `sort_pairs_ref`   -- a stable sort of (token, choice) pairs by expert id and the per-expert
  histogram: what a caller of the reference does with `jnp.argsort` / `jnp.bincount` before
  `ragged_dot` (the reference itself has no dispatch op on GPU).
* `gather_rows_ref`  -- ragged_gather, `x[indices]`
  (tokamax/_src/ops/ragged_gather/base.py:26-30), written as a scatter by position.
* `combine_ref`      -- ragged_gather_reduce, a gate-weighted sum of each token's top-k rows
  in float32 (tokamax/_src/ops/ragged_gather_reduce/base.py:26-37).
* `ragged_gather_ref`, `ragged_scatter_ref`, `ragged_gather_reduce_ref` -- the three
  permutation ops with the reference's own signatures
  (tokamax/_src/ops/ragged_gather/base.py:26-30, ragged_scatter/base.py:26-36,
  ragged_gather_reduce/base.py:26-37).
* `cyclic_ragged_dot_ref` -- ragged dot where segment i uses rhs[i % G]; equals the plain
  oracle applied per segment.
Integer results (positions, counts) are exact by construction; parity of the float part is
unpinned (no stored reference outputs exist).
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import ragged_dot_ref as ref


def sort_pairs_ref(expert_ids: np.ndarray, num_experts: int):
  """Returns (pos int32 [P], counts int32 [E]): pos[p] = rank of pair p in a stable sort by
  expert id; ids outside [0, E) get -1 and are not counted."""
  ids = np.asarray(expert_ids).reshape(-1).astype(np.int64)
  valid = (ids >= 0) & (ids < num_experts)
  counts = np.bincount(ids[valid], minlength=num_experts).astype(np.int32)
  order = np.argsort(np.where(valid, ids, num_experts), kind="stable")
  pos = np.empty(ids.shape[0], np.int32)
  pos[order] = np.arange(ids.shape[0], dtype=np.int32)
  pos[~valid] = -1
  return pos, counts


def gather_rows_ref(src: torch.Tensor, pos: np.ndarray, top_k: int) -> torch.Tensor:
  out = torch.zeros((len(pos), src.shape[1]), dtype=src.dtype)
  for p, d in enumerate(pos):
    if d >= 0:
      out[d] = src[p // top_k]
  return out


def combine_ref(rows: torch.Tensor, pos: np.ndarray, gates: torch.Tensor, num_tokens: int,
                top_k: int) -> torch.Tensor:
  y = torch.zeros((num_tokens, rows.shape[1]), dtype=torch.float32)
  g = gates.reshape(num_tokens, top_k).float()
  for t in range(num_tokens):
    for k in range(top_k):
      d = pos[t * top_k + k]
      if d >= 0:
        y[t] += g[t, k] * rows[d].float()
  return y.to(rows.dtype)


def _index_rows(x: torch.Tensor, indices) -> torch.Tensor:
  """`x[indices]` with array-indexing rules: negative indices wrap once, the rest is clamped."""
  idx = torch.as_tensor(np.asarray(indices)).long()
  idx = torch.where(idx < 0, idx + x.shape[0], idx).clamp(0, x.shape[0] - 1)
  return x[idx]


def ragged_gather_ref(x: torch.Tensor, indices, start=None, end=None) -> torch.Tensor:
  """ragged_gather/base.py:26-30: start and end are ignored."""
  del start, end
  return _index_rows(x, indices)


def ragged_scatter_ref(x: torch.Tensor, indices, start, end) -> torch.Tensor:
  """ragged_scatter/base.py:26-36: rows whose index is outside [start, end) are zero."""
  idx = torch.as_tensor(np.asarray(indices)).long()
  lo, hi = int(np.asarray(start).reshape(-1)[0]), int(np.asarray(end).reshape(-1)[0])
  mask = (idx >= lo) & (idx < hi)
  return torch.where(mask[:, None], _index_rows(x, indices), torch.zeros((), dtype=x.dtype))


def ragged_gather_reduce_ref(x: torch.Tensor, indices, topk_weights, valid_rows_mask,
                             reduce_group_size: int) -> torch.Tensor:
  """ragged_gather_reduce/base.py:26-37: float32 products, masked, summed per group of
  `reduce_group_size` consecutive rows, cast to x.dtype."""
  out = _index_rows(x, indices).float() * torch.as_tensor(np.asarray(topk_weights)).float()[:, None]
  mask = torch.as_tensor(np.asarray(valid_rows_mask)).bool()
  out = torch.where(mask[:, None], out, torch.zeros(()))
  out = out.reshape(-1, reduce_group_size, out.shape[-1])
  return out.sum(dim=1).to(x.dtype)


def cyclic_ragged_dot_ref(rows: torch.Tensor, rhs: torch.Tensor, segment_sizes, out_dtype=None):
  seg = np.asarray(segment_sizes).astype(np.int64)
  g = rhs.shape[0]
  expanded = rhs[[i % g for i in range(len(seg))]]
  return ref.ragged_dot_ref(rows, expanded, seg, out_dtype=out_dtype)


def ep_plan_ref(counts_all: np.ndarray, rank: int) -> dict:
  """Offsets of one expert-parallel step as rank `rank` derives them from the all-gathered
  per-expert pair counts `counts_all` int [W, G] (experts sharded contiguously, G/W per rank).
  This layer has no counterpart in the reference; the layout it restates is the one declared in
  include/tokamax_b200.h: a rank's receive buffer is ordered (local expert, source rank), its
  return buffer holds its own pairs in expert-sorted order, rows are sent local-expert major.
  Returns the tables of the device plan under their names."""
  c = np.maximum(np.asarray(counts_all).astype(np.int64), 0)
  w, g = c.shape
  gl = g // w
  send_off_all = np.cumsum(c, 1) - c                       # [src, e]: src's first sorted position of e
  within = np.cumsum(c, 0) - c                             # [src, e]: rows of earlier sources, same expert
  per_expert = c.sum(0)                                    # [e]
  pe = per_expert.reshape(w, gl)
  expert_start = (np.cumsum(pe, 1) - pe).reshape(-1)       # first row of e in its owner's receive buffer
  mine = slice(rank * gl, (rank + 1) * gl)
  seg_start = np.empty((gl, w + 1), np.int64)
  seg_start[:, :w] = (expert_start[mine][None, :] + within[:, mine]).T
  seg_start[:, w] = expert_start[mine] + per_expert[mine]
  ret_off = send_off_all[:, mine].T                        # [local e, src]
  v_to_e = np.array([(v % w) * gl + v // w for v in range(g)])
  vcount = c[rank][v_to_e]
  vstart = np.concatenate([[0], np.cumsum(vcount)])
  i32 = lambda a: np.asarray(a, np.int32)
  return dict(group_sizes=i32(per_expert[mine]), vstart=i32(vstart), src_off=i32(send_off_all[rank][v_to_e]),
              dst_row=i32((expert_start + within[rank])[v_to_e]), seg_start=i32(seg_start), ret_off=i32(ret_off))


def ep_reference_words_ref(ids_all, num_experts: int) -> list:
  """Reference words of the once-per-rank dispatch (include/tokamax_b200.h,
  tkmx_ep_moe_fused_once_per_rank) for every rank's receive buffer.

  `ids_all`: per source rank an int array [T, top_k] of global expert ids (ids outside
  [0, num_experts) are dropped pairs).  Of a token's pairs on one REMOTE rank only the one with the
  lowest (expert, pair index) is shipped; the word of every other such row is
  (local expert of that original + 1) << 24 | the original's receive-buffer row, and 0 for rows
  that arrive themselves (originals, and every row a rank sends to itself).
  Returns per rank an int64 array over its used receive-buffer rows."""
  w = len(ids_all)
  g = num_experts
  gl = g // w
  counts = np.zeros((w, g), np.int64)
  sorted_pos = []
  for s, ids in enumerate(ids_all):
    pos, cnt = sort_pairs_ref(np.asarray(ids), g)
    sorted_pos.append(np.asarray(pos).reshape(-1))
    counts[s] = cnt
  per_expert = counts.sum(0)
  pe = per_expert.reshape(w, gl)
  expert_start = (np.cumsum(pe, 1) - pe).reshape(-1)
  within = np.cumsum(counts, 0) - counts
  send_off = np.cumsum(counts, 1) - counts
  out = [np.zeros(int(pe[d].sum()), np.int64) for d in range(w)]

  def recv_row(s, pair, e):
    return int(expert_start[e] + within[s, e] + sorted_pos[s][pair] - send_off[s, e])

  for s, ids in enumerate(ids_all):
    ids = np.asarray(ids)
    t, top_k = ids.shape
    for tok in range(t):
      for j in range(top_k):
        e = int(ids[tok, j])
        if e < 0 or e >= g:
          continue
        d = e // gl
        if d == s:
          continue
        pair = tok * top_k + j
        best = min((int(ids[tok, jj]), tok * top_k + jj) for jj in range(top_k)
                   if 0 <= int(ids[tok, jj]) < g and int(ids[tok, jj]) // gl == d)
        if best[1] != pair:
          out[d][recv_row(s, pair, e)] = ((best[0] - d * gl + 1) << 24) | recv_row(s, best[1], best[0])
  return out
