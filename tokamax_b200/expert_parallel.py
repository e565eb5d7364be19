"""Expert-parallel MoE layer: dispatch all-to-all -> local grouped GEMM -> combine all-to-all.

The reference has no such layer (sharding is the caller's `shard_map`; its only
expert-parallel affordances are `group_offset` / `num_actual_groups`,
tokamax/_src/ops/ragged_dot/pallas_mosaic_tpu_kernel.py:85-86,
pallas_mosaic_tpu_v2.py:89-93).  This is the caller side for one process per GPU over
`torch.distributed` (NCCL over NVLink): experts are sharded contiguously, rank r owns
experts [r*G/W, (r+1)*G/W).

Per call on every rank:
  1. counting sort of the (token, choice) pairs by expert id      (kernel: moe_sort_pairs)
  2. all-to-all of the per-expert counts int32[W, G/W]
  3. pack token rows in expert order                              (kernel: moe_gather_rows)
  4. all-to-all of the rows; they land ordered (source rank, local expert)
  5. grouped GEMM over those segments as they lie, segment i using expert i % (G/W)
                                                                  (kernel: ragged_dot_fwd_cyclic)
  6. reverse all-to-all of the output rows (no reorder needed either way)
  7. per token: sum_k gate_k * y_k in float32                     (kernel: moe_combine)

The split sizes of the row exchanges are host integers (all_to_all_single wants lists), so
step 2 ends with one device-to-host read per call.

With `exchange="fused"` (the default on CUDA tensors) steps 2-6 are three launches with no
collective-library call and no device-to-host read: every rank holds a receive buffer and a
return buffer in peer-mapped ("symmetric") memory; `tkmx_ep_exchange_plan` all-gathers the
counts through peer stores, passes a bounded flag barrier and derives every offset of the step
on the device; `tkmx_ep_moe_fused` is ONE kernel in which two warps of every CTA push this
rank's token rows into the owners' receive buffers (plain stores over NVLink, expert by
expert, with per-expert arrival counters) while the other warps multiply the experts whose
rows have arrived and store each finished row straight into its source rank's return buffer;
`tkmx_cross_rank_barrier` ends the step.  `exchange="nccl"` keeps the all-to-all form
described above.

`forward_with_residuals` / `backward` give the layer's gradients through the all-to-all
exchange: cotangent rows travel to the experts' owners, dlhs rows travel back, drhs stays local.

The compute steps go through a small backend object; the default one calls the CUDA
kernels and has no other path.  Tests that run the exchange logic on CPU ranks (gloo)
pass their own backend.
"""

from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist


class CudaBackend:
  """Steps 1, 3, 5, 7 on the B200 kernels (C ABI of include/tokamax_b200.h)."""

  def __init__(self, config=None, reserve_sms: int = 0):
    """config: a `_capi.Config` for the grouped GEMM, or None for a size-based choice.
    reserve_sms: leave this many SMs free of the persistent GEMM kernel, so that
    communication kernels running beside it are not starved of SMs."""
    from tokamax_b200 import _capi
    self._capi = _capi
    self._config = config
    self._reserve_sms = reserve_sms
    _capi.load()

  def _gemm_config(self, rows: int, segments: int, n: int):
    if self._config is not None:
      return self._config
    # CTA pairs (256-row tiles) once the average segment fills most of a pair tile.
    pair = n >= 128 and segments > 0 and rows / segments >= 192
    cfg = self._capi.Config(collective=1 if pair else 0)
    if self._reserve_sms:
      sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
      cfg.max_ctas = max(2, (sms - self._reserve_sms) // 2 * 2)
    return cfg

  def sort_pairs(self, expert_ids: torch.Tensor, num_experts: int):
    ids = expert_ids.reshape(-1)
    if ids.dtype != torch.int32:
      ids = ids.to(torch.int32)
    return self._capi.moe_sort_pairs(ids.contiguous(), num_experts)

  def gather_rows(self, tokens: torch.Tensor, pos: torch.Tensor, top_k: int) -> torch.Tensor:
    return self._capi.moe_gather_rows(tokens.contiguous(), pos, top_k)

  def expert_gemm(self, rows: torch.Tensor, rhs_local: torch.Tensor, segment_sizes: torch.Tensor):
    out = torch.empty((rows.shape[0], rhs_local.shape[2]), dtype=rows.dtype, device=rows.device)
    self._capi.ragged_dot_fwd_cyclic(
        rows, rhs_local, segment_sizes, out,
        config=self._gemm_config(rows.shape[0], segment_sizes.numel(), rhs_local.shape[2]))
    return out

  def combine(self, rows: torch.Tensor, pos: torch.Tensor, gates: torch.Tensor, num_tokens: int,
              top_k: int) -> torch.Tensor:
    return self._capi.moe_combine(rows, pos, gates.to(torch.float32).contiguous(), num_tokens, top_k)

  def expert_gemm_dlhs(self, dout_rows: torch.Tensor, rhs_local: torch.Tensor, segment_sizes: torch.Tensor):
    """d(rows)[i, :] = dout_rows[i, :] @ rhs_local[expert(i)]^T over the same segments: the
    forward kernel with the weights read as stored ([G, K, N] is "[G, n_out, contraction]")."""
    out = torch.empty((dout_rows.shape[0], rhs_local.shape[1]), dtype=dout_rows.dtype, device=dout_rows.device)
    self._capi.ragged_dot_fwd_cyclic(
        dout_rows, rhs_local, segment_sizes, out, rhs_layout=self._capi.RHS_GNK,
        config=self._gemm_config(dout_rows.shape[0], segment_sizes.numel(), rhs_local.shape[1]))
    return out

  def expert_gemm_drhs(self, rows: torch.Tensor, dout_rows: torch.Tensor, segment_sizes: torch.Tensor,
                       local_experts: int):
    """d(rhs_local)[e] = sum over the segments of expert e of rows^T @ dout_rows, float32."""
    seg = torch.empty((segment_sizes.numel(), rows.shape[1], dout_rows.shape[1]), dtype=torch.float32,
                      device=rows.device)
    self._capi.ragged_dot_drhs(rows, dout_rows, segment_sizes, seg)
    return seg.reshape(-1, local_experts, rows.shape[1], dout_rows.shape[1]).sum(0)


@dataclasses.dataclass
class DispatchPlan:
  """What `combine` needs to undo `dispatch`."""

  pos: torch.Tensor             # int32 [T*top_k]: position of each pair in expert-sorted order
  send_splits: list[int]        # rows sent to each rank
  recv_splits: list[int]        # rows received from each rank
  segment_sizes: torch.Tensor   # int32 [W * G/W]: rows per (source rank, local expert)
  num_tokens: int
  top_k: int
  local_group_sizes: torch.Tensor | None = None   # int32 [G/W] when the exchange computed it itself

  @property
  def group_sizes(self) -> torch.Tensor:
    """Rows per local expert (the column sums of the received [source, expert] counts)."""
    if self.local_group_sizes is not None:
      return self.local_group_sizes
    w = len(self.recv_splits)
    return self.segment_sizes.reshape(w, -1).sum(0).to(torch.int32)


class ExpertParallelMoE:
  """One expert-parallel grouped-GEMM layer.

  Args:
    rhs_local: this rank's expert weights [G/W, K, N].
    num_experts: global expert count G.
    group: process group (default: the world).
    backend: object with sort_pairs / gather_rows / expert_gemm / combine (default: CudaBackend).
    num_chunks: with more than one rank, cut the local experts into this many chunks and
      overlap each chunk's exchanges with the neighbouring chunks' GEMMs (1 = no overlap).
  """

  def __init__(self, rhs_local: torch.Tensor, num_experts: int, group=None, backend=None,
               num_chunks: int = 4, exchange: str | None = None):
    self.group = group
    self.num_chunks = num_chunks
    self._fused = None
    self._seq = 0
    self.gemm_config = None          # a `_capi.Config` for the fused kernel's GEMM, or None for a size-based choice
    # Fused exchange: send a token once per destination RANK and let the owner copy the rows of
    # its other experts there.  None = whenever there is more than one rank and the sizes fit
    # the reference words (measured on 4 GPUs: 2.06 against 2.26 ms per step); set before the
    # first call.
    self.once_per_rank = None
    self.timeout_ns = 2_000_000_000  # budget of every cross-rank flag wait
    self.gemm_events = None          # set to a list to collect (start, end) CUDA events around the grouped GEMM
    self.launches_last_call = 0      # kernels of this library launched by the last call
    self.world = dist.get_world_size(group) if dist.is_initialized() else 1
    self.rank = dist.get_rank(group) if dist.is_initialized() else 0
    if num_experts % self.world:
      raise ValueError("num_experts must be divisible by the world size")
    self.num_experts = num_experts
    self.local_experts = num_experts // self.world
    if rhs_local.shape[0] != self.local_experts:
      raise ValueError(f"rhs_local must hold {self.local_experts} experts, got {rhs_local.shape[0]}")
    self.rhs_local = rhs_local
    if exchange is None:
      exchange = "fused" if (backend is None and rhs_local.is_cuda) else "nccl"
    if exchange not in ("fused", "nccl"):
      raise ValueError("exchange must be 'fused' or 'nccl'")
    if exchange == "fused" and backend is not None:
      raise ValueError("the fused exchange runs on the CUDA kernels only")
    self.exchange = exchange
    if backend is None:
      # With overlapped NCCL exchanges, keep a few SMs free for the communication kernels.
      reserve = 20 if (self.world > 1 and num_chunks > 1 and exchange == "nccl") else 0
      backend = CudaBackend(reserve_sms=reserve)
    self.backend = backend

  def _all_to_all(self, out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits):
    if self.world == 1:
      out.copy_(inp)
    else:
      dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

  def _exchange_async(self, outs: list, ins: list):
    """Asynchronous all-to-all of per-peer tensor views (ins[d] goes to rank d, outs[s] comes
    from rank s) as one batch of point-to-point operations; returns the work handles."""
    outs[self.rank].copy_(ins[self.rank])
    ops = []
    for peer in range(self.world):
      if peer == self.rank:
        continue
      if ins[peer].numel():
        ops.append(dist.P2POp(dist.isend, ins[peer], dist.get_global_rank(self.group, peer)
                              if self.group is not None else peer, self.group))
      if outs[peer].numel():
        ops.append(dist.P2POp(dist.irecv, outs[peer], dist.get_global_rank(self.group, peer)
                              if self.group is not None else peer, self.group))
    return dist.batch_isend_irecv(ops) if ops else []

  def _check_counts(self, sent: torch.Tensor, received: torch.Tensor, num_pairs: int) -> None:
    """Refuses a step whose exchanged counts cannot be right, on every rank at once (the
    verdict is all-reduced, so no rank walks into a row exchange the others have left):
    a negative count, a total that differs from this rank's number of routed pairs (rows
    dropped or invented by the sort), or rows announced as sent that nobody announces as received.  `sent` / `received` are host int tensors
    [W, G/W] (what this rank sends to / receives from each rank, per local expert)."""
    bad = int(sent.min()) < 0 or int(received.min()) < 0 or int(sent.sum()) != num_pairs
    totals = torch.tensor([int(sent.sum()), int(received.sum()), 1 if bad else 0], dtype=torch.int64)
    if self.world > 1:
      totals = totals.to(self.rhs_local.device)
      dist.all_reduce(totals, group=self.group)
      totals = totals.cpu()
    if int(totals[2]) != 0 or int(totals[0]) != int(totals[1]):
      raise RuntimeError(
          "expert-parallel dispatch: inconsistent per-expert counts across ranks "
          f"(rows announced as sent {int(totals[0])}, as received {int(totals[1])}, "
          f"ranks with invalid counts {int(totals[2])}); the step was not run")

  def dispatch(self, tokens: torch.Tensor, expert_ids: torch.Tensor):
    """Returns (rows [R, K] in (source rank, local expert) order, DispatchPlan)."""
    t, top_k = expert_ids.shape
    w, gl = self.world, self.local_experts
    pos, counts = self.backend.sort_pairs(expert_ids, self.num_experts)
    counts = counts.reshape(w, gl)                         # [dest rank, expert]
    recv_counts = torch.empty_like(counts)                 # [source rank, expert]
    self._all_to_all(recv_counts, counts, None, None)
    valid = ((expert_ids >= 0) & (expert_ids < self.num_experts)).sum().reshape(1, 1).expand(1, gl).to(counts.dtype)
    host_counts = torch.cat([counts, recv_counts, valid]).cpu()     # the one host read
    self._check_counts(host_counts[:w], host_counts[w:2 * w], int(host_counts[2 * w, 0]))
    send_splits = [int(v) for v in host_counts[:w].sum(1)]
    recv_splits = [int(v) for v in host_counts[w:2 * w].sum(1)]
    packed = self.backend.gather_rows(tokens, pos, top_k)  # expert order == (dest rank, expert)
    if w == 1:
      recv = packed
    else:
      recv = torch.empty((sum(recv_splits), tokens.shape[1]), dtype=tokens.dtype, device=tokens.device)
      self._all_to_all(recv, packed, recv_splits, send_splits)
    plan = DispatchPlan(pos, send_splits, recv_splits, recv_counts.reshape(-1).to(torch.int32).contiguous(),
                        t, top_k)
    return recv, plan

  def combine(self, out_rows: torch.Tensor, gates: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
    if self.world == 1:
      ret = out_rows
    else:
      ret = torch.empty((plan.num_tokens * plan.top_k, out_rows.shape[1]), dtype=out_rows.dtype,
                        device=out_rows.device)
      self._all_to_all(ret, out_rows, plan.send_splits, plan.recv_splits)
    return self.backend.combine(ret, plan.pos, gates, plan.num_tokens, plan.top_k)

  @property
  def exchange_name(self) -> str:
    if self.exchange == "fused":
      if self._fused is not None and self._fused["once"]:
        return "fused (peer stores inside the GEMM kernel; a token crosses to a rank once)"
      return "fused (peer stores inside the GEMM kernel)"
    return "nccl all-to-all" if self.world > 1 else "local (gather, GEMM, combine)"

  @property
  def gemm_kernel_name(self) -> str:
    if self.exchange == "fused":
      return "tkmx::ragged_gemm_kernel<kRowsBN, 256, pair, expert-parallel>"
    return "tkmx::ragged_gemm_kernel<kRowsBN, 256, pair>"

  def check_overflow(self) -> None:
    """Raises if a kernel of an earlier call reported a problem (a timed-out cross-rank wait, a
    row aimed outside a receive buffer).  Synchronises the device."""
    from tokamax_b200 import _capi
    _capi.device_status()

  def _gemm_bracket(self):
    """(start, end) events of the current stream when `gemm_events` collects them."""
    if self.gemm_events is None:
      return None
    pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    self.gemm_events.append(pair)
    return pair

  def __call__(self, tokens: torch.Tensor, expert_ids: torch.Tensor, gates: torch.Tensor):
    if self.exchange == "fused":
      return self.forward_fused(tokens, expert_ids, gates)
    if self.world > 1 and self.num_chunks > 1:
      return self.forward_pipelined(tokens, expert_ids, gates)
    rows, plan = self.dispatch(tokens, expert_ids)
    ev = self._gemm_bracket()
    if ev:
      ev[0].record()
    out_rows = self.backend.expert_gemm(rows, self.rhs_local, plan.segment_sizes)
    if ev:
      ev[1].record()
    self.launches_last_call = 6     # 3 sort + gather + GEMM + combine
    return self.combine(out_rows, gates, plan), plan

  # ------------------------------------------------------------------ backward
  def forward_with_residuals(self, tokens: torch.Tensor, expert_ids: torch.Tensor, gates: torch.Tensor):
    """The layer through the all-to-all exchange (no chunking), keeping what `backward` needs:
    the received rows, the returned expert outputs and the dispatch plan."""
    rows, plan = self.dispatch(tokens, expert_ids)
    out_rows = self.backend.expert_gemm(rows, self.rhs_local, plan.segment_sizes)
    if self.world == 1:
      ret = out_rows
    else:
      ret = torch.empty((plan.num_tokens * plan.top_k, out_rows.shape[1]), dtype=out_rows.dtype,
                        device=out_rows.device)
      self._all_to_all(ret, out_rows, plan.send_splits, plan.recv_splits)
    y = self.backend.combine(ret, plan.pos, gates, plan.num_tokens, plan.top_k)
    return y, dict(rows=rows, ret=ret, plan=plan, gates=gates)

  def backward(self, dy: torch.Tensor, ctx: dict):
    """Gradients of y = sum_k gate_k * (token @ rhs[expert_k]) given dy [T, N].

    Shards like the forward: the gate-weighted cotangent rows travel to the experts' owners
    (same splits as the dispatch), dlhs rows travel back and are summed per token, drhs stays
    local.  Returns (d_tokens [T, K], d_rhs_local [G/W, K, N] float32, d_gates [T, top_k]
    float32).  Row bookkeeping outside the GEMMs (gate scaling, the permutation by `pos`) is
    done with torch indexing on the device."""
    plan, gates, rows, ret = ctx["plan"], ctx["gates"], ctx["rows"], ctx["ret"]
    t, top_k = plan.num_tokens, plan.top_k
    pos = plan.pos.long()
    token_of = torch.arange(t * top_k, device=dy.device) // top_k
    valid = pos >= 0
    # d(ret)[pos[p]] = gate[p] * dy[token(p)];  d(gate)[p] = <ret[pos[p]], dy[token(p)]>
    g_flat = gates.reshape(-1).to(torch.float32)
    d_ret = torch.zeros((t * top_k, dy.shape[1]), dtype=ret.dtype, device=dy.device)
    d_ret[pos[valid]] = (g_flat[valid, None] * dy[token_of[valid]].float()).to(ret.dtype)
    d_gates = torch.zeros(t * top_k, dtype=torch.float32, device=dy.device)
    d_gates[valid] = (ret[pos[valid]].float() * dy[token_of[valid]].float()).sum(1)
    # cotangent rows to the owners: the forward's return exchange run backwards
    if self.world == 1:
      d_out_rows = d_ret
    else:
      d_out_rows = torch.empty((sum(plan.recv_splits), dy.shape[1]), dtype=d_ret.dtype, device=dy.device)
      self._all_to_all(d_out_rows, d_ret, plan.recv_splits, plan.send_splits)
    d_rows = self.backend.expert_gemm_dlhs(d_out_rows, self.rhs_local, plan.segment_sizes)
    d_rhs = self.backend.expert_gemm_drhs(rows, d_out_rows, plan.segment_sizes, self.local_experts)
    # dlhs rows back to the tokens' ranks, summed per token
    if self.world == 1:
      d_packed = d_rows
    else:
      d_packed = torch.empty((t * top_k, d_rows.shape[1]), dtype=d_rows.dtype, device=dy.device)
      self._all_to_all(d_packed, d_rows, plan.send_splits, plan.recv_splits)
    ones = torch.ones(t * top_k, dtype=torch.float32, device=dy.device)
    d_tokens = self.backend.combine(d_packed, plan.pos, ones, t, top_k)
    return d_tokens, d_rhs, d_gates.reshape(t, top_k)

  # ------------------------------------------------------------------ pipelined form
  def forward_pipelined(self, tokens: torch.Tensor, expert_ids: torch.Tensor, gates: torch.Tensor):
    """Same result as dispatch -> GEMM -> combine, with the local experts cut into
    `num_chunks` chunks: while chunk c is multiplied, the rows of chunk c+1 are already
    arriving and the outputs of chunk c-1 are already leaving (asynchronous all-to-alls on
    the communication stream), so only the first and last exchange are exposed."""
    t, top_k = expert_ids.shape
    w, gl = self.world, self.local_experts
    chunks = min(self.num_chunks, gl)
    while gl % chunks:
      chunks -= 1
    ce = gl // chunks
    pos, counts = self.backend.sort_pairs(expert_ids, self.num_experts)
    counts = counts.reshape(w, gl)
    recv_counts = torch.empty_like(counts)
    self._all_to_all(recv_counts, counts, None, None)
    valid = ((expert_ids >= 0) & (expert_ids < self.num_experts)).sum().reshape(1, 1).expand(1, gl).to(counts.dtype)
    host_all = torch.cat([counts, recv_counts, valid]).cpu()        # the one host read
    host = torch.stack([host_all[:w], host_all[w:2 * w]])
    self._check_counts(host[0], host[1], int(host_all[2 * w, 0]))
    send_c = host[0].reshape(w, chunks, ce).sum(2)                   # [dest, chunk] rows
    recv_c = host[1].reshape(w, chunks, ce).sum(2)                   # [src, chunk] rows
    send_off = (host[0].reshape(-1).cumsum(0) - host[0].reshape(-1)).reshape(w, gl)  # packed-row offsets
    packed = self.backend.gather_rows(tokens, pos, top_k)
    k = tokens.shape[1]
    n = self.rhs_local.shape[2]
    ret = torch.empty((t * top_k, n), dtype=tokens.dtype, device=tokens.device)

    def send_views(buf, c):
      return [buf[int(send_off[d, c * ce]): int(send_off[d, c * ce]) + int(send_c[d, c])] for d in range(w)]

    def start_dispatch(c):
      rows = torch.empty((int(recv_c[:, c].sum()), k), dtype=tokens.dtype, device=tokens.device)
      outs = list(rows.split([int(v) for v in recv_c[:, c]]))
      return rows, self._exchange_async(outs, send_views(packed, c))

    inflight = start_dispatch(0)
    back = []
    seg_all = recv_counts.to(torch.int32).reshape(w, chunks, ce)
    for c in range(chunks):
      rows, works = inflight
      if c + 1 < chunks:
        inflight = start_dispatch(c + 1)        # enqueued before this chunk's GEMM
      for wk in works:
        wk.wait()
      seg = seg_all[:, c, :].reshape(-1).contiguous()
      out_rows = self.backend.expert_gemm(rows, self.rhs_local[c * ce:(c + 1) * ce], seg)
      ins = list(out_rows.split([int(v) for v in recv_c[:, c]]))
      back.append((self._exchange_async(send_views(ret, c), ins), out_rows, rows))
    for works, _, _ in back:
      for wk in works:
        wk.wait()
    y = self.backend.combine(ret, pos, gates, t, top_k)
    plan = DispatchPlan(pos, [int(v) for v in host[0].sum(1)], [int(v) for v in host[1].sum(1)],
                        recv_counts.reshape(-1).to(torch.int32).contiguous(), t, top_k)
    return y, plan

  # ------------------------------------------------------------------ fused form
  def _fused_state(self, tokens: torch.Tensor, top_k: int):
    """Buffers of the fused exchange, allocated once per (token count, top_k, row widths): the
    receive buffer is sized for the worst case (every pair of every rank routed here), the
    return buffer for this rank's own pairs.  With more than one rank they live in peer-mapped
    ("symmetric") memory and every rank learns every rank's addresses."""
    from tokamax_b200 import _capi
    t, k = tokens.shape
    n = self.rhs_local.shape[2]
    fits = self.local_experts <= 254 and self.world * t * top_k <= 1 << 24
    if self.once_per_rank and self.world > 1 and not fits:
      raise NotImplementedError("once_per_rank serves up to 254 local experts and 2^24 receive-buffer rows")
    once = self.world > 1 and fits and self.once_per_rank is not False
    key = (t, top_k, k, n, tokens.dtype, once)
    if self._fused is not None and self._fused["key"] == key:
      return self._fused
    dev = tokens.device
    w, g, gl = self.world, self.num_experts, self.local_experts
    if w > _capi.EP_MAX_WORLD:
      raise NotImplementedError(f"the fused exchange serves up to {_capi.EP_MAX_WORLD} ranks")
    pairs = t * top_k
    cap = w * pairs
    shapes = dict(recv=((cap, k), tokens.dtype), arrive=((_capi.ep_arrive_words(g, w, once),), torch.int32),
                  ret=((pairs, n), tokens.dtype), counts=((w, g), torch.int32), flags=((w,), torch.int32))
    if once:
      shapes["refs"] = ((cap,), torch.int32)
    bufs, ptrs = {}, {}
    if w > 1:
      import torch.distributed._symmetric_memory as symm_mem
      group = self.group if self.group is not None else dist.group.WORLD
      for name, (shape, dtype) in shapes.items():
        bufs[name] = symm_mem.empty(shape, dtype=dtype, device=dev)
        if name in ("arrive", "counts", "flags"):
          bufs[name].zero_()
        ptrs[name] = [int(p) for p in symm_mem.rendezvous(bufs[name], group).buffer_ptrs]
      torch.cuda.synchronize(dev)
      dist.barrier(group)     # every rank's flags are zero before anyone's first step
    else:
      for name, (shape, dtype) in shapes.items():
        bufs[name] = torch.zeros(shape, dtype=dtype, device=dev) if name != "recv" else torch.empty(
            shape, dtype=dtype, device=dev)
        ptrs[name] = [bufs[name].data_ptr()]
    table = torch.zeros((_capi.EP_TAB_ROWS, _capi.EP_MAX_WORLD), dtype=torch.int64)
    for row, name in ((_capi.EP_TAB_RECV, "recv"), (_capi.EP_TAB_ARRIVE, "arrive"), (_capi.EP_TAB_RET, "ret"),
                      (_capi.EP_TAB_COUNTS, "counts"), (_capi.EP_TAB_FLAGS, "flags"), (_capi.EP_TAB_REFS, "refs")):
      if name not in bufs:
        continue
      for r in range(w):
        # addresses above 2^63 would not fit int64: CUDA virtual addresses are far below
        table[row, r] = ptrs[name][r]
    self._fused = dict(
        key=key, cap=cap, bufs=bufs, table=table.to(dev), once=once,
        plan=torch.zeros(_capi.ep_plan_ints(g, w), dtype=torch.int32, device=dev),
        pos=torch.empty(pairs, dtype=torch.int32, device=dev),
        sorted_pair=torch.zeros(pairs, dtype=torch.int32, device=dev),
        my_counts=torch.empty(g, dtype=torch.int32, device=dev),
        sort_ws=torch.empty(max(_capi.moe_sort_workspace_bytes(pairs, g), 4), dtype=torch.uint8, device=dev))
    return self._fused

  def _fused_config(self, pairs: int):
    from tokamax_b200 import _capi
    if self.gemm_config is not None:
      return self.gemm_config
    # CTA pairs (256-row tiles) once the average expert fills most of a pair tile.
    mean_rows = pairs * self.world / max(self.local_experts, 1)
    return _capi.Config(collective=1 if mean_rows >= 192 else 0)

  def forward_fused(self, tokens: torch.Tensor, expert_ids: torch.Tensor, gates: torch.Tensor,
                    phases: tuple[int, ...] = (3,)):
    """sort -> counts exchange + plan -> ONE kernel that sends this rank's rows, multiplies what
    has arrived and returns finished rows -> barrier -> gate-weighted combine.  Seven launches,
    no host read, no collective-library call.

    The returned plan's `pos` aliases a buffer that the next call overwrites.  `phases` splits
    the fused kernel into launches of its parts, (1, 2) = send everything, then multiply (a
    cross-rank barrier is put between them): the form the tests use to tell the two halves
    apart."""
    from tokamax_b200 import _capi
    if not tokens.is_cuda:
      raise NotImplementedError("the fused exchange runs on CUDA tensors only (no CPU fallback)")
    t, top_k = expert_ids.shape
    st = self._fused_state(tokens, top_k)
    w, g = self.world, self.num_experts
    b = st["bufs"]
    ids = expert_ids.reshape(-1)
    if ids.dtype != torch.int32:
      ids = ids.to(torch.int32)
    tokens = tokens.contiguous()
    _capi.moe_sort_pairs_inverse(ids.contiguous(), g, st["pos"], st["sorted_pair"], st["my_counts"], st["sort_ws"])
    self._seq += 1
    once = st["once"]
    ids = ids.contiguous()
    _capi.ep_exchange_plan(st["my_counts"], st["table"], b["counts"], b["flags"], b["arrive"], st["plan"], g, w,
                           self.rank, self._seq, self.timeout_ns, once_per_rank=once)
    cfg = self._fused_config(t * top_k)
    n = self.rhs_local.shape[2]
    launches = 3 + 1
    ev = self._gemm_bracket()
    if ev:
      ev[0].record()
    for i, ph in enumerate(phases):
      if i > 0:
        self._seq += 1
        _capi.cross_rank_barrier(st["table"], b["flags"], w, self.rank, self._seq, self.timeout_ns)
        launches += 1
      if once:   # the product form also copies duplicates (bit 2); a multiply-only launch copies first
        ph = 7 if ph == 3 else (6 if ph == 2 else ph)
      _capi.ep_moe_fused(tokens, st["sorted_pair"], b["recv"], self.rhs_local, st["plan"], st["table"],
                         b["arrive"], top_k, g, w, self.rank, n, phases=ph, config=cfg,
                         expert_ids=ids if once else None, pair_pos=st["pos"] if once else None)
      launches += 1
    if ev:
      ev[1].record()
    self._seq += 1
    _capi.cross_rank_barrier(st["table"], b["flags"], w, self.rank, self._seq, self.timeout_ns)
    y = self.backend.combine(b["ret"], st["pos"], gates, t, top_k)
    self.launches_last_call = launches + 2
    plan = DispatchPlan(st["pos"], [], [0] * w, st["plan"][:0], t, top_k,
                        local_group_sizes=st["plan"][:self.local_experts])
    return y, plan


class HostPipeline:
  """The layer on PINNED HOST buffers, step after step: tokens, routing and gates are copied to
  the device, the layer runs, the result is copied back -- with the copies of one step running
  beside the computation of its neighbours (a copy-in stream, the caller's stream, a copy-out
  stream; `depth` device staging slots).  A serving loop calls `submit` once per step and reads
  a step's output after waiting for the event `submit` returned (or after `drain`).

  Nothing is skipped: every step's inputs cross PCIe in that step and its output is written to
  host memory; what the pipeline removes is the idle time of the copy engines while the GPU
  computes and of the GPU while they copy."""

  def __init__(self, layer: ExpertParallelMoE, depth: int = 2):
    if depth < 1:
      raise ValueError("depth must be at least 1")
    self.layer = layer
    self.depth = depth
    self._slots = None
    self._next = 0
    self._copy_in = None
    self._copy_out = None

  def _make_slots(self, h_tok, h_ids, h_gates):
    dev = self.layer.rhs_local.device
    self._copy_in = torch.cuda.Stream(device=dev)
    self._copy_out = torch.cuda.Stream(device=dev)
    self._slots = []
    for _ in range(self.depth):
      self._slots.append(dict(
          tok=torch.empty(h_tok.shape, dtype=h_tok.dtype, device=dev),
          ids=torch.empty(h_ids.shape, dtype=h_ids.dtype, device=dev),
          gates=torch.empty(h_gates.shape, dtype=h_gates.dtype, device=dev),
          in_ready=torch.cuda.Event(), computed=torch.cuda.Event(), out_done=torch.cuda.Event(), used=False))

  def submit(self, h_tok: torch.Tensor, h_ids: torch.Tensor, h_gates: torch.Tensor, h_out: torch.Tensor):
    """Enqueues one step; returns the CUDA event after which `h_out` holds its result."""
    for h in (h_tok, h_ids, h_gates, h_out):
      if h.is_cuda or not h.is_pinned():
        raise ValueError("HostPipeline takes pinned host tensors")
    if self._slots is None or self._slots[0]["tok"].shape != h_tok.shape or self._slots[0]["ids"].shape != h_ids.shape:
      self.drain()
      self._make_slots(h_tok, h_ids, h_gates)
    slot = self._slots[self._next % self.depth]
    self._next += 1
    main = torch.cuda.current_stream(self.layer.rhs_local.device)
    if slot["used"]:
      self._copy_in.wait_event(slot["computed"])     # the step that last read this slot is done with it
    with torch.cuda.stream(self._copy_in):
      slot["tok"].copy_(h_tok, non_blocking=True)
      slot["ids"].copy_(h_ids, non_blocking=True)
      slot["gates"].copy_(h_gates, non_blocking=True)
      slot["in_ready"].record(self._copy_in)
    main.wait_event(slot["in_ready"])
    y, _ = self.layer(slot["tok"], slot["ids"], slot["gates"])
    slot["computed"].record(main)
    slot["used"] = True
    self._copy_out.wait_event(slot["computed"])
    with torch.cuda.stream(self._copy_out):
      h_out.copy_(y, non_blocking=True)
      slot["out_done"].record(self._copy_out)
    y.record_stream(self._copy_out)
    return slot["out_done"]

  def drain(self) -> None:
    """Waits until every submitted step's output is in host memory."""
    for s in (self._copy_in, self._copy_out):
      if s is not None:
        s.synchronize()
