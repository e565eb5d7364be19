"""The sort entry point that brings its own scratch (`tkmx_moe_sort_pairs_static`).

It exists for hosts that cannot obtain device memory when the call is made -- a server that
gave all of it to its own arena at start-up, a custom-call handler that was handed no
scratch buffer -- so it takes no workspace and allocates nothing.  The check: through the C
ABI it returns exactly what `tkmx_moe_sort_pairs` returns with a caller workspace, on two
calls in a row (the built-in scratch is reused, with whatever the first call left in it),
and it refuses sizes beyond its fixed scratch with a clear error instead of running.

Collected last on purpose, so a failure here cannot hide the other tests' results.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ids(num_pairs, num_experts, seed):
  rng = np.random.default_rng(seed)
  p = rng.random(num_experts) ** 2
  return torch.from_numpy(rng.choice(num_experts, num_pairs, p=p / p.sum()).astype(np.int32)).cuda()


def test_static_scratch_sort_matches_workspace_sort_twice_in_a_row():
  from tokamax_b200 import _capi
  _capi.load()
  # two different problems back to back: the second one sees the first one's leftovers
  for num_pairs, num_experts, seed in ((65536, 256, 0), (40000, 1000, 1)):
    ids = _ids(num_pairs, num_experts, seed)
    want_pos, want_counts = _capi.moe_sort_pairs(ids, num_experts)
    pos = torch.full((num_pairs,), -7, dtype=torch.int32, device="cuda")
    counts = torch.full((num_experts,), -7, dtype=torch.int32, device="cuda")
    # Warm-up call: the first call on a device looks up the scratch array's address (and, in a
    # fresh process, is when CUDA loads the library image onto the device).
    _capi.moe_sort_pairs_static(ids, num_experts, pos, counts)
    torch.cuda.synchronize()
    pos.fill_(-7)
    counts.fill_(-7)
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    _capi.moe_sort_pairs_static(ids, num_experts, pos, counts)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before      # nothing was taken from torch's pool
    assert free_after >= free_before                    # ... and nothing from the device behind its back
    assert torch.equal(pos, want_pos)
    assert torch.equal(counts, want_counts)
    # immediately again, same inputs: identical
    pos2 = torch.empty_like(pos)
    counts2 = torch.empty_like(counts)
    _capi.moe_sort_pairs_static(ids, num_experts, pos2, counts2)
    torch.cuda.synchronize()
    assert torch.equal(pos2, want_pos) and torch.equal(counts2, want_counts)
  _capi.device_status()


def test_static_scratch_sort_refuses_sizes_beyond_its_scratch():
  from tokamax_b200 import _capi
  # ceil(600000 / 1024) * 1024 experts = 600064 entries > 262144
  ids = torch.zeros(600000, dtype=torch.int32, device="cuda")
  pos = torch.empty(600000, dtype=torch.int32, device="cuda")
  counts = torch.empty(1024, dtype=torch.int32, device="cuda")
  with pytest.raises(NotImplementedError, match="built-in scratch"):
    _capi.moe_sort_pairs_static(ids, 1024, pos, counts)
  # the same size is fine with a caller workspace
  p2, c2 = _capi.moe_sort_pairs(ids, 1024)
  assert int(c2[0]) == 600000 and torch.equal(p2, torch.arange(600000, dtype=torch.int32, device="cuda"))
