"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle.

Cases follow the reference's shared ragged-dot test-suite
(tokamax/_src/ops/ragged_dot/test_base.py:152-344) and the ragged group patterns of its
Blackwell kernel tests (pallas_mosaic_gpu_kernel_sm100_fp8_quant_test.py:317-328).
Tolerance for bf16 inputs with fp32 accumulation: max abs/rel error 2e-2; integer
bookkeeping: bit-exact.
"""

import json
import os

import numpy as np
import pytest
import torch

from oracle import ragged_dot_ref as ref
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
  from tokamax_b200 import _capi
  _capi.load()  # fails loudly if the CUDA library has not been built
  assert torch.cuda.is_available()
  return _capi


@pytest.fixture(scope="module")
def tk():
  import tokamax_b200
  return tokamax_b200


def _dev(*ts):
  return [t.cuda() for t in ts]


def _gs_dev(gs):
  return torch.as_tensor(np.asarray(gs, np.int32)).cuda()


def _fwd(capi, lhs, rhs, gs, out_dtype=torch.bfloat16, rhs_layout=0, **cfg):
  m = lhs.shape[0]
  n = rhs.shape[2] if rhs_layout == 0 else rhs.shape[1]
  out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
  config = capi.Config(**cfg) if cfg else None
  capi.ragged_dot_fwd(lhs.cuda(), rhs.cuda(), _gs_dev(gs), out, rhs_layout=rhs_layout, config=config)
  capi.device_status()
  return out


def _dlhs(capi, dout, rhs, gs, out_dtype=torch.bfloat16, **cfg):
  out = torch.full((dout.shape[0], rhs.shape[1]), float("nan"), dtype=out_dtype, device="cuda")
  capi.ragged_dot_dlhs(dout.cuda(), rhs.cuda(), _gs_dev(gs), out, config=capi.Config(**cfg) if cfg else None)
  capi.device_status()
  return out


def _drhs(capi, lhs, dout, gs, out_dtype=torch.bfloat16, **cfg):
  out = torch.full((len(gs), lhs.shape[1], dout.shape[1]), float("nan"), dtype=out_dtype, device="cuda")
  capi.ragged_dot_drhs(lhs.cuda(), dout.cuda(), _gs_dev(gs), out, config=capi.Config(**cfg) if cfg else None)
  capi.device_status()
  return out


# ---------------------------------------------------------------- reference suite cases
def test_simple(capi):
  g, m, k, n = 8, 1024, 128, 256
  lhs, rhs, _, _ = helpers.seeded_inputs("test_simple", m, k, n, g)
  gs = [m // g] * g
  out = _fwd(capi, lhs, rhs, gs, out_dtype=torch.float32)
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, np.array(gs), out_dtype=torch.float32),
                       atol=1e-5, rtol=1e-5, what="fwd f32 out")


def test_padded(capi):
  g, m, k, n = 8, 1024, 128, 256
  lhs, rhs, _, rng = helpers.seeded_inputs("test_padded", m, k, n, g)
  gs = rng.integers(0, m // g, (g,), np.int32)
  out = _fwd(capi, lhs, rhs, gs)
  want = ref.ragged_dot_ref(lhs, rhs, gs)
  helpers.assert_close(out, want, what="padded")
  assert (out[int(gs.sum()):] == 0).all(), "rows past sum(group_sizes) must be zero"


def test_zero_group_sizes_all_patterns(capi):
  """All 2^8 zero / non-zero patterns (test_base.py:172-185), forward and both gradients."""
  g, m, k, n = 8, 1024, 128, 256
  lhs, rhs, dout, rng = helpers.seeded_inputs("test_zero_group_sizes", m, k, n, g)
  base_gs = rng.integers(1, m // g, (g,), np.int32)
  dl, dr, dd = _dev(lhs, rhs, dout)
  for i in range(2 ** g):
    mask = np.unpackbits(np.uint8(i))
    gs = np.where(mask, base_gs, 0).astype(np.int32)
    gsd = _gs_dev(gs)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.ragged_dot_fwd(dl, dr, gsd, out)
    helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, gs), what=f"fwd gs={gs.tolist()}")
    if i % 8 == 5 or i in (0, 255):
      dlhs = torch.full((m, k), float("nan"), dtype=torch.bfloat16, device="cuda")
      drhs = torch.full((g, k, n), float("nan"), dtype=torch.bfloat16, device="cuda")
      capi.ragged_dot_dlhs(dd, dr, gsd, dlhs)
      capi.ragged_dot_drhs(dl, dd, gsd, drhs)
      want_dlhs, want_drhs = ref.ragged_dot_vjp_ref(lhs, rhs, gs, dout)
      helpers.assert_close(dlhs, want_dlhs, what=f"dlhs gs={gs.tolist()}")
      helpers.assert_close(drhs, want_drhs, what=f"drhs gs={gs.tolist()}")
  capi.device_status()


RAGGED_PATTERNS = [
    (33, 67, 50, 80, 70, 60, 90, 62),
    (1, 7, 199, 1, 100, 50, 151, 3),
    (0, 130, 0, 200, 0, 98, 84, 0),
    (512,),
    (1,) * 8,
    (127, 129, 128, 1, 255, 257, 64, 63),
]


@pytest.mark.parametrize("pattern", RAGGED_PATTERNS, ids=[str(i) for i in range(len(RAGGED_PATTERNS))])
@pytest.mark.parametrize("block_n,collective", [(64, 0), (128, 0), (256, 0), (128, 1), (256, 1)])
def test_ragged_patterns_all_ops(capi, pattern, block_n, collective):
  g = len(pattern)
  m, k, n = 1024, 192, 320
  lhs, rhs, dout, _ = helpers.seeded_inputs(f"ragged{pattern}", m, k, n, g)
  gs = np.array(pattern, np.int32)
  cfg = dict(block_n=block_n, collective=collective)
  helpers.assert_close(_fwd(capi, lhs, rhs, gs, **cfg), ref.ragged_dot_ref(lhs, rhs, gs), what="fwd")
  rt = rhs.transpose(1, 2).contiguous()
  helpers.assert_close(_fwd(capi, lhs, rt, gs, rhs_layout=1, **cfg),
                       ref.ragged_dot_ref(lhs, rhs, gs), what="fwd rhs[g,n,k]")
  want_dlhs, want_drhs = ref.ragged_dot_vjp_ref(lhs, rhs, gs, dout)
  helpers.assert_close(_dlhs(capi, dout, rhs, gs, **cfg), want_dlhs, what="dlhs")
  helpers.assert_close(_drhs(capi, lhs, dout, gs, **cfg), want_drhs, what="drhs")


@pytest.mark.parametrize("collective", [0, 1])
@pytest.mark.parametrize("shape", [(1000, 328, 200), (130, 72, 8), (77, 8, 1000), (513, 520, 136)])
def test_unaligned_tails(capi, shape, collective):
  """K and N that are multiples of 8 but not of the tile sizes; M arbitrary."""
  m, k, n = shape
  gs = np.array([m // 3, 0, m // 2, m - m // 3 - m // 2 - 5], np.int32)
  lhs, rhs, dout, _ = helpers.seeded_inputs(f"tails{shape}", m, k, n, len(gs), scale=0.2)
  cfg = dict(collective=collective)
  helpers.assert_close(_fwd(capi, lhs, rhs, gs, **cfg), ref.ragged_dot_ref(lhs, rhs, gs), what="fwd")
  want_dlhs, want_drhs = ref.ragged_dot_vjp_ref(lhs, rhs, gs, dout)
  helpers.assert_close(_dlhs(capi, dout, rhs, gs, **cfg), want_dlhs, what="dlhs")
  helpers.assert_close(_drhs(capi, lhs, dout, gs, **cfg), want_drhs, what="drhs")


@pytest.mark.parametrize("collective", [0, 1])
@pytest.mark.parametrize("stages", [2, 3, 5])
@pytest.mark.parametrize("minor,width", [(0, 1), (0, 4), (1, 2), (1, 8)])
def test_config_space_is_numerically_neutral(capi, stages, minor, width, collective):
  g, m, k, n = 6, 1536, 448, 640
  lhs, rhs, dout, rng = helpers.seeded_inputs("cfgspace", m, k, n, g)
  gs = np.array(ref.generate_group_sizes(m=m - 100, num_groups=g, seed=3), np.int32)
  cfg = dict(block_n=128, num_stages=stages, grid_minor_dim=minor, grid_tile_width=width,
             collective=collective)
  helpers.assert_close(_fwd(capi, lhs, rhs, gs, **cfg), ref.ragged_dot_ref(lhs, rhs, gs), what="fwd")
  want_dlhs, want_drhs = ref.ragged_dot_vjp_ref(lhs, rhs, gs, dout)
  helpers.assert_close(_dlhs(capi, dout, rhs, gs, **cfg), want_dlhs, what="dlhs")
  helpers.assert_close(_drhs(capi, lhs, dout, gs, **cfg), want_drhs, what="drhs")


@pytest.mark.parametrize("out_type", [None, torch.bfloat16, torch.float32])
def test_preferred_element_type(tk, out_type):
  g, m, k, n = 8, 1024, 128, 256
  lhs, rhs, _, _ = helpers.seeded_inputs("test_preferred_element_type", m, k, n, g)
  gs = torch.tensor([m // g] * g, dtype=torch.int32)
  out = tk.ragged_dot(lhs.cuda(), rhs.cuda(), gs.cuda(), preferred_element_type=out_type)
  assert out.dtype == (out_type or torch.bfloat16)
  want = ref.ragged_dot_ref(lhs, rhs, gs.numpy(), out_dtype=torch.float32)
  tol = dict(atol=0.01, rtol=0.005) if out.dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
  helpers.assert_close(out, want, **tol)


def test_f16_inputs(capi):
  g, m, k, n = 4, 512, 128, 128
  lhs, rhs, _, _ = helpers.seeded_inputs("f16", m, k, n, g, dtype=torch.float16)
  gs = np.array([100, 200, 12, 150], np.int32)
  out = _fwd(capi, lhs, rhs, gs, out_dtype=torch.float16)
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, gs), atol=5e-3, rtol=5e-3)


def test_group_sizes_forms(tk):
  """int32 / int64 tensors, a GroupSizes wrapper and a Python list give the same result."""
  g, m, k, n = 8, 1024, 128, 256
  lhs, rhs, _, _ = helpers.seeded_inputs("test_group_sizes", m, k, n, g)
  sizes = [m // g] * g
  want = ref.ragged_dot_ref(lhs, rhs, np.array(sizes))
  dl, dr = lhs.cuda(), rhs.cuda()
  forms = [torch.tensor(sizes, dtype=torch.int32).cuda(), torch.tensor(sizes, dtype=torch.int64).cuda(),
           tk.RaggedDotGroupSizes(torch.tensor(sizes, dtype=torch.int32).cuda(), (1,) * g), sizes]
  for f in forms:
    helpers.assert_close(tk.ragged_dot(dl, dr, f), want)


@pytest.mark.parametrize("m,k,n", [(1024, 128, 256), (128, 64, 128)])
@pytest.mark.parametrize("activation", [None, torch.relu, torch.tanh])
def test_vjp(tk, m, k, n, activation):
  """Value and both gradients through autograd (test_base.py:259-293): forward against
  the f32 reference, gradients with atol 0.02 / rtol 0.005 after a bf16 cotangent."""
  g = 8
  lhs, rhs, _, _ = helpers.seeded_inputs("test_vjp", m, k, n, g)
  gs = np.array([m // g] * g, np.int32)
  a = lhs.cuda().requires_grad_(True)
  b = rhs.cuda().requires_grad_(True)
  out = tk.ragged_dot(a, b, torch.from_numpy(gs).cuda(), preferred_element_type=torch.float32,
                      activation=activation, precision="BF16_BF16_F32")
  a_ref = lhs.float().requires_grad_(True)
  b_ref = rhs.float().requires_grad_(True)
  pre = torch.zeros(m, n)
  off = ref.group_offsets(gs, m)
  pre = torch.cat([a_ref[off[i]:off[i + 1]] @ b_ref[i] for i in range(g)])
  want = activation(pre) if activation is not None else pre
  helpers.assert_close(out, want, atol=1e-5, rtol=1e-5, what="forward")
  dout = ((want - want.mean()) / want.std()).detach().bfloat16().float()
  ga, gb = torch.autograd.grad(out, (a, b), dout.cuda())
  ra, rb = torch.autograd.grad(want, (a_ref, b_ref), dout)
  assert ga.dtype == torch.bfloat16 and gb.dtype == torch.bfloat16
  helpers.assert_close(ga, ra, atol=0.02, rtol=0.005, what="dlhs")
  helpers.assert_close(gb, rb, atol=0.02, rtol=0.005, what="drhs")


def test_against_committed_goldens(capi):
  gold = helpers.load_golden()
  for name in ("ragged", "even", "single"):
    lhs, rhs, dout = gold[f"{name}.lhs"], gold[f"{name}.rhs"], gold[f"{name}.dout"]
    gs = gold[f"{name}.group_sizes"]
    helpers.assert_close(_fwd(capi, lhs, rhs, gs), gold[f"{name}.fwd"], what=f"{name} fwd")
    helpers.assert_close(_dlhs(capi, dout, rhs, gs), gold[f"{name}.dlhs"], what=f"{name} dlhs")
    helpers.assert_close(_drhs(capi, lhs, dout, gs), gold[f"{name}.drhs"], what=f"{name} drhs")


def test_relaunch_is_bit_identical(capi):
  g, m, k, n = 16, 4096, 512, 768
  lhs, rhs, dout, _ = helpers.seeded_inputs("determinism", m, k, n, g)
  gs = np.array(ref.generate_group_sizes(m=m, num_groups=g, seed=1), np.int32)
  a, b = _fwd(capi, lhs, rhs, gs), _fwd(capi, lhs, rhs, gs)
  assert torch.equal(a, b)
  c, d = _drhs(capi, lhs, dout, gs), _drhs(capi, lhs, dout, gs)
  assert torch.equal(c, d)


def test_does_not_write_outside_output(capi):
  """Canary rows around the output stay intact (stores are row- and column-exact)."""
  g, m, k, n = 5, 700, 128, 200
  lhs, rhs, _, _ = helpers.seeded_inputs("canary", m, k, n, g)
  gs = np.array([100, 0, 333, 7, 200], np.int32)
  buf = torch.full((m + 16, n), 7.0, dtype=torch.bfloat16, device="cuda")
  out = buf[8:8 + m]
  capi.ragged_dot_fwd(lhs.cuda(), rhs.cuda(), _gs_dev(gs), out)
  capi.device_status()
  assert (buf[:8] == 7.0).all() and (buf[8 + m:] == 7.0).all()
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, gs))


def test_degenerate_sizes(capi):
  lhs, rhs, dout, _ = helpers.seeded_inputs("degenerate", 64, 32, 16, 2)
  out = _fwd(capi, lhs, rhs, [0, 0])
  assert (out == 0).all()
  drhs = _drhs(capi, lhs, dout, [0, 0])
  assert (drhs == 0).all()
  # group sizes that overshoot the matrix are clamped, negative ones count as empty
  out = _fwd(capi, lhs, rhs, [50, 50])
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, np.array([50, 50])))
  out = _fwd(capi, lhs, rhs, [-5, 40])
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, np.array([-5, 40])))


# ---------------------------------------------------------------- 8-bit weights
QDTYPES = [torch.float8_e4m3fn, torch.int8]


def _f8_workspace(capi, m, k, n, g):
  """Scratch that switches the e4m3-weight forward to the native fp8 tensor-core kernel."""
  need = capi.workspace_bytes(0, m, k, n, g, torch.float8_e4m3fn)
  assert need >= 2 * m * k + 4 * m
  return torch.empty(need, dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("qdtype,native", [(torch.float8_e4m3fn, False), (torch.float8_e4m3fn, True),
                                           (torch.int8, False), (torch.int8, True)],
                         ids=["fp8", "fp8native", "int8", "int8native"])
@pytest.mark.parametrize("block_n,collective", [(128, 0), (256, 0), (256, 1)])
@pytest.mark.parametrize("pattern", [(33, 67, 50, 80, 70, 60, 90, 62), (0, 130, 0, 200, 0, 98, 84, 0),
                                     (1, 7, 199, 1, 100, 50, 151, 3), (700,)])
def test_quantized_weights(capi, qdtype, native, block_n, collective, pattern):
  """fp8-e4m3 / int8 weights with one fp32 scale per (expert, output channel): the kernel
  against dequantise-then-dot on the SAME (q, scale), tolerance 5e-2.  `native` passes the
  workspace that selects the 8-bit tensor-core kernel (activations split into two e4m3 terms
  for fp8 weights, into two int8 terms for int8 weights)."""
  g = len(pattern)
  m, k, n = 768, 448, 384
  rng = np.random.default_rng(sum(str(pattern).encode()))
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  q, scale = ref.quantize_tensor_ref(w, qdtype)
  gs = np.array(pattern, np.int32)
  out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd(lhs.cuda(), q.cuda(), _gs_dev(gs), out, rhs_scale=scale.cuda(),
                      config=capi.Config(block_n=block_n, collective=collective),
                      workspace=_f8_workspace(capi, m, k, n, g) if native else None)
  capi.device_status()
  want = ref.ragged_dot_ref(lhs, q, gs, rhs_scale=scale, out_dtype=torch.float32)
  helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="w8 fwd")
  # and against the scaled-GMM form (matmul on raw q, scale applied to the fp32 product)
  helpers.assert_close(out, ref.scaled_gmm_ref(lhs, q, scale, gs, out_dtype=torch.float32),
                       atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="w8 fwd vs scaled gmm")
  assert (out[int(gs.sum()):] == 0).all()


@pytest.mark.parametrize("qdtype,native", [(torch.float8_e4m3fn, False), (torch.float8_e4m3fn, True),
                                           (torch.int8, False), (torch.int8, True)],
                         ids=["fp8", "fp8native", "int8", "int8native"])
def test_quantized_every_code_point(capi, qdtype, native):
  """Every 8-bit code (fp8: all 254 finite encodings incl. subnormals; int8: -128..127) is
  expanded exactly: with lhs = identity rows the output reproduces q * scale.  (Native fp8
  kernel: the row scale is a power of two, so a one-hot row splits exactly as well.)"""
  k, n = 64, 256
  codes = torch.arange(256, dtype=torch.int32)
  if qdtype == torch.float8_e4m3fn:
    q8 = codes.to(torch.uint8).view(torch.float8_e4m3fn)
    finite = torch.isfinite(q8.float())
    q8 = torch.where(finite, q8.float(), torch.zeros(())).to(torch.float8_e4m3fn)
  else:
    q8 = (codes - 128).to(torch.int8)
  q = q8.reshape(1, 1, 256).expand(1, k, n).contiguous()
  scale = torch.ones(1, n)
  lhs = torch.zeros(128, k, dtype=torch.bfloat16)
  lhs[torch.arange(k), torch.arange(k)] = 1.0   # row i picks weight row i
  out = torch.empty(128, n, dtype=torch.float32, device="cuda")
  capi.ragged_dot_fwd(lhs.cuda(), q.cuda(), _gs_dev([128]), out, rhs_scale=scale.cuda(),
                      workspace=_f8_workspace(capi, 128, k, n, 1) if native else None)
  capi.device_status()
  want = lhs.float() @ q[0].float()
  if native and qdtype == torch.int8:
    # the int8 split's row scale is max|a| / 127, not a power of two: one rounding of 127 * s
    torch.testing.assert_close(out.cpu(), want, rtol=1e-6, atol=1e-5)
  else:
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("collective", [0, 1])
def test_native_fp8_activation_split_accuracy(capi, collective):
  """The native fp8 kernel represents each activation by two e4m3 terms under a per-row
  power-of-two scale.  With activations spanning a wide dynamic range (log-normal magnitudes,
  a few large outliers per row) the float32 result stays within 4e-3 relative Frobenius error
  of the exact dequantise-then-dot, i.e. the split keeps bf16-like precision; one e4m3 term
  alone would be off by ~3e-2."""
  g, m, k, n = 4, 1024, 2048, 512
  rng = np.random.default_rng(77)
  a = rng.normal(0, 1, (m, k)) * np.exp(rng.normal(0, 1.5, (m, k)))
  a[:, ::97] *= 50.0
  lhs = torch.from_numpy(a.astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  q, scale = ref.quantize_tensor_ref(w, torch.float8_e4m3fn)
  gs = np.array([300, 0, 500, 224], np.int32)
  out = torch.empty((m, n), dtype=torch.float32, device="cuda")
  capi.ragged_dot_fwd(lhs.cuda(), q.cuda(), _gs_dev(gs), out, rhs_scale=scale.cuda(),
                      config=capi.Config(block_n=256, collective=collective),
                      workspace=_f8_workspace(capi, m, k, n, g))
  capi.device_status()
  want = ref.ragged_dot_ref(lhs, q, gs, rhs_scale=scale, out_dtype=torch.float32)
  rel = float((out.cpu() - want).norm() / want.norm())
  assert rel < 4e-3, rel


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
def test_native_fp8_short_tiles_every_row_count(capi, block_n, out_dtype):
  """Groups of 1, 2, ... 130 rows: every short-tile row count (operands swapped, accumulator
  transposed) and the hand-over to full tiles, with a ragged last column tile (n = 336) and
  a contraction that ends inside a 128-deep block (k = 320)."""
  sizes = list(range(1, 131)) + [0, 300, 5]
  g, k, n = len(sizes), 320, 336
  m = sum(sizes) + 77
  rng = np.random.default_rng(321)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  q, scale = ref.quantize_tensor_ref(w, torch.float8_e4m3fn)
  gs = np.array(sizes, np.int32)
  out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
  capi.ragged_dot_fwd(lhs.cuda(), q.cuda(), _gs_dev(gs), out, rhs_scale=scale.cuda(),
                      config=capi.Config(block_n=block_n), workspace=_f8_workspace(capi, m, k, n, g))
  capi.device_status()
  want = ref.ragged_dot_ref(lhs, q, gs, rhs_scale=scale, out_dtype=torch.float32)
  helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="short tiles")
  assert (out[int(gs.sum()):] == 0).all()


def test_native_fp8_falls_back_without_usable_workspace(capi):
  """A short workspace, or k not a multiple of 16, takes the converter kernel (same result up
  to the 5e-2 tolerance) instead of failing."""
  g, m, n = 2, 256, 256
  rng = np.random.default_rng(5)
  for k, ws_bytes in [(192, 1024), (200, 1 << 20)]:
    lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
    w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
    q, scale = ref.quantize_tensor_ref(w, torch.float8_e4m3fn)
    gs = np.array([100, 156], np.int32)
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    capi.ragged_dot_fwd(lhs.cuda(), q.cuda(), _gs_dev(gs), out, rhs_scale=scale.cuda(),
                        workspace=torch.empty(ws_bytes, dtype=torch.uint8, device="cuda"))
    capi.device_status()
    want = ref.ragged_dot_ref(lhs, q, gs, rhs_scale=scale, out_dtype=torch.float32)
    helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL)


def test_quantized_through_api(tk):
  g, m, k, n = 4, 512, 256, 256
  rng = np.random.default_rng(9)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  gs = np.array([100, 0, 212, 150], np.int32)
  for qdtype in QDTYPES:
    qa = tk.quantize_per_channel(w.cuda(), qdtype)
    # The device quantiser and the oracle's agree up to division rounding on the device;
    # kernel and oracle are then fed the SAME (q, scale).
    q_chk, s_chk = ref.quantize_tensor_ref(w, qdtype)
    torch.testing.assert_close(qa.channel_scale().cpu(), s_chk, rtol=1e-6, atol=0)
    assert (qa.qvalue.cpu().float() == q_chk.float()).float().mean() > 0.999
    q_ref, s_ref = qa.qvalue.cpu(), qa.channel_scale().cpu()
    want = ref.ragged_dot_ref(lhs, q_ref, gs, rhs_scale=s_ref, out_dtype=torch.float32)
    out = tk.ragged_dot(lhs.cuda(), qa, torch.from_numpy(gs).cuda())
    assert out.dtype == torch.bfloat16
    helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL)
    # raw 8-bit rhs + rhs_scale keyword, in the [G, 1, 1, N] form of the TPU GMM-v2 route
    from tokamax_b200.ragged_dot import api
    op = api.IMPLEMENTATIONS["b200"]
    out2 = op(lhs.cuda(), qa.qvalue, group_sizes=torch.from_numpy(gs).cuda(),
              rhs_scale=qa.channel_scale().reshape(g, 1, 1, n))
    assert torch.equal(out, out2)
    # against the unquantised result the error is the quantisation error: small but not zero
    dense = ref.ragged_dot_ref(lhs, w, gs, out_dtype=torch.float32)
    rel = (out.float().cpu() - dense).norm() / dense.norm()
    assert rel < (0.05 if qdtype == torch.float8_e4m3fn else 0.02)


# ---------------------------------------------------------------- MoE dispatch / combine
@pytest.mark.parametrize("t,top_k,e", [(8192, 8, 256), (1000, 2, 8), (77, 3, 1000), (5000, 1, 64)])
def test_moe_sort_pairs_bit_exact(capi, t, top_k, e):
  from oracle import moe_ref
  rng = np.random.default_rng(t)
  p = rng.random(e) ** 3
  ids = rng.choice(e, (t, top_k), p=p / p.sum()).astype(np.int32)
  if t == 1000:
    ids[::50, 0] = -1
    ids[::70, 1] = e + 5          # out-of-range ids are dropped
  pos, counts = capi.moe_sort_pairs(torch.from_numpy(ids).cuda().reshape(-1), e)
  want_pos, want_counts = moe_ref.sort_pairs_ref(ids, e)
  assert np.array_equal(counts.cpu().numpy(), want_counts)
  assert np.array_equal(pos.cpu().numpy(), want_pos)
  pos2, _ = capi.moe_sort_pairs(torch.from_numpy(ids).cuda().reshape(-1), e)
  assert torch.equal(pos, pos2)   # deterministic


def test_moe_gather_and_combine(capi):
  from oracle import moe_ref
  rng = np.random.default_rng(4)
  t, k, n, top_k, e = 300, 256, 136, 4, 16
  tokens = torch.from_numpy(rng.normal(0, 1, (t, k)).astype(np.float32)).bfloat16()
  ids = rng.integers(0, e, (t, top_k)).astype(np.int32)
  gates = torch.from_numpy(rng.random((t, top_k)).astype(np.float32))
  pos, _ = capi.moe_sort_pairs(torch.from_numpy(ids).cuda().reshape(-1), e)
  rows = capi.moe_gather_rows(tokens.cuda(), pos, top_k)
  assert torch.equal(rows.cpu(), moe_ref.gather_rows_ref(tokens, pos.cpu().numpy(), top_k))   # byte-exact copy
  outs = torch.from_numpy(rng.normal(0, 1, (t * top_k, n)).astype(np.float32)).bfloat16()
  y = capi.moe_combine(outs.cuda(), pos, gates.cuda(), t, top_k)
  want = moe_ref.combine_ref(outs, pos.cpu().numpy(), gates, t, top_k)
  helpers.assert_close(y, want, atol=2e-2, rtol=1e-2, what="combine")


@pytest.mark.parametrize("collective", [0, 1])
def test_cyclic_groups_forward(capi, collective):
  """Segments in (source, expert) order: segment i multiplies by rhs[i % G]."""
  from oracle import moe_ref
  g, cycles, m, k, n = 4, 3, 1400, 192, 320
  lhs, rhs, _, rng = helpers.seeded_inputs("cyclic", m, k, n, g)
  seg = rng.integers(0, 200, g * cycles).astype(np.int32)
  seg[5] = 0
  out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd_cyclic(lhs.cuda(), rhs.cuda(), _gs_dev(seg), out, config=capi.Config(collective=collective))
  capi.device_status()
  helpers.assert_close(out, moe_ref.cyclic_ragged_dot_ref(lhs, rhs, seg), what="cyclic fwd")


def test_group_window_forward(capi):
  """Computing a buffer in windows of groups gives the same result as one call, and rows
  of groups outside the window are left alone."""
  g, m, k, n = 12, 1500, 128, 256
  lhs, rhs, _, rng = helpers.seeded_inputs("window", m, k, n, g)
  gs = rng.integers(0, 220, g).astype(np.int32)
  want = ref.ragged_dot_ref(lhs, rhs, gs)
  out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
  dl, dr, dg = lhs.cuda(), rhs.cuda(), _gs_dev(gs)
  for begin in (0, 4, 8):
    capi.ragged_dot_fwd_cyclic(dl, dr, dg, out, zero_initialize=False, segment_begin=begin, segment_count=4)
    off = ref.group_offsets(gs, m)
    done = int(off[begin + 4])
    helpers.assert_close(out[:done], want[:done], what=f"window up to group {begin + 4}")
    assert (out[done:] == 7.0).all()
  capi.device_status()


def test_native_fp8_cyclic_and_window(capi):
  """The native fp8 kernel behind the cyclic / windowed entry point: segments cycling over
  4 weight slabs, then the same buffer computed in two windows of segments."""
  g, cycles, m, k, n = 4, 3, 1400, 256, 384
  rng = np.random.default_rng(41)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  q, scale = ref.quantize_tensor_ref(w, torch.float8_e4m3fn)
  seg = rng.integers(0, 200, g * cycles).astype(np.int32)
  seg[5] = 0
  off = ref.group_offsets(seg, m)
  want = torch.zeros((m, n), dtype=torch.float32)
  for i in range(g * cycles):
    s0, s1 = int(off[i]), int(off[i + 1])
    if s1 > s0:
      want[s0:s1] = (lhs[s0:s1].float() @ q[i % g].float()) * scale[i % g][None, :]
  ws = _f8_workspace(capi, m, k, n, g)
  out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd_cyclic(lhs.cuda(), q.cuda(), _gs_dev(seg), out, rhs_scale=scale.cuda(), workspace=ws)
  capi.device_status()
  helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="fp8 cyclic")
  out2 = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
  for begin, count in ((0, 7), (7, 5)):
    capi.ragged_dot_fwd_cyclic(lhs.cuda(), q.cuda(), _gs_dev(seg), out2, rhs_scale=scale.cuda(),
                               zero_initialize=False, segment_begin=begin, segment_count=count, workspace=ws)
  capi.device_status()
  done = int(off[-1])
  assert torch.equal(out2[:done], out[:done]) and (out2[done:] == 7.0).all()


def test_expert_parallel_layer_world1(tk):
  """The whole layer on one GPU against a dense top-k MoE on the same inputs."""
  from tokamax_b200.expert_parallel import ExpertParallelMoE
  from tokamax_b200.ragged_dot import arg_specs
  t, k, n, g, top_k = 512, 256, 384, 16, 4
  rng = np.random.default_rng(8)
  tokens = torch.from_numpy(rng.normal(0, 1, (t, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  ids_np, gates_np = arg_specs.topk_routing(t, g, top_k, seed=1)
  layer = ExpertParallelMoE(rhs.cuda(), g)
  y, plan = layer(tokens.cuda(), torch.from_numpy(ids_np).cuda(), torch.from_numpy(gates_np).cuda())
  assert torch.equal(plan.group_sizes.cpu().long(), torch.bincount(torch.from_numpy(ids_np).reshape(-1).long(), minlength=g))
  want = torch.zeros(t, n)
  for j in range(top_k):
    w = rhs[torch.from_numpy(ids_np[:, j]).long()].float()
    want += torch.from_numpy(gates_np[:, j, None]) * torch.einsum("tk,tkn->tn", tokens.float(), w).bfloat16().float()
  helpers.assert_close(y, want, what="expert-parallel layer, world 1")


def test_expert_parallel_backward_world1(tk):
  """Gradients of the layer on one GPU (dlhs and drhs kernels over the dispatched rows)
  against autograd through a dense float32 top-k MoE."""
  from tokamax_b200.expert_parallel import ExpertParallelMoE
  from tokamax_b200.ragged_dot import arg_specs
  t, k, n, g, top_k = 512, 256, 384, 16, 4
  rng = np.random.default_rng(18)
  tokens = torch.from_numpy(rng.normal(0, 1, (t, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  dy = torch.from_numpy(rng.normal(0, 1, (t, n)).astype(np.float32)).bfloat16()
  ids_np, gates_np = arg_specs.topk_routing(t, g, top_k, seed=2)
  ids, gates = torch.from_numpy(ids_np), torch.from_numpy(gates_np)
  layer = ExpertParallelMoE(rhs.cuda(), g)
  y, ctx = layer.forward_with_residuals(tokens.cuda(), ids.cuda(), gates.cuda())
  d_tok, d_rhs, d_gates = layer.backward(dy.cuda(), ctx)
  x = tokens.float().requires_grad_(True)
  w = rhs.float().requires_grad_(True)
  gt = gates.float().requires_grad_(True)
  yr = torch.zeros(t, n)
  for j in range(top_k):
    yr = yr + gt[:, j, None] * torch.einsum("tk,tkn->tn", x, w[ids[:, j].long()])
  (yr * dy.float()).sum().backward()
  helpers.assert_close(y, yr.detach(), what="forward with residuals")
  rel = lambda a, b: float((a.float().cpu() - b).abs().max() / b.abs().max())
  assert rel(d_tok, x.grad) < 3e-2 and rel(d_rhs, w.grad) < 3e-2 and rel(d_gates, gt.grad) < 3e-2, (
      rel(d_tok, x.grad), rel(d_rhs, w.grad), rel(d_gates, gt.grad))
  assert d_rhs.dtype == torch.float32 and d_tok.dtype == torch.bfloat16


# ---------------------------------------------------------------- bookkeeping, bit-exact
KAT = json.load(open(os.path.join(helpers.GOLDEN_DIR, "group_info_kat.json")))["cases"]


@pytest.mark.parametrize("case", KAT, ids=[c["name"] for c in KAT])
def test_group_info_device_known_answers(capi, case):
  got = capi.group_info_aligned(_gs_dev(case["group_sizes"]), case["tile"], case["tid_size"], case["align_tile"])
  for f, v in got.items():
    assert v.cpu().tolist() == case[f], f


def test_group_info_device_vs_oracle_random(capi):
  rng = np.random.default_rng(21)
  for _ in range(50):
    g = int(rng.integers(1, 300))
    gs = (rng.integers(0, 400, g) * (rng.random(g) > 0.3)).astype(np.int32)
    tile = int(rng.choice([8, 32, 64, 128, 256]))
    tasks = int(-(-max(int(gs.sum()), 1) // tile) + g - 1)
    got = capi.group_info_aligned(_gs_dev(gs), tile, tasks, 8)
    want = ref.group_info_aligned_ref(gs, tile, tasks, 8)
    for f in want:
      assert np.array_equal(got[f].cpu().numpy(), want[f]), (f, g, tile)


# ---------------------------------------------------------------- expert-parallel keyword arguments
@pytest.mark.parametrize("offset", [0, 4, 8, 12, -4])
@pytest.mark.parametrize("quantised", [False, True], ids=["bf16", "fp8"])
def test_group_offset_window(tk, capi, offset, quantised):
  """`group_offset`: group_sizes of the 12 global groups, rhs with the 4 local experts that
  start at global group `offset`; rows of the other groups are zeros (gmm_v2_test.py:71-99).
  With zero_initialize=False only the window's rows are defined."""
  from tokamax_b200.ragged_dot import api
  op = api.IMPLEMENTATIONS["b200"]
  g_global, g_local, m, k, n = 12, 4, 1400, 256, 384
  rng = np.random.default_rng(offset + 100)
  gs = np.array([100, 0, 212, 150, 3, 77, 0, 256, 129, 128, 1, 200], np.int32)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g_local, k, n)).astype(np.float32)).bfloat16()
  if quantised:
    q, scale = ref.quantize_tensor_ref(w, torch.float8_e4m3fn)
    rhs_arg, kw = q.cuda(), {"rhs_scale": scale.cuda()}
    atol, rtol = helpers.Q_ATOL, helpers.Q_RTOL
  else:
    q, scale = w, None
    rhs_arg, kw = w.cuda(), {}
    atol, rtol = 2e-2, 2e-2
  want = ref.scaled_gmm_ref(lhs, q, scale, gs, out_dtype=torch.float32, group_offset=offset)
  out = op(lhs.cuda(), rhs_arg, group_sizes=torch.from_numpy(gs).cuda(),
           group_offset=torch.tensor([offset], dtype=torch.int32), **kw)
  capi.device_status()
  helpers.assert_close(out, want, atol=atol, rtol=rtol)
  off = ref.group_offsets(gs, m)
  lo, hi = (int(off[min(max(offset, 0), g_global)]), int(off[min(max(offset + g_local, 0), g_global)]))
  assert (out[:lo] == 0).all() and (out[hi:] == 0).all()
  out2 = op(lhs.cuda(), rhs_arg, group_sizes=torch.from_numpy(gs).cuda(), group_offset=offset,
            zero_initialize=False, **kw)
  assert torch.equal(out2[lo:hi], out[lo:hi])
  with pytest.raises(NotImplementedError):
    op(lhs.cuda(), rhs_arg, group_sizes=torch.from_numpy(gs).cuda(), group_offset=2, **kw)


# ---------------------------------------------------------------- short tiles in pair mode
@pytest.mark.parametrize("mode", ["fwd", "dlhs"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
def test_pair_mode_short_tiles_every_remainder(capi, mode, out_dtype):
  """CTA pairs on 256-row tiles: the last tile of a group runs with swapped MMA operands when
  it holds at most 192 rows.  Groups of 256 + r rows for r = 1 .. 255 in steps of 7 (plus
  the hand-over sizes 191-193 and tiny groups) hit every path, with a ragged last column
  tile and a contraction that is not a multiple of 64."""
  sizes = [256 + r for r in range(1, 256, 7)] + [191, 192, 193, 1, 15, 16, 17, 0, 33]
  g = len(sizes)
  m = sum(sizes) + 40
  k, n = 200, 328
  rng = np.random.default_rng(17)
  gs = np.array(sizes, np.int32)
  cfg = capi.Config(block_n=256, collective=1)
  if mode == "fwd":
    lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
    rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    capi.ragged_dot_fwd(lhs.cuda(), rhs.cuda(), _gs_dev(gs), out, config=cfg)
    want = ref.ragged_dot_ref(lhs, rhs, gs, out_dtype=torch.float32)
  else:
    dout = torch.from_numpy(rng.normal(0, 1, (m, n)).astype(np.float32)).bfloat16()
    rhs = torch.from_numpy(rng.normal(0, n ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
    out = torch.full((m, k), float("nan"), dtype=out_dtype, device="cuda")
    capi.ragged_dot_dlhs(dout.cuda(), rhs.cuda(), _gs_dev(gs), out, config=cfg)
    want = ref.ragged_dot_ref(dout, rhs.transpose(1, 2).contiguous(), gs, out_dtype=torch.float32)
  capi.device_status()
  helpers.assert_close(out, want, what=f"pair short tiles {mode}")
  assert (out[int(gs.sum()):] == 0).all()


# ---------------------------------------------------------------- tile scheduling
@pytest.mark.parametrize("dynamic", ["0", "1"])
@pytest.mark.parametrize("collective", [0, 1])
def test_static_and_dynamic_scheduling_agree(capi, monkeypatch, dynamic, collective):
  """Every contraction under both schedules (round-robin deal; tile numbers drawn from a
  global counter and passed to all roles of a CTA pair): same results, bit for bit, because
  a tile's arithmetic does not depend on which CTA runs it.  Launched several times so that
  counter words are reused."""
  monkeypatch.setenv("TKMX_DYNAMIC", dynamic)
  g, m, k, n = 9, 2600, 320, 600
  rng = np.random.default_rng(99)
  gs = np.array([300, 0, 515, 64, 1, 700, 129, 256, 600], np.int32)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  dout = torch.from_numpy(rng.normal(0, 1, (m, n)).astype(np.float32)).bfloat16()
  cfg = capi.Config(block_n=256, collective=collective)
  dl, dr, dd, dg = lhs.cuda(), rhs.cuda(), dout.cuda(), _gs_dev(gs)
  for _ in range(3):
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.ragged_dot_fwd(dl, dr, dg, out, config=cfg)
    dlhs = torch.full((m, k), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.ragged_dot_dlhs(dd, dr, dg, dlhs, config=cfg)
    drhs = torch.full((g, k, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.ragged_dot_drhs(dl, dd, dg, drhs, config=cfg)
  capi.device_status()
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, gs, out_dtype=torch.float32), what="fwd")
  helpers.assert_close(dlhs, ref.ragged_dot_ref(dout, rhs.transpose(1, 2).contiguous(), gs,
                                                out_dtype=torch.float32), what="dlhs")
  want_drhs = torch.zeros((g, k, n), dtype=torch.float32)
  off = ref.group_offsets(gs, m)
  for i in range(g):
    s0, s1 = int(off[i]), int(off[i + 1])
    want_drhs[i] = lhs[s0:s1].float().T @ dout[s0:s1].float()
  helpers.assert_close(drhs, want_drhs, what="drhs")
  # the other schedule gives the same bits
  monkeypatch.setenv("TKMX_DYNAMIC", "1" if dynamic == "0" else "0")
  out2 = torch.empty_like(out)
  capi.ragged_dot_fwd(dl, dr, dg, out2, config=cfg)
  drhs2 = torch.empty_like(drhs)
  capi.ragged_dot_drhs(dl, dd, dg, drhs2, config=cfg)
  capi.device_status()
  assert torch.equal(out, out2) and torch.equal(drhs, drhs2)


def test_dynamic_scheduling_counter_words_wrap(capi, monkeypatch):
  """More launches than there are tile-counter words (256), on two streams, so that words are
  reused by later launches while earlier ones may still run: every launch must see a fresh
  counter (all tiles computed exactly once)."""
  monkeypatch.setenv("TKMX_DYNAMIC", "1")
  g, m, k, n = 5, 1100, 128, 512
  rng = np.random.default_rng(5)
  gs = np.array([200, 300, 0, 333, 260], np.int32)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16().cuda()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16().cuda()
  dg = _gs_dev(gs)
  want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd(lhs, rhs, dg, want, config=capi.Config(block_n=256, collective=1))
  streams = [torch.cuda.Stream(), torch.cuda.Stream()]
  outs = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(8)]
  torch.cuda.synchronize()
  for i in range(640):
    with torch.cuda.stream(streams[i % 2]):
      capi.ragged_dot_fwd(lhs, rhs, dg, outs[i % 8], config=capi.Config(block_n=256, collective=i % 3 != 0))
  torch.cuda.synchronize()
  capi.device_status()
  for o in outs:
    assert torch.equal(o, want)


def test_relaunch_with_identical_parameters(capi, monkeypatch):
  """A launch replayed with exactly the same parameters -- same tile-counter word and epoch,
  as a captured CUDA graph does -- computes every tile again: the last unit of a launch puts
  its counter back to zero.  Checked by replaying a graph over changing inputs."""
  monkeypatch.setenv("TKMX_DYNAMIC", "1")
  g, m, k, n = 4, 900, 128, 512
  rng = np.random.default_rng(12)
  gs = np.array([300, 0, 333, 200], np.int32)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16().cuda()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16().cuda()
  dg = _gs_dev(gs)
  out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
  cfg = capi.Config(block_n=256, collective=1)
  capi.ragged_dot_fwd(lhs, rhs, dg, out, config=cfg)     # first call outside the capture
  torch.cuda.synchronize()
  graph = torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph):
    capi.ragged_dot_fwd(lhs, rhs, dg, out, config=cfg)
  for i in range(4):
    lhs.copy_(torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16())
    out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    want = ref.ragged_dot_ref(lhs.cpu(), rhs.cpu(), gs, out_dtype=torch.float32)
    helpers.assert_close(out, want, what=f"replay {i}")
  capi.device_status()


# ---------------------------------------------------------------- fused gate/up activation
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh", "swigluoai", "silu_and_mul_with_clamp"])
@pytest.mark.parametrize("block_n,collective", [(128, 0), (256, 0), (256, 1), (128, 1)])
def test_fused_gateup_activation(capi, act, block_n, collective):
  """act(tmp[:, :n/2]) * tmp[:, n/2:] fused into the epilogue, against the oracle; the
  reference's tolerance for the unquantised path is 5e-2 (gmm_v2_test.py:1277-1282).  n/2 = 328
  is not a multiple of the half tile, groups are ragged and rows past the groups are zeros."""
  g, m, k, n = 5, 900, 192, 656
  rng = np.random.default_rng(len(act) + block_n)
  lhs = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.uniform(-1, 1, (g, k, n)).astype(np.float32)).bfloat16()
  gs = np.array([130, 0, 301, 77, 256], np.int32)
  out = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd_gateup(lhs.cuda(), rhs.cuda(), _gs_dev(gs), out, act,
                             config=capi.Config(block_n=block_n, collective=collective))
  capi.device_status()
  want = ref.gateup_ref(lhs, rhs, gs, act, out_dtype=torch.float32)
  helpers.assert_close(out, want, atol=5e-2, rtol=5e-2, what=f"gateup {act}")
  assert (out[int(gs.sum()):] == 0).all()


@pytest.mark.parametrize("collective", [0, 1])
@pytest.mark.parametrize("act", [None, "silu"])
def test_rhs_bias(capi, collective, act):
  """`rhs_bias`: bias[group] added to the float32 product of the group's rows (rows of no
  group stay zero), alone and under the fused gate/up activation; ragged groups so that
  full, short (swapped) and zero-fill tiles all take the bias path."""
  from tokamax_b200.ragged_dot import api
  g, m, k, n = 6, 1500, 192, 656
  rng = np.random.default_rng(7 + collective)
  lhs = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.uniform(-1, 1, (g, k, n)).astype(np.float32)).bfloat16()
  bias = torch.from_numpy(rng.normal(0, 2, (g, 1, n)).astype(np.float32)).bfloat16()
  gs = np.array([300, 0, 513, 77, 256, 100], np.int32)
  out_cols = n // 2 if act else n
  out = torch.full((m, out_cols), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd_epilogue(lhs.cuda(), rhs.cuda(), _gs_dev(gs), out, rhs_bias=bias[:, 0].float().cuda(),
                               activation=act, config=capi.Config(block_n=256, collective=collective))
  capi.device_status()
  if act:
    want = ref.gateup_ref(lhs, rhs, gs, act, out_dtype=torch.float32, rhs_bias=bias)
  else:
    want = ref.scaled_gmm_ref(lhs, rhs, None, gs, out_dtype=torch.float32, rhs_bias=bias)
  helpers.assert_close(out, want, atol=5e-2, rtol=5e-2, what="rhs_bias")
  assert (out[int(gs.sum()):] == 0).all()
  # through the op, with the reference's [G, 1, N] bias
  op = api.IMPLEMENTATIONS["b200"]
  out2 = op(lhs.cuda(), rhs.cuda(), group_sizes=torch.from_numpy(gs).cuda(), rhs_bias=bias.cuda(),
            fuse_gateup_activation=act)
  helpers.assert_close(out2, want, atol=5e-2, rtol=5e-2, what="rhs_bias through the op")


@pytest.mark.parametrize("act", [None, "silu", "swigluoai"])
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_fp8_weights_fused_epilogue(capi, tk, act, with_bias):
  """Gate/up activation and rhs_bias in the native fp8 kernel: full tiles, short (swapped)
  tiles and zero-fill rows, against dequantise -> dot -> (+ bias) -> activation on the same
  (q, scale); tolerance of the quantised path."""
  if act is None and not with_bias:
    pytest.skip("plain forward is covered elsewhere")
  from tokamax_b200.ragged_dot import api
  g, m, k, n = 7, 1300, 320, 704            # n / 2 = 352: a multiple of 16, not of 128
  rng = np.random.default_rng(23)
  lhs = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).bfloat16()
  w = torch.from_numpy(rng.uniform(-1, 1, (g, k, n)).astype(np.float32)).bfloat16()
  q, scale = ref.quantize_tensor_ref(w, torch.float8_e4m3fn)
  bias = torch.from_numpy(rng.normal(0, 2, (g, n)).astype(np.float32)) if with_bias else None
  gs = np.array([300, 0, 40, 129, 7, 256, 500], np.int32)
  tmp = ref.scaled_gmm_ref(lhs, q, scale, gs, out_dtype=torch.float32, rhs_bias=bias)
  if act == "silu":
    want = torch.nn.functional.silu(tmp[:, :n // 2]) * tmp[:, n // 2:]
  elif act == "swigluoai":
    gt, up = tmp[:, :n // 2].clamp(max=7.0), tmp[:, n // 2:].clamp(-7.0, 7.0)
    want = (up + 1.0) * (gt * torch.sigmoid(1.702 * gt))
  else:
    want = tmp
  out = torch.full((m, want.shape[1]), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd_epilogue(lhs.cuda(), q.cuda(), _gs_dev(gs), out, rhs_scale=scale.cuda(),
                               rhs_bias=None if bias is None else bias.cuda(), activation=act,
                               config=capi.Config(block_n=256), workspace=_f8_workspace(capi, m, k, n, g))
  capi.device_status()
  helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="fp8 fused epilogue")
  assert (out[int(gs.sum()):] == 0).all()
  op = api.IMPLEMENTATIONS["b200"]
  out2 = op(lhs.cuda(), tk.QArray(q.cuda(), scale.reshape(g, 1, n).cuda()), group_sizes=torch.from_numpy(gs).cuda(),
            rhs_bias=None if bias is None else bias.reshape(g, 1, n).cuda(), fuse_gateup_activation=act)
  helpers.assert_close(out2, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="fp8 fused epilogue via op")
  with pytest.raises(NotImplementedError):   # the converter kernel (no workspace) has no epilogue extras
    capi.ragged_dot_fwd_epilogue(lhs.cuda(), q.cuda(), _gs_dev(gs), out, rhs_scale=scale.cuda(),
                                 rhs_bias=None if bias is None else bias.cuda(), activation=act)


def test_fused_gateup_through_op(tk):
  from tokamax_b200.ragged_dot import api
  op = api.IMPLEMENTATIONS["b200"]
  g, m, k, n = 4, 512, 128, 512
  rng = np.random.default_rng(3)
  lhs = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.uniform(-1, 1, (g, k, n)).astype(np.float32)).bfloat16()
  gs = np.array([100, 156, 0, 200], np.int32)
  out = op(lhs.cuda(), rhs.cuda(), group_sizes=torch.from_numpy(gs).cuda(), fuse_gateup_activation="silu",
           preferred_element_type=torch.float32)
  assert out.shape == (m, n // 2) and out.dtype == torch.float32
  helpers.assert_close(out, ref.gateup_ref(lhs, rhs, gs, "silu", out_dtype=torch.float32), atol=5e-2, rtol=5e-2)
  # unfused composition gives the same numbers up to the bf16 rounding of the intermediate
  tmp = tk.ragged_dot(lhs.cuda(), rhs.cuda(), torch.from_numpy(gs).cuda()).float()
  unfused = torch.nn.functional.silu(tmp[:, :n // 2]) * tmp[:, n // 2:]
  helpers.assert_close(out, unfused.cpu(), atol=5e-2, rtol=5e-2)
  with pytest.raises(NotImplementedError):
    op(lhs.cuda(), rhs.cuda(), group_sizes=torch.from_numpy(gs).cuda(), fuse_gateup_activation="relu")


# ---------------------------------------------------------------- error behaviour
def test_error_behaviour(tk, capi):
  lhs, rhs, _, _ = helpers.seeded_inputs("errors", 64, 32, 16, 2)
  gs = torch.tensor([32, 32], dtype=torch.int32).cuda()
  with pytest.raises(ValueError, match="Unknown implementation"):
    tk.ragged_dot(lhs.cuda(), rhs.cuda(), gs, implementation="xla")
  with pytest.raises(ValueError, match="reduction dimension"):
    tk.ragged_dot(lhs.cuda()[:, :16].contiguous(), rhs.cuda(), gs)
  with pytest.raises(NotImplementedError):
    tk.ragged_dot(lhs.cuda(), rhs.cuda(), gs, group_offset=torch.zeros(1, dtype=torch.int32))
  with pytest.raises(NotImplementedError):
    tk.ragged_dot(lhs.float().cuda(), rhs.float().cuda(), gs)
  with pytest.raises(NotImplementedError):  # K not a multiple of 8: rows are not 16-byte aligned
    tk.ragged_dot(lhs.cuda()[:, :28].contiguous(), rhs.cuda()[:, :28].contiguous(), gs)
  out = tk.ragged_dot(lhs.cuda(), rhs.cuda(), gs, implementation="mosaic")
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, np.array([32, 32])))


# ---------------------------------------------------------------- headline sizes
def _sampled_rows_check(capi, m, k, n, gs, name, rows=96):
  """Full-size run; the CPU oracle is evaluated on a sample of rows per group."""
  g = len(gs)
  gen = torch.Generator(device="cuda").manual_seed(0)
  lhs = torch.randn(m, k, device="cuda", generator=gen).bfloat16()
  rhs = (torch.randn(g, k, n, device="cuda", generator=gen) * k ** -0.5).bfloat16()
  gsd = _gs_dev(gs)
  out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd(lhs, rhs, gsd, out)
  capi.device_status()
  off = ref.group_offsets(np.asarray(gs), m)
  rng = np.random.default_rng(0)
  nz = [i for i in range(g) if off[i + 1] > off[i]]
  for gi in rng.choice(nz, size=min(6, len(nz)), replace=False):
    lo, hi = int(off[gi]), int(off[gi + 1])
    pick = np.unique(np.concatenate([[lo, hi - 1], rng.integers(lo, hi, rows // 6)]))
    want = lhs[pick].float().cpu() @ rhs[gi].float().cpu()
    helpers.assert_close(out[pick], want, what=f"{name} group {gi}")
  assert torch.isfinite(out.float()).all()
  assert (out[int(off[-1]):] == 0).all()
  # linearity: scaling lhs by 2 scales the output by exactly 2 (power-of-two scaling is exact)
  out2 = torch.empty_like(out)
  capi.ragged_dot_fwd(lhs * 2, rhs, gsd, out2)
  assert torch.equal(out2, out * 2)


def test_cfg1_full(capi):
  from tokamax_b200.ragged_dot import arg_specs
  w = arg_specs.workload("cfg1")
  rng = np.random.default_rng(0)
  lhs = torch.from_numpy(rng.standard_normal((w.m, w.k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy((rng.standard_normal((w.g, w.k, w.n)) / 16).astype(np.float32)).bfloat16()
  helpers.assert_close(_fwd(capi, lhs, rhs, w.group_sizes), ref.ragged_dot_ref(lhs, rhs, np.array(w.group_sizes)))


def test_cfg2_mixtral_full_size_properties(capi):
  from tokamax_b200.ragged_dot import arg_specs
  w = arg_specs.workload("cfg2")
  _sampled_rows_check(capi, w.m, w.k, w.n, w.group_sizes, "cfg2")


def test_cfg3_deepseek_fp8_full_size_properties(capi, tk):
  """cfg3 at full size (fp8-e4m3 weights, 256 experts, Zipf-routed groups from 9 to 3806
  rows) through the native fp8 kernel: sampled rows of small, medium and large groups against
  dequantise-then-dot on the same (q, scale); exact linearity under power-of-two scaling of
  the activations (the row scales are powers of two); agreement with the converter kernel."""
  from tokamax_b200.ragged_dot import arg_specs
  w = arg_specs.workload("cfg3")
  gen = torch.Generator(device="cuda").manual_seed(3)
  lhs = torch.randn(w.m, w.k, device="cuda", generator=gen).bfloat16()
  q = torch.empty(w.g, w.k, w.n, device="cuda", dtype=torch.float8_e4m3fn)
  scale = torch.empty(w.g, w.n, device="cuda", dtype=torch.float32)
  for g0 in range(0, w.g, 16):   # quantise in slices to bound temporaries
    wt = (torch.randn(16, w.k, w.n, device="cuda", generator=gen) * w.k ** -0.5).bfloat16()
    qa = tk.quantize_per_channel(wt, torch.float8_e4m3fn)
    q[g0:g0 + 16] = qa.qvalue
    scale[g0:g0 + 16] = qa.channel_scale()
    del wt, qa
  gsd = _gs_dev(w.group_sizes)
  ws = _f8_workspace(capi, w.m, w.k, w.n, w.g)
  out = torch.full((w.m, w.n), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd(lhs, q, gsd, out, rhs_scale=scale, workspace=ws)
  capi.device_status()
  assert torch.isfinite(out.float()).all()
  off = ref.group_offsets(np.asarray(w.group_sizes), w.m)
  sizes = np.asarray(w.group_sizes)
  order = np.argsort(sizes)
  rng = np.random.default_rng(0)
  for gi in (order[0], order[len(order) // 2], order[-1], order[-2], order[3]):
    lo, hi = int(off[gi]), int(off[gi + 1])
    pick = np.unique(np.concatenate([[lo, hi - 1], rng.integers(lo, hi, 12)]))
    want = (lhs[pick].float().cpu() @ q[gi].float().cpu()) * scale[gi].cpu()[None, :]
    helpers.assert_close(out[pick], want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what=f"cfg3 group {gi}")
  out2 = torch.empty_like(out)
  capi.ragged_dot_fwd(lhs * 4, q, gsd, out2, rhs_scale=scale, workspace=ws)
  assert torch.equal(out2, out * 4)
  capi.ragged_dot_fwd(lhs, q, gsd, out2, rhs_scale=scale)            # converter kernel, no workspace
  capi.device_status()
  rel = float((out2.float() - out.float()).norm() / out.float().norm())
  assert rel < 1e-2, rel


def test_cfg4_qwen_backward_full_size(capi):
  """dlhs and drhs at full size, every one of the 128 groups: against per-group float32
  products (computed on the device in true float32, TF32 off) within 2e-2 + 2e-2*|x|; four
  groups also against the same products on the host."""
  from tokamax_b200.ragged_dot import arg_specs
  w = arg_specs.workload("cfg4")
  gen = torch.Generator(device="cuda").manual_seed(1)
  lhs = torch.randn(w.m, w.k, device="cuda", generator=gen).bfloat16()
  rhs = (torch.randn(w.g, w.k, w.n, device="cuda", generator=gen) * w.k ** -0.5).bfloat16()
  dout = torch.randn(w.m, w.n, device="cuda", generator=gen).bfloat16()
  gsd = _gs_dev(w.group_sizes)
  dlhs = torch.empty(w.m, w.k, dtype=torch.bfloat16, device="cuda")
  drhs = torch.empty(w.g, w.k, w.n, dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_dlhs(dout, rhs, gsd, dlhs)
  capi.ragged_dot_drhs(lhs, dout, gsd, drhs)
  capi.device_status()
  off = ref.group_offsets(np.asarray(w.group_sizes), w.m)
  for gi in (0, 17, 63, 127):
    lo, hi = int(off[gi]), int(off[gi + 1])
    want_dl = dout[lo:hi].float().cpu() @ rhs[gi].float().cpu().T
    helpers.assert_close(dlhs[lo:hi], want_dl, what=f"dlhs group {gi}")
    want_dr = lhs[lo:hi].float().cpu().T @ dout[lo:hi].float().cpu()
    helpers.assert_close(drhs[gi], want_dr, what=f"drhs group {gi}")
  tf32 = torch.backends.cuda.matmul.allow_tf32
  torch.backends.cuda.matmul.allow_tf32 = False
  try:
    worst = 0.0
    for gi in range(w.g):
      lo, hi = int(off[gi]), int(off[gi + 1])
      want_dl = dout[lo:hi].float() @ rhs[gi].float().T
      want_dr = lhs[lo:hi].float().T @ dout[lo:hi].float()
      for got, want in ((dlhs[lo:hi], want_dl), (drhs[gi], want_dr)):
        ratio = ((got.float() - want).abs() / (helpers.BF16_ATOL + helpers.BF16_RTOL * want.abs())).max().item()
        worst = max(worst, ratio)
    assert worst <= 1.0, f"worst error / tolerance over all groups: {worst}"
  finally:
    torch.backends.cuda.matmul.allow_tf32 = tf32


# ---------------------------------------------------------------- host-buffer pipeline
@pytest.mark.parametrize("chunk_bytes", [1 << 16, 1 << 20, 1 << 30])
def test_host_pipeline_matches_device_call(tk, capi, chunk_bytes):
  """Operands in pinned host memory, copies pipelined with the per-chunk GEMMs: the result is
  bit-identical to one device call on the same data and within tolerance of the oracle,
  whatever the chunking; rows past sum(group_sizes) come back as zeros."""
  g, m, k, n = 12, 1500, 256, 384
  rng = np.random.default_rng(11)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16().pin_memory()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16().pin_memory()
  gs = np.array([100, 0, 212, 150, 3, 0, 0, 400, 129, 128, 1, 200], np.int32)
  pipe = tk.HostRaggedDot(chunk_bytes=chunk_bytes)
  out = torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()
  for _ in range(2):  # second call reuses the staging buffers
    got = pipe(lhs, rhs, torch.from_numpy(gs), out=out)
    torch.cuda.synchronize()
  assert got is out
  dev_out = tk.ragged_dot(lhs.cuda(), rhs.cuda(), torch.from_numpy(gs).cuda())
  capi.device_status()
  assert torch.equal(out, dev_out.cpu())
  helpers.assert_close(out, ref.ragged_dot_ref(lhs, rhs, gs, out_dtype=torch.float32))
  assert (out[int(gs.sum()):] == 0).all()


@pytest.mark.parametrize("qdtype", QDTYPES, ids=["fp8", "int8"])
def test_host_pipeline_quantised_weights(tk, qdtype):
  """8-bit weights cross PCIe as stored; each chunk goes through the expanding kernel."""
  g, m, k, n = 6, 900, 256, 384
  rng = np.random.default_rng(31)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16().pin_memory()
  w = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  q, scale = ref.quantize_tensor_ref(w, qdtype)
  gs = np.array([100, 0, 212, 150, 300, 90], np.int32)
  pipe = tk.HostRaggedDot(chunk_bytes=1 << 17)
  out = pipe(lhs, tk.QArray(q.pin_memory(), scale.reshape(g, 1, n)), torch.from_numpy(gs))
  torch.cuda.synchronize()
  want = ref.ragged_dot_ref(lhs, q, gs, rhs_scale=scale, out_dtype=torch.float32)
  helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL)
  assert (out[int(gs.sum()):] == 0).all()


def test_host_pipeline_edge_cases(tk):
  k, n = 64, 128
  lhs = torch.randn(300, k).bfloat16().pin_memory()
  rhs = torch.randn(3, k, n).bfloat16().pin_memory()
  # sizes that overrun m are clamped like the device kernel clamps them
  out = tk.ragged_dot_host(lhs, rhs, [200, 200, 50])
  torch.cuda.synchronize()
  want = ref.ragged_dot_ref(lhs, rhs, np.array([200, 100, 0]), out_dtype=torch.float32)
  helpers.assert_close(out, want)
  # all groups empty: zeros
  out = tk.ragged_dot_host(lhs, rhs, [0, 0, 0])
  torch.cuda.synchronize()
  assert (out == 0).all()
  with pytest.raises(ValueError):
    tk.ragged_dot_host(lhs.cuda(), rhs, [100, 100, 100])
  with pytest.raises(ValueError):
    tk.ragged_dot_host(lhs, rhs, [100, 100])


# ---------------------------------------------------------------- ragged_gather / scatter / gather_reduce
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
def test_ragged_gather_and_scatter_bit_exact(dtype):
  """The reference's base tests (ragged_gather/base_test.py:28-40: x [512, 128], 400 indices,
  start 3, end 338) plus negative and out-of-range indices; byte moves, so bit-exact."""
  from oracle import moe_ref
  from tokamax_b200 import ragged_gather as rg
  rng = np.random.default_rng(0)
  x = torch.from_numpy(rng.normal(0, 1, (512, 128)).astype(np.float32)).to(dtype)
  idx = rng.integers(0, 512, 400).astype(np.int32)
  idx[:6] = [-1, -512, 511, 0, 600, -700]
  start, end = np.array([3], np.int32), np.array([338], np.int32)
  got = rg.ragged_gather(x.cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(start).cuda(),
                         torch.from_numpy(end).cuda())
  assert torch.equal(got.cpu(), moe_ref.ragged_gather_ref(x, idx, start, end))
  got = rg.ragged_scatter(x.cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(start).cuda(),
                          torch.from_numpy(end).cuda())
  want = moe_ref.ragged_scatter_ref(x, idx, start, end)
  assert torch.equal(got.cpu(), want)
  assert (want == 0).all(dim=1).sum() > 100  # the window really masks rows
  # 0-d start / end, as the reference's signature also allows
  got = rg.ragged_scatter(x.cuda(), torch.from_numpy(idx).cuda(), torch.tensor(3), torch.tensor(338))
  assert torch.equal(got.cpu(), want)
  with pytest.raises(ValueError):
    rg.ragged_gather(x.cuda(), torch.from_numpy(idx).cuda(), start, end, implementation="mosaic_tpu")


@pytest.mark.parametrize("group", [1, 4, 8])
def test_ragged_gather_reduce(group):
  """ragged_gather_reduce/base_test.py:28-50 shape (x [512, 128], 512 rows, groups of 4) in
  bf16, with a mask that drops rows; float32 accumulation in the reference's order."""
  from oracle import moe_ref
  from tokamax_b200 import ragged_gather as rg
  rng = np.random.default_rng(group)
  x = torch.from_numpy(rng.normal(0, 1, (512, 128)).astype(np.float32)).bfloat16()
  idx = rng.integers(0, 512, 512).astype(np.int32)
  w = rng.normal(0, 1, 512).astype(np.float32)
  mask = rng.random(512) > 0.2
  got = rg.ragged_gather_reduce(x.cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(w).cuda(),
                                torch.from_numpy(mask).cuda(), reduce_group_size=group)
  want = moe_ref.ragged_gather_reduce_ref(x, idx, w, mask, group)
  assert got.shape == (512 // group, 128) and got.dtype == torch.bfloat16
  helpers.assert_close(got, want.float(), atol=2e-2, rtol=2e-2)
  with pytest.raises(ValueError):
    rg.ragged_gather_reduce(x.cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(w).cuda(),
                            torch.from_numpy(mask).cuda(), reduce_group_size=7)


# ---------------------------------------------------------------- fused `activation=`
@pytest.mark.parametrize("collective", [0, 1])
@pytest.mark.parametrize("name", ["relu", "silu", "gelu_tanh", "gelu_erf", "tanh", "sigmoid"])
def test_fused_elementwise_activation(capi, name, collective):
  """`activation=` computed on the float32 accumulator inside the kernel
  (tokamax/_src/ops/ragged_dot/api.py:108-113): every store path (TMA-stored full blocks,
  predicated ragged blocks, swapped short tiles, zero-fill rows) against act(float32 product)."""
  import torch.nn.functional as F
  g, m, k, n = 5, 1400, 160, 520
  rng = np.random.default_rng(sum(name.encode()) + collective)
  lhs = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
  rhs = torch.from_numpy(rng.normal(0, k ** -0.5, (g, k, n)).astype(np.float32)).bfloat16()
  gs = np.array([512, 0, 300, 40, 415], np.int32)          # 133 trailing rows of no group
  fns = {"relu": torch.relu, "silu": F.silu, "gelu_tanh": lambda x: F.gelu(x, approximate="tanh"),
         "gelu_erf": F.gelu, "tanh": torch.tanh, "sigmoid": torch.sigmoid}
  out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
  capi.ragged_dot_fwd_epilogue(lhs.cuda(), rhs.cuda(), _gs_dev(gs), out, element_activation=name,
                               config=capi.Config(block_n=256, collective=collective))
  capi.device_status()
  pre = ref.ragged_dot_ref(lhs, rhs, gs, out_dtype=torch.float32)
  helpers.assert_close(out, fns[name](pre), what=f"fused {name}")


def test_activation_argument_is_fused_when_recognised(tk, capi):
  """Through the public call: a recognised callable runs inside the kernel (bit-equal to the
  epilogue entry point), an unknown one is applied after the kernel, and with
  return_residuals the kernel is left unfused (the residual is the pre-activation result)."""
  import torch.nn.functional as F
  from tokamax_b200.ragged_dot import api
  from tokamax_b200.ragged_dot import b200 as b200_lib
  g, m, k, n = 4, 640, 128, 256
  lhs, rhs, _, _ = helpers.seeded_inputs("fused-act", m, k, n, g, scale=0.3)
  gs = np.array([200, 100, 40, 300], np.int32)
  gsd = _gs_dev(gs)
  got = tk.ragged_dot(lhs.cuda(), rhs.cuda(), gsd, activation=F.silu)
  bound = b200_lib.B200RaggedDot().bind(lhs.cuda(), rhs.cuda(), group_sizes=gsd)
  direct = torch.empty_like(got)
  capi.ragged_dot_fwd_epilogue(lhs.cuda(), rhs.cuda(), gsd, direct, element_activation="silu",
                               config=bound.default_config.to_capi())
  assert torch.equal(got, direct)
  pre = ref.ragged_dot_ref(lhs, rhs, gs, out_dtype=torch.float32)
  helpers.assert_close(got, F.silu(pre), what="activation=silu")
  odd = lambda x: x * 2 + 1
  helpers.assert_close(tk.ragged_dot(lhs.cuda(), rhs.cuda(), gsd, activation=odd), odd(pre.bfloat16().float()),
                       what="unknown callable, applied after the kernel")
  assert b200_lib.fusable_activation(odd) is None
  op = api.IMPLEMENTATIONS["b200"]
  out, res = op(lhs.cuda(), rhs.cuda(), group_sizes=gsd, activation=torch.relu, return_residuals=True)
  helpers.assert_close(res, pre, what="residuals are the pre-activation product")
  assert torch.equal(out, torch.relu(res))


def test_two_launches_on_one_tile_counter_word_report_a_conflict(capi, monkeypatch):
  """Dynamic scheduling hands every launch one of a fixed set of tile-counter words.  If two
  launches that overlap on the device are given the same word, neither may silently skip
  tiles: the one that sees the other's epoch stops and the status word reports it."""
  monkeypatch.setenv("TKMX_SCHED_SLOT", "7")
  monkeypatch.setenv("TKMX_DYNAMIC", "1")
  g, m, k, n = 8, 16384, 1024, 2048
  gen = torch.Generator(device="cuda").manual_seed(3)
  lhs = torch.randn(m, k, device="cuda", generator=gen).bfloat16()
  rhs = (torch.randn(g, k, n, device="cuda", generator=gen) * k ** -0.5).bfloat16()
  gsd = _gs_dev([m // g] * g)
  outs = [torch.zeros(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
  streams = [torch.cuda.Stream(), torch.cuda.Stream()]
  cfg = capi.Config(block_n=256, collective=0, max_ctas=64)     # both launches fit on the device together
  capi.device_status()
  torch.cuda.synchronize()
  for _ in range(4):
    for s, o in zip(streams, outs):
      with torch.cuda.stream(s):
        capi.ragged_dot_fwd(lhs, rhs, gsd, o, config=cfg)
  torch.cuda.synchronize()
  monkeypatch.delenv("TKMX_SCHED_SLOT")
  want = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
  conflict = False
  try:
    capi.device_status()
  except RuntimeError as e:
    assert "tile-counter word" in str(e)
    conflict = True
  capi.ragged_dot_fwd(lhs, rhs, gsd, want, config=cfg)
  capi.device_status()                                           # the device keeps working
  if not conflict:     # the launches happened not to overlap: then both results must be complete
    assert torch.equal(outs[0], want) and torch.equal(outs[1], want)


# ---------------------------------------------------------------- expert-parallel affordances of drhs
@pytest.mark.parametrize("collective", [0, 1])
def test_drhs_group_window_num_actual_groups(capi, collective):
  """`num_actual_groups` + `group_offset` of the drhs (tgmm) call: global group_sizes, only the
  local experts' slabs are produced (reference_tgmm, gmm_v2_test.py:109-160)."""
  from tokamax_b200.ragged_dot import b200 as b200_lib
  from tokamax_b200.ragged_dot import base as base_lib
  g, m, k, n = 8, 1100, 256, 320
  lhs, _, dout, rng = helpers.seeded_inputs("drhs-window", m, k, n, g)
  gs = np.array([100, 0, 257, 64, 300, 129, 0, 200], np.int32)      # 50 rows of no group
  want = ref.ragged_dot_ref(lhs, dout, gs, dims=ref.RAGGED_CONTRACTING, out_dtype=torch.float32)
  for begin, count in ((0, 8), (2, 4), (5, 3), (3, 0), (7, 1)):
    out = torch.full((count, k, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.ragged_dot_drhs(lhs.cuda(), dout.cuda(), _gs_dev(gs), out, group_begin=begin,
                         config=capi.Config(block_n=256, collective=collective))
    capi.device_status()
    if count:
      helpers.assert_close(out, want[begin:begin + count], what=f"drhs window [{begin}, {begin + count})")
  op = b200_lib.B200RaggedDot(num_actual_groups=4)
  out = op(lhs.cuda(), dout.cuda(), group_sizes=_gs_dev(gs), group_offset=torch.tensor([2]),
           ragged_dot_dimension_numbers=base_lib.RAGGED_CONTRACTING_DOT_DIM_NUMS)
  assert tuple(out.shape) == (4, k, n)
  helpers.assert_close(out, want[2:6], what="num_actual_groups through the op")
  with pytest.raises(ValueError):
    op(lhs.cuda(), dout.cuda(), group_sizes=_gs_dev(gs), group_offset=torch.tensor([6]),
       ragged_dot_dimension_numbers=base_lib.RAGGED_CONTRACTING_DOT_DIM_NUMS)


def test_as_qarray_and_vjp_with_quantised_rhs(tk, capi):
  """AsQArray is quantised next to the kernel call (tokamax/_src/quantization.py:39-72); with a
  quantised rhs the backward pass still gives dlhs (from the dequantised weights), as the
  reference's vjp does (base.py:434-446)."""
  g, m, k, n = 4, 512, 256, 384
  lhs, w, dout, _ = helpers.seeded_inputs("asq", m, k, n, g, scale=0.3)
  gs = np.array([100, 200, 12, 200], np.int32)
  for qtype in (torch.float8_e4m3fn, torch.int8):
    lazy = tk.AsQArray(w.cuda(), qtype)
    qa = lazy.as_qarray()       # the same (q, scale) goes to the oracle: the quantiser is not under test
    want = ref.ragged_dot_ref(lhs, qa.qvalue.cpu(), gs, rhs_scale=qa.channel_scale().cpu(), out_dtype=torch.float32)
    out = tk.ragged_dot(lhs.cuda(), lazy, _gs_dev(gs))
    helpers.assert_close(out, want, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what=f"AsQArray {qtype}")
  qa = tk.quantize_per_channel(w.cuda(), torch.float8_e4m3fn)
  a = lhs.cuda().requires_grad_(True)
  out = tk.ragged_dot(a, qa, _gs_dev(gs))
  (dl,) = torch.autograd.grad(out, (a,), dout.cuda())
  deq = (qa.qvalue.float() * qa.scale.float()).bfloat16()
  want_dl = ref.ragged_dot_ref(dout, deq.cpu(), gs, dims=ref.TRANS_RHS, out_dtype=torch.float32)
  helpers.assert_close(dl, want_dl, atol=helpers.Q_ATOL, rtol=helpers.Q_RTOL, what="dlhs with quantised rhs")


# ---------------------------------------------------------------- fused output quantisation
@pytest.mark.parametrize("sub", [64, 128, 256])
@pytest.mark.parametrize("collective,act", [(0, None), (1, "relu"), (1, None)])
def test_fused_output_quantisation(capi, sub, collective, act):
  """The epilogue returns (q, scale) by the reference's rule
  (pallas_mosaic_gpu_kernel_sm100_fp8_quant.py:800-844): per row and `sub` columns
  scale = max|x| / 448, q = e4m3(x / scale).  Scales against the float32 oracle; q * scale
  against the oracle within e4m3's 2^-4 relative step of the block maximum; empty rows q = 0,
  scale = 1."""
  g, m, k, n = 5, 1100, 192, 512
  lhs, rhs, _, _ = helpers.seeded_inputs(f"quant-out-{sub}", m, k, n, g, scale=0.3)
  gs = np.array([300, 0, 260, 77, 400], np.int32)           # 63 rows of no group
  q = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda").to(torch.float8_e4m3fn)
  qs = torch.full((m, n // sub), float("nan"), dtype=torch.float32, device="cuda")
  capi.ragged_dot_fwd_quant_out(lhs.cuda(), rhs.cuda(), _gs_dev(gs), q, qs, sub, element_activation=act,
                                config=capi.Config(block_n=256, collective=collective))
  capi.device_status()
  pre = ref.ragged_dot_ref(lhs, rhs, gs, out_dtype=torch.float32)
  if act == "relu":
    pre = torch.relu(pre)
  blocks = pre.reshape(m, n // sub, sub)
  amax = blocks.abs().amax(dim=2)
  want_scale = torch.where(amax == 0, torch.ones(()), amax / 448.0)
  torch.testing.assert_close(qs.cpu(), want_scale, rtol=1e-4, atol=1e-7)
  deq = (q.float().cpu().reshape(m, n // sub, sub) * qs.cpu()[:, :, None])
  err = (deq - blocks).abs()
  assert bool((err <= amax[:, :, None] * 2.0 ** -4 + 1e-6).all()), float(err.max())
  rows = int(gs.sum())
  assert (q[rows:].float() == 0).all() and (qs[rows:] == 1).all()


def test_chained_ragged_dots_through_a_quantised_intermediate(tk, capi):
  """dot1 with `epilogue_quant_qtype` returns a QArray that dot2 consumes as its lhs; against
  the chain with a bf16 intermediate (the reference's chained test,
  pallas_mosaic_gpu_kernel_sm100_fp8_quant_test.py:490-553: relative mean error < 0.1)."""
  from tokamax_b200.ragged_dot import api
  from tokamax_b200.ragged_dot import b200 as b200_lib
  g, m, k, n = 8, 512, 256, 512
  lhs, w1, _, rng = helpers.seeded_inputs("chain", m, k, n, g, scale=0.2)
  w2 = torch.from_numpy(rng.normal(0, 0.05, (g, n, n)).astype(np.float32)).bfloat16()
  gs = np.asarray(tk.generate_ragged_dot_group_sizes(m=m, num_groups=g), np.int32)
  gsd = _gs_dev(gs)
  op = api.IMPLEMENTATIONS["b200"]
  cfg = b200_lib.Config(block_m=128, block_n=256, block_k=64, num_stages=4,
                        epilogue_quant_qtype=torch.float8_e4m3fn, epilogue_quant_subchannel_size=128)
  fused_op = b200_lib.B200RaggedDot(config=cfg)
  h = fused_op(lhs.cuda(), w1.cuda(), group_sizes=gsd, activation=torch.relu)
  assert isinstance(h, tk.QArray) and h.qvalue.dtype == torch.float8_e4m3fn
  assert tuple(h.scale.shape) == (m, n // 128)
  y_fused = op(h, w2.cuda(), group_sizes=gsd)
  h_plain = op(lhs.cuda(), w1.cuda(), group_sizes=gsd, activation=torch.relu)
  y_base = op(h_plain, w2.cuda(), group_sizes=gsd)
  count = int(gs.sum())
  f, b = y_fused[:count].float(), y_base[:count].float()
  assert float((f - b).abs().mean() / b.abs().mean().clamp(min=1e-6)) < 0.1
