"""GPU parity: the CUDA kernels, called through the C ABI (ctypes), against
 (1) fixtures produced by the reference's own eager modules (tests/golden/),
 (2) the CPU oracle on seeded inputs, including the edge cases,
 (3) size-independent properties at the benchmark's full sizes.

Tolerances are the ones the specification states for fp16/bf16 kernels: outputs and scores within
max-abs 2e-2 AND scale-relative (max|d| / max|ref|) 1e-2; kept-index sets identical except at ties
within one fp16 ulp of the k-th key; selection on the kernels' own scores bit-exact.
"""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_NAMES, GQA_GOLDEN_NAMES, load_golden
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu

ABS_TOL = 2e-2
REL_TOL = 1e-2


@pytest.fixture(scope="module")
def ops(built_lib):
  if not torch.cuda.is_available():
    pytest.fail("the GPU parity tests need a CUDA device")
  from flashtensor_b200 import ops as _ops
  return _ops


def close(got, ref, what):
  e = O.errors(got, ref)
  assert e["abs_max"] <= ABS_TOL, f"{what}: max-abs {e['abs_max']:.3e} > {ABS_TOL}"
  assert e["scale_rel"] <= REL_TOL, f"{what}: scale-relative {e['scale_rel']:.3e} > {REL_TOL}"
  assert torch.isfinite(got.float()).all(), f"{what}: non-finite values"


def no_timeouts(ops):
  assert ops.device_status() == (0, 0)


# ------------------------------------------------------------------------------------------
# (1) golden fixtures from the reference
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_against_reference_fixture(ops, name):
  import flashtensor_b200 as ft
  g = load_golden(name)
  q, k, v = g["q"].cuda(), g["k"].cuda(), g["v"].cuda()
  H = q.shape[2]
  if name.startswith("attn"):
    outs = (ops.attn_fwd(q, k, v),)
  elif name.startswith("h2o"):
    outs = ops.h2o(q, k, v)
  elif name.startswith("kf"):
    outs = ops.keyformer(q, k, v, g["exp_rand"].cuda(), tau=g["tau"])
  elif name.startswith("roco"):
    outs = ops.roco(q, k, v)
  elif name.startswith("gemma2"):
    outs = (ft.Gemma2(logit_softcapping=g["softcap"], head_num=H, kv_head_num=H).forward(q, k, v),)
  elif name.startswith("snapkv"):
    outs = ft.SnapKV(kernel_size=g["kernel_size"], head_num=H, kv_head_num=H).forward(q, k, v)
  else:
    outs = ft.Corm(head_num=H, kv_head_num=H).forward(q, k, v, g["corm_mask"].cuda())
  torch.cuda.synchronize()
  assert len(outs) == len(g["outs"])
  for i, (got, want) in enumerate(zip(outs, g["outs"])):
    assert tuple(got.shape) == tuple(want.shape)
    if want.dtype == torch.bool:
      # a keep decision may differ from the reference's only where it hangs on rounding: some
      # probability within 1e-3 (relative) of its threshold
      _, _, margin = O.corm(g["q"], g["k"], g["v"], g["corm_mask"])
      differ = got.cpu() != want
      assert got.dtype == torch.bool and want.any() and not want.all()
      assert torch.all((margin[differ] - 1).abs() < 1e-3), f"{int(differ.sum())} decisions differ off the threshold"
      continue
    close(got, want, f"{name} output {i}")
  no_timeouts(ops)


@pytest.mark.parametrize("name", GQA_GOLDEN_NAMES)
def test_grouped_query_against_reference_fixture(ops, name):
  # fixtures from the reference's own AttnH2O / Attn modules (cases/attn_h2o.py:20-89,
  # cases/attn.py:20-63) in their 2-D layout, K/V heads shared by groups of query heads
  import flashtensor_b200 as ft
  g = load_golden(name)
  H, Hkv, causal = g["head_num"], g["kv_head_num"], bool(g["masked"])
  q, k, v = g["q"].cuda(), g["k"].cuda(), g["v"].cuda()
  assert q.dim() == 2 and q.shape[1] == H * 128 and k.shape[1] == Hkv * 128
  if name.startswith("gqa_attn"):
    outs = (ft.Attn(head_num=H, kv_head_num=Hkv, causal=causal)(q, k, v),)
  else:
    outs = ft.H2O(head_num=H, kv_head_num=Hkv, causal=causal)(q, k, v)
  torch.cuda.synchronize()
  assert len(outs) == len(g["outs"])
  for i, (got, want) in enumerate(zip(outs, g["outs"])):
    assert tuple(got.shape) == tuple(want.shape)
    close(got, want, f"{name} output {i}")
  no_timeouts(ops)


# ------------------------------------------------------------------------------------------
# (2) oracle parity on seeded inputs
# ------------------------------------------------------------------------------------------
SHAPES = [
    # B, Sq, Skv, H, causal
    (1, 128, 128, 1, True),
    (1, 1, 1, 1, True),          # a single token
    (2, 200, 200, 3, True),      # ragged: not a multiple of the tile
    (1, 100, 333, 2, True),      # q_len != kv_len, both ragged
    (1, 128, 640, 2, True),      # chunked prefill: short query block over a long cache
    (1, 300, 300, 2, False),     # unmasked form (cases/attn.py forward_wo_mask, bench/*.mlir)
    (1, 257, 257, 1, True),      # one row past a 256-row block
    (1, 1024, 1024, 4, True),    # configuration C1's shape with fewer heads
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_attn_and_h2o_vs_oracle(ops, shape, dtype):
  B, Sq, Skv, H, causal = shape
  q, k, v = O.make_inputs("h2o", B, Sq, Skv, H, 128, dtype, seed=Sq + Skv)
  ref_out, ref_score = O.h2o(q, k, v, causal)
  qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
  out = ops.attn_fwd(qd, kd, vd, causal=causal)
  out2, score = ops.h2o(qd, kd, vd, causal=causal)
  torch.cuda.synchronize()
  close(out, ref_out, "attn out")
  assert torch.equal(out, out2), "H2O's output must be the attention kernel's output"
  close(score, ref_score, "h2o_score")
  # every probability row sums to one, so the scores of a head sum to the number of query rows
  torch.testing.assert_close(score.sum(-1).cpu(), torch.full((B, H), float(Sq)), rtol=1e-4, atol=1e-3)
  no_timeouts(ops)


@pytest.mark.parametrize("shape", [(1, 4100, 4100, 2, True), (1, 3000, 5000, 3, True), (1, 4200, 4200, 2, False),
                                   (2, 4096, 4096, 1, True)])
def test_long_sequences_with_few_heads_vs_oracle(ops, shape):
  # few (batch, head) units and long sequences: the forward kernel divides every work item's key
  # range over several CTAs (partial results merged in part order) and the column pass divides the
  # query rows (partial sums added in range order); ragged, rectangular and unmasked shapes
  B, Sq, Skv, H, causal = shape
  dtype = torch.bfloat16 if H == 3 else torch.float16
  q, k, v = O.make_inputs("roco", B, Sq, Skv, H, 128, dtype, seed=Sq)
  ref_out, ref_sum, ref_sq = O.roco(q, k, v, causal)
  qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
  out, lse = ops.attn_fwd(qd, kd, vd, causal=causal, return_lse=True)
  out2, ssum, ssq = ops.roco(qd, kd, vd, causal=causal)
  torch.cuda.synchronize()
  close(out, ref_out, "out")
  assert torch.equal(out, out2)
  close(ssum, ref_sum, "roco_score")
  close(ssq, ref_sq, "roco_sq_score")
  torch.testing.assert_close(ssum.sum(-1).cpu(), torch.full((B, H), float(Sq)), rtol=1e-4, atol=1e-2)
  # the row statistic the forward kernel returns is the base-2 log-sum-exp of the scaled logits
  s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / 128 ** 0.5
  if causal:
    s = s + torch.triu(torch.full((Sq, Skv), float("-inf")), diagonal=Skv - Sq + 1)
  torch.testing.assert_close(lse.cpu(), torch.logsumexp(s, -1) * 1.4426950408889634, rtol=1e-4, atol=2e-3)
  # run-to-run identical, whatever order the parts finish in
  assert torch.equal(out, ops.attn_fwd(qd, kd, vd, causal=causal))
  assert torch.equal(ssum, ops.roco(qd, kd, vd, causal=causal)[1])
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 384, 384, 2), (2, 1000, 1000, 3), (1, 200, 456, 2)])
def test_roco_vs_oracle(ops, shape, dtype):
  B, Sq, Skv, H = shape
  q, k, v = O.make_inputs("roco", B, Sq, Skv, H, 128, dtype, seed=7)
  ref = O.roco(q, k, v)
  got = ops.roco(q.cuda(), k.cuda(), v.cuda())
  torch.cuda.synchronize()
  for g, r, n in zip(got, ref, ("out", "roco_score", "roco_sq_score")):
    close(g, r, n)
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 256, 256, 2), (2, 640, 640, 2), (1, 130, 300, 1), (1, 100, 333, 2)])
def test_keyformer_vs_oracle(ops, shape, dtype):
  B, Sq, Skv, H = shape
  q, k, v, er = O.make_inputs("keyformer", B, Sq, Skv, H, 128, dtype, seed=9)
  ref_out, ref_score = O.keyformer(q, k, v, er, tau=1.5)
  out, score = ops.keyformer(q.cuda(), k.cuda(), v.cuda(), er.cuda(), tau=1.5)
  torch.cuda.synchronize()
  close(out, ref_out, "out")
  close(score, ref_score, "kf_score")
  torch.testing.assert_close(score.sum(-1).cpu(), torch.full((B, H), float(Sq)), rtol=1e-4, atol=1e-3)
  no_timeouts(ops)


@pytest.mark.parametrize("skv", [4100, 4101])
def test_keyformer_long_sequence_with_few_heads_vs_oracle(ops, skv):
  # two heads of a long sequence: the forward kernel splits key ranges, the column pass splits
  # query ranges (partial sums per range, added in range order).  A row length of 4100 floats is
  # one TMA can describe (the passes stage the noise operand in shared memory), 4101 is not (they
  # read it with plain loads).
  B, H, Sq = 1, 2, 4100
  q, k, v, er = O.make_inputs("keyformer", B, Sq, skv, H, 128, torch.float16, seed=skv)
  ref_out, ref_score = O.keyformer(q, k, v, er, tau=1.5)
  out, score = ops.keyformer(q.cuda(), k.cuda(), v.cuda(), er.cuda(), tau=1.5)
  torch.cuda.synchronize()
  close(out, ref_out, "out")
  close(score, ref_score, "kf_score")
  torch.testing.assert_close(score.sum(-1).cpu(), torch.full((B, H), float(Sq)), rtol=1e-4, atol=1e-3)
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 256, 256, 2), (2, 640, 640, 3), (1, 100, 333, 2)])
def test_keyformer_seeded_noise_vs_oracle(ops, shape, dtype):
  # Gumbel noise generated in the kernels from a seed; the oracle restates the generator, turns it
  # into the exp_rand operand of the unmodified Keyformer definition, and must agree
  import flashtensor_b200 as ft
  B, Sq, Skv, H = shape
  q, k, v = O.make_inputs("attn", B, Sq, Skv, H, 128, dtype, seed=19)
  seed = 0x1234567_89ABCDEF
  er = O.keyformer_seeded_exp_rand(seed, B, H, Sq, Skv)
  ref_out, ref_score = O.keyformer(q, k, v, er, tau=1.5)
  model = ft.KeyFormer(tau=1.5, head_num=H, kv_head_num=H)
  out, score, idx = model.seeded(q.cuda(), k.cuda(), v.cuda(), seed, k_keep=Skv // 4)
  torch.cuda.synchronize()
  close(out, ref_out, "out")
  close(score, ref_score, "kf_score (seeded)")
  # the operand path fed with the same noise gives the same scores
  _, score_op = ops.keyformer(q.cuda(), k.cuda(), v.cuda(), er.cuda(), tau=1.5)
  torch.testing.assert_close(score, score_op, rtol=1e-4, atol=1e-5)
  # a different seed gives different scores; the same seed reproduces bit for bit
  _, score2 = model.seeded(q.cuda(), k.cuda(), v.cuda(), seed + 1)
  _, score3 = model.seeded(q.cuda(), k.cuda(), v.cuda(), seed)
  assert not torch.equal(score, score2) and torch.equal(score, score3)
  assert np.array_equal(idx.cpu().numpy(), O.keyformer_select(score.cpu().numpy(), Skv // 4))
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 128, 1), (2, 1000, 3), (1, 4096, 2), (1, 77, 2)])
def test_sima_vs_oracle(ops, shape, dtype):
  B, S, H = shape
  q, k, v = O.make_inputs("sima", B, S, S, H, 128, dtype, seed=5)
  ref = O.sima(q, k, v)
  out16 = ops.sima_fwd(q.cuda(), k.cuda(), v.cuda())
  out32 = ops.sima_fwd(q.cuda(), k.cuda(), v.cuda(), out_dtype=torch.float32)
  torch.cuda.synchronize()
  # outputs are ~1/S: "relative" is scale-relative (element-wise relative error of numbers near
  # fp16's subnormal range means nothing)
  close(out32, ref, "sima f32 out")
  close(out16, ref, "sima 16-bit out")
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(10, 700, 8), (3, 1000, 32), (80, 512, 1), (2, 1664, 40)])
def test_sima_with_many_units_vs_oracle(ops, shape, dtype):
  # enough (batch, head) units that the single persistent kernel runs (groups of four CTAs walk the
  # units, each CTA a quarter of the sequence); ragged lengths, a quarter with no tile at all
  B, S, H = shape
  q, k, v = O.make_inputs("sima", B, S, S, H, 128, dtype, seed=S)
  ref = O.sima(q, k, v)
  qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
  out16 = ops.sima_fwd(qd, kd, vd)
  out32 = ops.sima_fwd(qd, kd, vd, out_dtype=torch.float32)
  torch.cuda.synchronize()
  close(out32, ref, "sima f32 out")
  close(out16, ref, "sima 16-bit out")
  assert torch.equal(out32, ops.sima_fwd(qd, kd, vd, out_dtype=torch.float32))   # run-to-run identical
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 128, 1), (2, 1000, 3), (1, 4096, 4), (3, 2500, 2)])
def test_ea_vs_oracle(ops, shape, dtype):
  # bench/ea.mlir:13-17: softmax over the features of q, softmax over the sequence of k
  import flashtensor_b200 as ft
  B, S, H = shape
  g = torch.Generator().manual_seed(S + H)
  q = (2 * torch.randn(B, S, H, 128, generator=g)).to(dtype)
  k = (2 * torch.randn(B, S, H, 128, generator=g)).to(dtype)
  v = torch.randn(B, S, H, 128, generator=g).to(dtype)
  ref = O.ea(q, k, v)
  out16 = ft.EA(head_num=H, kv_head_num=H)(q.cuda(), k.cuda(), v.cuda())
  out32 = ops.ea_fwd(q.cuda(), k.cuda(), v.cuda(), out_dtype=torch.float32)
  torch.cuda.synchronize()
  close(out32, ref, "ea f32 out")
  close(out16, ref, "ea 16-bit out")
  # a sequence-axis softmax that is dominated by one late key: exercises the column maximum
  k2 = k.clone()
  k2[:, S - 1] += 6
  close(ops.ea_fwd(q.cuda(), k2.cuda(), v.cuda(), out_dtype=torch.float32), O.ea(q, k2, v), "ea peaked k")
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 4096, 2), (32, 2048, 8), (2, 1100, 1)])
def test_ea_keys_that_grow_along_the_sequence(ops, shape, dtype):
  # Every 128 keys the level of K steps up by more than the kernel lets a value exceed the running
  # per-column reference of its slab of the sequence, so the reference is raised (and what has been
  # accumulated is rescaled) again and again; one feature steps down instead, one is left alone.
  B, S, H = shape
  g = torch.Generator().manual_seed(7 * S + H)
  q = torch.randn(B, S, H, 128, generator=g).to(dtype)
  k = torch.randn(B, S, H, 128, generator=g)
  v = torch.randn(B, S, H, 128, generator=g).to(dtype)
  level = 10.0 * (torch.arange(S) // 128).to(torch.float32)
  k = k + level[None, :, None, None]
  k[..., 5] -= 2 * level[None, :, None]
  k[..., 6] -= level[None, :, None]
  k = k.to(dtype)
  ref = O.ea(q, k, v)
  close(ops.ea_fwd(q.cuda(), k.cuda(), v.cuda(), out_dtype=torch.float32), ref, "ea growing k, f32 out")
  close(ops.ea_fwd(q.cuda(), k.cuda(), v.cuda()), ref, "ea growing k, 16-bit out")
  no_timeouts(ops)


@pytest.mark.parametrize("ea", [False, True])
def test_linear_attention_blocks_at_the_reference_bench_shapes(ops, ea):
  # bench/sima.mlir / bench/ea.mlir: x [B, 784, 128] f32, 4 heads of 32; B reduced from 64 for the CPU oracle
  from flashtensor_b200.blocks import EABlock, SimABlock
  for (B, N, C) in [(3, 784, 128), (2, 100, 64), (1, 33, 32)]:
    g = torch.Generator().manual_seed(N + C)
    x = torch.randn(B, N, C, generator=g)
    w_qkv = torch.randn(3 * C, C, generator=g) / C ** 0.5
    b_qkv = torch.randn(3 * C, generator=g) * 0.1
    w_o = torch.randn(C, C, generator=g) / C ** 0.5
    b_o = torch.randn(C, generator=g) * 0.1
    ref = O.linear_attention_block(x, w_qkv, b_qkv, w_o, b_o, ea)
    block = EABlock() if ea else SimABlock()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
      got = block(*(t.cuda() for t in (x, w_qkv, b_qkv, w_o, b_o)))
    finally:
      torch.backends.cuda.matmul.allow_tf32 = prev
    e = O.errors(got, ref)
    assert e["scale_rel"] <= 1e-4, e
    # the core alone, on strided views, against the same line-by-line restatement without projections
    q = torch.randn(B, N, 3, C // 32, 32, generator=g)
    ref_core = O.linear_attention_core(q[:, :, 0], q[:, :, 1], q[:, :, 2], ea)
    qd = q.cuda()
    core = ops.linattn32_fwd(qd[:, :, 0], qd[:, :, 1], qd[:, :, 2], ea=ea)
    e = O.errors(core, ref_core)
    assert e["scale_rel"] <= 2e-5, e
    assert torch.equal(core, ops.linattn32_fwd(qd[:, :, 0], qd[:, :, 1], qd[:, :, 2], ea=ea))
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("direction", [1.0, -1.0])
def test_logits_that_keep_growing_or_shrinking(ops, dtype, direction):
  # keys scaled by a ramp along the sequence: the running maximum of a row keeps moving (or the
  # first tile dominates everything after it), which drives the kernel's exponent-reference
  # update and its rescaling of O and of the row sum
  for (B, Sq, Skv, H, causal) in [(1, 384, 384, 2, True), (1, 200, 456, 2, True), (1, 300, 300, 1, False),
                                  (2, 1024, 1024, 2, True)]:
    q, k, v = O.make_inputs("h2o", B, Sq, Skv, H, 128, dtype, seed=3)
    ramp = direction * (1 + torch.arange(Skv).float() / 16).view(1, Skv, 1, 1)
    k = (k.float() * ramp).to(dtype)
    ref_out, ref_score = O.h2o(q, k, v, causal)
    out, score = ops.h2o(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    torch.cuda.synchronize()
    close(out, ref_out, "out")
    close(score, ref_score, "score")
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sibling_cases_vs_oracle(ops, dtype):
  # Gemma-2 soft-capping, SnapKV pooling and CORM thresholds on ragged and rectangular shapes
  import flashtensor_b200 as ft
  for (B, Sq, Skv, H) in [(2, 200, 200, 3), (1, 130, 390, 2), (1, 1024, 1024, 2)]:
    q, k, v = O.make_inputs("attn", B, Sq, Skv, H, 128, dtype, seed=Sq)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    for cap, qs in ((50.0, 1.0), (30.0, 16.0)):      # the second one drives logits deep into the cap
      qq = (q.float() * qs).to(dtype)
      out = ft.Gemma2(logit_softcapping=cap, head_num=H, kv_head_num=H)(qq.cuda(), kd, vd)
      close(out, O.gemma2(qq, k, v, cap), f"gemma2 cap {cap}")
    for ks in (1, 5, 9):
      out, score = ft.SnapKV(kernel_size=ks, head_num=H, kv_head_num=H)(qd, kd, vd)
      ref_out, ref_score = O.snapkv(q, k, v, ks)
      close(out, ref_out, "snapkv out")
      close(score, ref_score, f"snapkv score k={ks}")
    mask = O.corm_mask(Sq, Skv)
    out, keep = ft.Corm(head_num=H, kv_head_num=H)(qd, kd, vd, mask.cuda())
    ref_out, ref_keep, margin = O.corm(q, k, v, mask)
    close(out, ref_out, "corm out")
    differ = keep.cpu() != ref_keep
    assert torch.all((margin[differ] - 1).abs() < 1e-3)
    assert differ.float().mean() < 0.01
  no_timeouts(ops)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_grouped_query_attention(ops, dtype):
  # kv_head_num < head_num (cases/attn.py, cases/attn_h2o.py): shared K/V heads, group-mean score
  import flashtensor_b200 as ft
  for (B, Sq, Skv, H, Hkv) in [(1, 256, 256, 8, 2), (2, 200, 333, 6, 3), (1, 1024, 1024, 4, 1)]:
    g = torch.Generator().manual_seed(Sq + H)
    q = torch.randn(B, Sq, H, 128, generator=g).to(dtype)
    k = torch.randn(B, Skv, Hkv, 128, generator=g).to(dtype)
    v = torch.randn(B, Skv, Hkv, 128, generator=g).to(dtype)
    ref_out, ref_score = O.h2o_gqa(q, k, v)
    model = ft.H2O(head_num=H, kv_head_num=Hkv)
    out, score = model(q.cuda(), k.cuda(), v.cuda())
    assert score.shape == (B, Hkv, Skv)
    close(out, ref_out, "gqa out")
    close(score, ref_score, "gqa score")
    out_a = ft.Attn(head_num=H, kv_head_num=Hkv)(q.cuda(), k.cuda(), v.cuda())
    assert torch.equal(out_a, out)
    k_keep = Skv // 8
    _, _, idx = model.select(q.cuda(), k.cuda(), v.cuda(), k_keep, 16)
    assert idx.shape == (B, Hkv, k_keep + 16)
    assert np.array_equal(idx.cpu().numpy(), O.h2o_select(score.cpu().numpy(), k_keep, 16))
  with pytest.raises(AssertionError):
    ft.RoCo(head_num=8, kv_head_num=2)
  no_timeouts(ops)


def test_host_pipeline(ops):
  # the host-buffer front end delivers the same bits as direct calls, for more calls than slots
  import flashtensor_b200 as ft
  from flashtensor_b200.host import HostPipeline
  model = ft.H2O(head_num=4, kv_head_num=4)
  fn = lambda q, k, v: model.select(q, k, v, 32, 16)
  calls = []
  for s in range(5):
    g = torch.Generator().manual_seed(100 + s)
    ins = [torch.randn(1, 384, 4, 128, generator=g).half().pin_memory() for _ in range(3)]
    want = [t.cpu() for t in fn(*[t.cuda() for t in ins])]
    outs = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in want]
    calls.append((ins, outs, want))
  pipe = HostPipeline(fn, [t.cuda() for t in calls[0][0]], depth=2)
  pipe.begin()
  for ins, outs, _ in calls:
    pipe.submit(ins, outs)
  pipe.drain()
  for _, outs, want in calls:
    for o, w in zip(outs, want):
      assert torch.equal(o, w)
  with pytest.raises(ValueError):
    pipe.submit([t.clone() for t in calls[0][0]], calls[0][1])  # not pinned
  no_timeouts(ops)


def test_layouts_strided_and_2d(ops):
  # heads sliced out of a larger buffer (non-contiguous), and the 2-D [S, H*D] layout of cases/attn.py
  B, S, H = 2, 256, 4
  q, k, v = O.make_inputs("h2o", B, S, S, H, 128, torch.float16, seed=3)
  big = [torch.zeros(B, S, H + 2, 128, dtype=torch.float16, device="cuda") for _ in range(3)]
  views = []
  for buf, t in zip(big, (q, k, v)):
    buf[:, :, 1:H + 1] = t.cuda()
    views.append(buf[:, :, 1:H + 1])
  assert not views[0].is_contiguous()
  ref_out, ref_score = O.h2o(q, k, v)
  out, score = ops.h2o(*views)
  close(out, ref_out, "strided out")
  close(score, ref_score, "strided score")
  # an output that starts on a 16-byte but not a 32-byte boundary (the epilogue's narrower stores)
  flat = torch.zeros(B * S * H * 128 + 8, dtype=torch.float16, device="cuda")
  odd = flat[8:].view(B, S, H, 128)
  assert odd.data_ptr() % 32 == 16
  ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), out=odd)
  assert torch.equal(odd, ops.attn_fwd(q.cuda(), k.cuda(), v.cuda()))
  q2, k2, v2 = (t[0].reshape(S, H * 128).cuda() for t in (q, k, v))
  out2 = ops.attn_fwd(q2, k2, v2)
  assert out2.shape == (S, H * 128)
  close(out2.view(1, S, H, 128), O.attn(q[:1], k[:1], v[:1]), "2-D layout out")
  no_timeouts(ops)


def test_per_case_callables_and_builder(ops):
  import flashtensor_b200 as ft
  q, k, v, er = O.make_inputs("keyformer", 1, 256, 256, 4, 128, torch.float16, seed=21)
  qd, kd, vd, erd = q.cuda(), k.cuda(), v.cuda(), er.cuda()
  out = ft.Attn(head_num=4, kv_head_num=4)(qd, kd, vd)
  o2, s2 = ft.H2O(head_num=4, kv_head_num=4).forward(qd, kd, vd)
  o3, s3 = ft.KeyFormer(tau=1.5, head_num=4, kv_head_num=4).forward(qd, kd, vd, erd)
  o4, s4, sq4 = ft.B200Builder("RoCo", head_num=4, kv_head_num=4).build_callable()(qd, kd, vd)
  assert torch.equal(out, o2) and torch.equal(out, o3) and torch.equal(out, o4)
  close(out, O.attn(q, k, v), "Attn")
  close(s2, O.h2o(q, k, v)[1], "H2O score")
  close(s3, O.keyformer(q, k, v, er, 1.5)[1], "KeyFormer score")
  close(sq4, O.roco(q, k, v)[2], "RoCo sq score")
  prep = ft.H2O(head_num=2, kv_head_num=2).prepare(batch_size=1, q_len=128, kv_len=128)
  assert prep["output"] == ["out", "h2o_score"] and prep["input"]["q"].shape == (1, 128, 2, 128)
  with pytest.raises(RuntimeError):
    ft.H2O(head_num=8, kv_head_num=8)(qd, kd, vd)       # head count mismatch


# ------------------------------------------------------------------------------------------
# selection
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S,k_keep,recent", [(256, 32, 16), (1024, 128, 64), (4096, 512, 256), (777, 100, 50)])
def test_h2o_selection(ops, S, k_keep, recent):
  B, H = 1, 4
  q, k, v = O.make_inputs("h2o", B, S, S, H, 128, torch.float16, seed=S)
  out, score, idx = ops.h2o(q.cuda(), k.cuda(), v.cuda(), k_keep=k_keep, recent=recent)
  torch.cuda.synchronize()
  idx = idx.cpu().numpy()
  assert idx.shape == (B, H, k_keep + recent) and idx.dtype == np.int32
  # integer work on the kernel's own scores: bit-exact against the oracle's rule
  assert np.array_equal(idx, O.h2o_select(score.cpu().numpy(), k_keep, recent))
  # against the oracle's scores: identical except inside the one-ulp tie band
  ref_score = O.h2o(q, k, v)[1].numpy()
  want = O.h2o_select(ref_score, k_keep, recent)
  O.check_index_sets(idx[:, :, :k_keep], want[:, :, :k_keep], ref_score, k_keep, S - recent)
  assert np.array_equal(idx[:, :, k_keep:], want[:, :, k_keep:])
  no_timeouts(ops)


def test_selection_with_many_exact_ties(ops):
  # constant scores: every key ties; the lowest indices must win, for every k
  from flashtensor_b200 import _lib
  score = torch.ones(2, 3, 1000, device="cuda")
  for k_keep in (1, 7, 999, 1000):
    idx = ops.select_topk(score, k_keep).cpu().numpy()
    assert np.array_equal(idx, np.broadcast_to(np.arange(k_keep, dtype=np.int32), (2, 3, k_keep)))
  # two-level scores with a tie straddling the cut
  s = torch.zeros(1, 1, 64, device="cuda")
  s[0, 0, [5, 9, 40]] = 2.0
  s[0, 0, [3, 20, 21, 50]] = 1.0
  assert ops.select_topk(s, 5).cpu().tolist() == [[[3, 5, 9, 20, 40]]]
  idx = ops.select_topk(s, 2, mode=_lib.SELECT_TOPK_RECENT, recent=30).cpu().tolist()[0][0]
  assert idx == [5, 9] + list(range(34, 64))
  # denormals, zeros and large values keep their order
  s = torch.tensor([[[0.0, 1e-45, 1e-38, 3e38, 1.0, 0.0]]], device="cuda")
  assert ops.select_topk(s, 4).cpu().tolist() == [[[1, 2, 3, 4]]]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_roco_and_keyformer_selection(ops, dtype):
  B, S, H, k_keep = 2, 1024, 3, 128
  q, k, v, er = O.make_inputs("keyformer", B, S, S, H, 128, dtype, seed=31)
  qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
  out, ssum, ssq, idx = ops.roco(qd, kd, vd, k_keep=k_keep)
  idx = idx.cpu().numpy()
  assert np.array_equal(idx, O.roco_select(ssum.cpu().numpy(), ssq.cpu().numpy(), k_keep, S))
  _, rs, rq = O.roco(q, k, v)
  mean, _ = O.roco_stats(rs.numpy(), rq.numpy(), S)
  O.check_index_sets(idx, O.roco_select(rs.numpy(), rq.numpy(), k_keep, S), mean, k_keep)
  out, score, idx = ops.keyformer(qd, kd, vd, er.cuda(), tau=1.5, k_keep=S // 4)
  idx = idx.cpu().numpy()
  assert np.array_equal(idx, O.keyformer_select(score.cpu().numpy(), S // 4))
  ref = O.keyformer(q, k, v, er, 1.5)[1].numpy()
  O.check_index_sets(idx, O.keyformer_select(ref, S // 4), ref, S // 4)
  no_timeouts(ops)


def test_kv_cache_compaction(ops):
  # bit-exact gather of the kept rows, on the index sets a selection produces and on strided caches
  B, S, H, k_keep, recent = 2, 640, 3, 80, 32
  q, k, v = O.make_inputs("h2o", B, S, S, H, 128, torch.bfloat16, seed=41)
  kd, vd = k.cuda(), v.cuda()
  _, _, idx = ops.h2o(q.cuda(), kd, vd, k_keep=k_keep, recent=recent)
  ko, vo = ops.gather_kv(kd, vd, idx)
  assert ko.shape == (B, k_keep + recent, H, 128)
  gi = idx.long().permute(0, 2, 1)[..., None].expand(-1, -1, -1, 128)    # [B, n, H, 128]
  assert torch.equal(ko, torch.gather(kd, 1, gi)) and torch.equal(vo, torch.gather(vd, 1, gi))
  big_k = torch.randn(B, S, H + 1, 128, device="cuda").bfloat16()
  big_v = torch.randn(B, S, H + 1, 128, device="cuda").bfloat16()
  ko, vo = ops.gather_kv(big_k[:, :, 1:], big_v[:, :, 1:], idx)
  assert torch.equal(ko, torch.gather(big_k[:, :, 1:], 1, gi)) and torch.equal(vo, torch.gather(big_v[:, :, 1:], 1, gi))


# ------------------------------------------------------------------------------------------
# determinism and error behaviour on the device
# ------------------------------------------------------------------------------------------
def test_bitwise_reproducible(ops):
  q, k, v = O.make_inputs("roco", 2, 1536, 1536, 4, 128, torch.bfloat16, seed=77)
  qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
  a = ops.roco(qd, kd, vd, k_keep=192)
  b = ops.roco(qd, kd, vd, k_keep=192)
  for x, y in zip(a, b):
    assert torch.equal(x, y)
  s1 = ops.sima_fwd(qd, kd, vd)
  s2 = ops.sima_fwd(qd, kd, vd)
  assert torch.equal(s1, s2)


def test_errors_raise_and_leave_the_device_usable(ops):
  from flashtensor_b200 import _lib
  q = torch.zeros(1, 256, 2, 128, dtype=torch.float16, device="cuda")
  with pytest.raises(_lib.AsukaError, match="BAD_SHAPE"):
    ops.attn_fwd(q, q[:, :128], q[:, :128])               # causal with fewer keys than queries
  with pytest.raises(_lib.AsukaError, match="BAD_DTYPE"):
    ops.attn_fwd(q, q.bfloat16(), q)
  with pytest.raises(_lib.AsukaError, match="BAD_ARGUMENT"):
    ops.h2o(q, q, q, k_keep=250, recent=16)               # k_keep > S - recent
  with pytest.raises(_lib.AsukaError, match="MISALIGNED"):
    flat = torch.zeros(256 * 2 * 128 + 8, dtype=torch.float16, device="cuda")
    ops.attn_fwd(flat[4:4 + 256 * 2 * 128].view(1, 256, 2, 128), q, q)
  out = ops.attn_fwd(q, q, q)                             # still works afterwards
  torch.cuda.synchronize()
  assert torch.count_nonzero(out) == 0
  no_timeouts(ops)


class _Banded:
  """Tensors carved out of one pattern-filled device buffer with untouched bands around each, to
  catch stores that land outside an output or a workspace (the ragged ends are the risk)."""
  BAND = 8192

  def __init__(self, total_bytes):
    self.buf = torch.full((total_bytes,), 0xA5, dtype=torch.uint8, device="cuda")
    self.off = self.BAND
    self.spans = []

  def take(self, shape, dtype):
    n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
    assert self.off + n + self.BAND <= self.buf.numel()
    t = self.buf[self.off:self.off + n].view(dtype).view(*shape)
    self.spans.append((self.off, self.off + n))
    self.off += (n + self.BAND + 255) // 256 * 256
    return t

  def bands_untouched(self):
    keep = torch.ones(self.buf.numel(), dtype=torch.bool, device="cuda")
    for lo, hi in self.spans:
      keep[lo:hi] = False
    return bool((self.buf[keep] == 0xA5).all())


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[1] * s[2] > 1] + [(1, 130, 130, 1, True)])
def test_no_store_lands_outside_outputs_or_workspace(ops, shape):
  import ctypes
  from flashtensor_b200 import _lib
  B, Sq, Skv, H, causal = shape
  q, k, v = (t.cuda() for t in O.make_inputs("roco", B, Sq, Skv, H, 128, torch.bfloat16, seed=5))
  k_keep = max(1, Skv // 8)
  recent = min(16, Skv - k_keep)
  mem = _Banded(64 << 20)
  lib = _lib.load()

  def ws_for(**kw):
    p = _lib.CaseParams(ops._desc(q), ops._desc(k), ops._desc(v))
    n = ctypes.c_size_t(0)
    assert lib.asuka_b200_case_workspace_bytes_split(ctypes.byref(p), ctypes.byref(n)) == 0
    return mem.take((n.value,), torch.uint8)

  # H2O with the recent window, RoCo with statistics, Keyformer with both noise sources
  o1, s1, i1 = ops.h2o(q, k, v, causal=causal, k_keep=k_keep, recent=recent, workspace=ws_for(),
                       out=mem.take((B, Sq, H, 128), torch.bfloat16), score=mem.take((B, H, Skv), torch.float32),
                       idx=mem.take((B, H, k_keep + recent), torch.int32))
  r = ops.roco(q, k, v, causal=causal, k_keep=k_keep, return_stats=True, workspace=ws_for(),
               out=mem.take((B, Sq, H, 128), torch.bfloat16), score=mem.take((B, H, Skv), torch.float32),
               score_sq=mem.take((B, H, Skv), torch.float32), idx=mem.take((B, H, k_keep), torch.int32),
               roco_mean=mem.take((B, H, Skv), torch.float32), roco_std=mem.take((B, H, Skv), torch.float32))
  er = 1 + torch.randn(B, H, Sq, Skv, device="cuda").abs()
  k1 = ops.keyformer(q, k, v, er, tau=1.5, causal=causal, k_keep=k_keep, workspace=ws_for(),
                     out=mem.take((B, Sq, H, 128), torch.bfloat16), score=mem.take((B, H, Skv), torch.float32),
                     idx=mem.take((B, H, k_keep), torch.int32))
  k2 = ops.keyformer(q, k, v, None, tau=1.5, seed=11, causal=causal, k_keep=k_keep, workspace=ws_for(),
                     out=mem.take((B, Sq, H, 128), torch.bfloat16), score=mem.take((B, H, Skv), torch.float32),
                     idx=mem.take((B, H, k_keep), torch.int32))
  o5 = ops.attn_fwd(q, k, v, causal=causal, out=mem.take((B, Sq, H, 128), torch.bfloat16))
  torch.cuda.synchronize()
  assert mem.bands_untouched(), "a kernel wrote outside its outputs or workspace"
  # and the banded buffers hold the same results as freshly allocated ones
  ref = ops.h2o(q, k, v, causal=causal, k_keep=k_keep, recent=recent)
  assert torch.equal(o1, ref[0]) and torch.equal(s1, ref[1]) and torch.equal(i1, ref[2])
  assert torch.equal(o5, ref[0]) and torch.equal(r[0], ref[0]) and torch.equal(k1[0], ref[0]) and torch.equal(k2[0], ref[0])
  # SimA / EA with their workspaces (16-bit output through TMA stores, f32 output through plain stores)
  if Sq == Skv:
    for entry in ("asuka_b200_sima_fwd", "asuka_b200_ea_fwd"):
      for odt in (torch.bfloat16, torch.float32):
        out = mem.take((B, Sq, H, 128), odt)
        p = _lib.SimaParams(ops._desc(q), ops._desc(k), ops._desc(v), ops._desc(out))
        n = ctypes.c_size_t(0)
        assert lib.asuka_b200_sima_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == 0
        ws = mem.take((max(n.value, 256),), torch.uint8)
        st = getattr(lib, entry)(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(ws.numel()),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert st == 0
    torch.cuda.synchronize()
    assert mem.bands_untouched(), "a SimA / EA kernel wrote outside its outputs or workspace"
  no_timeouts(ops)


@pytest.mark.parametrize("causal", [True, False])
def test_roco_mean_and_std_outputs(ops, causal):
  # the per-key mean and standard deviation the selection ranks by, as tensors: bit-exact against
  # the oracle's plain f32 evaluation on the kernel's own sums, within tolerance against the oracle's
  import flashtensor_b200 as ft
  from flashtensor_b200 import _lib
  for (B, Sq, Skv, H) in [(2, 384, 384, 3), (1, 200, 456, 2)]:
    q, k, v = O.make_inputs("roco", B, Sq, Skv, H, 128, torch.bfloat16, seed=Sq)
    k_keep = Skv // 8
    model = ft.RoCo(head_num=H, kv_head_num=H, causal=causal)
    out, ssum, ssq, idx, mean, std = model.select(q.cuda(), k.cuda(), v.cuda(), k_keep, return_stats=True)
    torch.cuda.synchronize()
    want_mean, want_std = O.roco_stats(ssum.cpu().numpy(), ssq.cpu().numpy(), Sq, causal)
    assert np.array_equal(mean.cpu().numpy(), want_mean) and np.array_equal(std.cpu().numpy(), want_std)
    assert np.array_equal(idx.cpu().numpy(), O.roco_select(ssum.cpu().numpy(), ssq.cpu().numpy(), k_keep, Sq, causal))
    _, rs, rq = O.roco(q, k, v, causal)
    ref_mean, ref_std = O.roco_stats(rs.numpy(), rq.numpy(), Sq, causal)
    close(mean, torch.from_numpy(ref_mean), "roco mean")
    close(std, torch.from_numpy(ref_std), "roco std")
    O.check_index_sets(idx.cpu().numpy(), O.roco_select(rs.numpy(), rq.numpy(), k_keep, Sq, causal), ref_mean, k_keep)
    # the stand-alone selection entry gives the same
    idx2, mean2, std2 = ops.select_topk(ssum, k_keep, mode=_lib.SELECT_ROCO, score_sq=ssq, q_len=Sq,
                                        causal=causal, return_stats=True)
    assert torch.equal(idx2, idx) and torch.equal(mean2, mean) and torch.equal(std2, std)
  no_timeouts(ops)


def test_a_slice_of_the_units_reproduces_the_whole_problem(ops):
  # one GPU's share of a problem split by (batch, head): same outputs as the units of the unsplit
  # run, including the seeded Keyformer noise, which is keyed by the unit's index in the whole problem
  import flashtensor_b200 as ft
  from flashtensor_b200 import sharding
  B, S, H, seed, k_keep = 2, 640, 6, 77, 80
  q, k, v = (t.cuda() for t in O.make_inputs("attn", B, S, S, H, 128, torch.float16, seed=8))
  whole = ft.KeyFormer(tau=1.5, head_num=H, kv_head_num=H).seeded(q, k, v, seed, k_keep)
  world = 4
  for rank in range(world):
    lo, hi = sharding.unit_range(B * H, rank, world)
    qs, ks, vs = (sharding.shard_bshd(t, rank, world) for t in (q, k, v))
    part = ft.KeyFormer(tau=1.5, head_num=hi - lo, kv_head_num=hi - lo).seeded(qs, ks, vs, seed, k_keep, unit_offset=lo)
    assert torch.equal(part[0], sharding.shard_bshd(whole[0], rank, world))
    assert torch.equal(part[1], sharding.shard_bhs(whole[1], rank, world))
    assert torch.equal(part[2], sharding.shard_bhs(whole[2], rank, world))
  parts = [ft.H2O(head_num=3, kv_head_num=3)(*(sharding.shard_bshd(t, r, world) for t in (q, k, v)))[1] for r in range(world)]
  assert torch.equal(sharding.gather_units(parts, B, H), ft.H2O(head_num=H, kv_head_num=H)(q, k, v)[1])
  no_timeouts(ops)


def test_an_expired_wait_is_reported_and_leaves_the_device_usable(ops):
  # a wait that nothing will ever satisfy, with a 2 ms limit: the kernel gives up and returns, the
  # status read reports the time-out once and clears it, and the next call works
  import ctypes
  from flashtensor_b200 import _lib
  lib = _lib.load()
  no_timeouts(ops)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  assert lib.asuka_b200_selftest_wait_timeout(2000, stream) == 0
  w = (ctypes.c_uint32 * 2)()
  assert lib.asuka_b200_device_status(w) == -9          # ASUKA_ERR_DEVICE_TIMEOUT
  assert (w[0], w[1]) == (1, 99)
  with pytest.raises(_lib.AsukaError, match="DEVICE_TIMEOUT"):
    lib.asuka_b200_selftest_wait_timeout(1000, stream)
    ops.device_status()
  no_timeouts(ops)                                      # cleared by the read
  assert lib.asuka_b200_selftest_wait_timeout(0, stream) == -10
  q = torch.randn(1, 256, 2, 128, device="cuda").half()
  out = ops.attn_fwd(q, q, q)
  torch.cuda.synchronize()
  assert torch.isfinite(out.float()).all()


# ------------------------------------------------------------------------------------------
# (3) full benchmark sizes: size-independent properties
# ------------------------------------------------------------------------------------------
def test_full_size_h2o_properties(ops):
  # configuration C2: B=1, H=32, S=4096, fp16, k = S/8 + 256 recent
  B, S, H = 1, 4096, 32
  g = torch.Generator(device="cuda").manual_seed(0)
  q = torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float16)
  k = torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float16)
  v = torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float16)
  out, score, idx = ops.h2o(q, k, v, k_keep=S // 8, recent=256)
  torch.cuda.synchronize()
  # (a) a head's scores sum to the number of query rows
  torch.testing.assert_close(score.sum(-1), torch.full((B, H), float(S), device="cuda"), rtol=1e-4, atol=0.05)
  # (b) causality: the first 1024 rows equal the computation on the first 1024 tokens alone (up to
  # rounding: the shorter problem may divide its key ranges differently over the CTAs)
  out_p, score_p = ops.h2o(q[:, :1024], k[:, :1024], v[:, :1024])
  torch.testing.assert_close(out[:, :1024].float(), out_p.float(), rtol=0, atol=4e-3)
  # (c) a constant V gives a constant output
  vc = torch.full_like(v, 0.5)
  oc = ops.attn_fwd(q, k, vc)
  torch.testing.assert_close(oc.float(), torch.full_like(oc, 0.5).float(), rtol=0, atol=2e-3)
  # (d) the first row attends to key 0 only
  torch.testing.assert_close(out[:, 0].float(), v[:, 0].float(), rtol=0, atol=1e-3)
  # (e) index sets: ascending, in range, the recent window present, exact on the kernel's scores
  idx_np = idx.cpu().numpy()
  assert np.all(np.diff(idx_np, axis=-1) > 0) and idx_np.min() >= 0 and idx_np.max() == S - 1
  assert np.array_equal(idx_np[..., -256:], np.broadcast_to(np.arange(S - 256, S), (B, H, 256)))
  assert np.array_equal(idx_np, O.h2o_select(score.cpu().numpy(), S // 8, 256))
  # (f) one head against the oracle (the whole configuration takes the CPU ~10 s)
  ref_out, ref_score = O.h2o(q[:, :, :1].cpu(), k[:, :, :1].cpu(), v[:, :, :1].cpu())
  close(out[:, :, :1], ref_out, "C2 head 0 out")
  close(score[:, :1], ref_score, "C2 head 0 score")
  no_timeouts(ops)


def test_full_size_roco_and_sima_properties(ops):
  # RoCo at C4's sequence length and dtype (fewer heads: the property does not depend on them)
  B, S, H = 2, 4096, 8
  g = torch.Generator(device="cuda").manual_seed(1)
  q, k, v = (torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.bfloat16) for _ in range(3))
  out, ssum, ssq = ops.roco(q, k, v)
  torch.testing.assert_close(ssum.sum(-1), torch.full((B, H), float(S), device="cuda"), rtol=1e-4, atol=0.05)
  assert torch.all(ssq <= ssum * 1.0001 + 1e-6) and torch.all(ssq >= 0)
  # key S-1 is seen by the last row only: sum = p, sumsq = p^2
  torch.testing.assert_close(ssq[..., -1], ssum[..., -1] ** 2, rtol=1e-4, atol=1e-9)
  # SimA at C5's sequence length: invariance to the scale of K and of Q, linearity in V
  B, S, H = 1, 8192, 4
  q, k = (torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float16) for _ in range(2))
  v = (torch.rand(B, S, H, 128, generator=g, device="cuda") * 2 - 1).half()
  o = ops.sima_fwd(q, k, v, out_dtype=torch.float32)
  scale = o.abs().max()
  assert torch.equal(ops.sima_fwd(q, k * 2, v, out_dtype=torch.float32), o)      # exact: powers of two
  assert torch.equal(ops.sima_fwd(q * 4, k, v, out_dtype=torch.float32), o)
  torch.testing.assert_close(ops.sima_fwd(q, k, v * 2, out_dtype=torch.float32), 2 * o, rtol=0, atol=float(scale) * 1e-5)
  # every L1-normalised channel of Q sums (in absolute value) to one: with K = sign pattern of
  # ones and V = ones, out[s, e] = sum_d Qn[s, d]
  ones = torch.ones_like(q)
  o1 = ops.sima_fwd(q, ones, ones, out_dtype=torch.float32)
  qn = q.float() / q.float().abs().sum(1, keepdim=True)
  torch.testing.assert_close(o1, qn.sum(-1, keepdim=True).expand_as(o1), rtol=0, atol=float(o1.abs().max()) * 2e-3)
  no_timeouts(ops)


# ------------------------------------------------------------------------------------------
# (4) the benchmark configurations at their own size: whole configuration on the GPU, a few
#     (batch, head) units of it against the CPU oracle
# ------------------------------------------------------------------------------------------
def _gpu_inputs(B, S, H, dtype, seed, uniform_v=False):
  g = torch.Generator(device="cuda").manual_seed(seed)
  q = torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float32).to(dtype)
  k = torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float32).to(dtype)
  if uniform_v:
    v = (torch.rand(B, S, H, 128, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(dtype)
  else:
    v = torch.randn(B, S, H, 128, generator=g, device="cuda", dtype=torch.float32).to(dtype)
  return q, k, v


def _unit(t, b, h):
  """[B,S,H,D] -> the (b, h) unit as a CPU tensor [1,S,1,D]."""
  return t[b:b + 1, :, h:h + 1].cpu()


def test_full_size_keyformer_units_vs_oracle(ops):
  # configuration C3: fp16 B=4 H=32 S=2048, tau 1.5, top-k = S/4, both noise sources
  import flashtensor_b200 as ft
  B, S, H, tau, k_keep = 4, 2048, 32, 1.5, 512
  q, k, v = _gpu_inputs(B, S, H, torch.float16, 3)
  model = ft.KeyFormer(tau=tau, head_num=H, kv_head_num=H)
  units = [(0, 0), (3, 17)]
  # (a) the exp_rand operand of cases/kernels/kf.py:48
  g = torch.Generator(device="cuda").manual_seed(33)
  er = 1 + torch.randn(B, H, S, S, generator=g, device="cuda").abs()
  out, score, idx = model.select(q, k, v, er, k_keep)
  torch.cuda.synchronize()
  for b, h in units:
    ref_out, ref_score = O.keyformer(_unit(q, b, h), _unit(k, b, h), _unit(v, b, h), er[b:b + 1, h:h + 1].cpu(), tau)
    close(out[b:b + 1, :, h:h + 1], ref_out, f"C3 operand unit ({b},{h}) out")
    close(score[b:b + 1, h:h + 1], ref_score, f"C3 operand unit ({b},{h}) kf_score")
    got_idx = idx[b:b + 1, h:h + 1].cpu().numpy()
    assert np.array_equal(got_idx, O.keyformer_select(score[b:b + 1, h:h + 1].cpu().numpy(), k_keep))
    O.check_index_sets(got_idx, O.keyformer_select(ref_score.numpy(), k_keep), ref_score.numpy(), k_keep)
  del er
  # (b) Gumbel noise generated in the kernels from a seed
  seed = 2024
  out2, score2, idx2 = model.seeded(q, k, v, seed, k_keep)
  torch.cuda.synchronize()
  assert torch.equal(out2, out)
  for b, h in units:
    er_u = O.keyformer_seeded_exp_rand(seed, B, H, S, S, units=[b * H + h])[None]
    ref_out, ref_score = O.keyformer(_unit(q, b, h), _unit(k, b, h), _unit(v, b, h), er_u, tau)
    close(score2[b:b + 1, h:h + 1], ref_score, f"C3 seeded unit ({b},{h}) kf_score")
    got_idx = idx2[b:b + 1, h:h + 1].cpu().numpy()
    assert np.array_equal(got_idx, O.keyformer_select(score2[b:b + 1, h:h + 1].cpu().numpy(), k_keep))
    O.check_index_sets(got_idx, O.keyformer_select(ref_score.numpy(), k_keep), ref_score.numpy(), k_keep)
  torch.testing.assert_close(score2.sum(-1), torch.full((B, H), float(S), device="cuda"), rtol=1e-4, atol=0.05)
  no_timeouts(ops)


def test_full_size_roco_units_vs_oracle(ops):
  # configuration C4: bf16 B=2 H=40 S=4096, top-k = S/8 by mean, ties by standard deviation
  import flashtensor_b200 as ft
  B, S, H, k_keep = 2, 4096, 40, 512
  q, k, v = _gpu_inputs(B, S, H, torch.bfloat16, 4)
  out, ssum, ssq, idx = ft.RoCo(head_num=H, kv_head_num=H).select(q, k, v, k_keep)
  torch.cuda.synchronize()
  assert np.array_equal(idx.cpu().numpy(), O.roco_select(ssum.cpu().numpy(), ssq.cpu().numpy(), k_keep, S))
  for b, h in [(0, 0), (1, 23)]:
    ref_out, rs, rq = O.roco(_unit(q, b, h), _unit(k, b, h), _unit(v, b, h))
    close(out[b:b + 1, :, h:h + 1], ref_out, f"C4 unit ({b},{h}) out")
    close(ssum[b:b + 1, h:h + 1], rs, f"C4 unit ({b},{h}) roco_score")
    close(ssq[b:b + 1, h:h + 1], rq, f"C4 unit ({b},{h}) roco_sq_score")
    mean, _ = O.roco_stats(rs.numpy(), rq.numpy(), S)
    O.check_index_sets(idx[b:b + 1, h:h + 1].cpu().numpy(), O.roco_select(rs.numpy(), rq.numpy(), k_keep, S),
                       mean, k_keep)
  no_timeouts(ops)


def test_full_size_sima_units_vs_oracle(ops):
  # configuration C5: fp16 B=8 H=32 S=8192, V ~ U(-1,1), non-causal; 16-bit and f32 outputs
  B, S, H = 8, 8192, 32
  q, k, v = _gpu_inputs(B, S, H, torch.float16, 5, uniform_v=True)
  out16 = ops.sima_fwd(q, k, v)
  torch.cuda.synchronize()
  refs = {}
  for b, h in [(0, 0), (5, 9), (7, 31)]:
    refs[(b, h)] = O.sima(_unit(q, b, h), _unit(k, b, h), _unit(v, b, h))
    close(out16[b:b + 1, :, h:h + 1], refs[(b, h)], f"C5 unit ({b},{h}) 16-bit out")
  del out16
  out32 = ops.sima_fwd(q, k, v, out_dtype=torch.float32)
  torch.cuda.synchronize()
  for (b, h), ref in refs.items():
    close(out32[b:b + 1, :, h:h + 1], ref, f"C5 unit ({b},{h}) f32 out")
  no_timeouts(ops)


def test_graphed_call_replays_the_same_bits(ops):
  # the CUDA-graph front end records a case once per input set and replays it: same results as
  # direct calls, also after the inputs' contents change in place and with two sets alternating
  import flashtensor_b200 as ft
  from flashtensor_b200.host import GraphedCall
  g = torch.Generator().manual_seed(5)
  mk = lambda: [torch.randn(1, 640, 4, 128, generator=g).half().cuda() for _ in range(3)]
  a, b = mk(), mk()
  h2o = ft.H2O(head_num=4, kv_head_num=4)
  case = lambda q, k, v: h2o.select(q, k, v, 80, 48)   # forward, column scores and selection
  graphed = GraphedCall(case, max_graphs=2)
  for ins in (a, b, a):
    want = [t.clone() for t in case(*ins)]
    got = graphed(*ins)
    torch.cuda.synchronize()
    for w_, g_ in zip(want, got):
      assert torch.equal(w_, g_)
  a[0].copy_(torch.randn(1, 640, 4, 128, generator=g).half())
  want = [t.clone() for t in case(*a)]
  got = graphed(*a)
  torch.cuda.synchronize()
  for w_, g_ in zip(want, got):
    assert torch.equal(w_, g_)
  assert len(graphed.cache) == 2 and graphed.launches > 0
  no_timeouts(ops)
