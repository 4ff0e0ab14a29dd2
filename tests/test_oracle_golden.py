"""CPU: the oracle restatement against fixtures produced by the reference's own modules, and the
self-defined (unpinned) parts of the oracle against brute-force definitions."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_NAMES, GQA_GOLDEN_NAMES, load_golden
from oracle import attn_oracle as O


def _run_oracle(name, g):
  q, k, v = g["q"], g["k"], g["v"]
  if name.startswith("attn"):
    return (O.attn(q, k, v),)
  if name.startswith("h2o"):
    return O.h2o(q, k, v)
  if name.startswith("kf"):
    return O.keyformer(q, k, v, g["exp_rand"], g["tau"])
  if name.startswith("roco"):
    return O.roco(q, k, v)
  if name.startswith("gemma2"):
    return (O.gemma2(q, k, v, g["softcap"]),)
  if name.startswith("snapkv"):
    return O.snapkv(q, k, v, g["kernel_size"])
  if name.startswith("corm"):
    return O.corm(q, k, v, g["corm_mask"])[:2]
  raise AssertionError(name)


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_matches_reference_fixture(name):
  g = load_golden(name)
  outs = _run_oracle(name, g)
  assert len(outs) == len(g["outs"])
  for got, want in zip(outs, g["outs"]):
    assert got.shape == want.shape
    if want.dtype == torch.bool:
      assert torch.equal(got, want)
      continue
    # same torch ops in the same order on the same host: differences are rounding noise only
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", GQA_GOLDEN_NAMES)
def test_grouped_query_oracle_matches_reference_fixture(name):
  # cases/attn_h2o.py AttnH2O / cases/attn.py Attn in their own 2-D layout, K/V heads < query heads
  g = load_golden(name)
  H, Hkv, causal = g["head_num"], g["kv_head_num"], bool(g["masked"])
  q4 = g["q"].view(1, -1, H, 128)
  k4, v4 = g["k"].view(1, -1, Hkv, 128), g["v"].view(1, -1, Hkv, 128)
  out, score = O.h2o_gqa(q4, k4, v4, causal)
  torch.testing.assert_close(out.reshape(q4.shape[1], H * 128), g["outs"][0], rtol=1e-5, atol=1e-6)
  if len(g["outs"]) > 1:
    assert g["outs"][1].shape == (Hkv, k4.shape[1])
    torch.testing.assert_close(score[0], g["outs"][1], rtol=1e-5, atol=1e-6)


def test_causal_mask_convention():
  # key j visible to query i iff j <= i + (kv_len - q_len): cases/kernels/attn.py:22-23
  q, k, v = O.make_inputs("attn", 1, 3, 5, 1, 128, torch.float16, 0)
  _, probs = O._scores_probs(q, k, True)
  vis = probs[0, 0] > 0
  want = torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 0], [1, 1, 1, 1, 1]], dtype=torch.bool)
  assert torch.equal(vis, want)


def test_score_columns_sum_to_rows():
  q, k, v = O.make_inputs("h2o", 2, 64, 64, 2, 128, torch.float16, 1)
  _, s = O.h2o(q, k, v)
  torch.testing.assert_close(s.sum(-1), torch.full((2, 2), 64.0), rtol=1e-5, atol=1e-4)
  _, s1, s2 = O.roco(q, k, v)
  torch.testing.assert_close(s1, s)
  assert torch.all(s2 <= s1 + 1e-6)


def test_sima_matches_elementwise_definition():
  q, k, v = O.make_inputs("sima", 1, 40, 40, 2, 128, torch.float16, 2)
  out = O.sima(q, k, v)
  qf, kf, vf = q.double(), k.double(), v.double()
  for h in range(2):
    qn = qf[0, :, h] / qf[0, :, h].abs().sum(0, keepdim=True)
    kn = kf[0, :, h] / kf[0, :, h].abs().sum(0, keepdim=True)
    want = qn @ (kn.T @ vf[0, :, h])
    torch.testing.assert_close(out[0, :, h].double(), want, rtol=1e-4, atol=1e-6)
  # scaling K (or Q) by a constant changes nothing: the L1 normalisation removes it
  torch.testing.assert_close(O.sima(q, (k.float() * 4).half(), v), out, rtol=1e-4, atol=1e-6)


def test_h2o_select_rule():
  score = np.array([[[5, 1, 5, 3, 9, 0, 0, 0]]], dtype=np.float32)
  idx = O.h2o_select(score, 2, 3)            # candidates 0..4, keep 2 + last 3
  assert idx.tolist() == [[[0, 4, 5, 6, 7]]]  # 9, then the FIRST of the two 5s
  assert O.keyformer_select(score, 3).tolist() == [[[0, 2, 4]]]


def test_roco_stats_and_select():
  S, q_len = 6, 4                             # kv_len - q_len = 2: n_j = 4,4,4,3,2,1
  ssum = np.arange(1, 7, dtype=np.float32).reshape(1, 1, S)
  ssq = ssum ** 2
  mean, std = O.roco_stats(ssum, ssq, q_len)
  n = np.array([4, 4, 4, 3, 2, 1], dtype=np.float32)
  np.testing.assert_allclose(mean[0, 0], ssum[0, 0] / n, rtol=1e-6)
  np.testing.assert_allclose(std[0, 0] ** 2, np.maximum(ssq[0, 0] / n - (ssum[0, 0] / n) ** 2, 0), rtol=1e-5)
  assert O.roco_select(ssum, ssq, 2, q_len).tolist() == [[[4, 5]]]
  # equal means: the larger std wins, then the lower index
  ssum = np.ones((1, 1, 4), dtype=np.float32)
  ssq = np.array([[[1, 3, 3, 2]]], dtype=np.float32)
  assert O.roco_select(ssum, ssq, 2, 1).tolist() == [[[1, 2]]]  # q_len 1: every n_j is 1


def test_tie_rule_comparator():
  keys = np.array([[[1.0, 2.0, 2.0005, 3.0, 0.5]]], dtype=np.float32)
  want = O.keyformer_select(keys, 2)          # {2, 3}
  assert want.tolist() == [[[2, 3]]]
  assert O.check_index_sets(want, want, keys, 2) == 0
  near = np.array([[[1, 3]]], dtype=np.int32)  # 2.0 vs 2.0005: within one fp16 ulp (2^-10 * 2)
  assert O.check_index_sets(near, want, keys, 2) == 2
  far = np.array([[[0, 3]]], dtype=np.int32)
  with pytest.raises(AssertionError):
    O.check_index_sets(far, want, keys, 2)


def test_seeded_noise_generator():
  x = np.arange(1 << 16, dtype=np.uint32)
  h = O.hash_u32(x)
  assert len(np.unique(h)) == len(x)                      # a bijection never collides
  assert int(O.hash_u32(np.uint32(0))) == 0               # 0 is the mixer's fixed point
  w = O.keyformer_seeded_bits(3, 1, 2, 64, 128)
  assert w.shape == (1, 2, 64, 128)
  assert len(np.unique(w[0, 0])) == 64 * 128               # distinct word per logit of a head
  assert not np.array_equal(w[0, 0], w[0, 1])              # heads differ
  assert not np.array_equal(w, O.keyformer_seeded_bits(4, 1, 2, 64, 128))
  assert np.array_equal(w, O.keyformer_seeded_bits(3, 1, 2, 64, 128))
  assert np.array_equal(O.keyformer_seeded_bits(3, 1, 2, 64, 128, units=[1])[0], w[0, 1])   # one unit alone
  # known answers of the mixer and of the word of a logit (computed once from the definition in
  # the oracle's docstring and frozen here; the kernels are compared with the oracle on the GPU)
  assert [int(O.hash_u32(np.uint32(x))) for x in (1, 2, 0xDEADBEEF, 0xFFFFFFFF)] == \
      [0x688990C0, 0xD1132181, 0xE628C683, 0x6768824A]
  kat = O.keyformer_seeded_bits(0x123456789ABCDEF, 2, 3, 4, 8)
  assert kat[1, 2, 3, :4].tolist() == [1103299651, 1057166858, 2759986128, 2888210570]
  assert kat[0, 0, 0, :2].tolist() == [6164005, 4144588518]
  # uniform bytes (chi-square, 255 degrees of freedom: mean 255, sigma 22.6) and no visible
  # correlation between the noise of neighbouring keys or neighbouring query rows
  big = O.keyformer_seeded_bits(7, 1, 1, 1024, 1024)[0, 0]
  n = big.size
  for byte in (big >> np.uint32(24), big & np.uint32(255)):
    cnt = np.bincount(byte.ravel(), minlength=256)
    assert ((cnt - n / 256) ** 2 / (n / 256)).sum() < 255 + 5 * 22.6
  u = ((big >> np.uint32(9)).astype(np.float64) + 0.5) * 2.0 ** -23
  assert abs(np.corrcoef(u[:, :-1].ravel(), u[:, 1:].ravel())[0, 1]) < 0.01
  assert abs(np.corrcoef(u[:-1].ravel(), u[1:].ravel())[0, 1]) < 0.01
  er = O.keyformer_seeded_exp_rand(3, 2, 2, 256, 256)
  assert er.shape == (2, 2, 256, 256) and torch.all(er > 0) and torch.isfinite(er).all()
  g = -er.double().log()                                   # Gumbel(0,1): mean 0.5772, var pi^2/6
  assert abs(g.mean().item() - 0.5772) < 0.02 and abs(g.var().item() - 1.6449) < 0.05
