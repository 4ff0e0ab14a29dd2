"""Per-case callables with the reference's signatures.

Each class mirrors the eager module of the same name in the reference (``cases/kernels/attn.py``,
``h2o.py``, ``kf.py``, ``roco.py``): same constructor arguments, same ``forward`` arguments and
return order, same ``prepare`` dictionary, and a module-level ``get_model``-style factory.  The
body of ``forward`` is the hand-written sm_100a kernel library instead of PyTorch eager or a
generated Triton kernel.  ``SimA`` and ``EA`` have no Python counterpart in the reference (only
``bench/sima.mlir`` and ``bench/ea.mlir``); their signature follows the other cases.  The sibling
cases ``Gemma2``, ``SnapKV`` and ``Corm`` mirror ``cases/kernels/{gemma2,snapkv,corm}.py``.

The ``select`` methods are additions the benchmark configuration defines (the reference stops at
the scores): they return the kept key indices as ascending int32.
"""
import torch

from . import ops


class _Case:
  output_names = ["out"]
  allow_gqa = False

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128):
    if head_dim != 128:
      raise ValueError("the sm_100a kernels are built for head_dim = 128")
    self.kv_head_num = kv_head_num
    self.head_num = head_num
    self.head_dim = head_dim
    self.hidden_size = head_num * head_dim
    self.kv_hidden_size = kv_head_num * head_dim
    self.group_size = self.head_num // self.kv_head_num
    # the reference's 4-D cases assert group_size == 1 (cases/kernels/h2o.py:16); its 2-D case
    # scripts (cases/attn.py, cases/attn_h2o.py) run grouped-query attention, supported here by
    # the classes that set `allow_gqa`
    assert self.head_num % self.kv_head_num == 0
    assert self.group_size == 1 or self.allow_gqa, "grouped-query attention: Attn, Gemma2, H2O only"

  def __call__(self, *args, **kwargs):
    return self.forward(*args, **kwargs)

  # nn.Module-style no-ops so that scripts written for the reference keep working
  def eval(self):
    return self

  def to(self, *_args, **_kwargs):
    return self

  def _check(self, q):
    if q.dim() == 4 and q.shape[2] != self.head_num:
      raise RuntimeError(f"expected {self.head_num} heads, got {q.shape[2]}")

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    """Random inputs of the case's shapes, as ``prepare`` in cases/kernels/h2o.py:41-58."""
    device = torch.cuda.current_device() if device is None else device
    shape_q = (batch_size, q_len, self.head_num, self.head_dim)
    shape_kv = (batch_size, kv_len, self.kv_head_num, self.head_dim)
    q = torch.randn(shape_q, dtype=dtype, device=device)
    k = torch.randn(shape_kv, dtype=dtype, device=device)
    v = torch.randn(shape_kv, dtype=dtype, device=device)
    return {"input": {"q": q, "k": k, "v": v}, "output": list(self.output_names)}

  # ---- the bookkeeping the reference's Kernel object carries (python/asuka/partition/kernel.py)
  @property
  def input_names(self):
    """Positional input order of the callable (Kernel.inputs, kernel.py:78-93)."""
    return list(self.prepare(1, 8, 8, device="cpu")["input"].keys())

  def get_flops(self, batch_size=1, q_len=4096, kv_len=4096):
    """Dense flop count of the case's contractions, 2*m*k*n per dot with no credit for the causal
    mask -- the convention of Kernel.get_flops (kernel.py:155-159).  The algorithmic count the
    benchmark reports (unmasked region only) is utils.causal_flops."""
    return 4 * batch_size * self.head_num * q_len * kv_len * self.head_dim

  def get_mem_size(self, batch_size=1, q_len=4096, kv_len=4096):
    """Elements (not bytes) of all inputs and outputs, as Kernel.get_mem_size (kernel.py:161-175)."""
    ins = self.prepare(1, 8, 8, device="cpu")["input"]
    n = 0
    for name in ins:
      if name in ("q",):
        n += batch_size * q_len * self.head_num * self.head_dim
      elif name in ("k", "v"):
        n += batch_size * kv_len * self.kv_head_num * self.head_dim
      elif name == "exp_rand":
        n += batch_size * self.head_num * q_len * kv_len
      elif name == "corm_mask":
        n += q_len * kv_len
    n += batch_size * q_len * self.head_num * self.head_dim                      # out
    n += (len(self.output_names) - 1) * batch_size * self.kv_head_num * kv_len   # per-key outputs
    return n

  def prepare_dummy_inputs(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    """Positional list of random inputs, as Kernel.prepare_dummy_inputs (kernel.py:181-195)."""
    return list(self.prepare(batch_size, q_len, kv_len, dtype, device)["input"].values())


class Attn(_Case):
  """cases/kernels/attn.py:7-34.  ``causal=False`` gives ``forward_wo_mask`` of cases/attn.py;
  kv_head_num < head_num is the grouped-query form of cases/attn.py:20-42."""
  output_names = ["out"]
  allow_gqa = True

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.causal = causal

  def forward(self, q, k, v):
    self._check(q)
    return ops.attn_fwd(q, k, v, causal=self.causal)


class Gemma2(_Case):
  """cases/kernels/gemma2.py: attention with soft-capped logits, cap * tanh(logits / cap)."""
  output_names = ["out"]
  allow_gqa = True

  def __init__(self, logit_softcapping=50.0, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.logit_softcapping = logit_softcapping
    self.causal = causal

  def forward(self, q, k, v):
    self._check(q)
    return ops.attn_fwd(q, k, v, causal=self.causal, softcap=self.logit_softcapping)


class H2O(_Case):
  """cases/kernels/h2o.py:7-38: returns (out, h2o_score [B,Hkv,Skv] f32).  With kv_head_num <
  head_num the score is the mean over each group of query heads (cases/attn_h2o.py:42-46)."""
  output_names = ["out", "h2o_score"]
  allow_gqa = True

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.causal = causal

  def forward(self, q, k, v):
    self._check(q)
    return ops.h2o(q, k, v, causal=self.causal)

  def select(self, q, k, v, k_keep, recent):
    """(out, h2o_score, idx): keep the `k_keep` heaviest keys of [0, S-recent) plus the last
    `recent` keys."""
    self._check(q)
    return ops.h2o(q, k, v, causal=self.causal, k_keep=k_keep, recent=recent)


class SnapKV(_Case):
  """cases/kernels/snapkv.py: (out, snapkv_score), the H2O column sums smoothed by a moving
  average of `kernel_size` keys."""
  output_names = ["out", "snapkv_score"]

  def __init__(self, kernel_size=5, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.kernel_size = kernel_size
    self.causal = causal

  def forward(self, q, k, v):
    self._check(q)
    out, score = ops.h2o(q, k, v, causal=self.causal)
    return out, ops.pool_scores(score, self.kernel_size)


class Corm(_Case):
  """cases/kernels/corm.py: (out, corm_score) with corm_score[b,h,j] = any_i(p_ij >= corm_mask[i,j])."""
  output_names = ["out", "corm_score"]

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.causal = causal

  def forward(self, q, k, v, corm_mask):
    self._check(q)
    out, lse = ops.attn_fwd(q, k, v, causal=self.causal, return_lse=True)
    from . import _lib
    keep = ops.col_scores(q, k, lse, mode=_lib.SCORE_CORM, causal=self.causal, corm_mask=corm_mask)
    return out, keep

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    ret = super().prepare(batch_size, q_len, kv_len, dtype, device)
    dev = ret["input"]["q"].device
    # row i of the threshold is 1 / (i + 1), cases/kernels/corm.py:46-48
    rows = 1.0 / torch.arange(1, q_len + 1, dtype=torch.float32, device=dev)
    ret["input"]["corm_mask"] = rows[:, None].expand(q_len, kv_len).contiguous()
    return ret


class KeyFormer(_Case):
  """cases/kernels/kf.py:7-42: returns (out, kf_score); ``tau`` is a constructor constant."""
  output_names = ["out", "kf_score"]

  def __init__(self, tau=1.5, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.tau = tau
    self.causal = causal

  def forward(self, q, k, v, exp_rand):
    self._check(q)
    return ops.keyformer(q, k, v, exp_rand, tau=self.tau, causal=self.causal)

  def select(self, q, k, v, exp_rand, k_keep):
    self._check(q)
    return ops.keyformer(q, k, v, exp_rand, tau=self.tau, causal=self.causal, k_keep=k_keep)

  def seeded(self, q, k, v, seed, k_keep=0, unit_offset=0):
    """(out, kf_score[, idx]) with Gumbel(0,1) noise generated inside the kernels from `seed`
    (the UNIT_GUMBEL generator op of bench/keyformer.mlir:17) instead of an `exp_rand` operand.
    `unit_offset`: index of the first (batch, head) unit of these tensors within the whole problem
    when they are one GPU's slice of it (flashtensor_b200.sharding.unit_range)."""
    self._check(q)
    return ops.keyformer(q, k, v, None, tau=self.tau, seed=seed, causal=self.causal, k_keep=k_keep,
                         unit_offset=unit_offset)

  def prepare(self, batch_size=1, q_len=4096, kv_len=4096, dtype=torch.float16, device=None):
    ret = super().prepare(batch_size, q_len, kv_len, dtype, device)
    q = ret["input"]["q"]
    # the case's own noise, cases/kernels/kf.py:48
    ret["input"]["exp_rand"] = 1 + torch.randn(batch_size, self.head_num, q_len, kv_len,
                                               dtype=torch.float32, device=q.device).abs()
    return ret


class RoCo(_Case):
  """cases/kernels/roco.py:7-48: returns (out, roco_score, roco_sq_score)."""
  output_names = ["out", "roco_score", "roco_sq_score"]

  def __init__(self, kv_head_num=32, head_num=32, head_dim=128, causal=True):
    super().__init__(kv_head_num, head_num, head_dim)
    self.causal = causal

  def forward(self, q, k, v):
    self._check(q)
    return ops.roco(q, k, v, causal=self.causal)

  def select(self, q, k, v, k_keep, return_stats=False):
    """(out, roco_score, roco_sq_score, idx[, mean, std]): the `k_keep` keys of largest mean
    probability over the query rows that attend to them, ties broken by larger standard deviation,
    then lower index; `return_stats` adds the per-key mean and standard deviation [B,H,Skv] f32."""
    self._check(q)
    return ops.roco(q, k, v, causal=self.causal, k_keep=k_keep, return_stats=return_stats)


class SimA(_Case):
  """bench/sima.mlir:13-17: out = L1norm(q) (L1norm(k)^T v), normalised over the sequence axis."""
  output_names = ["out"]

  def forward(self, q, k, v):
    self._check(q)
    return ops.sima_fwd(q, k, v)

  def get_flops(self, batch_size=8, q_len=8192, kv_len=None):
    """K^T V and Q M: 2 * S * D * D each per (batch, head)."""
    return 4 * batch_size * self.head_num * q_len * self.head_dim * self.head_dim

  def prepare(self, batch_size=8, q_len=8192, kv_len=None, dtype=torch.float16, device=None):
    ret = super().prepare(batch_size, q_len, q_len, dtype, device)
    v = ret["input"]["v"]
    ret["input"]["v"] = (torch.rand(v.shape, dtype=torch.float32, device=v.device) * 2 - 1).to(dtype)
    return ret


class EA(SimA):
  """bench/ea.mlir:13-17: out = softmax(q over features) (softmax(k over the sequence)^T v)."""

  def forward(self, q, k, v):
    self._check(q)
    return ops.ea_fwd(q, k, v)

  def prepare(self, batch_size=8, q_len=8192, kv_len=None, dtype=torch.float16, device=None):
    return _Case.prepare(self, batch_size, q_len, q_len, dtype, device)


CASES = {"EA": EA, "Attn": Attn, "Gemma2": Gemma2, "SnapKV": SnapKV, "Corm": Corm, "H2O": H2O, "KeyFormer": KeyFormer, "RoCo": RoCo, "SimA": SimA}


def get_model(name="H2O", **kwargs):
  """Factory in the spirit of each reference module's ``get_model()``."""
  return CASES[name](**kwargs)
