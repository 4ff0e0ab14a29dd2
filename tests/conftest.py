import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def load_golden(name):
  """Fixture written by tests/golden/make_golden.py from the reference's own eager modules."""
  z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
  dtype = torch.bfloat16 if str(z["dtype"]) == "bf16" else torch.float16
  d = {"dtype": dtype}
  for key in ("q", "k", "v"):
    d[key] = torch.from_numpy(z[key].copy()).view(dtype)
  if "exp_rand" in z.files:
    d["exp_rand"] = torch.from_numpy(z["exp_rand"].copy())
    d["tau"] = float(z["tau"])
  for key in ("corm_mask",):
    if key in z.files:
      d[key] = torch.from_numpy(z[key].copy())
  for key in ("softcap", "kernel_size", "head_num", "kv_head_num", "masked"):
    if key in z.files:
      d[key] = z[key].item()
  d["outs"] = [torch.from_numpy(z[f"out{i}"].copy()) for i in range(4) if f"out{i}" in z.files]
  return d


GOLDEN_NAMES = ["attn_f16_s256", "attn_f16_q128_kv320", "h2o_f16_b2_s192", "kf_f16_s256",
                "roco_bf16_s256", "gemma2_f16_s256", "snapkv_f16_s256", "corm_f16_s256"]
# grouped-query fixtures from the reference's 2-D scripts (cases/attn.py, cases/attn_h2o.py):
# q [q_len, H*128], k and v [kv_len, Hkv*128]
GQA_GOLDEN_NAMES = ["gqa_h2o_f16_s256_h8_kv2", "gqa_h2o_bf16_q100_kv333_h6_kv3",
                    "gqa_h2o_f16_s200_h4_kv1_nomask", "gqa_attn_f16_s320_h6_kv2"]


@pytest.fixture(scope="session")
def built_lib():
  """The in-tree CUDA library, built if missing (nvcc cross-compiles without a GPU)."""
  from flashtensor_b200 import build
  return build.build()
