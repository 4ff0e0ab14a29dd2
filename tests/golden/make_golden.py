"""Generates the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Run once where the reference checkout is mounted:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports the reference's own eager modules (cases/kernels/{attn,h2o,kf,roco,gemma2,snapkv,corm}.py),
unmodified,
runs their ``forward`` on the CPU in fp32 on seeded inputs that were first rounded to fp16/bf16,
and stores inputs (16-bit) and outputs (fp32) as compressed .npz files.  The tests compare the CPU
oracle (oracle/attn_oracle.py) and the CUDA kernels against these files; neither the tests nor the
product read the reference checkout at run time.

The reference modules evaluate ``torch.cuda.current_device()`` in a default argument at class
definition time, which raises on a host without a driver; it is replaced by a stub that returns
"cpu" for the duration of the import.  Nothing else of the reference is touched.

The grouped-query fixtures come from the reference's 2-D scripts cases/attn.py (``Attn``) and
cases/attn_h2o.py (``AttnH2O``).  Those import ``onnx`` and ``onnxsim`` at module top (for the
export their ``main`` does); neither package is needed by ``forward``, so empty stand-in modules
are registered under those names for the duration of the import.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, module, class, B, Sq, Skv, H, dtype, seed
CASES = [
    ("attn_f16_s256", "attn", "Attn", 1, 256, 256, 2, torch.float16, 11),
    ("attn_f16_q128_kv320", "attn", "Attn", 1, 128, 320, 1, torch.float16, 12),
    ("h2o_f16_b2_s192", "h2o", "H2O", 2, 192, 192, 2, torch.float16, 13),
    ("kf_f16_s256", "kf", "KeyFormer", 1, 256, 256, 2, torch.float16, 14),
    ("roco_bf16_s256", "roco", "RoCo", 1, 256, 256, 2, torch.bfloat16, 15),
    ("gemma2_f16_s256", "gemma2", "Gemma2", 1, 256, 256, 2, torch.float16, 16),
    ("snapkv_f16_s256", "snapkv", "SnapKV", 1, 256, 256, 2, torch.float16, 17),
    ("corm_f16_s256", "corm", "Corm", 1, 256, 256, 2, torch.float16, 18),
]

# name, script, class, q_len, kv_len, head_num, kv_head_num, masked, dtype, seed
# (2-D layout of the scripts: q [q_len, H*128], k and v [kv_len, Hkv*128])
GQA_CASES = [
    ("gqa_h2o_f16_s256_h8_kv2", "attn_h2o", "AttnH2O", 256, 256, 8, 2, True, torch.float16, 21),
    ("gqa_h2o_bf16_q100_kv333_h6_kv3", "attn_h2o", "AttnH2O", 100, 333, 6, 3, True, torch.bfloat16, 22),
    ("gqa_h2o_f16_s200_h4_kv1_nomask", "attn_h2o", "AttnH2O", 200, 200, 4, 1, False, torch.float16, 23),
    ("gqa_attn_f16_s320_h6_kv2", "attn", "Attn", 320, 320, 6, 2, True, torch.float16, 24),
]


def bits16(t):
  return t.view(torch.int16).numpy().copy()


def main(ref_root):
  sys.path.insert(0, os.path.join(ref_root, "cases"))
  real = torch.cuda.current_device
  torch.cuda.current_device = lambda: "cpu"
  try:
    mods = {m: importlib.import_module(f"kernels.{m}")
            for m in ("attn", "h2o", "kf", "roco", "gemma2", "snapkv", "corm")}
  finally:
    torch.cuda.current_device = real
  for name, mod, cls, B, Sq, Skv, H, dtype, seed in CASES:
    model = getattr(mods[mod], cls)(kv_head_num=H, head_num=H, head_dim=128)
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, Sq, H, 128, generator=g).to(dtype)
    k = torch.randn(B, Skv, H, 128, generator=g).to(dtype)
    v = torch.randn(B, Skv, H, 128, generator=g).to(dtype)
    args = [q.float(), k.float(), v.float()]
    save = {"q": bits16(q), "k": bits16(k), "v": bits16(v),
            "dtype": np.array("bf16" if dtype == torch.bfloat16 else "f16")}
    if cls == "KeyFormer":
      er = 1 + torch.randn(B, H, Sq, Skv, generator=g).abs()
      args.append(er)
      save["exp_rand"] = er.numpy()
      save["tau"] = np.float32(model.tau)
    if cls == "Corm":
      cm = torch.ones(Sq, Skv)
      for i in range(Sq):                 # as the reference's prepare, cases/kernels/corm.py:46-48
        cm[i] /= i + 1
      args.append(cm)
      save["corm_mask"] = cm.numpy()
    if cls == "Gemma2":
      # N(0,1) inputs never reach the cap of 50; scale q so that the tanh actually bends the logits
      q = (q.float() * 12).to(dtype)
      args[0] = q.float()
      save["q"] = bits16(q)
      save["softcap"] = np.float32(model.logit_softcapping)
    if cls == "SnapKV":
      save["kernel_size"] = np.int32(model.kernel_size)
    with torch.no_grad():
      outs = model.forward(*args)
    outs = outs if isinstance(outs, tuple) else (outs,)
    for i, o in enumerate(outs):
      save[f"out{i}"] = o.numpy() if o.dtype == torch.bool else o.float().numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **save)
    print(name, [tuple(o.shape) for o in outs], os.path.getsize(path) // 1024, "KiB")
  make_gqa(ref_root)


def make_gqa(ref_root):
  """Fixtures from the unmodified AttnH2O / Attn modules of the reference's 2-D scripts."""
  stubs = {}
  for name in ("onnx", "onnxsim"):
    if name not in sys.modules:
      stubs[name] = sys.modules[name] = types.ModuleType(name)
  try:
    sys.path.insert(0, os.path.join(ref_root, "cases"))
    scripts = {m: importlib.import_module(m) for m in ("attn_h2o", "attn")}
  finally:
    for name in stubs:
      del sys.modules[name]
  for name, script, cls, q_len, kv_len, H, Hkv, masked, dtype, seed in GQA_CASES:
    model = getattr(scripts[script], cls)(Hkv, H, 128, masked)
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(q_len, H * 128, generator=g).to(dtype)
    k = torch.randn(kv_len, Hkv * 128, generator=g).to(dtype)
    v = torch.randn(kv_len, Hkv * 128, generator=g).to(dtype)
    with torch.no_grad():
      outs = model.forward(q.float(), k.float(), v.float())
    outs = outs if isinstance(outs, tuple) else (outs,)
    save = {"q": bits16(q), "k": bits16(k), "v": bits16(v),
            "dtype": np.array("bf16" if dtype == torch.bfloat16 else "f16"),
            "head_num": np.int32(H), "kv_head_num": np.int32(Hkv), "masked": np.int32(masked)}
    for i, o in enumerate(outs):
      save[f"out{i}"] = o.float().numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **save)
    print(name, [tuple(o.shape) for o in outs], os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
  if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
  main(sys.argv[1])
