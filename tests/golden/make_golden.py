"""Generates the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Run once where the reference checkout is mounted:

    python tests/golden/make_golden.py /root/reference

It imports the reference's own eager modules (cases/kernels/{attn,h2o,kf,roco,gemma2,snapkv,corm}.py),
unmodified,
runs their ``forward`` on the CPU in fp32 on seeded inputs that were first rounded to fp16/bf16,
and stores inputs (16-bit) and outputs (fp32) as compressed .npz files.  The tests compare the CPU
oracle (oracle/attn_oracle.py) and the CUDA kernels against these files; neither the tests nor the
product read the reference checkout at run time.

The reference modules evaluate ``torch.cuda.current_device()`` in a default argument at class
definition time, which raises on a host without a driver; it is replaced by a stub that returns
"cpu" for the duration of the import.  Nothing else of the reference is touched.
"""
import importlib
import os
import sys

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


if __name__ == "__main__":
  main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
