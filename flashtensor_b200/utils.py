"""Timing and error-metric helpers with the reference's conventions (python/asuka/utils.py)."""
import time

import numpy as np
import torch


def perf(label, f, args, kwargs={}, gflops=None, mem_gb=None, run=10, warmup=4, quiet=False):
  """Wall-clock timing between synchronisations, avg/min/max ms -- python/asuka/utils.py:28-58."""
  torch.cuda.synchronize()
  for _ in range(warmup):
    torch.cuda.synchronize()
    f(*args, **kwargs)
    torch.cuda.synchronize()
  ms = []
  for _ in range(run):
    torch.cuda.synchronize()
    tik = time.time()
    f(*args, **kwargs)
    torch.cuda.synchronize()
    ms.append((time.time() - tik) * 1000.0)
  res = {"label": label, "avg_ms": float(np.mean(ms)), "min_ms": float(np.min(ms)),
         "max_ms": float(np.max(ms)), "run": run, "warmup": warmup}
  msg = f"[{label}] avg {res['avg_ms']:.4f} ms, min {res['min_ms']:.4f} ms, max {res['max_ms']:.4f} ms"
  if gflops is not None:
    res["gflops_per_s"] = gflops / (res["avg_ms"] / 1000.0)
    msg += f", {res['gflops_per_s']} gflops/s"
  if mem_gb is not None:
    res["gb_per_s"] = mem_gb / (res["avg_ms"] / 1000.0)
    msg += f", {res['gb_per_s']} gb/s"
  if not quiet:
    print(msg + f" ({run} runs, {warmup} warmups)")
  return res


def loss(out, ref, remove_zero=False):
  """Mismatch count for integers; abs/rel max/mean for floats -- python/asuka/utils.py:61-76."""
  assert out.shape == ref.shape, f"{out.shape=} {ref.shape=}"
  if out.dtype in {torch.int32, torch.int64}:
    err_num = torch.sum(out != ref).item()
    return {"err_num": err_num, "err": err_num / out.numel()}
  diff = (out.float() - ref.float())
  deno = ref.float().abs()
  if remove_zero:
    deno = deno.clone()
    deno[deno == 0] = 1.0
  return {"abs_max": diff.abs().max().item(), "abs_mean": diff.abs().mean().item(),
          "rel_max": (diff / deno).abs().max().item(), "rel_mean": (diff / deno).abs().mean().item(),
          "remove_zero": remove_zero}


def causal_flops(B, H, Sq, Skv, D=128, causal=True):
  """Flops of the two contractions of the eager definition over the unmasked region only:
  query i sees keys 0 .. i + (Skv - Sq)."""
  off = Skv - Sq
  visible = Sq * (off + 1) + Sq * (Sq - 1) // 2 if causal else Sq * Skv
  return 4 * B * H * D * visible


def sima_flops(B, H, S, D=128):
  return 4 * B * H * S * D * D
