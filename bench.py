#!/usr/bin/env python
"""Benchmark of the fused-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--case h2o|attn|roco|keyformer|keyformer_seeded|sima|ea]
    python bench.py --impl reference ...      # the reference's CPU eager path on the host cores

One "step" is one call of the case on one batch of synthetic inputs.  The default workload is the
configuration the headline metric is quoted on: H2O prefill, fp16, B=1, H=32, S=4096, D=128, keep
top-k = S/8 heavy hitters plus the last 256 tokens.  With N GPUs every rank runs that workload on
its own (batch, head) units (weak scaling: global batch = N), there is no collective on the data
path, and the time is the maximum over ranks of the device time.

Rank 0 prints ONE JSON line:
  value        algorithmic TFLOP/s of the whole job, inputs resident in HBM
  e2e          the same metric through the public per-case callable with HOST buffers: the timed
               region holds, for every step, the host->device copies of q, k, v from pinned memory
               and the device->host copies of every result; the package's host front end
               (flashtensor_b200.host.HostPipeline) keeps two calls in flight on three streams
  roofline     the dominant kernel (attention forward) timed alone with CUDA events
  cpu_baseline the CPU oracle port timed on a bounded sample of the same workload (rank 0, N=1)
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused_attn_tflops"
UNIT = "TFLOP/s"

# name -> (B, H, S, dtype, description)
WORKLOADS = {
    "attn": dict(B=1, H=32, S=1024, dtype="f16", desc="plain causal attention B1 H32 S1024 D128 (GPU run in fp16)"),
    "h2o": dict(B=1, H=32, S=4096, dtype="f16", k_keep=512, recent=256,
                desc="H2O prefill fp16 B1 H32 S4096 D128, top-k S/8 + 256 recent"),
    "keyformer": dict(B=4, H=32, S=2048, dtype="f16", k_keep=512, tau=1.5,
                      desc="Keyformer prefill fp16 B4 H32 S2048 D128 tau 1.5, top-k S/4, exp_rand operand"),
    "keyformer_seeded": dict(B=4, H=32, S=2048, dtype="f16", k_keep=512, tau=1.5, seed=2024,
                             desc="Keyformer prefill fp16 B4 H32 S2048 D128 tau 1.5, top-k S/4, Gumbel noise from seed"),
    "roco": dict(B=2, H=40, S=4096, dtype="bf16", k_keep=512,
                 desc="RoCo prefill bf16 B2 H40 S4096 D128, top-k S/8 by mean then std"),
    "sima": dict(B=8, H=32, S=8192, dtype="f16", desc="SimA fp16 B8 H32 S8192 D128 non-causal"),
    "ea": dict(B=8, H=32, S=8192, dtype="f16", desc="EA fp16 B8 H32 S8192 D128 (softmax over features of q, over the sequence of k)"),
}
STREAMING = ("sima", "ea")   # HBM-bound two-pass programs: no S x S product

# DRAM bytes per launch of the attention-forward kernel at the H2O workload, from the ncu capture
# summarised in profiles/attn_fwd_h2o_c2.md (dram__bytes_read.sum + dram__bytes_write.sum).
FWD_DRAM_TRAFFIC_BYTES = 160818944


E2E_DEPTH = 2


def peaks():
  """Measured peaks of this pool's B200s, else the documented fallback."""
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  try:
    with open(path) as f:
      p = json.load(f)
    return {"hbm_gbs": float(p["hbm_gbs"]), "tf_burst": float(p["bf16_tflops"]),
            "tf_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
  except Exception:
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "source": "fallback"}


def flops_of(case, w, batch):
  from flashtensor_b200 import utils
  if case in STREAMING:
    return utils.sima_flops(batch, w["H"], w["S"])
  return utils.causal_flops(batch, w["H"], w["S"], w["S"])


def io_bytes_of(case, w, batch):
  """Compulsory traffic: every input and output once at its storage width."""
  n = batch * w["S"] * w["H"] * 128 * 2
  total = 4 * n
  if case in ("h2o", "keyformer", "keyformer_seeded"):
    total += batch * w["H"] * w["S"] * 4
  if case == "roco":
    total += 2 * batch * w["H"] * w["S"] * 4
  if case == "keyformer":
    total += batch * w["H"] * w["S"] * w["S"] * 4
  return total


class ClockSampler:
  """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""
  FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
            "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_index):
    self.rows, self.windows, self.proc = [], [], None
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
           "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except Exception:
      self.proc = None

  def _read(self):
    for line in self.proc.stdout:
      self.rows.append((time.time(), line.strip()))

  def window(self, t0, t1):
    self.windows.append((t0, t1))

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    time.sleep(0.08)
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except Exception:
      self.proc.kill()
    sm, smax, reasons, n_in = [], None, set(), 0
    for ts, line in self.rows:
      parts = [x.strip() for x in line.split(",")]
      if len(parts) < 10:
        continue
      inside = any(t0 - 0.02 <= ts <= t1 + 0.06 for t0, t1 in self.windows)
      try:
        smax = float(parts[3])
        if inside:
          n_in += 1
          sm.append(float(parts[2]))
          for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                               parts[6:10]):
            if val.lower().startswith("active"):
              reasons.add(name)
      except ValueError:
        continue
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
            "reasons": sorted(reasons), "samples": n_in}


def make_inputs(case, w, batch, device, seed):
  dtype = torch.float16 if w["dtype"] == "f16" else torch.bfloat16
  g = torch.Generator(device=device).manual_seed(seed)
  shape = (batch, w["S"], w["H"], 128)
  q = torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(dtype)
  k = torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(dtype)
  if case == "sima":
    v = (torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 2 - 1).to(dtype)
  else:
    v = torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(dtype)
  ins = [q, k, v]
  if case == "keyformer":
    ins.append(1 + torch.randn(batch, w["H"], w["S"], w["S"], generator=g, device=device).abs())
  return ins


def build_step(case, w):
  """The public per-case callable a user of the reference would call."""
  import flashtensor_b200 as ft
  H = w["H"]
  if case == "attn":
    m = ft.Attn(head_num=H, kv_head_num=H)
    return lambda q, k, v: (m(q, k, v),)
  if case == "h2o":
    m = ft.H2O(head_num=H, kv_head_num=H)
    return lambda q, k, v: m.select(q, k, v, w["k_keep"], w["recent"])
  if case == "roco":
    m = ft.RoCo(head_num=H, kv_head_num=H)
    return lambda q, k, v: m.select(q, k, v, w["k_keep"])
  if case == "keyformer":
    m = ft.KeyFormer(tau=w["tau"], head_num=H, kv_head_num=H)
    return lambda q, k, v, er: m.select(q, k, v, er, w["k_keep"])
  if case == "keyformer_seeded":
    m = ft.KeyFormer(tau=w["tau"], head_num=H, kv_head_num=H)
    return lambda q, k, v: m.seeded(q, k, v, w["seed"], w["k_keep"])
  m = (ft.EA if case == "ea" else ft.SimA)(head_num=H, kv_head_num=H)
  return lambda q, k, v: (m(q, k, v),)


def timed_loop(fn, steps, begin=None, join=None):
  """Device time of `steps` back-to-back calls on torch's current stream (the launching stream).
  `begin` / `join` order side streams after the first event and before the second one."""
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  torch.cuda.synchronize()
  t0 = time.time()
  e0.record()
  if begin:
    begin()
  for i in range(steps):
    fn(i)
  if join:
    join()
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1), t0, time.time()


def cpu_oracle_sample(case, w, heads, threads):
  """One timed pass of the CPU oracle port over `heads` heads of one batch element."""
  from oracle import attn_oracle as O
  torch.set_num_threads(threads)
  dtype = torch.float16 if w["dtype"] == "f16" else torch.bfloat16
  ins = O.make_inputs("sima" if case in STREAMING else ("keyformer" if case == "keyformer" else "h2o"),
                      1, w["S"], w["S"], heads, 128, dtype, seed=0)
  ins = [t.float() for t in ins]
  t0 = time.time()
  if case == "attn":
    O.attn(*ins)
  elif case == "h2o":
    _, s = O.h2o(*ins)
    O.h2o_select(s.numpy(), w["k_keep"], w["recent"])
  elif case == "roco":
    _, s, s2 = O.roco(*ins)
    O.roco_select(s.numpy(), s2.numpy(), w["k_keep"], w["S"])
  elif case in ("keyformer", "keyformer_seeded"):
    if case == "keyformer_seeded":
      ins = ins[:3] + [O.keyformer_seeded_exp_rand(w["seed"], 1, heads, w["S"], w["S"])]
    _, s = O.keyformer(*ins, tau=w["tau"])
    O.keyformer_select(s.numpy(), w["k_keep"])
  elif case == "ea":
    O.ea(*ins)
  else:
    O.sima(*ins)
  dt = time.time() - t0
  from flashtensor_b200 import utils
  fl = utils.sima_flops(1, heads, w["S"]) if case in STREAMING else utils.causal_flops(1, heads, w["S"], w["S"])
  return dt, fl


def run_reference(args, w, rank):
  """The reference's own CPU implementation of the path: its eager definition, restated in
  oracle/ (the reference checkout is not present on the benchmark host), all host threads."""
  if rank != 0:
    return
  threads = os.cpu_count() or 1
  # bounded sample: as many heads per step as keep the whole run near two minutes
  dt1, _ = cpu_oracle_sample(args.case, w, 1, threads)
  heads = max(1, min(w["H"], int(120.0 / max(1, args.steps + args.warmup) / max(dt1, 1e-3))))
  for _ in range(args.warmup):
    cpu_oracle_sample(args.case, w, heads, threads)
  dts, fl = [], 0
  for _ in range(args.steps):
    dt, fl = cpu_oracle_sample(args.case, w, heads, threads)
    dts.append(dt)
  mean = sum(dts) / len(dts)
  value = fl / mean / 1e12
  sample = f"{heads} of {w['H']} heads of one batch element per step, all kernels of the case incl. selection"
  line = {
      "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
      "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
      "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
      "config": {"workload": w["desc"], "sample": sample},
      "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }
  print(json.dumps(line), flush=True)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=200)
  ap.add_argument("--warmup", type=int, default=10)
  ap.add_argument("--case", default="h2o", choices=sorted(WORKLOADS))
  ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
  ap.add_argument("--no-cpu-baseline", action="store_true")
  args = ap.parse_args()
  args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
  w = WORKLOADS[args.case]

  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))

  if args.impl == "reference":
    run_reference(args, w, rank)
    return

  if not torch.cuda.is_available():
    raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
  import torch.distributed as dist
  from flashtensor_b200 import ops
  torch.cuda.set_device(local_rank)
  device = torch.device("cuda", local_rank)
  if world > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  def max_over_ranks(x):
    if world == 1:
      return x
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()

  step = build_step(args.case, w)
  batch = w["B"]                       # per rank; the global batch is batch * world
  flops_rank = flops_of(args.case, w, batch)
  in_bytes = sum(t.numel() * t.element_size() for t in make_inputs(args.case, dict(w, S=128), 1, device, 0))
  del in_bytes
  # rotate over enough input sets that a step never finds its inputs in the 126 MB L2
  probe = make_inputs(args.case, w, batch, device, seed=1000 * rank)
  set_bytes = sum(t.numel() * t.element_size() for t in probe)
  n_sets = max(2, min(4, int(300e6 // set_bytes) + 1)) if set_bytes < 1.2e9 else 2
  sets = [probe] + [make_inputs(args.case, w, batch, device, seed=1000 * rank + s) for s in range(1, n_sets)]
  sampler = ClockSampler(local_rank) if rank == 0 else None

  # ---- (1) device-resident throughput -----------------------------------------------------
  for i in range(args.warmup):
    step(*sets[i % n_sets])
  barrier()
  launches0 = ops.launch_count()
  ms, t0, t1 = timed_loop(lambda i: step(*sets[i % n_sets]), args.steps)
  launches = ops.launch_count() - launches0
  barrier()
  if sampler:
    sampler.window(t0, t1)
  ms = max_over_ranks(ms)
  ms_per_step = ms / args.steps
  value = flops_rank * world / (ms_per_step * 1e-3) / 1e12

  # ---- (2) end to end through the public callable with host buffers ------------------------
  # Host buffers go through the package's host front end: copy-in, the case and copy-out run on
  # three streams with two calls in flight, so a steady stream of calls is bound by the slower
  # copy direction.  Every step still copies all its inputs in and all its results out.
  from flashtensor_b200.host import HostPipeline
  host_in = [t.cpu().pin_memory() for t in sets[0]]
  first = step(*sets[0])
  host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in first]
  del first
  h2d = sum(t.numel() * t.element_size() for t in host_in)
  d2h = sum(t.numel() * t.element_size() for t in host_out)
  pipe = HostPipeline(step, sets[0], depth=E2E_DEPTH, device=device)

  def e2e_step(_i):
    pipe.submit(host_in, host_out)

  e2e_steps = max(3, min(args.steps, 50))
  for i in range(3):
    e2e_step(i)
  pipe.drain()
  barrier()
  ms_e, t0, t1 = timed_loop(e2e_step, e2e_steps, begin=pipe.begin, join=pipe.join)
  pipe.drain()
  barrier()
  if sampler:
    sampler.window(t0, t1)
  ms_e = max_over_ranks(ms_e) / e2e_steps
  e2e_value = flops_rank * world / (ms_e * 1e-3) / 1e12

  # ---- (3) the dominant kernel alone, for the roofline -------------------------------------
  pk = peaks()
  if args.case in STREAMING:
    ms_k, t0, t1 = ms, None, None          # one HBM-bound pipeline: the step is the kernel chain
    algo = io_bytes_of(args.case, w, batch)
    achieved = algo / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": ("ea_colmax + " if args.case == "ea" else "") +
                "sima_stats + sima_reduce + sima_out (whole step)",
                "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                "algorithmic_bytes_per_launch": algo}
  else:
    outs_k = [torch.empty_like(s[0]) for s in sets]
    kern = lambda i: ops.attn_fwd(sets[i % n_sets][0], sets[i % n_sets][1], sets[i % n_sets][2],
                                  causal=True, return_lse=True, out=outs_k[i % n_sets])
    for i in range(3):
      kern(i)
    barrier()
    ms_k, t0, t1 = timed_loop(kern, args.steps)
    barrier()
    if sampler:
      sampler.window(t0, t1)
    us_kernel = ms_k / args.steps * 1e3
    achieved = flops_rank / (us_kernel * 1e-6) / 1e12
    sustained = ms_k > 1000.0
    peak = pk["tf_sustained"] if sustained else pk["tf_burst"]
    roofline = {"bound": "tensor", "kernel": "attn_fwd_kernel", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": FWD_DRAM_TRAFFIC_BYTES if args.case == "h2o" else None,
                "peak_source": pk["source"] + (" sustained" if sustained else " burst"),
                "us_per_launch": us_kernel, "algorithmic_flops_per_launch": flops_rank,
                "frac_of_nominal_2250": achieved / 2250.0,
                "executed_flops_per_step": flops_rank * (1.5 if args.case != "attn" else 1.0)}

  clocks = sampler.stop() if sampler else None
  status = ops.device_status()

  # ---- (4) CPU baseline: the oracle port on a bounded sample (rank 0, N = 1) ---------------
  cpu = None
  if rank == 0 and world == 1 and not args.no_cpu_baseline:
    threads = os.cpu_count() or 1
    dt1, _ = cpu_oracle_sample(args.case, w, 1, threads)             # warm-up and size estimate
    heads = max(1, min(w["H"], int(4.0 / max(dt1, 1e-3))))            # ~4 s per pass
    passes, spent, fl_total = 0, 0.0, 0
    while spent < 12.0 and passes < 64:                               # ~12-20 s of CPU work in all
      dt, fl = cpu_oracle_sample(args.case, w, heads, threads)
      spent += dt
      fl_total += fl
      passes += 1
    cpu = {"value": fl_total / spent / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": f"{heads} of {w['H']} heads of one batch element x {passes} passes ({spent:.1f} s), "
                     "all kernels of the case incl. selection"}

  if rank == 0:
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "us_per_call": ms_per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["desc"], "global_batch": batch * world, "per_gpu_units": batch * w["H"],
                   "parallelism": f"(batch,head) units sharded over {world} GPU(s), no collective",
                   "l2": f"inputs rotate over {n_sets} sets of {set_bytes / 1e6:.0f} MB (L2 is 126 MB), no flush"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e, "steps": e2e_steps,
                "pipeline": f"flashtensor_b200.host.HostPipeline, {E2E_DEPTH} calls in flight (copy-in / case / copy-out streams)"},
        "gpu_launches": launches,
        "roofline": roofline,
        "cpu_baseline": cpu,
        "clocks": clocks,
        "frac_of_nominal_2250": value / world / 2250.0,
        "device_timeouts": status[0],
    }
    print(json.dumps(line), flush=True)
  if world > 1:
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
