#!/usr/bin/env python
"""Benchmark of the fused-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--case h2o|attn|roco|keyformer|keyformer_seeded|sima|ea]
    python bench.py --impl reference ...      # the reference's CPU eager path on the host cores

One "step" is one call of the case on one batch of synthetic inputs.  The default workload is the
configuration the headline metric is quoted on: H2O prefill, fp16, B=1, H=32, S=4096, D=128, keep
top-k = S/8 heavy hitters plus the last 256 tokens.  With N GPUs that ONE configuration is split by
(batch, head): rank r owns a contiguous range of the B*H units (flashtensor_b200.sharding), its
slices are resident before the timed region, there is no collective on the data path, and the time
of a step is the maximum over ranks of the device time (strong scaling).  `--scaling weak` runs the
whole configuration on every rank instead (independent replicas); the default N>1 run reports that
number too, as the secondary key `replicas`.

Rank 0 prints ONE JSON line:
  value        algorithmic TFLOP/s of the whole job, inputs resident in HBM: median over `repeats`
               timed loops of `steps` calls each (per loop: maximum over ranks); each call
               replays the CUDA graph of the case's kernels for that input set (--no-graphs:
               calls the case directly, which at small shapes measures the host)
  e2e          the same metric through the public per-case callable with HOST buffers: the timed
               region holds, for every step, the host->device copies of q, k, v from pinned memory
               and the device->host copies of every result; the package's host front end
               (flashtensor_b200.host.HostPipeline) keeps two calls in flight on three streams
  roofline     the dominant kernel (attention forward) timed alone with CUDA events
  cpu_baseline the CPU oracle port timed on a bounded sample of the same workload (rank 0, N=1)
  per_rank     every rank's own time per step, SM clock under load and throttle reasons
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

E2E_DEPTH = 2


def measured_dram_traffic(case):
  """DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of
  one profiler capture at this workload), read from the committed capture summary; None when no
  capture of this workload is on file."""
  import re
  name = {"h2o": "attn_fwd_h2o_c2.md"}.get(case)
  if name is None:
    return None
  try:
    with open(os.path.join(ROOT, "profiles", name)) as f:
      m = re.search(r"dram_bytes_per_launch\s*[:=]\s*(\d+)", f.read())
    return int(m.group(1)) if m else None
  except OSError:
    return None


def config_of(case, w, world, scaling):
  """The `config` object of the JSON line; a function of the workload and the launch alone, so the
  library arm and the reference arm print the same one."""
  units = w["B"] * w["H"]
  set_bytes = input_set_bytes(case, w, units if scaling == "weak" else -(-units // world))
  n_sets = n_input_sets(set_bytes)
  if scaling == "strong":
    par = (f"one configuration, its {units} (batch,head) units split over {world} GPU(s) in contiguous "
           "ranges, no collective")
    gb, per = w["B"], -(-units // world)
  else:
    par = f"{world} independent replica(s) of the configuration, no collective"
    gb, per = w["B"] * world, units
  return {"workload": w["desc"], "global_batch": gb, "per_gpu_units": per, "parallelism": par,
          "l2": f"inputs rotate over {n_sets} sets of {set_bytes / 1e6:.0f} MB per GPU (L2 is 126 MB), no flush"}


def input_set_bytes(case, w, units):
  n = 3 * units * w["S"] * 128 * 2
  if case == "keyformer":
    n += units * w["S"] * w["S"] * 4
  return n


def n_input_sets(set_bytes):
  """Enough input sets that a step never finds its inputs in the 126 MB L2."""
  return max(2, min(6, int(300e6 // set_bytes) + 1)) if set_bytes < 1.2e9 else 2


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

  def __init__(self, gpu_id):
    self.rows, self.windows, self.proc = [], [], None
    gpu_index = gpu_id
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
    return lambda q, k, v: m.seeded(q, k, v, w["seed"], w["k_keep"], unit_offset=w.get("unit_offset", 0))
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


_REF_MODELS = {}


def reference_eager_model(case, w, ref_root, heads):
  """The reference's own eager module for the case, imported unmodified from a checkout the user
  points at with --reference-root (cases/kernels/{attn,h2o,kf,roco}.py); None if there is none."""
  names = {"attn": ("attn", "Attn"), "h2o": ("h2o", "H2O"), "roco": ("roco", "RoCo"),
           "keyformer": ("kf", "KeyFormer"), "keyformer_seeded": ("kf", "KeyFormer")}
  if not ref_root or case not in names:
    return None
  key = (case, heads)
  if key not in _REF_MODELS:
    import importlib
    mod_name, cls = names[case]
    path = os.path.join(ref_root, "cases")
    if path not in sys.path:
      sys.path.insert(0, path)
    real = torch.cuda.current_device
    if not torch.cuda.is_available():
      torch.cuda.current_device = lambda: "cpu"   # evaluated in a default argument at import
    try:
      mod = importlib.import_module(f"kernels.{mod_name}")
    finally:
      torch.cuda.current_device = real
    _REF_MODELS[key] = getattr(mod, cls)(kv_head_num=heads, head_num=heads, head_dim=128)
  return _REF_MODELS[key]


def cpu_oracle_sample(case, w, heads, threads, ref_root=None):
  """One timed pass of the CPU implementation over `heads` heads of one batch element: the
  reference's own eager module when a checkout was given, else the oracle port of it; the
  selection always comes from the oracle (the reference has none)."""
  from oracle import attn_oracle as O
  torch.set_num_threads(threads)
  ref_model = reference_eager_model(case, w, ref_root, heads)
  dtype = torch.float16 if w["dtype"] == "f16" else torch.bfloat16
  ins = O.make_inputs("sima" if case in STREAMING else ("keyformer" if case == "keyformer" else "h2o"),
                      1, w["S"], w["S"], heads, 128, dtype, seed=0)
  ins = [t.float() for t in ins]
  t0 = time.time()
  with torch.no_grad():
    if case == "keyformer_seeded":
      ins = ins[:3] + [O.keyformer_seeded_exp_rand(w["seed"], 1, heads, w["S"], w["S"])]
    if ref_model is not None:
      outs = ref_model.forward(*ins)
      outs = outs if isinstance(outs, tuple) else (outs,)
    elif case == "attn":
      outs = (O.attn(*ins),)
    elif case == "h2o":
      outs = O.h2o(*ins)
    elif case == "roco":
      outs = O.roco(*ins)
    elif case in ("keyformer", "keyformer_seeded"):
      outs = O.keyformer(*ins, tau=w["tau"])
    elif case == "ea":
      outs = (O.ea(*ins),)
    else:
      outs = (O.sima(*ins),)
  if case == "h2o":
    O.h2o_select(outs[1].numpy(), w["k_keep"], w["recent"])
  elif case == "roco":
    O.roco_select(outs[1].numpy(), outs[2].numpy(), w["k_keep"], w["S"])
  elif case in ("keyformer", "keyformer_seeded"):
    O.keyformer_select(outs[1].numpy(), w["k_keep"])
  dt = time.time() - t0
  from flashtensor_b200 import utils
  fl = utils.sima_flops(1, heads, w["S"]) if case in STREAMING else utils.causal_flops(1, heads, w["S"], w["S"])
  return dt, fl


def run_reference(args, w, rank, world):
  """The reference's own CPU implementation of the path, all host threads: its eager module when
  --reference-root points at a checkout, else the restatement of it in oracle/."""
  if rank != 0:
    return
  threads = os.cpu_count() or 1
  ref_root = args.reference_root
  kind = "reference" if reference_eager_model(args.case, w, ref_root, 1) is not None else "port"
  # bounded sample: as many heads per step as keep the whole run near two minutes
  dt1, _ = cpu_oracle_sample(args.case, w, 1, threads, ref_root)
  heads = max(1, min(w["H"], int(120.0 / max(1, args.steps + args.warmup) / max(dt1, 1e-3))))
  for _ in range(args.warmup):
    cpu_oracle_sample(args.case, w, heads, threads, ref_root)
  dts, fl = [], 0
  for _ in range(args.steps):
    dt, fl = cpu_oracle_sample(args.case, w, heads, threads, ref_root)
    dts.append(dt)
  mean = sum(dts) / len(dts)
  value = fl / mean / 1e12
  sample = f"{heads} of {w['H']} heads of one batch element per step, all kernels of the case incl. selection"
  line = {
      "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
      "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
      "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
      "config": config_of(args.case, w, world, args.scaling),
      "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample,
                       "arithmetic": "f32 on the host cores"},
      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }
  print(json.dumps(line), flush=True)


def gpu_uuid(index):
  try:
    return "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
  except Exception:
    return str(index)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=10)
  ap.add_argument("--repeats", type=int, default=0, help="timed loops of --steps calls (0: ten)")
  ap.add_argument("--case", default="h2o", choices=sorted(WORKLOADS))
  ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
  ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                  help="strong: one configuration split by (batch, head) over the GPUs; weak: a replica per GPU")
  ap.add_argument("--reference-root", default=os.environ.get("ASUKA_REFERENCE_ROOT"),
                  help="a checkout of the reference: the CPU legs then time its own eager modules")
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--no-graphs", action="store_true",
                  help="call the case directly for every timed step instead of replaying its CUDA graph")
  args = ap.parse_args()
  args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
  w = WORKLOADS[args.case]

  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))

  if args.impl == "reference":
    run_reference(args, w, rank, world)
    return

  if not torch.cuda.is_available():
    raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
  import torch.distributed as dist
  from flashtensor_b200 import ops, sharding
  torch.cuda.set_device(local_rank)
  device = torch.device("cuda", local_rank)
  if world > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  def gather_rows(xs):
    """[n] floats of this rank -> [world][n] on every rank."""
    t = torch.tensor(xs, device=device, dtype=torch.float64)
    if world == 1:
      return [t.tolist()]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]

  units = w["B"] * w["H"]
  flops_total = flops_of(args.case, w, w["B"])

  def local_inputs(seed, whole):
    """One input set of this rank: the whole configuration, or this rank's units of it folded
    into the head axis ([1, S, n_local, 128]; exact, every unit is independent)."""
    full = make_inputs(args.case, w, w["B"], device, seed)
    if whole:
      return full
    ins = [sharding.shard_bshd(t, rank, world) for t in full[:3]]
    if len(full) > 3:
      ins.append(sharding.shard_bhs(full[3], rank, world))
    return ins

  def measure(step, sets, repeats):
    """`repeats` timed loops of --steps calls; per loop the maximum over ranks; median over loops."""
    n_sets = len(sets)
    for i in range(args.warmup):
      step(*sets[i % n_sets])
    barrier()
    mine, t_begin = [], time.time()
    count = (lambda: step.launches) if hasattr(step, "launches") else ops.launch_count
    launches0 = count()
    for _ in range(repeats):
      barrier()
      ms, _, _ = timed_loop(lambda i: step(*sets[i % n_sets]), args.steps)
      mine.append(ms / args.steps)
    launches = (count() - launches0) // repeats
    t_end = time.time()
    barrier()
    rows = gather_rows(mine)                                     # [world][repeats]
    worst = [max(rows[r][i] for r in range(world)) for i in range(repeats)]
    return {"ms": statistics.median(worst), "min": min(worst), "max": max(worst),
            "per_rank": [statistics.median(r) for r in rows], "launches": launches,
            "window": (t_begin, t_end)}

  def run_mode(scaling, want_e2e):
    lo, hi = sharding.unit_range(units, rank, world)
    whole = scaling == "weak" or world == 1
    n_local = units if whole else hi - lo
    ww = w if whole else dict(w, H=n_local, unit_offset=lo)   # (the seeded noise is keyed by the global unit index)
    step = build_step(args.case, ww)
    set_bytes = input_set_bytes(args.case, w, n_local)
    n_sets = n_input_sets(set_bytes)
    sets = [local_inputs(1000 + s, whole) for s in range(n_sets)]
    res = {"n_local": n_local, "sets": sets, "step": step, "ww": ww, "whole": whole}
    step(*sets[0])
    torch.cuda.synchronize()
    t0 = time.time()
    for i in range(3):
      step(*sets[i % n_sets])
    torch.cuda.synchronize()
    est_ms = (time.time() - t0) / 3 * 1e3
    # ten loops by default: long enough for a median and a spread, short enough (~0.1 s) that the
    # clocks are those of a burst, like the measured peak the roofline divides by
    repeats = args.repeats if args.repeats > 0 else 10
    if world > 1:   # every rank must run the same number of loops
      t = torch.tensor([repeats], device=device)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      repeats = int(t.item())
    res["repeats"] = repeats
    resident_step = step
    if not args.no_graphs:
      # the kernels of a call, recorded once per input set and replayed: the host then spends one
      # launch per call instead of descriptors, allocations and up to four launches
      from flashtensor_b200.host import GraphedCall
      resident_step = GraphedCall(step, max_graphs=n_sets)
      for s_ in sets:
        resident_step(*s_)
      torch.cuda.synchronize()
    res["resident"] = measure(resident_step, sets, repeats)
    if want_e2e:
      from flashtensor_b200.host import HostPipeline
      host_in = [t.cpu().pin_memory() for t in sets[0]]
      first = step(*sets[0])
      host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in first]
      del first
      res["h2d"] = sum(t.numel() * t.element_size() for t in host_in)
      res["d2h"] = sum(t.numel() * t.element_size() for t in host_out)
      pipe = HostPipeline(step, sets[0], depth=E2E_DEPTH, device=device)
      e2e_steps = max(3, min(args.steps, 50))
      for i in range(3):
        pipe.submit(host_in, host_out)
      pipe.drain()
      mine, t_begin = [], time.time()
      for _ in range(3):
        barrier()
        ms_e, _, _ = timed_loop(lambda i: pipe.submit(host_in, host_out), e2e_steps, begin=pipe.begin, join=pipe.join)
        pipe.drain()
        mine.append(ms_e / e2e_steps)
      t_end = time.time()
      barrier()
      rows = gather_rows(mine)
      worst = [max(rows[r][i] for r in range(world)) for i in range(3)]
      res["e2e"] = {"ms": statistics.median(worst), "per_rank": [statistics.median(r) for r in rows],
                    "steps": e2e_steps, "window": (t_begin, t_end)}
      del pipe, host_in, host_out
    return res

  sampler = ClockSampler(gpu_uuid(local_rank))
  main_mode = run_mode(args.scaling, not args.no_e2e)
  ms_per_step = main_mode["resident"]["ms"]
  value = flops_total * (world if args.scaling == "weak" else 1) / (ms_per_step * 1e-3) / 1e12
  sampler.window(*main_mode["resident"]["window"])
  if "e2e" in main_mode:
    sampler.window(*main_mode["e2e"]["window"])

  # ---- the split against the unsplit run: every rank's outputs are the same bits as its units of
  # ---- the whole configuration computed on one GPU (not timed)
  shard_check = None
  if world > 1 and args.scaling == "strong":
    full = local_inputs(1000, True)
    outs_full = build_step(args.case, w)(*full)
    outs_mine = main_mode["step"](*main_mode["sets"][0])
    same, worst_rel, idx_rows = True, 0.0, 0
    for a, b in zip(outs_full, outs_mine):
      want = sharding.shard_bshd(a, rank, world) if a.dim() == 4 else sharding.shard_bhs(a, rank, world)
      same = same and bool(torch.equal(want, b))
      if want.dtype == torch.int32:
        idx_rows += int((want != b).any(dim=-1).sum().item())
      else:
        d = (want.float() - b.float()).abs().max() / want.float().abs().max().clamp_min(1e-30)
        worst_rel = max(worst_rel, float(d.item()))
    t = torch.tensor([0.0 if same else 1.0, worst_rel, float(idx_rows)], device=device, dtype=torch.float64)
    agg = t.clone()
    dist.all_reduce(agg, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    if agg[0].item() == 0:
      shard_check = "every rank's outputs equal, bit for bit, its units of the unsplit run"
    else:
      # a rank with few units splits its work items further (key ranges, query ranges), which
      # changes the order of the f32 sums: the comparison is then by tolerance
      shard_check = (f"ranks' outputs against their units of the unsplit run: max|d|/max|ref| {agg[1].item():.2e} "
                     f"(tolerance 1e-2), kept-index rows that differ (near-ties): {int(t[2].item())} of {units}")
    del full, outs_full, outs_mine

  # ---- the dominant kernel alone, for the roofline -----------------------------------------
  pk = peaks()
  sets, n_sets, ww = main_mode["sets"], len(main_mode["sets"]), main_mode["ww"]
  flops_local = flops_of(args.case, ww, 1 if not main_mode["whole"] else w["B"])
  if args.case in STREAMING:
    algo = io_bytes_of(args.case, ww, 1 if not main_mode["whole"] else w["B"])
    achieved = algo / (main_mode["resident"]["per_rank"][rank] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "sima_stats + sima_reduce + sima_out in EA mode (whole step)"
                if args.case == "ea" else "sima_fused_kernel (whole step: statistics, reduce and output in one launch)",
                "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                "algorithmic_bytes_per_launch": algo}
  else:
    outs_k = [torch.empty_like(s[0]) for s in sets]
    fwd = lambda q, k, v, o: ops.attn_fwd(q, k, v, causal=True, return_lse=True, out=o)
    if not args.no_graphs:   # (a direct call costs the host more than this kernel takes at small shapes)
      from flashtensor_b200.host import GraphedCall
      fwd = GraphedCall(fwd, max_graphs=n_sets)
    kern = lambda i: fwd(sets[i % n_sets][0], sets[i % n_sets][1], sets[i % n_sets][2], outs_k[i % n_sets])
    for i in range(max(3, n_sets)):
      kern(i)
    barrier()
    reps, t_begin = [], time.time()
    for _ in range(10):
      ms_k, _, _ = timed_loop(kern, args.steps)
      reps.append(ms_k / args.steps * 1e3)
    sampler.window(t_begin, time.time())
    barrier()
    us_kernel = statistics.median(reps)
    achieved = flops_local / (us_kernel * 1e-6) / 1e12
    peak = pk["tf_burst"]
    roofline = {"bound": "tensor", "kernel": "attn_fwd_kernel", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": measured_dram_traffic(args.case) if main_mode["whole"] else None,
                "peak_source": pk["source"] + " burst",
                "us_per_launch": us_kernel, "us_min": min(reps), "us_max": max(reps),
                "algorithmic_flops_per_launch": flops_local,
                "frac_of_nominal_2250": achieved / 2250.0,
                "executed_flops_per_step": flops_local * (1.5 if args.case != "attn" else 1.0)}

  # ---- secondary: independent replicas (the whole configuration on every GPU) ----------------
  replicas = None
  if world > 1 and args.scaling == "strong":
    main_mode["sets"] = sets = None
    torch.cuda.empty_cache()
    rep = run_mode("weak", False)
    replicas = {"value": flops_total * world / (rep["resident"]["ms"] * 1e-3) / 1e12, "unit": UNIT,
                "ms_per_step": rep["resident"]["ms"], "scaling": "weak",
                "per_rank_ms": rep["resident"]["per_rank"]}
    sampler.window(*rep["resident"]["window"])
    del rep

  clocks = sampler.stop()
  status = ops.device_status()

  # ---- every rank's own numbers ------------------------------------------------------------
  reason_bits = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
  mask = sum(1 << i for i, n in enumerate(reason_bits) if n in clocks["reasons"])
  rows = gather_rows([clocks["sm_mhz"] or 0.0, float(mask), float(clocks["samples"])])
  per_rank = []
  for r in range(world):
    entry = {"rank": r, "ms_per_step": main_mode["resident"]["per_rank"][r], "sm_mhz": rows[r][0],
             "reasons": [n for i, n in enumerate(reason_bits) if int(rows[r][1]) >> i & 1],
             "clock_samples": int(rows[r][2])}
    if "e2e" in main_mode:
      entry["e2e_ms_per_step"] = main_mode["e2e"]["per_rank"][r]
    per_rank.append(entry)
  if "e2e" in main_mode:
    h2d_rows = gather_rows([float(main_mode["h2d"]), float(main_mode["d2h"])])
    for r in range(world):
      per_rank[r]["h2d_gbs"] = h2d_rows[r][0] / (per_rank[r]["e2e_ms_per_step"] * 1e-3) / 1e9
    h2d_total = int(sum(x[0] for x in h2d_rows))
    d2h_total = int(sum(x[1] for x in h2d_rows))
  all_reasons = sorted({n for e in per_rank for n in e["reasons"]})

  # ---- CPU baseline: the CPU implementation on a bounded sample (rank 0, N = 1) --------------
  cpu = None
  if rank == 0 and world == 1 and not args.no_cpu_baseline:
    threads = os.cpu_count() or 1
    ref_root = args.reference_root
    kind = "reference" if reference_eager_model(args.case, w, ref_root, 1) is not None else "port"
    dt1, _ = cpu_oracle_sample(args.case, w, 1, threads, ref_root)    # warm-up and size estimate
    heads = max(1, min(w["H"], int(4.0 / max(dt1, 1e-3))))            # ~4 s per pass
    passes, spent, fl_total = 0, 0.0, 0
    while spent < 12.0 and passes < 64:                               # ~12-20 s of CPU work in all
      dt, fl = cpu_oracle_sample(args.case, w, heads, threads, ref_root)
      spent += dt
      fl_total += fl
      passes += 1
    cpu = {"value": fl_total / spent / 1e12, "unit": UNIT, "cores": threads, "kind": kind,
           "sample": f"{heads} of {w['H']} heads of one batch element x {passes} passes ({spent:.1f} s), "
                     "all kernels of the case incl. selection"}

  if rank == 0:
    res = main_mode["resident"]
    sm = clocks["sm_mhz"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "us_per_call": ms_per_step * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": config_of(args.case, w, world, args.scaling),
        "repeats": {"n": main_mode["repeats"], "steps_each": args.steps, "ms_per_step_median": res["ms"],
                    "ms_per_step_min": res["min"], "ms_per_step_max": res["max"],
                    "ms_times_sm_mhz": res["ms"] * sm if sm else None},
        "gpu_launches": res["launches"],
        "launch_mode": ("direct calls of the case" if args.no_graphs else
                        "CUDA graph of one call per input set, replayed (flashtensor_b200.host.GraphedCall)"),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "clocks": {"sm_mhz": sm, "sm_max_mhz": clocks["sm_max_mhz"], "reasons": all_reasons,
                   "samples": clocks["samples"]},
        "per_rank": per_rank,
        "frac_of_nominal_2250": value / world / 2250.0,
        "device_timeouts": status[0],
    }
    if "e2e" in main_mode:
      e = main_mode["e2e"]
      e2e_value = flops_total * (world if args.scaling == "weak" else 1) / (e["ms"] * 1e-3) / 1e12
      line["e2e"] = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_total,
                     "d2h_bytes_per_step": d2h_total, "ms_per_step": e["ms"], "steps": e["steps"],
                     "pipeline": f"flashtensor_b200.host.HostPipeline, {E2E_DEPTH} calls in flight "
                                 "(copy-in / case / copy-out streams); bytes are the whole job's, all ranks"}
    if shard_check:
      line["shard_check"] = shard_check
    if replicas:
      line["replicas"] = replicas
    print(json.dumps(line), flush=True)
  if world > 1:
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
