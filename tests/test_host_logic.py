"""CPU: the C-ABI library loads and exports what include/asuka_b200.h declares; host-side argument
validation returns its specific code before anything is launched; sharding and builder logic."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

from conftest import ROOT
from flashtensor_b200 import _lib, sharding, utils
from flashtensor_b200.builder import B200Builder, Builder


def _declared_symbols():
  text = open(os.path.join(ROOT, "include", "asuka_b200.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(asuka_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
  declared = _declared_symbols()
  assert len(declared) >= 14
  lib = ctypes.CDLL(built_lib)
  for name in declared:
    assert hasattr(lib, name), f"{name} is declared in the header but not exported"
  assert sorted(_lib.SYMBOLS) == declared, "ctypes prototypes and header disagree"
  assert _lib.load().asuka_b200_version() >= 100
  assert _lib.load().asuka_b200_strerror(-3) == b"bad shape"


def _t(shape, dtype=_lib.F16, ptr=0x1000, strides=None):
  d = _lib.Tensor()
  d.ptr, d.dtype, d.ndim = ptr, dtype, len(shape)
  st = 1
  for i in range(len(shape) - 1, -1, -1):
    d.shape[i] = shape[i]
    d.stride[i] = st if strides is None else strides[i]
    st *= shape[i]
  return d


def _attn(q=None, k=None, v=None, out=None, lse=None, scale=0.0, causal=1):
  shp = (1, 256, 2, 128)
  return _lib.AttnParams(q or _t(shp), k or _t(shp), v or _t(shp), out or _t(shp),
                         lse or _lib.Tensor(), scale, causal, 0.0)


def test_attn_validation_codes(built_lib):
  lib = _lib.load()
  call = lambda p: lib.asuka_b200_attn_fwd(ctypes.byref(p), None)
  assert lib.asuka_b200_attn_fwd(None, None) == -1                        # null params
  assert call(_attn(q=_t((1, 256, 2, 128), ptr=0))) == -1                 # null tensor
  assert call(_attn(q=_t((1, 256, 2, 128), dtype=_lib.F32))) == -2        # dtype
  assert call(_attn(k=_t((1, 256, 2, 128), dtype=_lib.BF16))) == -2       # mixed dtypes
  assert call(_attn(q=_t((1, 256, 2, 64)))) == -3                         # head_dim
  assert call(_attn(k=_t((1, 256, 4, 128)), v=_t((1, 256, 4, 128)))) == -3  # head count differs
  assert call(_attn(k=_t((1, 128, 2, 128)), v=_t((1, 128, 2, 128)))) == -3  # causal with Skv < Sq
  assert call(_attn(q=_t((1, 256, 2, 128), strides=(65536, 256, 128, 2)))) == -4
  assert call(_attn(q=_t((1, 256, 2, 128), strides=(65540, 260, 132, 1)))) == -4  # not 16-byte multiples
  assert call(_attn(q=_t((1, 256, 2, 128), ptr=0x1008))) == -5            # alignment
  assert call(_attn(scale=float("nan"))) == -10
  assert call(_attn(lse=_t((1, 2, 128), dtype=_lib.F32))) == -3           # lse shape


def test_select_and_case_validation_codes(built_lib):
  lib = _lib.load()
  score = _t((1, 2, 512), dtype=_lib.F32)
  idx = lambda n: _t((1, 2, n), dtype=_lib.I32)
  sel = lambda **kw: lib.asuka_b200_select_topk(ctypes.byref(_lib.SelectParams(
      kw.get("score", score), kw.get("sq", _lib.Tensor()), kw.get("idx", idx(64)),
      kw.get("k", 64), kw.get("recent", 0), kw.get("q_len", 512), kw.get("mode", 0))), None)
  assert sel(k=0) == -10
  assert sel(k=513, idx=idx(513)) == -10                                   # k > S
  assert sel(mode=1, recent=500, k=64, idx=idx(564)) == -10                # k > S - recent
  assert sel(mode=7) == -10
  assert sel(idx=idx(65)) == -3                                            # idx shape
  assert sel(mode=2) == -1                                                 # RoCo needs score_sq
  assert sel(score=_t((1, 2, 40000), dtype=_lib.F32), idx=idx(64)) == -11  # beyond the shared-memory limit
  # fused case: workspace too small is reported before any launch
  shp = (1, 256, 2, 128)
  cp = _lib.CaseParams(_t(shp), _t(shp), _t(shp), _t(shp), _t((1, 2, 256), dtype=_lib.F32),
                       _lib.Tensor(), _lib.Tensor(), _lib.Tensor(), 0.0, 1.0, 0, 1, 0, 0)
  need = ctypes.c_size_t(0)
  assert lib.asuka_b200_case_workspace_bytes(ctypes.byref(cp), ctypes.byref(need)) == 0
  assert need.value >= 2 * 256 * 4
  assert lib.asuka_b200_h2o(ctypes.byref(cp), ctypes.c_void_p(0x1000), 16, None) == -6
  assert lib.asuka_b200_h2o(ctypes.byref(cp), None, need.value, None) == -1
  # Keyformer: a bad temperature is refused (tau is 1.0 above, make it 0)
  cp.tau = 0.0
  assert lib.asuka_b200_keyformer(ctypes.byref(cp), ctypes.c_void_p(0x1000), need.value, None) == -10
  sp = _lib.SimaParams(_t(shp), _t(shp), _t((1, 128, 2, 128)), _t(shp))
  assert lib.asuka_b200_sima_workspace_bytes(ctypes.byref(sp), ctypes.byref(need)) == -3


def test_sibling_entry_points_validation_codes(built_lib):
  # every check below fails before anything is launched (no GPU needed)
  lib = _lib.load()
  f32 = lambda shape, **kw: _t(shape, dtype=_lib.F32, **kw)
  # score pooling: odd kernel size, distinct buffers
  s3 = f32((1, 2, 512))
  assert lib.asuka_b200_pool_scores(ctypes.byref(s3), ctypes.byref(f32((1, 2, 512), ptr=0x200000)), 4, None) == -10
  assert lib.asuka_b200_pool_scores(ctypes.byref(s3), ctypes.byref(s3), 5, None) == -10
  assert lib.asuka_b200_pool_scores(ctypes.byref(s3), ctypes.byref(f32((1, 2, 500), ptr=0x200000)), 5, None) == -3
  # cache compaction: index tensor must be [B, H, n] i32 and the outputs [B, n, H, 128]
  kv = _t((1, 256, 2, 128))
  gp = lambda **kw: lib.asuka_b200_gather_kv(ctypes.byref(_lib.GatherParams(
      kv, kv, kw.get("idx", _t((1, 2, 64), dtype=_lib.I32)), kw.get("ko", _t((1, 64, 2, 128), ptr=0x300000)),
      kw.get("vo", _t((1, 64, 2, 128), ptr=0x400000)))), None)
  assert gp(idx=_t((1, 3, 64), dtype=_lib.I32)) == -3
  assert gp(idx=_t((1, 2, 64), dtype=_lib.F32)) == -2
  assert gp(ko=_t((1, 32, 2, 128), ptr=0x300000)) == -3
  # linear attention at head_dim 32: f32 only, last axis 32, 16-byte aligned
  t32 = f32((2, 100, 4, 32))
  la = lambda **kw: lib.asuka_b200_linattn32_fwd(ctypes.byref(_lib.LinAttn32Params(
      kw.get("q", t32), kw.get("k", t32), kw.get("v", t32), kw.get("out", f32((2, 100, 4, 32), ptr=0x500000)),
      kw.get("ea", 0))), None)
  assert la(q=_t((2, 100, 4, 32))) == -2                       # 16-bit input
  assert la(k=f32((2, 100, 4, 64))) == -3
  assert la(v=f32((2, 100, 4, 32), ptr=0x1004)) == -5
  assert la(out=f32((2, 100, 4, 32), strides=(12800, 128, 32, 2), ptr=0x500000)) == -4
  assert la(ea=2) == -10
  # EA shares SimA's checks
  shp = (1, 256, 2, 128)
  sp = _lib.SimaParams(_t(shp), _t(shp), _t(shp), _t(shp, dtype=_lib.I32))
  assert lib.asuka_b200_ea_fwd(ctypes.byref(sp), ctypes.c_void_p(0x1000), 1 << 30, None) in (-2, -5, -3)
  sp = _lib.SimaParams(_t(shp), _t(shp), _t(shp), _t(shp, ptr=0x600000))
  assert lib.asuka_b200_ea_fwd(ctypes.byref(sp), ctypes.c_void_p(0x1000), 16, None) == -6
  assert lib.asuka_b200_ea_fwd(ctypes.byref(sp), None, 1 << 30, None) == -1


def test_ops_refuse_cpu_tensors(built_lib):
  from flashtensor_b200 import ops
  q = torch.zeros(1, 128, 1, 128, dtype=torch.float16)
  with pytest.raises(RuntimeError, match="no CPU path"):
    ops.attn_fwd(q, q, q)


def test_missing_library_is_loud(tmp_path, monkeypatch):
  monkeypatch.setattr(_lib, "_lib", None)
  monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
  with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
    _lib.load()


def test_unit_ranges_cover_everything():
  for n_units, ws in ((32, 8), (128, 8), (80, 8), (256, 8), (5, 2), (3, 4)):
    spans = [sharding.unit_range(n_units, r, ws) for r in range(ws)]
    assert spans[0][0] == 0 and spans[-1][1] == n_units
    for (a, b), (c, d) in zip(spans, spans[1:]):
      assert b == c
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1
  assert sharding.unit_range(32, 3, 8) == (12, 16)     # H2O config: 4 heads per GPU
  with pytest.raises(ValueError):
    sharding.unit_range(8, 8, 8)


def test_shard_roundtrip():
  t = torch.arange(2 * 5 * 3 * 4, dtype=torch.float32).reshape(2, 5, 3, 4)
  parts = [sharding.shard_bshd(t, r, 4) for r in range(4)]
  assert sum(p.shape[2] for p in parts) == 6
  cat = torch.cat([p[0] for p in parts], dim=1)          # [S, B*H, D]
  assert torch.equal(cat.reshape(5, 2, 3, 4).permute(1, 0, 2, 3), t)
  s = torch.arange(2 * 3 * 7, dtype=torch.float32).reshape(2, 3, 7)
  assert torch.equal(sharding.gather_units([sharding.shard_bhs(s, r, 4) for r in range(4)], 2, 3), s)


def test_flop_conventions():
  assert utils.causal_flops(1, 32, 4096, 4096) == 4 * 32 * 128 * (4096 * 4097 // 2)
  assert utils.causal_flops(1, 1, 2, 3) == 4 * 128 * (2 + 3)
  assert utils.causal_flops(1, 1, 2, 3, causal=False) == 4 * 128 * 6
  assert utils.sima_flops(8, 32, 8192) == 4 * 8 * 32 * 8192 * 128 * 128


def test_builder_interface():
  assert issubclass(B200Builder, Builder)
  with pytest.raises(ValueError):
    B200Builder("Performer")
  f = B200Builder("H2O").build_callable()
  with pytest.raises(RuntimeError):
    f(torch.zeros(1), torch.zeros(1))                     # wrong arity
  class K:  # stands in for the reference's Kernel dataclass
    func_name = "RoCo"
  assert B200Builder(K()).case_name == "RoCo"


_GLOO_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from flashtensor_b200 import sharding
from oracle import attn_oracle as O
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, ws = dist.get_rank(), dist.get_world_size()
B, S, H = 2, 48, 3
q, k, v = O.make_inputs("h2o", B, S, S, H, 128, torch.float16, 0)
out_full, score_full = O.h2o(q, k, v)
# each rank computes only its (b,h) units, with the units folded into the head axis
ql, kl, vl = (sharding.shard_bshd(t, rank, ws) for t in (q, k, v))
out_l, score_l = O.h2o(ql, kl, vl)
lo, hi = sharding.unit_range(B * H, rank, ws)
want = out_full.permute(1, 0, 2, 3).reshape(S, B * H, 128)[:, lo:hi]
assert torch.allclose(out_l[0], want, atol=1e-6), "sharded output differs"
parts = [torch.empty(1, sharding.unit_range(B * H, r, ws)[1] - sharding.unit_range(B * H, r, ws)[0], S) for r in range(ws)]
dist.all_gather(parts, score_l.contiguous()) if len(set(p.shape for p in parts)) == 1 else None
if len(set(p.shape for p in parts)) == 1:
  assert torch.allclose(sharding.gather_units(parts, B, H), score_full, atol=1e-5)
t = torch.tensor([float(rank + 1)])
dist.all_reduce(t, op=dist.ReduceOp.MAX)     # the benchmark's max-over-ranks timing reduction
assert t.item() == ws
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_two_rank_sharding_over_gloo(tmp_path):
  script = tmp_path / "worker.py"
  script.write_text(_GLOO_WORKER)
  env = dict(os.environ, REPO_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", WORLD_SIZE="2")
  procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)),
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
  outs = [p.communicate(timeout=180)[0] for p in procs]
  for r, (p, o) in enumerate(zip(procs, outs)):
    assert p.returncode == 0, o
    assert f"ok {r}" in o


def test_case_bookkeeping_like_the_reference_kernel_object():
  # python/asuka/partition/kernel.py: positional inputs, dense flops (2*m*k*n per dot), sizes in elements
  import flashtensor_b200 as ft
  h2o = ft.H2O(head_num=32, kv_head_num=32)
  assert h2o.input_names == ["q", "k", "v"] and h2o.output_names == ["out", "h2o_score"]
  assert h2o.get_flops(1, 4096, 4096) == 274877906944           # 274.9 GF dense at the H2O configuration
  assert ft.RoCo(head_num=40, kv_head_num=40).get_flops(2, 4096, 4096) == 687194767360
  assert ft.Attn().get_flops(1, 1024, 1024) == 17179869184
  assert ft.SimA().get_flops(8, 8192) == 4 * 8 * 32 * 8192 * 128 * 128
  assert h2o.get_mem_size(1, 4096, 4096) == 4 * 4096 * 32 * 128 + 32 * 4096
  kf = ft.KeyFormer()
  assert kf.input_names == ["q", "k", "v", "exp_rand"]
  assert kf.get_mem_size(4, 2048, 2048) == 4 * 4 * 2048 * 32 * 128 + 4 * 32 * 2048 * 2048 + 4 * 32 * 2048
  args = ft.H2O(head_num=4, kv_head_num=2).prepare_dummy_inputs(2, 16, 24, device="cpu")
  assert [tuple(a.shape) for a in args] == [(2, 16, 4, 128), (2, 24, 2, 128), (2, 24, 2, 128)]


def test_new_entry_points_validate_before_touching_a_device(built_lib):
  # RoCo statistics outputs, the optional split scratch queries and the wait self-test: every check
  # below fails on the host, before a device is asked anything
  lib = _lib.load()
  score = _t((1, 2, 512), dtype=_lib.F32)
  sel = lambda **kw: lib.asuka_b200_select_topk(ctypes.byref(_lib.SelectParams(
      score, score, _t((1, 2, 64), dtype=_lib.I32), 64, 0, kw.get("q_len", 512), 2, kw.get("all_rows", 0),
      kw.get("mean", _lib.Tensor()), kw.get("std", _lib.Tensor()))), None)
  assert sel(mean=_t((1, 2, 500), dtype=_lib.F32)) == -3            # statistics have the scores' shape
  assert sel(std=_t((1, 2, 512), dtype=_lib.I32)) == -2
  assert sel(q_len=600) == -10                                      # more query rows than keys, causal count
  need = ctypes.c_size_t(0)
  assert lib.asuka_b200_attn_workspace_bytes(None, ctypes.byref(need)) == -1
  assert lib.asuka_b200_attn_workspace_bytes(ctypes.byref(_attn(q=_t((1, 256, 2, 64)))), ctypes.byref(need)) == -3
  assert lib.asuka_b200_col_scores_workspace_bytes(None, ctypes.byref(need)) == -1
  assert lib.asuka_b200_case_workspace_bytes_split(None, ctypes.byref(need)) == -1
  assert lib.asuka_b200_selftest_wait_timeout(0, None) == -10
  assert lib.asuka_b200_selftest_wait_timeout(200000, None) == -10


def test_both_benchmark_arms_print_the_same_config():
  import bench
  for case in ("h2o", "roco", "sima"):
    for world in (1, 8):
      a = bench.config_of(case, bench.WORKLOADS[case], world, "strong")
      b = bench.config_of(case, bench.WORKLOADS[case], world, "strong")
      assert a == b and set(a) == {"workload", "global_batch", "per_gpu_units", "parallelism", "l2"}
  assert bench.config_of("h2o", bench.WORKLOADS["h2o"], 8, "strong")["per_gpu_units"] == 4
  assert bench.config_of("h2o", bench.WORKLOADS["h2o"], 8, "weak")["global_batch"] == 8


def test_ctypes_structures_match_the_c_header(tmp_path):
  # the header is the contract; the Python binding restates every parameter block: compile a C
  # program against the header that prints sizes and field offsets, and compare
  import os
  import shutil
  import subprocess
  cc = shutil.which("gcc") or shutil.which("cc")
  if cc is None:
    pytest.skip("no C compiler")
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  blocks = {
      "asuka_tensor": (_lib.Tensor, ["ptr", "dtype", "ndim", "shape", "stride"]),
      "asuka_attn_params": (_lib.AttnParams, ["q", "lse", "softmax_scale", "causal", "softcap", "workspace", "workspace_bytes"]),
      "asuka_score_params": (_lib.ScoreParams, ["lse", "exp_rand", "tau", "seed", "mode", "corm_mask", "workspace", "seed_unit_offset"]),
      "asuka_select_params": (_lib.SelectParams, ["idx", "k_keep", "q_len", "mode", "all_rows", "mean", "std"]),
      "asuka_sima_params": (_lib.SimaParams, ["q", "out"]),
      "asuka_linattn32_params": (_lib.LinAttn32Params, ["out", "ea"]),
      "asuka_gather_params": (_lib.GatherParams, ["idx", "v_out"]),
      "asuka_case_params": (_lib.CaseParams, ["idx", "softmax_scale", "seed", "recent", "roco_mean", "roco_std", "seed_unit_offset"]),
  }
  lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "asuka_b200.h"', "int main(void) {"]
  for name, (_, fields) in blocks.items():
    lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
    for f in fields:
      lines.append(f'  printf("{name}.{f} %zu\\n", offsetof({name}, {f}));')
  lines += ["  return 0;", "}"]
  src = tmp_path / "layout.c"
  src.write_text("\n".join(lines))
  exe = tmp_path / "layout"
  subprocess.run([cc, "-I", os.path.join(root, "include"), str(src), "-o", str(exe)], check=True)
  got = dict(l.split() for l in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
  for name, (cls, fields) in blocks.items():
    assert int(got[name]) == ctypes.sizeof(cls), name
    for f in fields:
      assert int(got[f"{name}.{f}"]) == getattr(cls, f).offset, f"{name}.{f}"
