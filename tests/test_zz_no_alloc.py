"""The allocation-free H2O entry point (asuka_b200_h2o_static), called through the C ABI.

It exists for hosts that cannot give the library scratch memory and cannot let it allocate
(engine plug-ins whose enqueue hook must not allocate, processes whose memory pool already owns
the whole device).  Its scratch is a fixed array inside the library, shared by all calls, so the
check runs calls back to back and compares each with the ordinary entry point (asuka_b200_h2o,
caller-supplied workspace) on the same inputs, and with the CPU oracle.  The shapes include
grouped K/V heads (which park more in the array) and the largest problem the array admits.
"""
import ctypes

import numpy as np
import pytest
import torch

from flashtensor_b200 import _lib
from oracle import attn_oracle as O


def _desc(t):
  d = _lib.Tensor()
  if t is not None:
    d.ptr, d.ndim = t.data_ptr(), t.dim()
    d.dtype = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2, torch.int32: 3}[t.dtype]
    for i in range(t.dim()):
      d.shape[i], d.stride[i] = t.shape[i], t.stride(i)
  return d


def _params(q, k, v, out, score, idx, k_keep, recent):
  return _lib.CaseParams(_desc(q), _desc(k), _desc(v), _desc(out), _desc(score), _lib.Tensor(),
                         _lib.Tensor(), _desc(idx), 0.0, 1.0, 0, 1, k_keep, recent)


def test_static_entry_refuses_oversized_requests_before_any_launch(built_lib):
  # descriptors only: the size check is the first thing the entry point does, and on a host
  # without a GPU nothing could launch in any case
  lib = _lib.load()
  def fake(shape, dtype=0):
    d = _lib.Tensor()
    d.ptr, d.dtype, d.ndim = 0x10000, dtype, len(shape)
    st = 1
    for i in range(len(shape) - 1, -1, -1):
      d.shape[i], d.stride[i] = shape[i], st
      st *= shape[i]
    return d
  rows_ok, rows_bad = 524288, 524288 + 128
  for S, want in ((rows_bad, -11),):
    p = _lib.CaseParams(fake((1, S, 1, 128)), fake((1, S, 1, 128)), fake((1, S, 1, 128)),
                        fake((1, S, 1, 128)), fake((1, 1, S), 2), _lib.Tensor(), _lib.Tensor(),
                        _lib.Tensor(), 0.0, 1.0, 0, 1, 0, 0)
    assert lib.asuka_b200_h2o_static(ctypes.byref(p), None) == want
  assert rows_ok == 524288  # ASUKA_H2O_STATIC_MAX_ROWS in include/asuka_b200.h
  assert lib.asuka_b200_h2o_static(None, None) == -1
  # grouped K/V heads: 8 bytes per query row plus 4 bytes per (query head, key) must fit in 4 MiB
  B, S, H, Hkv = 1, 32768, 12, 4          # 393216 rows: 3 MiB of row statistics + 1.5 MiB of scores
  p = _lib.CaseParams(fake((B, S, H, 128)), fake((B, S, Hkv, 128)), fake((B, S, Hkv, 128)),
                      fake((B, S, H, 128)), fake((B, Hkv, S), 2), _lib.Tensor(), _lib.Tensor(),
                      _lib.Tensor(), 0.0, 1.0, 0, 1, 0, 0)
  assert lib.asuka_b200_h2o_static(ctypes.byref(p), None) == -11


@pytest.mark.gpu
def test_static_entry_matches_workspace_entry_twice_in_a_row(built_lib):
  assert torch.cuda.is_available()
  lib = _lib.load()
  dev = torch.device("cuda", 0)
  stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
  g = torch.Generator(device=dev).manual_seed(123)
  # (B, S, H, Hkv, k_keep, recent); the last shape is exactly ASUKA_H2O_STATIC_MAX_ROWS query rows
  shapes = [(1, 1024, 4, 4, 128, 64), (2, 640, 3, 3, 80, 32), (1, 777, 6, 2, 90, 40), (4, 4096, 32, 32, 512, 256)]
  for call, (B, S, H, Hkv, k_keep, recent) in enumerate(shapes):
    q = torch.randn(B, S, H, 128, generator=g, device=dev).half()
    k, v = (torch.randn(B, S, Hkv, 128, generator=g, device=dev).half() for _ in range(2))
    res = []
    for static in (False, True):
      # the caller owns every output; poison them so that stale data cannot pass
      out = torch.full((B, S, H, 128), float("nan"), dtype=torch.float16, device=dev)
      score = torch.full((B, Hkv, S), -1.0, dtype=torch.float32, device=dev)
      idx = torch.full((B, Hkv, k_keep + recent), -7, dtype=torch.int32, device=dev)
      p = _params(q, k, v, out, score, idx, k_keep, recent)
      if static:
        st = lib.asuka_b200_h2o_static(ctypes.byref(p), stream)
      else:
        n = ctypes.c_size_t(0)
        assert lib.asuka_b200_case_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == 0
        ws = torch.empty(n.value, dtype=torch.uint8, device=dev)
        st = lib.asuka_b200_h2o(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), n, stream)
      assert st == 0, lib.asuka_b200_strerror(st)
      torch.cuda.synchronize()
      res.append((out, score, idx))
    (o0, s0, i0), (o1, s1, i1) = res
    assert torch.isfinite(o1.float()).all() and (s1 >= 0).all() and (i1 >= 0).all()
    # same kernels on the same inputs: the tolerance of the other parity tests, met with room
    assert (o0.float() - o1.float()).abs().max().item() <= 2e-2, f"call {call}: out differs"
    assert (s0 - s1).abs().max().item() <= 2e-2 and ((s0 - s1).abs().max() / s0.abs().max()).item() <= 1e-2
    assert torch.equal(i0, i1), f"call {call}: kept indices differ"
    # against the CPU oracle: the whole problem when it is small, two units of the largest one
    units = [(b, h) for b in range(B) for h in range(Hkv)] if B * S * H <= 16384 else [(0, 0), (B - 1, Hkv - 1)]
    grp = H // Hkv
    for b, h in units:
      ref_out, ref_score = O.h2o_gqa(q[b:b + 1, :, h * grp:(h + 1) * grp].cpu(), k[b:b + 1, :, h:h + 1].cpu(),
                                     v[b:b + 1, :, h:h + 1].cpu())
      e = O.errors(o1[b:b + 1, :, h * grp:(h + 1) * grp], ref_out)
      assert e["abs_max"] <= 2e-2 and e["scale_rel"] <= 1e-2, (call, b, h, e)
      e = O.errors(s1[b:b + 1, h:h + 1], ref_score)
      assert e["abs_max"] <= 2e-2 and e["scale_rel"] <= 1e-2, (call, b, h, e)
      O.check_index_sets(i1[b:b + 1, h:h + 1, :k_keep].cpu().numpy(),
                         O.h2o_select(ref_score.numpy(), k_keep, recent)[..., :k_keep], ref_score.numpy(),
                         k_keep, S - recent)
  w = (ctypes.c_uint32 * 2)()
  assert lib.asuka_b200_device_status(w) == 0
