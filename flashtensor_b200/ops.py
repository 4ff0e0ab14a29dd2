"""Operator layer: torch tensors in, C-ABI calls, torch tensors out.

Outputs are allocated with torch.empty on the inputs' device and the work is enqueued on torch's
current stream without synchronising -- the contract of the reference's generated callables
(lib/Translate/to_triton.cpp:579-609).  Shape/dtype problems raise (as the TensorRT back end's
closure does, python/asuka/backend/tensorrt/builder.py:104-111); nothing falls back to PyTorch.
"""
import contextlib
import ctypes

import torch

from . import _lib
from ._lib import AsukaError  # noqa: F401  (re-exported)

_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32,
           torch.int32: _lib.I32, torch.uint8: _lib.U8, torch.bool: _lib.U8}


def _desc(t):
  """asuka_tensor descriptor of a torch tensor (None -> null descriptor)."""
  d = _lib.Tensor()
  if t is None:
    return d
  if t.dtype not in _DTYPES:
    raise TypeError(f"unsupported dtype {t.dtype}")
  if t.dim() > 5:
    raise ValueError("at most 5 dimensions")
  n = t.dim()
  d.ptr = t.data_ptr()
  d.dtype = _DTYPES[t.dtype]
  d.ndim = n
  d.shape[:n] = t.shape      # (slice assignment: one call instead of a Python loop; this function
  d.stride[:n] = t.stride()  #  is most of the host time of a call at small shapes)
  return d


_NO_SWITCH = contextlib.nullcontext()


def _on(dev):
  """Context that makes `dev` the current CUDA device (a no-op, and cheap, when it already is)."""
  return _NO_SWITCH if dev.index == torch.cuda.current_device() else torch.cuda.device(dev)


def _stream(t):
  if not t.is_cuda:
    raise RuntimeError("asuka_b200 kernels run on CUDA tensors only; there is no CPU path")
  return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _as4d(t):
  """Accept the 2-D [S, H*D] layout of cases/attn.py as [1, S, H, 128] (same memory)."""
  if t.dim() == 2:
    return t.view(1, t.shape[0], t.shape[1] // 128, 128)
  return t


def _same_device(*ts):
  dev = ts[0].device
  for t in ts:
    if t is None:
      continue
    if not t.is_cuda:
      raise RuntimeError("asuka_b200 kernels run on CUDA tensors only; there is no CPU path")
    if t.device != dev:
      raise RuntimeError("all tensors must be on the same device")


def _scratch(query, name, params, device):
  """Optional scratch a kernel can use to split its work items when a launch has too few of them
  to fill the device (None when it would not help).  The caching allocator keeps the block alive
  until the stream's work that uses it has run."""
  nbytes = ctypes.c_size_t(0)
  _lib.check(name, query(ctypes.byref(params), ctypes.byref(nbytes)))
  if nbytes.value == 0:
    return None
  return torch.empty((nbytes.value,), dtype=torch.uint8, device=device)


def attn_fwd(q, k, v, causal=True, softmax_scale=0.0, return_lse=False, out=None, softcap=0.0):
  """out = softmax(q k^T * scale (+ causal mask)) v.  q: [B,Sq,H,128]; k, v: [B,Skv,H,128].
  softcap > 0 applies cap * tanh(logits / cap) before the mask (cases/kernels/gemma2.py:30-33)."""
  lib = _lib.load()
  q4, k4, v4 = _as4d(q), _as4d(k), _as4d(v)
  _same_device(q4, k4, v4)
  with _on(q4.device):
    if out is None:
      out = torch.empty(q4.shape, dtype=q4.dtype, device=q4.device)
    lse = torch.empty((q4.shape[0], q4.shape[2], q4.shape[1]), dtype=torch.float32,
                      device=q4.device) if return_lse else None
    p = _lib.AttnParams(_desc(q4), _desc(k4), _desc(v4), _desc(_as4d(out)), _desc(lse),
                        float(softmax_scale), int(bool(causal)), float(softcap), None, 0)
    ws = _scratch(lib.asuka_b200_attn_workspace_bytes, "asuka_b200_attn_workspace_bytes", p, q4.device)
    if ws is not None:
      p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check("asuka_b200_attn_fwd", lib.asuka_b200_attn_fwd(ctypes.byref(p), _stream(q4)))
  out = out.view(q.shape) if q.dim() == 2 else out
  return (out, lse) if return_lse else out


def col_scores(q, k, lse, mode=_lib.SCORE_SUM, causal=True, softmax_scale=0.0, exp_rand=None,
               tau=1.0, seed=0, corm_mask=None, unit_offset=0):
  """Per-key reductions over the query rows of the attention probabilities: [B,H,Skv] f32 sums
  (and sums of squares in mode SCORE_SUM_SQ); in mode SCORE_CORM a bool tensor that is True where
  some probability reaches its threshold in `corm_mask` [Sq, Skv]."""
  lib = _lib.load()
  q4, k4 = _as4d(q), _as4d(k)
  _same_device(q4, k4, lse, exp_rand, corm_mask)
  B, Skv, H = k4.shape[0], k4.shape[1], k4.shape[2]
  with _on(q4.device):
    score = torch.empty((B, H, Skv), dtype=torch.bool if mode == _lib.SCORE_CORM else torch.float32,
                        device=q4.device)
    score_sq = torch.empty_like(score) if mode == _lib.SCORE_SUM_SQ else None
    p = _lib.ScoreParams(_desc(q4), _desc(k4), _desc(lse), _desc(score), _desc(score_sq),
                         _desc(exp_rand), float(softmax_scale), float(tau), int(seed),
                         int(bool(causal)), int(mode), _desc(corm_mask), None, 0, int(unit_offset))
    ws = _scratch(lib.asuka_b200_col_scores_workspace_bytes, "asuka_b200_col_scores_workspace_bytes", p, q4.device)
    if ws is not None:
      p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check("asuka_b200_col_scores", lib.asuka_b200_col_scores(ctypes.byref(p), _stream(q4)))
  return (score, score_sq) if score_sq is not None else score


def keyformer_rowstat(q, k, causal=True, softmax_scale=0.0, exp_rand=None, tau=1.5, seed=0, unit_offset=0):
  """Base-2 log-sum-exp per query row of the perturbed logits (s + g) / tau: [B,H,Sq] f32."""
  lib = _lib.load()
  q4, k4 = _as4d(q), _as4d(k)
  _same_device(q4, k4, exp_rand)
  with _on(q4.device):
    lse = torch.empty((q4.shape[0], q4.shape[2], q4.shape[1]), dtype=torch.float32, device=q4.device)
    p = _lib.ScoreParams(_desc(q4), _desc(k4), _desc(lse), _lib.Tensor(), _lib.Tensor(),
                         _desc(exp_rand), float(softmax_scale), float(tau), int(seed),
                         int(bool(causal)), _lib.SCORE_PERTURBED, _lib.Tensor(), None, 0, int(unit_offset))
    _lib.check("asuka_b200_keyformer_rowstat",
               lib.asuka_b200_keyformer_rowstat(ctypes.byref(p), _stream(q4)))
  return lse


def select_topk(score, k_keep, mode=_lib.SELECT_TOPK, recent=0, score_sq=None, q_len=0, causal=True,
                return_stats=False):
  """Kept key indices, ascending int32 [B,H,k_keep(+recent)].  Mode SELECT_ROCO ranks by the
  per-key mean (then standard deviation) of the probabilities over the rows that attend to the
  key -- all `q_len` rows when `causal` is False -- and with `return_stats` also returns
  (mean, std), both [B,H,S] f32."""
  lib = _lib.load()
  _same_device(score, score_sq)
  B, H, _ = score.shape
  n_out = k_keep + (recent if mode == _lib.SELECT_TOPK_RECENT else 0)
  with _on(score.device):
    idx = torch.empty((B, H, n_out), dtype=torch.int32, device=score.device)
    stats = return_stats and mode == _lib.SELECT_ROCO
    mean = torch.empty_like(score) if stats else None
    std = torch.empty_like(score) if stats else None
    p = _lib.SelectParams(_desc(score), _desc(score_sq), _desc(idx), int(k_keep), int(recent),
                          int(q_len), int(mode), int(not causal), _desc(mean), _desc(std))
    _lib.check("asuka_b200_select_topk", lib.asuka_b200_select_topk(ctypes.byref(p), _stream(score)))
  return (idx, mean, std) if stats else idx


def pool_scores(score, kernel_size):
  """SnapKV smoothing: avg_pool1d(score, kernel_size, padding=kernel_size // 2, stride=1) over keys."""
  lib = _lib.load()
  _same_device(score)
  with _on(score.device):
    out = torch.empty_like(score)
    a, b = _desc(score), _desc(out)
    _lib.check("asuka_b200_pool_scores",
               lib.asuka_b200_pool_scores(ctypes.byref(a), ctypes.byref(b), int(kernel_size), _stream(score)))
  return out


def gather_kv(k, v, idx):
  """Compact the KV cache to the kept keys: (k[b, idx[b,h,n], h, :], v alike) as [B, n, H, 128]."""
  lib = _lib.load()
  _same_device(k, v, idx)
  B, _, H, D = k.shape
  n = idx.shape[2]
  with _on(k.device):
    k_out = torch.empty((B, n, H, D), dtype=k.dtype, device=k.device)
    v_out = torch.empty_like(k_out)
    p = _lib.GatherParams(_desc(k), _desc(v), _desc(idx), _desc(k_out), _desc(v_out))
    _lib.check("asuka_b200_gather_kv", lib.asuka_b200_gather_kv(ctypes.byref(p), _stream(k)))
  return k_out, v_out


def sima_fwd(q, k, v, out_dtype=None, _entry="asuka_b200_sima_fwd"):
  """SimA: out = L1norm_seq(q) (L1norm_seq(k)^T v), [B,S,H,128]."""
  lib = _lib.load()
  q4, k4, v4 = _as4d(q), _as4d(k), _as4d(v)
  _same_device(q4, k4, v4)
  with _on(q4.device):
    out = torch.empty(q4.shape, dtype=out_dtype or q4.dtype, device=q4.device)
    p = _lib.SimaParams(_desc(q4), _desc(k4), _desc(v4), _desc(out))
    nbytes = ctypes.c_size_t(0)
    _lib.check("asuka_b200_sima_workspace_bytes",
               lib.asuka_b200_sima_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)))
    ws = torch.empty((max(nbytes.value, 16),), dtype=torch.uint8, device=q4.device)
    _lib.check(_entry, getattr(lib, _entry)(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()),
                                            ctypes.c_size_t(ws.numel()), _stream(q4)))
  return out.view(q.shape) if q.dim() == 2 else out


def ea_fwd(q, k, v, out_dtype=None):
  """EA (bench/ea.mlir:13-17): out = softmax_features(q) (softmax_seq(k)^T v), [B,S,H,128]."""
  return sima_fwd(q, k, v, out_dtype, _entry="asuka_b200_ea_fwd")


def linattn32_fwd(q, k, v, ea=False, out=None):
  """SimA (ea=False) or EA (ea=True) attention core at head_dim 32 in f32 (bench/sima.mlir:13-17,
  bench/ea.mlir:13-17).  q, k, v: [B, N, H, 32] f32, possibly strided views of a fused QKV tensor."""
  lib = _lib.load()
  _same_device(q, k, v, out)
  with _on(q.device):
    if out is None:
      out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    p = _lib.LinAttn32Params(_desc(q), _desc(k), _desc(v), _desc(out), int(bool(ea)))
    _lib.check("asuka_b200_linattn32_fwd", lib.asuka_b200_linattn32_fwd(ctypes.byref(p), _stream(q)))
  return out


def _case(fn_name, q, k, v, causal, softmax_scale, want_sq=False, exp_rand=None, tau=1.0, seed=0,
          k_keep=0, recent=0, n_idx=0, workspace=None, out=None, score=None, score_sq=None, idx=None,
          roco_mean=None, roco_std=None, unit_offset=0):
  lib = _lib.load()
  q4, k4, v4 = _as4d(q), _as4d(k), _as4d(v)
  _same_device(q4, k4, v4, exp_rand)
  # scores and indices are per key/value head (with grouped-query attention: the group mean)
  B, Skv, H = k4.shape[0], k4.shape[1], k4.shape[2]
  dev = q4.device
  with _on(dev):
    if out is None:
      out = torch.empty(q4.shape, dtype=q4.dtype, device=dev)
    if score is None:
      score = torch.empty((B, H, Skv), dtype=torch.float32, device=dev)
    if want_sq and score_sq is None:
      score_sq = torch.empty_like(score)
    if n_idx > 0 and idx is None:
      idx = torch.empty((B, H, n_idx), dtype=torch.int32, device=dev)
    p = _lib.CaseParams(_desc(q4), _desc(k4), _desc(v4), _desc(_as4d(out)), _desc(score),
                        _desc(score_sq), _desc(exp_rand), _desc(idx), float(softmax_scale),
                        float(tau), int(seed), int(bool(causal)), int(k_keep), int(recent),
                        _desc(roco_mean), _desc(roco_std), int(unit_offset))
    if workspace is None:
      nbytes = ctypes.c_size_t(0)
      _lib.check("asuka_b200_case_workspace_bytes_split",
                 lib.asuka_b200_case_workspace_bytes_split(ctypes.byref(p), ctypes.byref(nbytes)))
      workspace = torch.empty((max(nbytes.value, 16),), dtype=torch.uint8, device=dev)
    _lib.check(fn_name, getattr(lib, fn_name)(ctypes.byref(p), ctypes.c_void_p(workspace.data_ptr()),
                                              ctypes.c_size_t(workspace.numel()), _stream(q4)))
  if q.dim() == 2:
    # the 2-D scripts return out [q_len, H*128] and per-key tensors [Hkv, kv_len] (cases/attn_h2o.py:47)
    out = out.view(q.shape)
    score, score_sq, idx = (None if t is None else t[0] for t in (score, score_sq, idx))
  return out, score, score_sq, idx


def h2o(q, k, v, causal=True, softmax_scale=0.0, k_keep=0, recent=0, **buffers):
  """(out, h2o_score[, idx]) -- cases/kernels/h2o.py:18-38 plus the optional keep set."""
  n_idx = k_keep + recent if k_keep > 0 else 0
  out, score, _, idx = _case("asuka_b200_h2o", q, k, v, causal, softmax_scale, k_keep=k_keep,
                             recent=recent, n_idx=n_idx, **buffers)
  return (out, score, idx) if n_idx else (out, score)


def h2o_static(q, k, v, out, score, idx=None, causal=True, softmax_scale=0.0, k_keep=0, recent=0):
  """H2O through the entry point that allocates nothing: the caller supplies every output
  (`out`, `score`, optionally `idx`), and the scratch between the two kernels is the library's
  fixed device array.  For hosts that may not allocate on the call path (engine plug-ins, fully
  pre-reserved memory pools); limited to B*H*Sq <= 524288 rows, and calls on one device must not
  overlap.  This wrapper itself creates no tensors."""
  lib = _lib.load()
  q4, k4, v4 = _as4d(q), _as4d(k), _as4d(v)
  _same_device(q4, k4, v4, out, score, idx)
  with _on(q4.device):
    p = _lib.CaseParams(_desc(q4), _desc(k4), _desc(v4), _desc(_as4d(out)), _desc(score),
                        _lib.Tensor(), _lib.Tensor(), _desc(idx), float(softmax_scale), 1.0, 0,
                        int(bool(causal)), int(k_keep), int(recent), _lib.Tensor(), _lib.Tensor(), 0)
    _lib.check("asuka_b200_h2o_static", lib.asuka_b200_h2o_static(ctypes.byref(p), _stream(q4)))
  return (out, score, idx) if idx is not None else (out, score)


def roco(q, k, v, causal=True, softmax_scale=0.0, k_keep=0, return_stats=False, **buffers):
  """(out, roco_score, roco_sq_score[, idx[, mean, std]]) -- cases/kernels/roco.py:18-48; with a
  selection (`k_keep` > 0) and `return_stats`, also the per-key mean and standard deviation of the
  probabilities the selection ranks by, [B,H,Skv] f32."""
  if return_stats and k_keep > 0:
    k4 = _as4d(k)
    shape = (k4.shape[0], _as4d(q).shape[2], k4.shape[1])
    buffers.setdefault("roco_mean", torch.empty(shape, dtype=torch.float32, device=q.device))
    buffers.setdefault("roco_std", torch.empty(shape, dtype=torch.float32, device=q.device))
  out, score, sq, idx = _case("asuka_b200_roco", q, k, v, causal, softmax_scale, want_sq=True,
                              k_keep=k_keep, n_idx=k_keep, **buffers)
  if return_stats and k_keep > 0:
    return out, score, sq, idx, buffers["roco_mean"], buffers["roco_std"]
  return (out, score, sq, idx) if k_keep else (out, score, sq)


def keyformer(q, k, v, exp_rand=None, tau=1.5, seed=0, causal=True, softmax_scale=0.0, k_keep=0,
              **buffers):
  """(out, kf_score[, idx]) -- cases/kernels/kf.py:19-42; exp_rand=None uses the seeded noise
  (`unit_offset`: index of this call's first (batch, head) unit when it is a slice of a larger
  problem, so that the slice gets the noise the whole problem would have had)."""
  out, score, _, idx = _case("asuka_b200_keyformer", q, k, v, causal, softmax_scale,
                             exp_rand=exp_rand, tau=tau, seed=seed, k_keep=k_keep, n_idx=k_keep,
                             **buffers)
  return (out, score, idx) if k_keep else (out, score)


def device_status():
  """(count, last_site) of expired device-side waits since the last read; raises if non-zero."""
  lib = _lib.load()
  w = (ctypes.c_uint32 * 2)()
  st = lib.asuka_b200_device_status(w)
  _lib.check("asuka_b200_device_status", st)
  return int(w[0]), int(w[1])


def launch_count():
  return int(_lib.load().asuka_b200_launch_count())
