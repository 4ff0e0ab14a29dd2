"""The reference's SimA and EA benchmark programs as whole blocks (bench/sima.mlir, bench/ea.mlir).

``func @EA(%arg0 x[B,N,C], %arg1 w_qkv[3C,C], %arg2 b_qkv[3C], %arg3 w_o[C,C], %arg4 b_o[C])``:
a fused QKV projection with bias (lines 3-5), split into heads of 32 features (lines 6-12), the
linear-attention core (lines 13-17), and the output projection with bias (lines 18-22).

The two projections are plain GEMMs with a bias and go to cuBLAS through ``torch.addmm``; the
split / reshape / transpose between them and the core cost nothing, because the core kernel reads
q, k, v as strided views of the projection's output and writes the layout the output projection
reads.  The core is this library's kernel (``ops.linattn32_fwd``); there is no other path.
"""
import torch

from . import ops

HEAD_DIM = 32


class LinearAttentionBlock:
  """``block(x, w_qkv, b_qkv, w_o, b_o) -> [B, N, C]`` in f32, argument order as the mlir function."""

  def __init__(self, ea: bool):
    self.ea = ea

  def __call__(self, x, w_qkv, b_qkv, w_o, b_o):
    if x.dim() != 3 or x.dtype != torch.float32:
      raise RuntimeError("x must be [B, N, C] float32")
    B, N, C = x.shape
    if C % HEAD_DIM or tuple(w_qkv.shape) != (3 * C, C) or tuple(b_qkv.shape) != (3 * C,) or \
       tuple(w_o.shape) != (C, C) or tuple(b_o.shape) != (C,):
      raise RuntimeError("expected w_qkv [3C, C], b_qkv [3C], w_o [C, C], b_o [C] with C a multiple of 32")
    H = C // HEAD_DIM
    qkv = torch.addmm(b_qkv, x.reshape(B * N, C), w_qkv.t()).view(B, N, 3, H, HEAD_DIM)
    core = ops.linattn32_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], ea=self.ea)   # [B, N, H, 32]
    return torch.addmm(b_o, core.view(B * N, C), w_o.t()).view(B, N, C)


class SimABlock(LinearAttentionBlock):
  """bench/sima.mlir (with the normalised Q in the last product, as the SimA method defines it)."""

  def __init__(self):
    super().__init__(ea=False)


class EABlock(LinearAttentionBlock):
  """bench/ea.mlir."""

  def __init__(self):
    super().__init__(ea=True)
