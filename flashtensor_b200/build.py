"""Builds the sm_100a kernel library in-tree: flashtensor_b200/libasuka_b200.so.

Usage: python -m flashtensor_b200.build [--force] [--verbose]
nvcc cross-compiles without a GPU; the result is loaded with ctypes by flashtensor_b200._lib.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libasuka_b200.so")

SOURCES = ["capi.cu", "attn_fwd.cu", "col_scores.cu", "select_topk.cu", "score_ops.cu", "sima.cu", "linattn32.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]


def _flags():
  """The fixed flags plus whatever ASUKA_NVCC_FLAGS adds (e.g. -DASUKA_TUNE_ENV, which lets the
  environment variables ASUKA_FWD_PARTS / ASUKA_COL_CHUNKS force the work-item split factors for
  tuning runs)."""
  return NVCC_FLAGS + os.environ.get("ASUKA_NVCC_FLAGS", "").split()


def _nvcc():
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise RuntimeError("nvcc not found: the asuka_b200 kernel library cannot be built")


def _deps():
  return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))] + [
      os.path.join(PKG_DIR, "..", "include", "asuka_b200.h")]


def build(force=False, verbose=False):
  """Compile every .cu under csrc/ for sm_100a and link the shared library.  Returns its path."""
  nvcc = _nvcc()
  os.makedirs(OBJ_DIR, exist_ok=True)
  srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
  dep_mtime = max(os.path.getmtime(d) for d in _deps())
  objs, relink = [], force or not os.path.exists(LIB_PATH)
  for s in srcs:
    src = os.path.join(CSRC, s)
    obj = os.path.join(OBJ_DIR, s.replace(".cu", ".o"))
    objs.append(obj)
    stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), dep_mtime)
    if stale:
      cmd = [nvcc] + _flags() + ["-c", src, "-o", obj]
      res = subprocess.run(cmd, capture_output=True, text=True)
      log = res.stdout + res.stderr
      with open(obj + ".log", "w") as f:
        f.write(log)
      if verbose or res.returncode != 0:
        print(log, file=sys.stderr)
      if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {s}")
      relink = True
  if relink or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs):
    cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
      print(res.stdout + res.stderr, file=sys.stderr)
      raise RuntimeError("link failed")
  return LIB_PATH


if __name__ == "__main__":
  path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
  print(path)
