"""ctypes binding of libasuka_b200.so (the C ABI declared in include/asuka_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libasuka_b200.so")

F16, BF16, F32, I32, U8 = 0, 1, 2, 3, 4

SCORE_SUM, SCORE_SUM_SQ, SCORE_PERTURBED, SCORE_CORM = 0, 1, 2, 3
SELECT_TOPK, SELECT_TOPK_RECENT, SELECT_ROCO = 0, 1, 2

STATUS_NAMES = {
    0: "ASUKA_OK", -1: "ASUKA_ERR_NULL_POINTER", -2: "ASUKA_ERR_BAD_DTYPE", -3: "ASUKA_ERR_BAD_SHAPE",
    -4: "ASUKA_ERR_BAD_STRIDE", -5: "ASUKA_ERR_MISALIGNED", -6: "ASUKA_ERR_WORKSPACE_TOO_SMALL",
    -7: "ASUKA_ERR_UNSUPPORTED_ARCH", -8: "ASUKA_ERR_CUDA", -9: "ASUKA_ERR_DEVICE_TIMEOUT",
    -10: "ASUKA_ERR_BAD_ARGUMENT", -11: "ASUKA_ERR_TOO_LARGE",
}


class Tensor(ctypes.Structure):
  _fields_ = [("ptr", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
              ("shape", ctypes.c_int64 * 5), ("stride", ctypes.c_int64 * 5)]


class AttnParams(ctypes.Structure):
  _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("out", Tensor), ("lse", Tensor),
              ("softmax_scale", ctypes.c_float), ("causal", ctypes.c_int32),
              ("softcap", ctypes.c_float), ("workspace", ctypes.c_void_p),
              ("workspace_bytes", ctypes.c_uint64)]


class ScoreParams(ctypes.Structure):
  _fields_ = [("q", Tensor), ("k", Tensor), ("lse", Tensor), ("score", Tensor), ("score_sq", Tensor),
              ("exp_rand", Tensor), ("softmax_scale", ctypes.c_float), ("tau", ctypes.c_float),
              ("seed", ctypes.c_uint64), ("causal", ctypes.c_int32), ("mode", ctypes.c_int32),
              ("corm_mask", Tensor), ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
              ("seed_unit_offset", ctypes.c_uint32)]


class SelectParams(ctypes.Structure):
  _fields_ = [("score", Tensor), ("score_sq", Tensor), ("idx", Tensor), ("k_keep", ctypes.c_int32),
              ("recent", ctypes.c_int32), ("q_len", ctypes.c_int32), ("mode", ctypes.c_int32),
              ("all_rows", ctypes.c_int32), ("mean", Tensor), ("std", Tensor)]


class SimaParams(ctypes.Structure):
  _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("out", Tensor)]


class LinAttn32Params(ctypes.Structure):
  _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("out", Tensor), ("ea", ctypes.c_int32)]


class GatherParams(ctypes.Structure):
  _fields_ = [("k", Tensor), ("v", Tensor), ("idx", Tensor), ("k_out", Tensor), ("v_out", Tensor)]


class CaseParams(ctypes.Structure):
  _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("out", Tensor), ("score", Tensor),
              ("score_sq", Tensor), ("exp_rand", Tensor), ("idx", Tensor),
              ("softmax_scale", ctypes.c_float), ("tau", ctypes.c_float), ("seed", ctypes.c_uint64),
              ("causal", ctypes.c_int32), ("k_keep", ctypes.c_int32), ("recent", ctypes.c_int32),
              ("roco_mean", Tensor), ("roco_std", Tensor), ("seed_unit_offset", ctypes.c_uint32)]


class AsukaError(RuntimeError):
  def __init__(self, fn, status, text):
    super().__init__(f"{fn} failed: {STATUS_NAMES.get(status, status)} ({text})")
    self.status = status


# name -> (restype, argtypes); every symbol include/asuka_b200.h declares
SYMBOLS = {
    "asuka_b200_version": (ctypes.c_int, []),
    "asuka_b200_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "asuka_b200_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32)]),
    "asuka_b200_launch_count": (ctypes.c_uint64, []),
    "asuka_b200_selftest_wait_timeout": (ctypes.c_int, [ctypes.c_uint32, ctypes.c_void_p]),
    "asuka_b200_attn_fwd": (ctypes.c_int, [ctypes.POINTER(AttnParams), ctypes.c_void_p]),
    "asuka_b200_attn_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(AttnParams), ctypes.POINTER(ctypes.c_size_t)]),
    "asuka_b200_col_scores": (ctypes.c_int, [ctypes.POINTER(ScoreParams), ctypes.c_void_p]),
    "asuka_b200_col_scores_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(ScoreParams), ctypes.POINTER(ctypes.c_size_t)]),
    "asuka_b200_keyformer_rowstat": (ctypes.c_int, [ctypes.POINTER(ScoreParams), ctypes.c_void_p]),
    "asuka_b200_select_topk": (ctypes.c_int, [ctypes.POINTER(SelectParams), ctypes.c_void_p]),
    "asuka_b200_pool_scores": (ctypes.c_int, [ctypes.POINTER(Tensor), ctypes.POINTER(Tensor), ctypes.c_int32, ctypes.c_void_p]),
    "asuka_b200_gather_kv": (ctypes.c_int, [ctypes.POINTER(GatherParams), ctypes.c_void_p]),
    "asuka_b200_sima_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(SimaParams), ctypes.POINTER(ctypes.c_size_t)]),
    "asuka_b200_sima_fwd": (ctypes.c_int, [ctypes.POINTER(SimaParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "asuka_b200_ea_fwd": (ctypes.c_int, [ctypes.POINTER(SimaParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "asuka_b200_linattn32_fwd": (ctypes.c_int, [ctypes.POINTER(LinAttn32Params), ctypes.c_void_p]),
    "asuka_b200_case_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(CaseParams), ctypes.POINTER(ctypes.c_size_t)]),
    "asuka_b200_case_workspace_bytes_split": (ctypes.c_int, [ctypes.POINTER(CaseParams), ctypes.POINTER(ctypes.c_size_t)]),
    "asuka_b200_h2o": (ctypes.c_int, [ctypes.POINTER(CaseParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "asuka_b200_h2o_static": (ctypes.c_int, [ctypes.POINTER(CaseParams), ctypes.c_void_p]),
    "asuka_b200_roco": (ctypes.c_int, [ctypes.POINTER(CaseParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "asuka_b200_keyformer": (ctypes.c_int, [ctypes.POINTER(CaseParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
}

_lib = None


def load():
  """Load the shared library once and set the prototypes of every exported symbol."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise ImportError(
          f"{LIB_PATH} is missing: build it with `python -m flashtensor_b200.build` "
          "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
      fn = getattr(lib, name)  # AttributeError if the library does not export it
      fn.restype = res
      fn.argtypes = args
    _lib = lib
  return _lib


def check(fn_name, status):
  if status != 0:
    text = load().asuka_b200_strerror(status).decode()
    raise AsukaError(fn_name, status, text)
