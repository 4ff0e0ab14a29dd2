"""Back-end plug-in: the reference's ``Builder`` interface over the sm_100a kernel library.

``python/asuka/backend/builder.py:7-14`` defines ``Builder(kernel)`` with an abstract
``build_callable() -> Callable``; the reference's only implementation is the TensorRT back end
(``python/asuka/backend/tensorrt/builder.py:13-151``).  ``B200Builder`` is the same plug-in for
this library: the callable takes tensors positionally, allocates its outputs with ``torch.empty``,
enqueues on the caller's current stream, and returns a tensor or a tuple in the case's output
order.  It accepts a case name (always available) or any object with a ``func_name`` attribute
naming one of the cases (the reference's ``Kernel`` carries one, partition/kernel.py:8-30).
"""
from abc import ABC, abstractmethod
from typing import Any, Callable

from . import cases


class Builder(ABC):
  """Same shape as python/asuka/backend/builder.py:7-14."""

  def __init__(self, kernel) -> None:
    self.kernel = kernel

  @abstractmethod
  def build_callable(self) -> Callable[..., Any]:
    pass


class B200Builder(Builder):

  def __init__(self, kernel, check_before_run=True, **case_kwargs) -> None:
    super().__init__(kernel)
    name = kernel if isinstance(kernel, str) else getattr(kernel, "func_name", None)
    if name not in cases.CASES:
      raise ValueError(f"no sm_100a kernels for {name!r}; known cases: {sorted(cases.CASES)}")
    self.case_name = name
    self.check_before_run = check_before_run
    self.case_kwargs = case_kwargs

  def build_callable(self) -> Callable[..., Any]:
    model = cases.CASES[self.case_name](**self.case_kwargs)
    n_in = 4 if self.case_name in ("KeyFormer", "Corm") else 3
    check = self.check_before_run

    def f(*args):
      if check:
        # the TensorRT back end raises RuntimeError on a mismatch (tensorrt/builder.py:104-111)
        if len(args) != n_in:
          raise RuntimeError(f"{self.case_name} takes {n_in} tensors, got {len(args)}")
        for a in args[:3]:
          if a.dtype != args[0].dtype:
            raise RuntimeError("q, k, v must share one dtype")
      return model.forward(*args)

    return f
