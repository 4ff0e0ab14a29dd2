"""flashtensor_b200: hand-written sm_100a kernels for the fused attention programs of
FlashTensor/Asuka (plain causal attention and its Gemma-2 / SnapKV / CORM siblings, H2O, Keyformer,
RoCo, SimA, EA), behind the reference's per-case callables and back-end plug-in interface.  The
CUDA library is mandatory: importing the operator layer without it raises."""
from . import _lib
from .builder import B200Builder, Builder
from .cases import CASES, EA, Attn, Corm, Gemma2, H2O, KeyFormer, RoCo, SimA, SnapKV, get_model

__all__ = ["EA", "Attn", "Gemma2", "SnapKV", "Corm", "H2O", "KeyFormer", "RoCo", "SimA", "CASES", "get_model", "Builder",
           "B200Builder", "_lib"]
