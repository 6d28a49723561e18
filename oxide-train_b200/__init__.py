"""B200-native (sm_100a) GEMM layer behind the reference trainer's matmul entry points.

``Tcgen05Gemm`` mirrors the reference's host type of the same name; the work is
done by ``libb200gemm.so`` (hand-written CUDA, built from ``csrc/``).
"""
from . import _lib
from ._lib import B200GemmError, GemmDesc
from .gemm import Tcgen05Gemm
from .lmhead import FusedLmHead
from . import moe
from . import parallel
from .moe import GroupedExpertFfn, GatedExpertFfn

__all__ = ["Tcgen05Gemm", "FusedLmHead", "GroupedExpertFfn", "GatedExpertFfn", "moe", "parallel", "B200GemmError", "GemmDesc", "_lib"]
