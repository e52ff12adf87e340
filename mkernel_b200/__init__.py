"""mkernel_b200: B200-native AllGather+GEMM, GEMM+ReduceScatter and GEMM+AllReduce behind the
operator interface of uccl-project/mKernel (``load_module.load(name)`` -> ``DistBuffer``,
``*_prepare``, ``*_launch``)."""
from . import _lib
from .load_module import load

__all__ = ["load", "_lib"]
