"""nncv_b200: the compiled vision-model forward of nncv, rebuilt for B200 (sm_100a).

The product is ``libnncv_b200.so`` (CUDA kernels + C++ host runtime behind the C ABI of
``include/nncv_b200.h``); this package is its host-side mirror for Python callers and tests.
"""
from .memref import (MemRefDescriptor1, MemRefDescriptor2, MemRefDescriptor4, MemRefFlatArray,
                     MemRefIndexer, MemRefMagicHead, make_descriptor)

__all__ = ["MemRefDescriptor1", "MemRefDescriptor2", "MemRefDescriptor4", "MemRefFlatArray",
           "MemRefIndexer", "MemRefMagicHead", "make_descriptor"]
