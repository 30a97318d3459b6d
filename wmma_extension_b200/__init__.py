"""B200-native TCEC SGEMM: error-corrected FP32 GEMM emulation on tcgen05 tensor cores.

``wmma_extension_b200.tcec`` binds the C ABI declared in ``include/tcec.h``.
"""
from . import tcec  # noqa: F401

__all__ = ["tcec"]
