"""Functional "fused" entry points with the reference's names and signatures
(quashkv/triton_kernels/__init__.py:17-28).  The module keeps the reference's name
so imports port unchanged; nothing here uses Triton — every function is a call
into the CUDA library, and ``HAS_TRITON`` is False.
"""

from .attention import CompressedBlock, fused_quantized_attention
from .compress import fused_compress_ip, fused_compress_mse
from .decompress import fused_decompress_ip, fused_decompress_mse

HAS_TRITON = False

__all__ = ["HAS_TRITON", "fused_compress_mse", "fused_compress_ip", "fused_decompress_mse",
           "fused_decompress_ip", "fused_quantized_attention", "CompressedBlock"]
