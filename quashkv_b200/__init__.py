"""quashkv_b200 — B200 (sm_100a) implementation of QuashKV's compressed-KV hot path.

Same public names as the reference package (quashkv/__init__.py:5-22); the hot
methods call hand-written CUDA kernels through ``libquashkv_b200.so``.
"""

__version__ = "0.1.0"

from .codebook import LloydMaxCodebook
from .engine import CompressedKVBlock, QuashKVEngine
from .mixed_precision import MixedPrecisionIPQuantizer, MixedPrecisionMSEQuantizer
from .nn_search import QuashIndex
from .packing import pack_bits, unpack_bits
from .quantizer import InnerProductQuantizer, MSEQuantizer

__all__ = [
    "LloydMaxCodebook", "MSEQuantizer", "InnerProductQuantizer", "QuashKVEngine", "CompressedKVBlock",
    "QuashIndex", "MixedPrecisionMSEQuantizer", "MixedPrecisionIPQuantizer", "pack_bits", "unpack_bits",
]
