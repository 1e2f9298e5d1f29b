from .api import CompressionFallbackWarning, compress, decompress
from .compressed_tensor import CompressedTensor

__all__ = ["CompressedTensor", "CompressionFallbackWarning", "compress", "decompress"]
