from .api import CompressionFallbackWarning, compress, decompress
from .compressed_tensor import CompressedTensor
from .pipeline import decompress_many

__all__ = ["CompressedTensor", "CompressionFallbackWarning", "compress", "decompress", "decompress_many"]
