"""entropack_b200: the entropack compression hot path on B200 (sm_100a) behind the reference's public API.

``compress`` / ``decompress``, the config classes and ``CompressedTensor`` keep the names, defaults and
byte layout of modelscope/entropack, so containers written by either side decode on the other. All
compute runs in hand-written CUDA kernels reached through a C ABI (``include/entropack_b200.h``);
there is no CPU or eager execution path.
"""
from .compression import CompressedTensor, CompressionFallbackWarning, compress, decompress, decompress_many
from .decode_ahead import DecodeAhead
from .linear import CompressedFP8Linear, CompressedINT8Linear, CompressedLinear, check_kernel_errors, prepare_decode_plans
from .registry import DispatchError
from .schemes import CompressionConfig, DFloat11Config, EntroPackLossyConfig, LatticeRANSConfig, RawConfig, TileANSConfig

__version__ = "0.1.0"

__all__ = [
    "CompressedFP8Linear", "CompressedINT8Linear", "CompressedLinear", "CompressedTensor", "CompressionConfig", "CompressionFallbackWarning", "DFloat11Config", "DecodeAhead", "DispatchError", "EntroPackLossyConfig",
    "LatticeRANSConfig", "RawConfig", "TileANSConfig",
    "__version__", "check_kernel_errors", "compress", "decompress", "decompress_many", "prepare_decode_plans",
]
