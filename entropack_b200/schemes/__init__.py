from ..registry import all_schemes
from .base import Scheme
from .config import CompressionConfig, RawConfig
from .lattice_rans import EntroPackLossyConfig, LatticeRANSConfig
from .tile_ans import TileANSConfig

__all__ = ["CompressionConfig", "EntroPackLossyConfig", "LatticeRANSConfig", "RawConfig", "Scheme", "TileANSConfig", "all_schemes"]
