from ..registry import all_schemes
from .base import Scheme
from .config import CompressionConfig, RawConfig
from .dfloat11 import DFloat11Config
from .lattice_rans import EntroPackLossyConfig, LatticeRANSConfig
from .tile_ans import TileANSConfig

__all__ = ["CompressionConfig", "DFloat11Config", "EntroPackLossyConfig", "LatticeRANSConfig", "RawConfig", "Scheme", "TileANSConfig", "all_schemes"]
