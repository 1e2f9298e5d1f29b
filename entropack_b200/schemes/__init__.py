from ..registry import all_schemes
from .base import Scheme
from .config import CompressionConfig, RawConfig
from .tile_ans import TileANSConfig

__all__ = ["CompressionConfig", "RawConfig", "Scheme", "TileANSConfig", "all_schemes"]
