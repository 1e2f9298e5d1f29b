"""Tile-ANS scheme. Stands in for entropack/schemes/tile_ans/__init__.py:8-50."""
import torch

from ..base import Scheme, packed_buffers, register_scheme
from ..checks import prepare_weight
from .format import OPTIONS_BY_DTYPE, PACKED_KEYS, TileANSConfig, TileBuffers, parse_layout_cached, validate_packed


class TileANSScheme(Scheme):
    name = "tile_ans"
    buffer_names = PACKED_KEYS
    priority = 100
    dtypes = tuple(OPTIONS_BY_DTYPE)

    def options_for(self, dtype):
        tile_elements, probability_bits = OPTIONS_BY_DTYPE[dtype]
        return {"tile_elements": tile_elements, "probability_bits": probability_bits,
                "raw_lane_threshold": TileANSConfig().raw_lane_threshold}

    def encode(self, weight: torch.Tensor, config: TileANSConfig) -> dict:
        weight = prepare_weight(weight, scheme=self.name)
        tile_elements = config.tile_elements
        if tile_elements == 0:
            tile_elements = 4096 if weight.numel() * weight.element_size() <= 32 * 1024 * 1024 else 8192
        source = weight.device
        lane, run_on = self.lane_for(weight, config.execution_backend)
        if source != run_on:
            weight = weight.to(run_on)
        buffers = lane.encode(
            weight=weight, tile_elements=tile_elements, probability_bits=config.probability_bits,
            raw_lane_threshold=config.raw_lane_threshold, threads_per_block=config.threads_per_block)
        return {key: value.to(source) for key, value in buffers._asdict().items()}

    def validate_buffers(self, buffers, shape, dtype):
        validate_packed(buffers, shape, dtype)

    def prime_host_metadata(self, buffers: dict) -> None:
        from .b200 import _lane_modes_host   # host-only helpers; importing them does not load the kernel library

        packed = packed_buffers(buffers, TileBuffers)
        parse_layout_cached(packed.layout)
        _lane_modes_host(packed)

    def decode(self, packed: dict, *, shape: tuple[int, ...], dtype: torch.dtype, config: TileANSConfig) -> torch.Tensor:
        buffers = packed_buffers(packed, TileBuffers)
        source = buffers.layout.device
        lane, run_on = self.lane_for(buffers.layout, config.execution_backend, gate_dtype=False)
        if source != run_on:
            buffers = TileBuffers._make(value.to(run_on) for value in buffers)
        out = lane.decode(buffers, dtype=dtype, threads_per_block=config.threads_per_block).reshape(shape)
        return out if out.device == source else out.to(source)


register_scheme(TileANSScheme())

__all__ = ["TileANSConfig", "TileANSScheme"]
