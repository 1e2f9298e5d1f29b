"""Tile-ANS scheme. Stands in for entropack/schemes/tile_ans/__init__.py:8-50."""
import torch

from ..base import Scheme, StreamingPlan, packed_buffers, register_scheme
from ..checks import prepare_weight
from .format import OPTIONS_BY_DTYPE, PACKED_KEYS, TileANSConfig, TileBuffers, num_tiles, parse_layout_cached, validate_packed


class TileStreamingPlan(StreamingPlan):
    """Tiles as streaming units: tile ``t`` reads streams ``lane * tiles + t`` of the payload (one byte range per byte
    lane for a run of tiles) and writes ``tile_elements`` whole elements."""

    streamed_buffer = "payload"
    granule = 8    # tiles per decode block

    def __init__(self, scheme: "TileANSScheme", buffers: TileBuffers, dtype: torch.dtype):
        tile_elements, _, num_lanes, num_elements = parse_layout_cached(buffers.layout)
        self.scheme, self.dtype, self.lanes = scheme, dtype, num_lanes
        self.units = num_tiles(num_elements, tile_elements)
        self.unit_output_bytes = tile_elements * num_lanes
        self.output_bytes = num_elements * num_lanes
        self.offsets = buffers.offsets.numpy()    # host view, uint32[lanes * tiles + 1], in 16-bit words

    def byte_ranges(self, first: int, count: int) -> list[tuple[int, int]]:
        ranges = []
        for lane in range(self.lanes):
            begin = 2 * int(self.offsets[lane * self.units + first])
            end = 2 * int(self.offsets[lane * self.units + first + count])
            if end > begin:
                ranges.append((begin, end))
        return ranges

    def decode_units(self, buffers: dict, output: torch.Tensor, first: int, count: int, config: TileANSConfig) -> None:
        self.scheme.lane().decode(packed_buffers(buffers, TileBuffers), dtype=self.dtype,
                                  threads_per_block=config.threads_per_block, out=output, tiles=(first, count))


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

    def streaming_plan(self, buffers: dict, *, shape, dtype):
        packed = packed_buffers(buffers, TileBuffers)
        if packed.layout.device.type != "cpu":
            return None
        return TileStreamingPlan(self, packed, dtype)

    def decode(self, packed: dict, *, shape: tuple[int, ...], dtype: torch.dtype, config: TileANSConfig,
               error: torch.Tensor | None = None) -> torch.Tensor:
        buffers = packed_buffers(packed, TileBuffers)
        source = buffers.layout.device
        lane, run_on = self.lane_for(buffers.layout, config.execution_backend, gate_dtype=False)
        if source != run_on:
            buffers = TileBuffers._make(value.to(run_on) for value in buffers)
        out = lane.decode(buffers, dtype=dtype, threads_per_block=config.threads_per_block, error=error).reshape(shape)
        return out if out.device == source else out.to(source)


register_scheme(TileANSScheme())

__all__ = ["TileANSConfig", "TileANSScheme"]
