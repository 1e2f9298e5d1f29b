"""DFloat11 scheme. Stands in for entropack/schemes/dfloat11/__init__.py:9-47."""
import torch

from ..base import Scheme, packed_buffers, register_scheme
from ..checks import prepare_weight
from .format import PACKED_KEYS, DFloat11Buffers, DFloat11Config, validate_packed


class DFloat11Scheme(Scheme):
    name = "dfloat11"
    buffer_names = PACKED_KEYS
    priority = 200
    dtypes = (torch.bfloat16,)

    def encode(self, weight: torch.Tensor, config: DFloat11Config) -> dict:
        weight = prepare_weight(weight, scheme=self.name, dtypes=self.dtypes)
        source = weight.device
        flat = weight.reshape(-1)
        lane, run_on = self.lane_for(flat, config.execution_backend)
        if source != run_on:
            flat = flat.to(run_on)
        codec = lane.build_codec(lane.exponent_counter(flat, config.threads_per_block))
        buffers = lane.encode(weight=flat, codec=codec, luts=lane.build_luts(codec), bytes_per_thread=config.bytes_per_thread,
                              threads_per_block=config.threads_per_block)
        return {key: value.to(source) for key, value in buffers._asdict().items()}

    def validate_buffers(self, buffers, shape, dtype):
        validate_packed(buffers, shape)

    def prime_host_metadata(self, buffers: dict) -> None:
        from .format import parse_layout_cached

        parse_layout_cached(buffers["layout"])

    def prepare_decode_plan(self, buffers: dict, *, shape: tuple[int, ...]) -> bool:
        from . import b200

        packed = packed_buffers(buffers, DFloat11Buffers)
        if packed.layout.device.type != "cuda" or getattr(packed.layout, "_dfloat11_decode_tables", None) is not None:
            return False
        b200.decode_tables(packed)
        return True

    def decode(self, packed: dict, *, shape: tuple[int, ...], dtype: torch.dtype, config: DFloat11Config,
               error: torch.Tensor | None = None) -> torch.Tensor:
        buffers = packed_buffers(packed, DFloat11Buffers)
        source = buffers.layout.device
        lane, run_on = self.lane_for(buffers.layout, config.execution_backend, gate_dtype=False)
        if source != run_on:
            buffers = DFloat11Buffers._make(value.to(run_on) for value in buffers)
        out = lane.decode(buffers, error=error).reshape(shape)
        return out if out.device == source else out.to(source)


register_scheme(DFloat11Scheme())

__all__ = ["DFloat11Config", "DFloat11Scheme"]
