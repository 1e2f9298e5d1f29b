"""EntroPack-Lossy scheme. Stands in for entropack/schemes/lattice_rans/__init__.py:13-58."""
import torch

from ..base import Scheme, packed_buffers, register_scheme
from ..checks import prepare_weight
from .format import (
    LATTICE_DIM, PACKED_KEYS, SUPPORTED_DTYPES, EntroPackLossyConfig, LatticeBuffers, LatticeRANSConfig,
    recommended_tile_elements, validate_packed,
)

__all__ = ["EntroPackLossyConfig", "LatticeRANSConfig", "LatticeRANSScheme"]


class LatticeRANSScheme(Scheme):
    name = "lattice_rans"
    buffer_names = PACKED_KEYS
    lossless = False
    priority = 0
    dtypes = SUPPORTED_DTYPES

    def encode(self, weight: torch.Tensor, config: EntroPackLossyConfig) -> dict:
        weight = prepare_weight(weight, scheme=self.name, ndim=2, dtypes=SUPPORTED_DTYPES, require_finite=True)
        target_bpp = min(float(config.target_bpp), 1.0 if weight.dtype == torch.bool else weight.element_size() * 8.0)
        shape, source = tuple(weight.shape), weight.device
        lane, run_on = self.lane_for(weight, config.execution_backend)
        if source != run_on:
            weight = weight.to(run_on)
        pad = -shape[1] % LATTICE_DIM
        if pad:
            weight = torch.cat([weight, weight.new_zeros(shape[0], pad)], dim=1)
        tile_elements = recommended_tile_elements(target_bpp) if config.tile_elements is None else int(config.tile_elements)
        packed = lane.encode(
            weight, target_bpp=target_bpp, prob_bits=None if config.prob_bits in (None, 0) else int(config.prob_bits),
            tile_elements=tile_elements, row_rdo_iterations=config.row_rdo_iterations,
            row_rdo_candidates=config.row_rdo_candidates, scale_search_iterations=config.scale_search_iterations,
            scale_search_max_vectors=config.scale_search_max_vectors)
        return {key: value.to(source) for key, value in packed._asdict().items()}

    def validate_buffers(self, buffers, shape, dtype):
        validate_packed(buffers, tuple(shape), dtype)

    def prime_host_metadata(self, buffers: dict) -> None:
        from ..base import cached_parse
        from .b200 import max_alphabet
        from .format import parse_layout

        cached_parse(buffers["layout"], parse_layout, "_lattice_rans_layout")
        max_alphabet(packed_buffers(buffers, LatticeBuffers))

    def prepare_decode_plan(self, buffers: dict, *, shape: tuple[int, ...]) -> bool:
        from . import b200

        packed = packed_buffers(buffers, LatticeBuffers)
        return packed.layout.device.type == "cuda" and b200.prepare_plan(packed, shape=tuple(shape))

    def decode(self, packed: dict, *, shape: tuple[int, ...], dtype: torch.dtype, config: EntroPackLossyConfig,
               error: torch.Tensor | None = None) -> torch.Tensor:
        buffers = packed_buffers(packed, LatticeBuffers)
        source = buffers.layout.device
        lane, run_on = self.lane_for(buffers.layout, config.execution_backend, gate_dtype=False)
        if source != run_on:
            buffers = LatticeBuffers._make(value.to(run_on) for value in buffers)
        out = lane.decode(buffers, shape=shape, dtype=dtype, threads_per_block=config.threads_per_block,
                          l2_prefetch=config.l2_prefetch, error=error)
        if shape and tuple(out.shape) != tuple(shape):
            out = out[: shape[0], : shape[1]]
        return out if out.device == source else out.to(source)


register_scheme(LatticeRANSScheme())
