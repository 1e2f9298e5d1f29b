"""EntroPack-Lossy container schema and config. Stands in for entropack/schemes/lattice_rans/format.py:25-312.

Buffers (container order):
  payload      u16[]            all tiles back to back
  offsets      u32[tiles + 1]   tile bounds in u16 words
  states       u32[tiles, 32]   final encoder states
  stream_meta  i32[17, 4]       per table: n_symbols, sym_min, freq_offset, alphabet
  freq_tables  u16[sum alphabets]  normalised frequencies of the non-empty tables, concatenated
  scales       f32[rows]        reconstruction scale per row
  layout       i64[3]           cols (padded to a multiple of 8), prob_bits, tile_elements

Table 0 codes the coset c of each 8-vector; table 1 + 2f + c codes field f (z0..z6, then m) of a
vector whose coset is c. Tiles hold max(32, tile_elements // 9) vectors.
"""
import logging
from dataclasses import dataclass
from typing import Annotated, ClassVar, NamedTuple

import torch

from ..base import cached_parse
from ..config import CompressionConfig, OneOf, Range
from ..tile_ans.format import NUM_STATES

logger = logging.getLogger("entropack_b200.lattice_rans")

SUPPORTED_PROB_BITS = (9, 10, 11, 12, 13, 14, 15)
ALPHABET_COARSEN_MARGIN = 1.05
SUBSAMPLE_SEED_MULTIPLIER = 1000003
LATTICE_DIM = 8
NUM_TABLES = 17
MIN_RMS = 1.0e-12
#: Scale-independent bytes the rate search adds to the coded size (layout 64 + stream_meta 408 + slack 384),
#: the byte model of the reference's eager lane (entropack/schemes/lattice_rans/eager.py:94-107).
MODEL_FIXED_BYTES = 64 + 408 + 384


@dataclass
class EntroPackLossyConfig(CompressionConfig):
    """Lossy compression of finite 2-D tensors at a requested bits-per-parameter."""

    #: Requested bits per input element in [0.001, 11], capped at 1 for bool and 8 for one-byte dtypes.
    target_bpp: Annotated[float, Range(0.001, 11.0)] = 4.0
    #: Probability-table precision; None or 0 selects it automatically (11 up to 7 bpp, else 12, growing on overflow).
    prob_bits: Annotated[int | None, OneOf(SUPPORTED_PROB_BITS, silent=(0,))] = None
    #: Symbols per tile; None selects by rate (32768 / 16384 / 8192 / 4096 for <= 2 / 4 / 7 / more bpp).
    tile_elements: Annotated[int | None, Range(1, None)] = None
    #: Per-row rate-distortion sweeps (0 = off, the reference default).
    row_rdo_iterations: Annotated[int, Range(0, 8)] = 0
    #: Candidate scales per row for the rate-distortion sweeps.
    row_rdo_candidates: Annotated[int, Range(1, None)] = 5
    #: Bisection steps of the scale search.
    scale_search_iterations: Annotated[int, Range(1, None)] = 12
    #: Sampling budget of the scale search, in 8-value vectors.
    scale_search_max_vectors: Annotated[int, Range(1, None)] = 262144
    #: Accepted for compatibility; the kernels pick their own block width.
    threads_per_block: Annotated[int | None, Range(1, None)] = None
    #: Accepted for compatibility; payload words are always staged through shared memory.
    l2_prefetch: bool = True

    #: Tile size of :meth:`low_latency`.
    LOW_LATENCY_TILE_ELEMENTS: ClassVar[int] = 8192

    @classmethod
    def low_latency(cls, target_bpp: float = 4.0, **fields) -> "EntroPackLossyConfig":
        """The configuration for layers that decode their weight on every forward at small batch sizes.

        A tile is 32 interleaved rANS chains that a decoder has to walk one step after the other, so the time to decode
        a layer of a few million weights is the length of one tile's chain, not the size of the layer. This preset
        stores tiles of 8192 symbols (910 vectors, 257 steps) instead of the 16384 (1820 vectors, 513 steps) that rates
        up to 4 bpp get by default: the chain halves, every tile still costs its 132 bytes of states and offset, so a
        3840 x 3840 layer at 4 bpp stores about 0.02 bpp more for the same error. It is an ordinary ``tile_elements``
        setting: containers written with it decode with the reference implementation like any other.

        It pays while all of a layer's tiles still decode side by side: a B200 holds 3552 of them at once (24 warps on each
        of 148 SMs), that is layers of up to about 29 million weights at 8192 symbols a tile. Measured at 4 bpp, one token:
        3840 x 3840 (14.7 M weights) 62 -> 46 us per forward; 3840 -> 10240 (39.3 M weights, 4800 half-length tiles, two
        rounds) 87 -> 91 us, so larger layers keep the default."""
        fields.setdefault("tile_elements", cls.LOW_LATENCY_TILE_ELEMENTS)
        return cls(target_bpp=target_bpp, **fields)


LatticeRANSConfig = EntroPackLossyConfig

SUPPORTED_DTYPES = (
    torch.float32, torch.float16, torch.bfloat16,
    torch.float8_e4m3fn, torch.float8_e4m3fnuz, torch.float8_e5m2, torch.float8_e5m2fnuz,
    torch.int64, torch.int32, torch.int16, torch.int8, torch.uint64, torch.uint32, torch.uint16, torch.uint8, torch.bool,
)
_INTEGER_DTYPES = frozenset({
    torch.int64, torch.int32, torch.int16, torch.int8, torch.uint64, torch.uint32, torch.uint16, torch.uint8,
})


class LatticeBuffers(NamedTuple):
    payload: torch.Tensor
    offsets: torch.Tensor
    states: torch.Tensor
    stream_meta: torch.Tensor
    freq_tables: torch.Tensor
    scales: torch.Tensor
    layout: torch.Tensor


PACKED_KEYS = LatticeBuffers._fields
_SCHEMA = {
    "payload": torch.uint16, "offsets": torch.uint32, "states": torch.uint32, "stream_meta": torch.int32,
    "freq_tables": torch.uint16, "scales": torch.float32, "layout": torch.int64,
}


def recommended_tile_elements(target_bpp: float) -> int:
    if target_bpp <= 2.0:
        return 32768
    if target_bpp <= 4.0:
        return 16384
    if target_bpp <= 7.0:
        return 8192
    return 4096


def resolve_prob_bits(prob_bits: int | None, target_bpp: float) -> tuple[int, bool]:
    if prob_bits in (None, 0):
        return (11 if float(target_bpp) <= 7.0 else 12), True
    return int(prob_bits), False


def vector_tile_elements(tile_elements: int) -> int:
    return max(32, tile_elements // 9)


def subsample_index(rows: int, cols: int, sub_rows: int) -> torch.Tensor | None:
    """Rows the rate search looks at: a seeded CPU permutation, identical to the reference's
    (entropack/schemes/lattice_rans/format.py:127-134). None when every row is used."""
    if sub_rows >= rows:
        return None
    generator = torch.Generator().manual_seed(rows * SUBSAMPLE_SEED_MULTIPLIER + cols)
    return torch.randperm(rows, generator=generator)[:sub_rows]


def snap_to_container(values: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """fp32 -> container cast with saturation (float formats clamp to their largest finite value,
    integers round half to even and clamp)."""
    if dtype == torch.float32:
        return values
    if dtype == torch.bool:
        return values.round() != 0
    if dtype in _INTEGER_DTYPES:
        edge = torch.tensor(float(torch.iinfo(dtype).max) + 1.0, dtype=values.dtype)
        high = float(torch.nextafter(edge, torch.full_like(edge, float("-inf"))))
        return values.round().clamp(float(torch.iinfo(dtype).min), high).to(dtype)
    limit = float(torch.finfo(dtype).max)
    return values.clamp(-limit, limit).to(dtype)


def make_layout(cols: int, prob_bits: int, tile_elements: int) -> torch.Tensor:
    return torch.tensor([cols, prob_bits, tile_elements], dtype=torch.int64)


def parse_layout(layout: torch.Tensor) -> dict:
    if layout.dtype != torch.int64 or layout.ndim != 1 or layout.numel() != 3:
        raise ValueError("lattice_rans layout must be int64[3]")
    cols, prob_bits, tile_elements = (int(v) for v in layout.detach().cpu().tolist())
    if cols <= 0 or cols % LATTICE_DIM != 0:
        raise ValueError("lattice_rans vector-plane format requires positive cols divisible by 8")
    if prob_bits not in SUPPORTED_PROB_BITS:
        raise ValueError(f"lattice_rans prob_bits {prob_bits} unsupported")
    if tile_elements <= 0:
        raise ValueError("lattice_rans tile_elements must be positive")
    return {"cols": cols, "prob_bits": prob_bits, "tile_elements": tile_elements}


def decode_geometry(buffers: dict, shape: tuple) -> dict:
    stored = cached_parse(buffers["layout"], parse_layout, "_lattice_rans_layout")
    rows = int(shape[0])
    tile_vectors = vector_tile_elements(stored["tile_elements"])
    vectors = rows * (stored["cols"] // LATTICE_DIM)
    return {**stored, "rows": rows, "n_streams": NUM_TABLES, "total_tiles": max(1, -(-vectors // tile_vectors))}


def validate_packed(buffers: dict, shape: tuple, dtype: torch.dtype) -> dict:
    """Structural check of a container (reads the small buffers back to the host)."""
    missing = [key for key in PACKED_KEYS if key not in buffers]
    if missing:
        raise ValueError(f"lattice_rans packed data is missing buffers: {missing}")
    extra = sorted(set(buffers) - set(PACKED_KEYS))
    if extra:
        raise ValueError(f"lattice_rans packed data has unexpected buffers: {extra}")
    if not all(isinstance(buffers[key], torch.Tensor) for key in PACKED_KEYS):
        raise TypeError("lattice_rans packed buffers must be torch.Tensor values")
    if dtype not in SUPPORTED_DTYPES:
        raise ValueError(f"lattice_rans does not support output dtype {dtype}")
    if len(shape) != 2 or any(not isinstance(d, int) or d <= 0 for d in shape):
        raise ValueError(f"lattice_rans shape must be non-empty 2D, got {shape}")
    if len({buffers[key].device for key in PACKED_KEYS}) != 1:
        raise ValueError("lattice_rans packed buffers must share one device")
    for key, expected in _SCHEMA.items():
        if not buffers[key].is_contiguous():
            raise ValueError(f"lattice_rans buffer '{key}' must be contiguous")
        if buffers[key].dtype != expected:
            raise ValueError(f"lattice_rans buffer '{key}' must be {expected}, got {buffers[key].dtype}")
    info = decode_geometry(buffers, shape)
    rows, cols = shape
    if not 0 <= info["cols"] - cols < LATTICE_DIM:
        raise ValueError(f"lattice_rans layout columns {info['cols']} do not match {(rows, cols)}")
    scales = buffers["scales"]
    if scales.ndim != 1 or scales.numel() != rows:
        raise ValueError(f"lattice_rans scales must be 1D with one entry per row, got {tuple(scales.shape)}")
    if not bool((torch.isfinite(scales) & (scales > 0)).all()):
        raise ValueError("lattice_rans scales must be finite and positive")
    tiles = info["total_tiles"]
    meta = buffers["stream_meta"]
    if tuple(meta.shape) != (NUM_TABLES, 4):
        raise ValueError(f"lattice_rans stream_meta must be ({NUM_TABLES},4), got {tuple(meta.shape)}")
    if tuple(buffers["states"].shape) != (tiles, NUM_STATES):
        raise ValueError("lattice_rans states shape does not match total_tiles")
    if buffers["offsets"].numel() != tiles + 1:
        raise ValueError("lattice_rans offsets length must be total_tiles+1")
    offsets = buffers["offsets"].detach().cpu().to(torch.int64)
    if int(offsets[0]) != 0 or int(offsets[-1]) != buffers["payload"].numel():
        raise ValueError("lattice_rans payload offsets endpoints are invalid")
    if bool((offsets[1:] < offsets[:-1]).any()):
        raise ValueError("lattice_rans payload offsets must be monotone")
    table_size = 1 << info["prob_bits"]
    meta_host = meta.detach().cpu().to(torch.int64)
    freq = buffers["freq_tables"].detach().cpu().to(torch.int64)
    cursor, counts = 0, []
    for table in range(NUM_TABLES):
        n_symbols, _sym_min, offset, alphabet = (int(v) for v in meta_host[table])
        if n_symbols < 0 or alphabet < 0 or offset < 0:
            raise ValueError("lattice_rans table metadata has a negative field")
        if offset != cursor or offset + alphabet > freq.numel():
            raise ValueError("lattice_rans frequency-table ranges must be contiguous")
        if (n_symbols == 0) != (alphabet == 0):
            raise ValueError("lattice_rans empty table metadata is inconsistent")
        if alphabet:
            if alphabet > table_size:
                raise ValueError("lattice_rans table alphabet exceeds probability precision")
            if int(freq[offset : offset + alphabet].sum()) != table_size:
                raise ValueError("lattice_rans normalized frequencies have an invalid sum")
        cursor += alphabet
        counts.append(n_symbols)
    if cursor != freq.numel():
        raise ValueError("lattice_rans frequency table has trailing entries")
    vectors = rows * (info["cols"] // LATTICE_DIM)
    if counts[0] != vectors or int(meta_host[0, 1]) != 0:
        raise ValueError("lattice_rans coset table metadata is invalid")
    if int(meta_host[0, 3]) > 2:
        # a coset is 0 or 1 and selects between two tables per field; the reference derives it by comparing the slot
        # with the first frequency (lattice_rans.cu, e8_decode_coset), so a third symbol can only come from corruption
        raise ValueError("lattice_rans coset table has more than two symbols")
    if counts[1] + counts[2] != vectors:
        raise ValueError("lattice_rans conditioned table counts do not cover all vectors")
    for field in range(8):
        if counts[1 + 2 * field] != counts[1] or counts[2 + 2 * field] != counts[2]:
            raise ValueError("lattice_rans conditioned table counts disagree across fields")
    return info
