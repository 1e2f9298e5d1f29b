"""Host orchestration of the EntroPack-Lossy encoder over the sm_100a kernels.

Follows the reference's encode flow (entropack/schemes/lattice_rans/cuda.py:436-597, eager.py:110-194):
row RMS -> geometric bisection of the lattice scale on a seeded row subsample, priced with the eager
lane's byte model -> full quantisation -> alphabet check (automatic prob_bits grows, otherwise the scale
is coarsened) -> least-squares row scales -> normalised tables -> rANS encode -> compaction.
All tensor-sized work runs on the GPU; the host sees only the 34-word min/max record and the compact
histogram of each pass (one device->host copy per bisection step).
"""
import ctypes
import math

import numpy as np
import torch

from ... import _native
from ..tile_ans.format import NUM_STATES
from .format import (
    ALPHABET_COARSEN_MARGIN, LATTICE_DIM, MODEL_FIXED_BYTES, NUM_TABLES, LatticeBuffers, logger, make_layout, resolve_prob_bits,
    subsample_index, vector_tile_elements,
)

_MINMAX_WORDS = 34
_HEADER_WORDS = 36          # min/max record, bins_used, one pad word: keeps the bins 16-byte aligned
_DEFAULT_BINS = 16384


class _Pass:
    """Device buffers for quantising one operand (the full tensor or the search subsample)."""

    def __init__(self, work: torch.Tensor, rms: torch.Tensor):
        self.work, self.rms = work, rms
        self.rows, self.cols = work.shape
        self.vectors = self.rows * (self.cols // LATTICE_DIM)
        self.is_bf16 = int(work.dtype == torch.bfloat16)
        device = work.device
        self.device = device
        self.fields = torch.empty((self.vectors, 8), dtype=torch.int16, device=device)
        self.cosets = torch.empty(self.vectors, dtype=torch.uint8, device=device)
        self._allocate_stats(_DEFAULT_BINS)

    def _allocate_stats(self, capacity: int) -> None:
        self.capacity = capacity
        self.stats = torch.empty(_HEADER_WORDS + capacity, dtype=torch.int32, device=self.device)

    def quantize(self, scale: float):
        """Quantise at ``scale`` and count symbols. Returns (minmax int32[34], bins int32[used]) on the host."""
        lib = _native.load()
        stream = _native.stream_handle(self.device)
        while True:
            stats_ptr = self.stats.data_ptr()
            _native.check(lib.ep_lattice_quantize(
                _native.ptr(self.work), self.is_bf16, _native.ptr(self.rms), self.rows, self.cols, float(scale),
                _native.ptr(self.fields), _native.ptr(self.cosets), stats_ptr, stream), "lattice_rans quantize")
            _native.check(lib.ep_lattice_histogram(
                _native.ptr(self.fields), _native.ptr(self.cosets), self.vectors, stats_ptr, stats_ptr + 4 * _HEADER_WORDS,
                self.capacity, stats_ptr + 4 * _MINMAX_WORDS, stream), "lattice_rans histogram")
            host = self.stats.cpu().numpy()
            used = int(host[_MINMAX_WORDS])
            if used <= self.capacity:
                return np.ascontiguousarray(host[:_MINMAX_WORDS]), np.ascontiguousarray(host[_HEADER_WORDS:_HEADER_WORDS + used])
            self._allocate_stats(used)

    def coded_bytes(self, minmax: np.ndarray, bins: np.ndarray, prob_bits: int, tile_elements: int) -> float:
        if minmax[33]:
            return math.inf  # a field left the int16 range: far too fine a scale for any table
        value = ctypes.c_double(0.0)
        _native.check(_native.load().ep_lattice_coded_bytes(
            minmax.ctypes.data, bins.ctypes.data, self.vectors, prob_bits, tile_elements, ctypes.addressof(value)),
            "lattice_rans size model")
        return value.value


def _row_rms(work: torch.Tensor) -> torch.Tensor:
    rows, cols = work.shape
    rms = torch.empty(rows, dtype=torch.float32, device=work.device)
    _native.check(_native.load().ep_lattice_row_rms(
        _native.ptr(work), int(work.dtype == torch.bfloat16), rows, cols, _native.ptr(rms), _native.stream_handle(work.device)),
        "lattice_rans row rms")
    return rms


def _bisect_scale(work, rms, target_bpp, prob_bits, tile_elements, iterations, max_vectors) -> float:
    rows, cols = work.shape
    sub_rows = max(1, min(rows, max_vectors // (cols // LATTICE_DIM)))
    index = subsample_index(rows, cols, sub_rows)
    if index is not None:
        index = index.to(work.device)
        work, rms = work.index_select(0, index).contiguous(), rms.index_select(0, index).contiguous()
    search = _Pass(work, rms)
    elements = sub_rows * cols
    lo, hi = 0.001, 8.0
    for _ in range(iterations):
        mid = math.sqrt(lo * hi)
        minmax, bins = search.quantize(mid)
        total = search.coded_bytes(minmax, bins, prob_bits, tile_elements) + sub_rows * 4 + MODEL_FIXED_BYTES
        if 8 * total / elements > target_bpp:
            lo = mid
        else:
            hi = mid
    return math.sqrt(lo * hi)


def encode(weight: torch.Tensor, *, target_bpp: float, prob_bits, tile_elements: int, row_rdo_iterations: int,
           scale_search_iterations: int, scale_search_max_vectors: int) -> LatticeBuffers:
    _native.require_cuda(weight)
    if row_rdo_iterations:
        raise NotImplementedError("per-row rate-distortion refinement (row_rdo_iterations > 0) is not implemented")
    if weight.shape[1] % LATTICE_DIM:
        raise ValueError(f"lattice_rans quantizes whole E8 vectors, so the column count must be a multiple of {LATTICE_DIM}; "
                         f"got cols={weight.shape[1]}")
    device = weight.device
    lib = _native.load()
    with torch.cuda.device(device):
        work = weight.contiguous() if weight.dtype == torch.bfloat16 else weight.float().contiguous()
        rows, cols = work.shape
        rms = _row_rms(work)
        if not bool(torch.isfinite(rms).all()):
            raise ValueError(
                f"lattice_rans normalizes rows in fp32, and the row RMS of this {weight.dtype} tensor overflowed; "
                "rescale the source, or use tile_ans, which has no numeric range limit")
        prob_bits, auto = resolve_prob_bits(prob_bits, target_bpp)
        full = _Pass(work, rms)
        if float(work.abs().amax()) == 0.0:
            scale = 1.0
            minmax, bins = full.quantize(scale)
        else:
            clamped = False
            while True:
                escalate = False
                scale = _bisect_scale(work, rms, target_bpp, prob_bits, tile_elements, scale_search_iterations,
                                      scale_search_max_vectors)
                while True:
                    minmax, bins = full.quantize(scale)
                    alphabet = 1 << 30 if minmax[33] else int(lib.ep_lattice_max_alphabet(minmax.ctypes.data))
                    if alphabet <= (1 << prob_bits):
                        break
                    if auto and prob_bits < 15:
                        prob_bits += 1
                        escalate = True
                        break
                    clamped = True
                    scale *= alphabet / (1 << prob_bits) * ALPHABET_COARSEN_MARGIN
                if not escalate:
                    if clamped:
                        logger.debug("lattice_rans coarsened the lattice scale to %.6g so a coordinate alphabet of %d fits the "
                                     "%d-entry rANS table; actual_bpp will fall below target_bpp", scale, alphabet, 1 << prob_bits)
                    break
        stream = _native.stream_handle(device)
        scales = torch.empty(rows, dtype=torch.float32, device=device)
        _native.check(lib.ep_lattice_refit_scales(
            _native.ptr(work), full.is_bf16, _native.ptr(full.fields), _native.ptr(full.cosets), _native.ptr(rms), float(scale),
            rows, cols, _native.ptr(scales), stream), "lattice_rans refit")

        meta_host = np.zeros((NUM_TABLES, 4), dtype=np.int32)
        freq_host = np.zeros(max(1, bins.size), dtype=np.uint16)
        entries = ctypes.c_int64(0)
        _native.check(lib.ep_lattice_tables(
            minmax.ctypes.data, bins.ctypes.data, full.vectors, prob_bits, meta_host.ctypes.data, freq_host.ctypes.data,
            freq_host.size, ctypes.addressof(entries)), "lattice_rans tables")
        freq_host = freq_host[: entries.value]
        stream_meta = torch.from_numpy(meta_host).to(device)
        freq_tables = torch.from_numpy(freq_host.copy()).to(device)

        tile_vectors = vector_tile_elements(tile_elements)
        tiles = max(1, -(-full.vectors // tile_vectors))
        scratch = torch.empty(tiles * tile_vectors * 9, dtype=torch.uint16, device=device)
        symbol_scratch = torch.empty(max(1, entries.value) * 2, dtype=torch.int32, device=device)
        word_counts = torch.empty(tiles, dtype=torch.uint32, device=device)
        states = torch.empty((tiles, NUM_STATES), dtype=torch.uint32, device=device)
        offsets = torch.empty(tiles + 1, dtype=torch.uint32, device=device)
        total = torch.empty(1, dtype=torch.int64, device=device)
        _native.check(lib.ep_lattice_encode(
            _native.ptr(full.fields), _native.ptr(full.cosets), full.vectors, _native.ptr(stream_meta), _native.ptr(freq_tables),
            entries.value, prob_bits, tile_elements, _native.ptr(symbol_scratch), _native.ptr(scratch), _native.ptr(word_counts),
            _native.ptr(states), stream), "lattice_rans encode")
        _native.check(lib.ep_exclusive_scan_u32(_native.ptr(word_counts), tiles, _native.ptr(offsets), _native.ptr(total), stream),
                      "lattice_rans offsets")
        total_words = int(total.item())
        if total_words >= 1 << 32:
            raise ValueError("lattice_rans payload exceeds uint32 offset capacity")
        payload = torch.empty(total_words, dtype=torch.uint16, device=device)
        if total_words:
            _native.check(lib.ep_compact_streams(_native.ptr(scratch), _native.ptr(offsets), _native.ptr(payload),
                                                 tile_vectors * 9, tiles, stream), "lattice_rans compaction")
    result = LatticeBuffers(
        payload=payload, offsets=offsets, states=states, stream_meta=stream_meta, freq_tables=freq_tables, scales=scales,
        layout=make_layout(cols, prob_bits, tile_elements).to(device))
    result.layout._lattice_rans_search_scale = scale
    return result
