"""Host orchestration of the EntroPack-Lossy encoder over the sm_100a kernels.

Follows the reference's encode flow (entropack/schemes/lattice_rans/cuda.py:436-597, eager.py:110-194):
row RMS -> geometric bisection of the lattice scale on a seeded row subsample, priced with the eager
lane's byte model -> full quantisation -> alphabet check (automatic prob_bits grows, otherwise the scale
is coarsened) -> least-squares row scales -> optional per-row rate-distortion refinement
(entropack/schemes/lattice_rans/rdo.py) -> normalised tables -> rANS encode -> compaction.
All tensor-sized work runs on the GPU; the host sees only the 34-word min/max record and the compact
histogram of each pass (one device->host copy per bisection step) and, under row refinement, the
rows x candidates matrices of distortions and rates.
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

EP_MORE_BINS = 1            # status of ep_lattice_search_scale: retry with the capacity it reports
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

    def summarize(self):
        """(minmax, bins) of the symbols already in ``fields`` / ``cosets`` (a mixture of candidate rows)."""
        lib = _native.load()
        stream = _native.stream_handle(self.device)
        while True:
            stats_ptr = self.stats.data_ptr()
            _native.check(lib.ep_lattice_minmax(_native.ptr(self.fields), _native.ptr(self.cosets), self.vectors, stats_ptr, stream),
                          "lattice_rans min/max")
            _native.check(lib.ep_lattice_histogram(
                _native.ptr(self.fields), _native.ptr(self.cosets), self.vectors, stats_ptr, stats_ptr + 4 * _HEADER_WORDS,
                self.capacity, stats_ptr + 4 * _MINMAX_WORDS, stream), "lattice_rans histogram")
            host = self.stats.cpu().numpy()
            used = int(host[_MINMAX_WORDS])
            if used <= self.capacity:
                return np.ascontiguousarray(host[:_MINMAX_WORDS]), np.ascontiguousarray(host[_HEADER_WORDS:_HEADER_WORDS + used])
            self._allocate_stats(used)

    def refit(self, scale: float):
        """Least-squares row scales and the squared error each row is left with, float32[rows] each, on the device."""
        scales = torch.empty(self.rows, dtype=torch.float32, device=self.device)
        row_sse = torch.empty(self.rows, dtype=torch.float32, device=self.device)
        _native.check(_native.load().ep_lattice_refit_rows(
            _native.ptr(self.work), self.is_bf16, _native.ptr(self.fields), _native.ptr(self.cosets), _native.ptr(self.rms),
            float(scale), self.rows, self.cols, _native.ptr(scales), _native.ptr(row_sse), _native.stream_handle(self.device)),
            "lattice_rans refit")
        return scales, row_sse

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
    # The bisection itself runs in the library (quantise, count, read back, price, halve the interval; one call instead
    # of a dozen round trips through Python): per step the midpoint sqrt(lo * hi) is kept when
    # 8 * (coded bytes + 4 bytes per row scale + fixed bytes) / elements stays within the target.
    scale, needed = ctypes.c_double(0.0), ctypes.c_int64(0)
    while True:
        status = _native.load().ep_lattice_search_scale(
            _native.ptr(search.work), search.is_bf16, _native.ptr(search.rms), search.rows, search.cols, _native.ptr(search.fields),
            _native.ptr(search.cosets), search.stats.data_ptr(), search.capacity, float(target_bpp), int(prob_bits), int(tile_elements),
            int(iterations), 0.001, 8.0, float(MODEL_FIXED_BYTES), ctypes.addressof(scale), ctypes.addressof(needed),
            _native.stream_handle(search.device))
        if status != EP_MORE_BINS:
            break
        search._allocate_stats(int(needed.value))   # alphabets wider than the bins: again with room for them
    _native.check(status, "lattice_rans rate search")
    return scale.value


# ---- per-row rate-distortion refinement (entropack/schemes/lattice_rans/rdo.py) -----------------------------
RATIO_SPAN = (0.70, 1.45)


def ratio_ladder(count: int) -> tuple[float, ...]:
    """Scale ratios priced per row: 1.0, then repeatedly the geometric midpoint of the widest log-gap inside
    RATIO_SPAN (rdo.ratio_ladder, rdo.py:12-22)."""
    points = [1.0]
    while len(points) < count:
        bounds = [RATIO_SPAN[0], *points, RATIO_SPAN[1]]
        widest = max(range(1, len(bounds)), key=lambda j: bounds[j] / bounds[j - 1])
        points.insert(widest - 1, (bounds[widest] * bounds[widest - 1]) ** 0.5)
    return tuple(points)


def _stream_counts(minmax: np.ndarray, bins: np.ndarray):
    """Per table: (counts int64[alphabet], first symbol). Table 0 is the coset; table 1 + st the coordinate streams."""
    coset_alphabet = int(minmax[32]) + 1
    streams = [(bins[:coset_alphabet].astype(np.int64), 0)]
    cursor = 2
    for st in range(NUM_TABLES - 1):
        low, high = int(minmax[2 * st]), int(minmax[2 * st + 1])
        if low == 0x7FFFFFFF:
            streams.append((np.zeros(0, dtype=np.int64), 0))
            continue
        width = high - low + 1
        streams.append((bins[cursor:cursor + width].astype(np.int64), low))
        cursor += width
    return streams


def _rate_table(streams, minima, maxima, device, alpha: float = 0.5):
    """Smoothed ideal code lengths of the current symbol statistics over every candidate's range
    (rdo.rate_costs, rdo.py:49-67): values float32, offsets int32[18], minima int32[17]."""
    tables, offsets = [], [0]
    for table, (counts, first) in enumerate(streams):
        width = maxima[table] - minima[table] + 1
        expanded = np.zeros(width, dtype=np.float64)
        if counts.size:
            at = first - minima[table]
            expanded[at:at + counts.size] = counts
        probability = (expanded + alpha) / (float(counts.sum()) + alpha * width)
        tables.append((-np.log2(probability)).astype(np.float32))
        offsets.append(offsets[-1] + width)
    return (torch.from_numpy(np.concatenate(tables)).to(device), torch.tensor(offsets, dtype=torch.int32, device=device),
            torch.tensor(minima, dtype=torch.int32, device=device))


def _choose_rate_tradeoff(distortion: np.ndarray, rates: np.ndarray, desired_rate: float) -> np.ndarray:
    """Per row, the candidate minimising distortion + lambda * rate, with lambda the smallest multiplier (found by
    doubling, then 20 bisection steps) whose total rate does not exceed ``desired_rate`` (rdo.choose_rate_tradeoff,
    rdo.py:123-143). float32 arithmetic, as in the reference."""
    row = np.arange(distortion.shape[0])
    best = distortion.argmin(1)
    if rates[row, best].sum(dtype=np.float32) <= desired_rate:
        return best
    choice, low = best, 0.0
    high = max(float(distortion.mean(dtype=np.float32)) * 1.0e-4, 1.0e-12)
    for _ in range(50):
        trial = (distortion + np.float32(high) * rates).argmin(1)
        if rates[row, trial].sum(dtype=np.float32) <= desired_rate:
            break
        high *= 2.0
    for _ in range(20):
        middle = high * 0.5 if low == 0.0 else math.sqrt(low * high)
        trial = (distortion + np.float32(middle) * rates).argmin(1)
        if rates[row, trial].sum(dtype=np.float32) > desired_rate:
            low = middle
        else:
            high = middle
            choice = trial
    return choice


def _optimize_rows(full: _Pass, baseline_stats, baseline_fit, scale: float, prob_bits: int, tile_elements: int, iterations: int,
                   candidate_count: int):
    """Row refinement (rdo.optimize_rows, rdo.py:146-162; call site eager.py:251-266): quantise the tensor at a ladder of
    scales around ``scale``, then repeatedly re-price every candidate row under the statistics of the current
    mixture and re-pick rows so that the modelled size stays at the baseline's. Returns the pass holding the chosen
    symbols, its (minmax, bins) and the chosen rows' fitted scales."""
    lib = _native.load()
    device, rows, cols = full.device, full.rows, full.cols
    stream = _native.stream_handle(device)
    ratios = ratio_ladder(candidate_count)
    baseline_index = ratios.index(1.0)
    passes, stats, fits = [], [], []
    for index, ratio in enumerate(ratios):
        if index == baseline_index:
            passes.append(full), stats.append(baseline_stats), fits.append(baseline_fit)
            continue
        candidate = _Pass(full.work, full.rms)
        candidate_stats = candidate.quantize(scale * ratio)
        if candidate_stats[0][33]:
            continue   # a field left the int16 range at this (finer) scale: not a usable candidate
        stats.append(candidate_stats)
        fits.append(candidate.refit(scale * ratio))
        passes.append(candidate)
    baseline_index = passes.index(full)
    streams_of = [_stream_counts(*item) for item in stats]
    minima, maxima = [0] * NUM_TABLES, [0] * NUM_TABLES
    for table in range(NUM_TABLES):
        alive = [(first, first + counts.size - 1) for counts, first in (streams[table] for streams in streams_of) if counts.size]
        if alive:
            minima[table], maxima[table] = min(a for a, _ in alive), max(b for _, b in alive)

    distortion = torch.stack([sse for _, sse in fits], dim=1).cpu().numpy()
    fitted = torch.stack([scales for scales, _ in fits], dim=1)
    field_pointers = torch.tensor([p.fields.data_ptr() for p in passes], dtype=torch.int64, device=device)
    coset_pointers = torch.tensor([p.cosets.data_ptr() for p in passes], dtype=torch.int64, device=device)
    chosen = _Pass(full.work, full.rms)
    rates_device = torch.empty((len(passes), rows), dtype=torch.float32, device=device)

    def select(choice: np.ndarray):
        choice_device = torch.from_numpy(choice.astype(np.int32)).to(device)
        _native.check(lib.ep_lattice_select_rows(
            _native.ptr(field_pointers), _native.ptr(coset_pointers), len(passes), _native.ptr(choice_device), rows, cols,
            _native.ptr(chosen.fields), _native.ptr(chosen.cosets), stream), "lattice_rans row selection")
        return chosen.summarize()

    def total_bytes(minmax, bins) -> float:
        return full.coded_bytes(minmax, bins, prob_bits, tile_elements) + rows * 4 + MODEL_FIXED_BYTES

    choice = np.full(rows, baseline_index, dtype=np.int64)
    row = np.arange(rows)
    target_bytes = total_bytes(*baseline_stats)
    minmax, bins = baseline_stats
    for iteration in range(iterations):
        if iteration == 0:
            current = _stream_counts(minmax, bins)   # the first mixture is the baseline itself
        values, offsets, table_minima = _rate_table(current, minima, maxima, device)
        for index, candidate in enumerate(passes):
            _native.check(lib.ep_lattice_row_rates(
                _native.ptr(candidate.fields), _native.ptr(candidate.cosets), rows, cols, _native.ptr(values), _native.ptr(offsets),
                _native.ptr(table_minima), _native.ptr(rates_device[index]), stream), "lattice_rans row rates")
        rates = np.ascontiguousarray(rates_device.cpu().numpy().T)
        current_rate = float(rates[row, choice].sum(dtype=np.float32))
        desired_rate = current_rate + 8.0 * (target_bytes - total_bytes(minmax, bins))
        choice = _choose_rate_tradeoff(distortion, rates, desired_rate)
        minmax, bins = select(choice)
        current = _stream_counts(minmax, bins)
    if iterations == 0:
        minmax, bins = select(choice)
    scales = fitted[torch.arange(rows, device=device), torch.from_numpy(choice).to(device)].contiguous()
    return chosen, minmax, bins, scales


def encode(weight: torch.Tensor, *, target_bpp: float, prob_bits, tile_elements: int, row_rdo_iterations: int,
           scale_search_iterations: int, scale_search_max_vectors: int, row_rdo_candidates: int = 5) -> LatticeBuffers:
    _native.require_cuda(weight)
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
        chosen, scales = full, None
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
                    chosen, scales = full, None
                    if alphabet <= (1 << prob_bits) and row_rdo_iterations > 0:
                        chosen, minmax, bins, scales = _optimize_rows(
                            full, (minmax, bins), full.refit(scale), scale, prob_bits, tile_elements, int(row_rdo_iterations),
                            int(row_rdo_candidates))
                        # mixing rows of finer candidates can widen an alphabet past the baseline's
                        alphabet = int(lib.ep_lattice_max_alphabet(minmax.ctypes.data))
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
        if scales is None:
            scales = torch.empty(rows, dtype=torch.float32, device=device)
            _native.check(lib.ep_lattice_refit_scales(
                _native.ptr(work), full.is_bf16, _native.ptr(full.fields), _native.ptr(full.cosets), _native.ptr(rms), float(scale),
                rows, cols, _native.ptr(scales), stream), "lattice_rans refit")
        full = chosen   # the symbols that get coded

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
