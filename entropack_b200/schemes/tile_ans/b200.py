"""Tile-ANS lane over the sm_100a kernel library.

Same entry points as the reference's lane modules (entropack/schemes/tile_ans/cuda.py:64,122):
``encode(*, weight, tile_elements, probability_bits, raw_lane_threshold, threads_per_block)`` and
``decode(buffers, *, dtype, threads_per_block)``. ``threads_per_block`` is accepted and ignored: the
kernels are compiled for one block shape.
"""
import ctypes

import numpy as np
import torch

from ... import _native
from .format import NUM_STATES, TileBuffers, make_layout, num_tiles, parse_layout_cached

_native_lib = _native.load


def _lane_modes_host(buffers: TileBuffers) -> np.ndarray:
    cached = getattr(buffers.layout, "_tile_ans_lane_modes", None)
    if cached is None:
        cached = np.ascontiguousarray(buffers.lane_modes.detach().cpu().numpy().astype(np.uint8))
        buffers.layout._tile_ans_lane_modes = cached
    return cached


def decode(buffers: TileBuffers, *, dtype: torch.dtype, threads_per_block: int | None = None,
           error: torch.Tensor | None = None, out: torch.Tensor | None = None,
           tiles: tuple[int, int] | None = None) -> torch.Tensor:
    """Decode to a flat tensor of ``dtype`` on the buffers' device. One kernel launch, no host sync.

    ``error``: optional int32[1] device tensor (zeroed by the caller) that receives a non-zero code if
    the bitstream is malformed; without it a malformed stream decodes to garbage silently, as in the
    reference. ``out``: the whole tensor's bytes (uint8) to decode into. ``tiles = (first, count)``: decode
    only those tiles, leaving the rest of ``out`` as it is; only their streams need to be in ``payload``."""
    payload = buffers.payload
    _native.require_cuda(payload)
    tile_elements, prob_bits, num_lanes, num_elements = parse_layout_cached(buffers.layout)
    modes = _lane_modes_host(buffers)
    if out is None:
        out = torch.empty(num_elements * num_lanes, dtype=torch.uint8, device=payload.device)
    elif out.dtype != torch.uint8 or out.numel() != num_elements * num_lanes or not out.is_contiguous() or out.device != payload.device:
        raise ValueError(f"tile_ans decode needs a contiguous uint8 output of {num_elements * num_lanes} bytes on {payload.device}")
    total_tiles = num_tiles(num_elements, tile_elements)
    first, count = (0, total_tiles) if tiles is None else tiles
    # the kernels index offsets and states by tile and lane: their lengths are checked here, on the host, for free
    coded_lanes = int((modes == 0).sum())
    if buffers.offsets.numel() != total_tiles * num_lanes + 1:
        raise ValueError(f"tile_ans offsets hold {buffers.offsets.numel()} entries, the layout needs {total_tiles * num_lanes + 1}")
    if buffers.states.numel() != total_tiles * coded_lanes * NUM_STATES:
        raise ValueError(f"tile_ans states hold {buffers.states.numel()} words, the layout needs {total_tiles * coded_lanes * NUM_STATES}")
    if buffers.decode_tables.numel() != num_lanes << prob_bits:
        raise ValueError(f"tile_ans decode_tables hold {buffers.decode_tables.numel()} entries, the layout needs {num_lanes << prob_bits}")
    with torch.cuda.device(payload.device):
        status = _native_lib().ep_tile_ans_decode_tiles(
            _native.ptr(payload), payload.numel(), _native.ptr(buffers.offsets), _native.ptr(buffers.states),
            _native.ptr(buffers.decode_tables), modes.ctypes.data, _native.ptr(out), num_elements, tile_elements,
            prob_bits, num_lanes, first, count, _native.ptr(error), _native.stream_handle(payload.device))
    _native.check(status, "tile_ans decode")
    return out.view(dtype)


def lane_histogram(weight: torch.Tensor) -> np.ndarray:
    """Per-byte-lane symbol counts, uint64[lanes, 256], on the host (one device->host copy)."""
    num_lanes = weight.element_size()
    histograms = torch.empty((num_lanes, 256), dtype=torch.int64, device=weight.device)
    with torch.cuda.device(weight.device):
        status = _native_lib().ep_tile_ans_histogram(
            _native.ptr(weight), weight.numel(), num_lanes, _native.ptr(histograms), _native.stream_handle(weight.device))
    _native.check(status, "tile_ans histogram")
    return np.ascontiguousarray(histograms.cpu().numpy().view(np.uint64))


def plan_tables(counts: np.ndarray, tile_elements: int, probability_bits: int, raw_lane_threshold: float):
    """(probability_bits, frequencies u16[lanes,256], cdfs u16[lanes,256], decode_tables u32[lanes,2^pb], modes u8[lanes])"""
    num_lanes = counts.shape[0]
    frequencies = np.zeros((num_lanes, 256), dtype=np.uint16)
    cdfs = np.zeros((num_lanes, 256), dtype=np.uint16)
    tables = np.zeros((num_lanes, 4096), dtype=np.uint32)
    modes = np.zeros(num_lanes, dtype=np.uint8)
    chosen = ctypes.c_int(0)
    status = _native_lib().ep_tile_ans_plan(
        counts.ctypes.data, num_lanes, tile_elements, float(raw_lane_threshold), int(probability_bits),
        ctypes.addressof(chosen), frequencies.ctypes.data, cdfs.ctypes.data, tables.ctypes.data, modes.ctypes.data)
    _native.check(status, "tile_ans table planning")
    size = 1 << chosen.value
    packed = np.ascontiguousarray(tables.reshape(-1)[: num_lanes * size].reshape(num_lanes, size))
    return chosen.value, frequencies, cdfs, packed, modes


def encode(*, weight: torch.Tensor, tile_elements: int, probability_bits: int, raw_lane_threshold: float,
           threads_per_block: int | None = None) -> TileBuffers:
    _native.require_cuda(weight)
    contiguous = weight.contiguous()
    num_elements = contiguous.numel()
    if num_elements == 0:
        raise ValueError("tile_ans does not support empty tensors")
    num_lanes = contiguous.element_size()
    device = contiguous.device
    counts = lane_histogram(contiguous)
    prob_bits, frequencies, cdfs, tables, modes = plan_tables(counts, tile_elements, probability_bits, raw_lane_threshold)
    tiles = num_tiles(num_elements, tile_elements)
    streams = tiles * num_lanes
    ans_lanes = int((modes == 0).sum())
    # the five small host arrays go up in one copy: tables (u32), layout (i64), frequencies and cdfs (u16), modes (u8)
    layout_host = make_layout(num_elements, num_lanes, tile_elements, prob_bits).numpy()
    pieces = [tables, layout_host, frequencies, cdfs, modes]
    starts, cursor = [], 0
    for piece in pieces:
        cursor = -(-cursor // 16) * 16
        starts.append(cursor)
        cursor += piece.nbytes
    staging = np.zeros(cursor, dtype=np.uint8)
    for start, piece in zip(starts, pieces):
        staging[start:start + piece.nbytes] = np.ascontiguousarray(piece).view(np.uint8).reshape(-1)
    uploaded = torch.from_numpy(staging).to(device)
    tables_dev, layout, frequencies_dev, cdfs_dev, modes_dev = (
        uploaded[start:start + piece.nbytes].view(torch.from_numpy(piece).dtype).view(piece.shape)
        for start, piece in zip(starts, pieces))
    states = torch.empty((tiles * ans_lanes, NUM_STATES), dtype=torch.uint32, device=device)
    word_counts = torch.empty(streams, dtype=torch.uint32, device=device)
    scratch = torch.empty(streams * tile_elements, dtype=torch.uint16, device=device)
    offsets = torch.empty(streams + 1, dtype=torch.uint32, device=device)
    total = torch.empty(1, dtype=torch.int64, device=device)
    lib = _native_lib()
    with torch.cuda.device(device):
        stream = _native.stream_handle(device)
        _native.check(lib.ep_tile_ans_encode(
            _native.ptr(contiguous), num_elements, num_lanes, tile_elements, prob_bits, _native.ptr(frequencies_dev),
            _native.ptr(cdfs_dev), modes.ctypes.data, _native.ptr(scratch), _native.ptr(word_counts), _native.ptr(states),
            stream), "tile_ans encode")
        _native.check(lib.ep_exclusive_scan_u32(
            _native.ptr(word_counts), streams, _native.ptr(offsets), _native.ptr(total), stream), "tile_ans offsets")
        total_words = int(total.item())
        if total_words >= 1 << 32:
            raise ValueError("tile_ans payload exceeds uint32 offset capacity")
        payload = torch.empty(total_words, dtype=torch.uint16, device=device)
        if total_words:
            _native.check(lib.ep_compact_streams(
                _native.ptr(scratch), _native.ptr(offsets), _native.ptr(payload), tile_elements, streams, stream),
                "tile_ans compaction")
    return TileBuffers(payload=payload, offsets=offsets, states=states, decode_tables=tables_dev, lane_modes=modes_dev, layout=layout)
