"""Decode many containers that sit in host memory, with upload, decode and download overlapped.

``decompress`` works on one container on the current stream, so a loop over a checkpoint's tensors
runs copy-in, kernel and copy-out one after the other. ``decompress_many`` puts the three on streams
of their own: while tensor *i* is being decoded, tensor *i + 1* is on its way to the GPU and tensor
*i - 1* on its way back (PCIe moves both directions at once). Headers and the small layout buffers are
parsed while the container is still in host memory, so nothing is read back from the device in
between. A large container whose scheme can decode independent pieces (Tile-ANS tiles) is not even
uploaded as a whole: its small buffers go first, then its payload in runs of tiles, each run decoded
and sent back while the next is on its way, so the download, the longer of the two transfers, starts
a fraction of a millisecond after the call and never waits for an upload again. The reference has no
counterpart: its ``decompress`` (entropack/compression/api.py:62-76) is the per-tensor call this
builds on.
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch

from ..schemes.config import CompressionConfig, validate_config
from .compressed_tensor import CompressedTensor

_streams: dict[int, tuple[torch.cuda.Stream, torch.cuda.Stream, torch.cuda.Stream]] = {}


def _streams_for(device: torch.device):
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _streams:
        _streams[index] = tuple(torch.cuda.Stream(device=index) for _ in range(3))
    return _streams[index]


def _transfer_order(containers: Sequence[CompressedTensor], *, with_download: bool) -> list[int]:
    """Order that keeps both PCIe directions busy (Johnson's rule for a two-stage flow shop, upload then
    download, the decode in between being short): containers that upload faster than they download go
    first, smallest upload first; the others follow, largest download first."""
    if not with_download:
        return list(range(len(containers)))
    sizes = [(c.entropack_quant_state.numel(), c.numel() * c.element_size()) for c in containers]
    first = sorted((i for i, (up, down) in enumerate(sizes) if up < down), key=lambda i: sizes[i][0])
    second = sorted((i for i, (up, down) in enumerate(sizes) if up >= down), key=lambda i: -sizes[i][1])
    return first + second


#: output bytes of one streamed piece, and of the first piece of a call (pieces double from there): large enough for
#: full PCIe efficiency, small enough that the first download starts early
PIECE_BYTES = 32 << 20
FIRST_PIECE_BYTES = 4 << 20
_COPY_ALIGNMENT = 256


def _piece_runs(plan, piece_bytes: int, first_piece_bytes: int) -> list[tuple[int, int]]:
    """Runs of units ``(first, count)`` whose output is about ``piece_bytes`` each, starting at multiples of the
    plan's granule; the first run is ``first_piece_bytes`` and the following ones double until they reach the target."""
    runs, first, wanted = [], 0, min(first_piece_bytes, piece_bytes)
    while first < plan.units:
        count = max(1, wanted // plan.unit_output_bytes)
        count = max(plan.granule, count // plan.granule * plan.granule)
        count = min(count, plan.units - first)
        runs.append((first, count))
        first += count
        wanted = min(2 * wanted, piece_bytes)
    return runs


def _decode_streamed(host: CompressedTensor, plan, item_config, device, streams, target: torch.Tensor,
                     first_piece_bytes: int):
    """Upload, decode and download one container in pieces. Returns (device-resident container, dense result)."""
    upload, compute, download = streams
    blob = host.entropack_quant_state
    streamed = host.buffers[plan.streamed_buffer]
    streamed_begin = streamed.data_ptr() - blob.data_ptr()
    streamed_end = streamed_begin + streamed.numel() * streamed.element_size()
    target_bytes = target.view(torch.uint8).reshape(-1)

    with torch.cuda.stream(upload):
        device_blob = torch.empty(blob.numel(), dtype=torch.uint8, device=device)
        for begin, end in ((0, streamed_begin), (streamed_end, blob.numel())):
            if end > begin:
                device_blob[begin:end].copy_(blob[begin:end], non_blocking=True)
    resident = host._remap(lambda _: device_blob)
    with torch.cuda.stream(compute):
        dense_bytes = torch.empty(plan.output_bytes, dtype=torch.uint8, device=device)
    device_blob.record_stream(compute)
    dense_bytes.record_stream(download)

    for first, count in _piece_runs(plan, PIECE_BYTES, first_piece_bytes):
        with torch.cuda.stream(upload):
            for begin, end in plan.byte_ranges(first, count):
                # whole 256-byte lines: the neighbours' bytes that come along are the same bytes they get anyway
                begin = streamed_begin + begin // _COPY_ALIGNMENT * _COPY_ALIGNMENT
                end = min(streamed_end, streamed_begin + -(-end // _COPY_ALIGNMENT) * _COPY_ALIGNMENT)
                device_blob[begin:end].copy_(blob[begin:end], non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(upload)
        compute.wait_event(uploaded)
        with torch.cuda.stream(compute):
            plan.decode_units(resident.buffers, dense_bytes, first, count, item_config)
            decoded = torch.cuda.Event()
            decoded.record(compute)
        download.wait_event(decoded)
        begin = first * plan.unit_output_bytes
        end = min(plan.output_bytes, (first + count) * plan.unit_output_bytes)
        with torch.cuda.stream(download):
            target_bytes[begin:end].copy_(dense_bytes[begin:end], non_blocking=True)
    return resident, dense_bytes.view(host.encoded_dtype).reshape(tuple(host.shape))


def decompress_many(blobs: Iterable[torch.Tensor | CompressedTensor], config: CompressionConfig | Sequence[CompressionConfig], *,
                    device: torch.device | str | int, out: Sequence[torch.Tensor] | None = None) -> list[torch.Tensor]:
    """Decode packed containers (``CompressedTensor`` objects or their ``entropack_quant_state`` blobs,
    ideally in pinned host memory) on ``device``.

    Returns the dense tensors on ``device``; with ``out`` (one host tensor per container, pinned for a
    true overlap) each result is also copied there, viewed as bytes if the dtypes differ. Work is
    queued on three internal streams; the call returns once everything has finished, and the calling
    stream is untouched.
    """
    device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    if device.type != "cuda":
        raise ValueError("decompress_many decodes on a CUDA device")
    blobs = list(blobs)
    configs = list(config) if isinstance(config, (list, tuple)) else [config] * len(blobs)
    if len(configs) != len(blobs):
        raise ValueError(f"{len(blobs)} containers but {len(configs)} configs")
    if out is not None and len(out) != len(blobs):
        raise ValueError(f"{len(blobs)} containers but {len(out)} output tensors")
    for item in {id(c): c for c in configs}.values():
        validate_config(item)

    upload, compute, download = _streams_for(device)
    entry = torch.cuda.current_stream(device)
    ready = torch.cuda.Event()
    ready.record(entry)
    for stream in (upload, compute, download):
        stream.wait_event(ready)   # whatever produced the blobs on the caller's stream is done first

    containers = [blob if isinstance(blob, CompressedTensor) else CompressedTensor.unpack(blob) for blob in blobs]
    results: list[torch.Tensor | None] = [None] * len(containers)
    keep_alive = []
    first_piece_bytes = FIRST_PIECE_BYTES
    for index in _transfer_order(containers, with_download=out is not None):
        host, item_config = containers[index], configs[index]
        if host.device.type != "cuda":
            host.scheme.prime_host_metadata(host.buffers)
        plan = None
        if (out is not None and host.device.type == "cpu" and host.encoded_dtype == host.dtype and out[index].is_contiguous()
                and out[index].device.type == "cpu" and out[index].numel() * out[index].element_size() == host.numel() * host.element_size()
                and host.numel() * host.element_size() >= 2 * PIECE_BYTES):
            plan = host.scheme.streaming_plan(host.buffers, shape=tuple(host.shape), dtype=host.encoded_dtype)
        if plan is not None:
            resident, dense = _decode_streamed(host, plan, item_config, device, (upload, compute, download), out[index],
                                               first_piece_bytes)
            first_piece_bytes = PIECE_BYTES
            results[index] = dense
            keep_alive.append(resident)
            continue
        with torch.cuda.stream(upload):
            resident = host.to(device, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(upload)
        compute.wait_event(uploaded)
        with torch.cuda.stream(compute):
            dense = resident.scheme.decode(resident.buffers, shape=tuple(resident.shape), dtype=resident.encoded_dtype,
                                           config=item_config).to(resident.dtype)
            decoded = torch.cuda.Event()
            decoded.record(compute)
        resident.entropack_quant_state.record_stream(compute)
        results[index] = dense
        keep_alive.append(resident)
        if out is not None:
            target = out[index]
            download.wait_event(decoded)
            with torch.cuda.stream(download):
                if target.dtype == dense.dtype:
                    target.reshape(dense.shape).copy_(dense, non_blocking=True)
                else:
                    target.view(torch.uint8).reshape(-1).copy_(dense.reshape(-1).view(torch.uint8), non_blocking=True)
            dense.record_stream(download)
    for stream in (upload, compute, download):
        stream.synchronize()
    for dense in results:
        dense.record_stream(entry)
    return results
