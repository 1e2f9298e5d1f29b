"""Decode many containers that sit in host memory, with upload, decode and download overlapped.

``decompress`` works on one container on the current stream, so a loop over a checkpoint's tensors
runs copy-in, kernel and copy-out one after the other. ``decompress_many`` puts the three on streams
of their own: while tensor *i* is being decoded, tensor *i + 1* is on its way to the GPU and tensor
*i - 1* on its way back (PCIe moves both directions at once). Headers and the small layout buffers are
parsed while the container is still in host memory, so nothing is read back from the device in
between. The reference has no counterpart: its ``decompress`` (entropack/compression/api.py:62-76)
is the per-tensor call this builds on.
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
    for index in _transfer_order(containers, with_download=out is not None):
        host, item_config = containers[index], configs[index]
        if host.device.type != "cuda":
            host.scheme.prime_host_metadata(host.buffers)
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
