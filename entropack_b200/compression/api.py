"""``compress`` / ``decompress``. Stands in for entropack/compression/api.py:18-76 (same fallback rules)."""
import logging
import warnings

import torch

from ..registry import DispatchError, get_scheme, name_for_config
from ..schemes.config import CompressionConfig, RawConfig, validate_config
from .compressed_tensor import CompressedTensor

logger = logging.getLogger("entropack_b200")


class CompressionFallbackWarning(RuntimeWarning):
    """Emitted when an encode failed and the tensor was stored uncompressed instead."""


def compress(tensor: torch.Tensor, config: CompressionConfig) -> CompressedTensor:
    """Compress ``tensor`` with the scheme ``config`` selects.

    An encode that fails on the data (not on the configuration or the backend) yields a ``raw``
    container plus a :class:`CompressionFallbackWarning`; its header records what was requested and why
    it failed. Invalid configurations raise, and so does a missing GPU / kernel library
    (:class:`DispatchError`): nothing ever runs on the CPU instead."""
    if isinstance(tensor, CompressedTensor):
        raise TypeError("compress expects an uncompressed tensor; decompress the container before recompressing")
    scheme = get_scheme(name_for_config(config))
    validate_config(config)
    try:
        packed = scheme.encode(tensor, config)
    except DispatchError:
        raise
    except Exception as error:  # noqa: BLE001 - mirrors the reference: any encode failure stores raw
        logger.warning("%s could not encode a %s %s tensor, storing it uncompressed: %s",
                       scheme.name, tuple(tensor.shape), tensor.dtype, error)
        return _store_raw(tensor, scheme.name, error)
    return CompressedTensor(header={"compress_method": scheme.name}, buffers=packed, shape=tuple(tensor.shape), dtype=tensor.dtype)


def _store_raw(tensor: torch.Tensor, requested: str, error: Exception) -> CompressedTensor:
    reason = f"{type(error).__name__}: {error}"
    warnings.warn(
        f"entropack stored a {tuple(tensor.shape)} {tensor.dtype} tensor uncompressed, at "
        f"{tensor.element_size() * 8} bits per parameter: compress_method={requested!r} failed with {reason}",
        CompressionFallbackWarning, stacklevel=3)
    return CompressedTensor(
        header={"compress_method": "raw", "requested": requested, "reason": reason},
        buffers=get_scheme("raw").encode(tensor, RawConfig()), shape=tuple(tensor.shape), dtype=tensor.dtype)


def decompress(compressed: CompressedTensor, config: CompressionConfig, *, check: bool = False) -> torch.Tensor:
    """Restore the dense tensor (container's shape and dtype, on the device holding its buffers).

    The decode kernels never fault on a malformed bitstream: they decode what they can and record what they saw in
    an error word. ``check=True`` (not part of the reference's signature) passes such a word, waits for the decode
    and raises ``ValueError`` if the kernels found bad stream offsets, a truncated or over-long payload or a corrupt
    table; without it a damaged container decodes to garbage silently, as it does in the reference."""
    validate_config(config)
    scheme = compressed.scheme
    if not check or scheme.name == "raw":
        restored = scheme.decode(compressed.buffers, shape=tuple(compressed.shape), dtype=compressed.encoded_dtype, config=config)
        return restored.to(compressed.dtype)
    from .. import _native

    device = next(iter(compressed.buffers.values())).device
    error = torch.zeros(1, dtype=torch.int32, device=device)
    restored = scheme.decode(compressed.buffers, shape=tuple(compressed.shape), dtype=compressed.encoded_dtype, config=config, error=error)
    _native.raise_stream_error(int(error.item()), f"{scheme.name} decode")
    return restored.to(compressed.dtype)
