"""ConvRot: a block-diagonal orthogonal rotation of the input features that flattens outliers before INT8
quantisation. Stands in for entropack/linear/convrot.py:9-61 (same function names and checks).

The rotation matrix of a group is the Kronecker power of a 4 x 4 sign matrix over sqrt(group); it is symmetric and
its own inverse, so activations, weight rows and the inverse weight rotation all go through one kernel
(``ep_convrot_rows``), which applies it as log4(group) radix-4 butterfly passes rather than as a matrix product.
"""
import math

import torch

from . import _native

__all__ = ["build_convrot_matrix", "choose_convrot_group", "is_convrot_group", "rotate_activation", "rotate_weight"]

_SEED = ((1.0, 1.0, 1.0, -1.0), (1.0, 1.0, -1.0, 1.0), (1.0, -1.0, 1.0, 1.0), (-1.0, 1.0, 1.0, 1.0))
_KINDS = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def is_convrot_group(value: object) -> bool:
    return type(value) is int and value >= 4 and value & (value - 1) == 0 and (value.bit_length() - 1) % 2 == 0


def choose_convrot_group(in_features: int, requested: int = 256) -> int | None:
    """The largest power of four, at most ``requested``, that divides ``in_features``; None when even 4 does not."""
    if not is_convrot_group(requested):
        raise ValueError(f"convrot group size must be a power of four at least 4, got {requested}")
    group = requested
    while group >= 4 and in_features % group:
        group //= 4
    return group if group >= 4 else None


def build_convrot_matrix(order: int, *, device: torch.device | str = "cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The dense ``order x order`` rotation (tests and documentation; the kernels never form it)."""
    seed = torch.tensor(_SEED, dtype=torch.float32)
    matrix = seed
    for _ in range(int(round(math.log(order, 4))) - 1):
        matrix = torch.kron(matrix, seed)
    return (matrix / math.sqrt(order)).to(device=device, dtype=dtype)


def _rotate_rows(rows: torch.Tensor, group: int) -> torch.Tensor:
    if rows.shape[-1] % group:
        raise ValueError(f"in_features {rows.shape[-1]} is not divisible by convrot group {group}")
    kind = _KINDS.get(rows.dtype)
    if kind is None:
        raise TypeError(f"convrot rotates bf16, fp16 or fp32 tensors, got {rows.dtype}")
    _native.require_cuda(rows)
    flat = rows.reshape(-1, rows.shape[-1]).contiguous()
    out = torch.empty_like(flat)
    if flat.numel():
        with torch.cuda.device(flat.device):
            status = _native.load().ep_convrot_rows(_native.ptr(flat), kind, flat.shape[0], flat.shape[1], int(group), _native.ptr(out),
                                                    _native.stream_handle(flat.device))
        _native.check(status, "convrot rotation")
    return out.reshape(rows.shape)


def rotate_activation(x: torch.Tensor, group: int) -> torch.Tensor:
    """``x @ R`` per group of features."""
    return _rotate_rows(x, group)


def rotate_weight(weight: torch.Tensor, group: int, *, inverse: bool = False) -> torch.Tensor:
    """``weight @ R.T`` per group (``inverse`` rotates back); R is symmetric and self-inverse, so both are the same pass."""
    del inverse
    return _rotate_rows(weight, group)
