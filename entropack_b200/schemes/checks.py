"""Input checks shared by the encoders. Stands in for entropack/schemes/checks.py:13-33."""
from collections.abc import Iterable

import torch

__all__ = ["prepare_weight"]

_EIGHT_BIT_FLOATS = frozenset({torch.float8_e4m3fn, torch.float8_e4m3fnuz, torch.float8_e5m2, torch.float8_e5m2fnuz})


def _all_finite(weight: torch.Tensor) -> bool:
    if not weight.dtype.is_floating_point:
        return True
    probe = weight.float() if weight.dtype in _EIGHT_BIT_FLOATS else weight
    low, high = torch.aminmax(probe)
    limit = float(torch.finfo(weight.dtype).max)
    return float(low) >= -limit and float(high) <= limit


def prepare_weight(weight: torch.Tensor, *, scheme: str, ndim: int | None = None,
                   dtypes: Iterable[torch.dtype] | None = None, require_finite: bool = False) -> torch.Tensor:
    if dtypes is not None and weight.dtype not in frozenset(dtypes):
        raise ValueError(f"{scheme} does not support dtype {weight.dtype}")
    if ndim is not None and weight.ndim != ndim:
        raise ValueError(f"{scheme} encode requires exactly {ndim}D input, got {weight.ndim}D")
    if weight.numel() == 0:
        raise ValueError(f"{scheme} does not support empty tensors")
    if require_finite and not _all_finite(weight):
        raise ValueError(f"{scheme} input must contain only finite values")
    return weight.contiguous()
