"""ctypes binding of ``libentropack_b200.so`` (the C ABI declared in ``include/entropack_b200.h``).

There is no fallback: if the library has not been built, or no CUDA device is present, every compute
entry point raises. ``python -m entropack_b200.build`` (or ``__graft_entry__.build()``) builds it.
"""
import contextlib
import ctypes
from pathlib import Path

import torch

LIBRARY_PATH = Path(__file__).resolve().parent / "lib" / "libentropack_b200.so"

EP_OK = 0
STREAM_ERRORS = {
    1: "stream offsets are out of range", 2: "payload is truncated", 3: "payload contains unread words",
    4: "raw lane payload length is invalid", 5: "a decoded table selector is out of range (corrupt coset table)",
    9: "a bounded wait inside a kernel ran out (tensor-core product, peer barrier or a bulk copy of the DFloat11 decode)",
}


class NativeLibraryError(RuntimeError):
    """The sm_100a kernel library is missing or reported a failure."""


_lib = None

_i64, _i32, _f64, _f32, _ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_float, ctypes.c_void_p

#: name -> argument types; every function returns int status unless listed in _RESTYPES
_PROTOTYPES = {
    "ep_abi_version": [],
    "ep_set_sm_limits": [_i32, _i32],
    "ep_tile_ans_decode": [_ptr, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i32, _i32, _ptr, _ptr],
    "ep_tile_ans_decode_tiles": [_ptr, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i32, _i32, _i64, _i64, _ptr, _ptr],
    "ep_tile_ans_histogram": [_ptr, _i64, _i32, _ptr, _ptr],
    "ep_tile_ans_plan": [_ptr, _i32, _i64, _f64, _i32, _ptr, _ptr, _ptr, _ptr, _ptr],
    "ep_tile_ans_encode": [_ptr, _i64, _i32, _i64, _i32, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "ep_exclusive_scan_u32": [_ptr, _i64, _ptr, _ptr, _ptr],
    "ep_compact_streams": [_ptr, _ptr, _ptr, _i64, _i64, _ptr],
    "ep_lattice_decode": [_ptr, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _ptr, _i32, _i64, _i64, _i32, _i64, _i32, _ptr, _i64, _i32, _ptr, _ptr],
    "ep_lattice_linear_forward": [_ptr, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _i64, _i32, _i64, _i32, _ptr, _i64, _i32, _ptr, _ptr,
                                  _i32, _ptr, _ptr, _ptr, _ptr],
    "ep_lattice_slot_tables_bytes": [_i32, _i32],
    "ep_lattice_build_slot_tables": [_ptr, _ptr, _i64, _i32, _i32, _ptr, _i64, _ptr],
    "ep_lattice_decode_scratch_bytes": [_i32, _i32],
    "ep_lattice_decode_static": [_ptr, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _ptr, _i32, _i64, _i64, _i32, _i64, _i32, _ptr, _ptr],
    "ep_lattice_decode_static_max_prob_bits": [],
    "ep_dfloat11_decode": [_ptr, _i32, _ptr, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _i32, _i32, _i32, _ptr, _i64, _ptr, _ptr],
    "ep_dfloat11_decode_tables_bytes": [_i32],
    "ep_dfloat11_build_decode_tables": [_ptr, _i32, _ptr, _i64, _ptr],
    "ep_dfloat11_histogram": [_ptr, _i64, _ptr, _ptr],
    "ep_dfloat11_build_code": [_ptr, _ptr, _ptr],
    "ep_dfloat11_build_luts": [_ptr, _ptr, _ptr, _i32, _ptr],
    "ep_dfloat11_chunks": [_i64],
    "ep_dfloat11_chunk_bits": [_ptr, _i64, _ptr, _ptr, _ptr],
    "ep_dfloat11_pack": [_ptr, _i64, _ptr, _ptr, _ptr, ctypes.c_uint64, _i32, _i32, _i32, ctypes.c_uint32, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "ep_linear_forward": [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr],
    "ep_linear_forward_scatter": [_ptr, _ptr, _ptr, _ptr, _ptr, _i32, _i64, _i64, _i64, _i64, _i64, _ptr, _ptr],
    "ep_peer_barrier": [_ptr, _i32, _i32, ctypes.c_uint32, _i64, _ptr, _ptr],
    "ep_linear_forward_fp8": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i32, _i64, _i64, _i64, _ptr, _ptr],
    "ep_quantize_rows_fp8": [_ptr, _i32, _i64, _i64, _ptr, _ptr, _ptr],
    "ep_linear_forward_int8": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i32, _i64, _i64, _i64, _ptr, _ptr],
    "ep_quantize_rows_int8": [_ptr, _i32, _i64, _i64, _ptr, _ptr, _ptr],
    "ep_convrot_rows": [_ptr, _i32, _i64, _i64, _i32, _ptr, _ptr],
    "ep_lattice_row_rms": [_ptr, _i32, _i64, _i64, _ptr, _ptr],
    "ep_lattice_quantize": [_ptr, _i32, _ptr, _i64, _i64, _f32, _ptr, _ptr, _ptr, _ptr],
    "ep_lattice_histogram": [_ptr, _ptr, _i64, _ptr, _ptr, _i64, _ptr, _ptr],
    "ep_lattice_bins_needed": [_ptr],
    "ep_lattice_max_alphabet": [_ptr],
    "ep_lattice_coded_bytes": [_ptr, _ptr, _i64, _i32, _i64, _ptr],
    "ep_lattice_search_scale": [_ptr, _i32, _ptr, _i64, _i64, _ptr, _ptr, _ptr, _i64, _f64, _i32, _i64, _i32, _f64, _f64, _f64, _ptr, _ptr, _ptr],
    "ep_lattice_tables": [_ptr, _ptr, _i64, _i32, _ptr, _ptr, _i64, _ptr],
    "ep_lattice_refit_scales": [_ptr, _i32, _ptr, _ptr, _ptr, _f32, _i64, _i64, _ptr, _ptr],
    "ep_lattice_refit_rows": [_ptr, _i32, _ptr, _ptr, _ptr, _f32, _i64, _i64, _ptr, _ptr, _ptr],
    "ep_lattice_minmax": [_ptr, _ptr, _i64, _ptr, _ptr],
    "ep_lattice_row_rates": [_ptr, _ptr, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr],
    "ep_lattice_select_rows": [_ptr, _ptr, _i32, _ptr, _i64, _i64, _ptr, _ptr, _ptr],
    "ep_lattice_encode_scratch_words": [_i64, _i64],
    "ep_lattice_encode": [_ptr, _ptr, _i64, _ptr, _ptr, _i64, _i32, _i64, _ptr, _ptr, _ptr, _ptr, _ptr],
}
_RESTYPES = {"ep_status_string": ctypes.c_char_p, "ep_last_cuda_error": ctypes.c_char_p}
_INT64_RESULTS = ("ep_lattice_decode_scratch_bytes", "ep_lattice_slot_tables_bytes", "ep_dfloat11_decode_tables_bytes", "ep_lattice_bins_needed", "ep_lattice_encode_scratch_words",
                  "ep_dfloat11_chunks")


def library_path() -> Path:
    return LIBRARY_PATH


def load():
    """Load the shared object once; raises NativeLibraryError when it has not been built."""
    global _lib
    if _lib is None:
        if not LIBRARY_PATH.exists():
            raise NativeLibraryError(
                f"{LIBRARY_PATH} is missing: build the sm_100a kernels with `python -m entropack_b200.build`; "
                "entropack_b200 has no CPU or eager fallback"
            )
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        for name, argtypes in _PROTOTYPES.items():
            function = getattr(lib, name)
            function.argtypes = argtypes
            function.restype = ctypes.c_int64 if name in _INT64_RESULTS else ctypes.c_int
        for name, restype in _RESTYPES.items():
            function = getattr(lib, name)
            function.restype = restype
        lib.ep_status_string.argtypes = [ctypes.c_int]
        _lib = lib
    return _lib


def exported_symbols() -> list[str]:
    return sorted(set(_PROTOTYPES) | set(_RESTYPES))


def check(status: int, what: str) -> None:
    if status != EP_OK:
        lib = load()
        detail = lib.ep_status_string(status).decode()
        if status == -3:
            detail += ": " + lib.ep_last_cuda_error().decode()
        if status in (-1, -2, -4, -5, -6):
            raise ValueError(f"{what}: {detail}")
        raise NativeLibraryError(f"{what}: {detail}")


def require_cuda(tensor: torch.Tensor | None = None) -> None:
    if not torch.cuda.is_available():
        raise NativeLibraryError("entropack_b200 needs a CUDA device (B200, sm_100a); torch.cuda.is_available() is False")
    if tensor is not None and tensor.device.type != "cuda":
        raise NativeLibraryError(f"kernel operand lives on {tensor.device}, expected a CUDA device")


def ptr(tensor: torch.Tensor | None) -> int | None:
    """Device (or pinned/host) address of a contiguous tensor; None stays a null pointer."""
    if tensor is None:
        return None
    if not tensor.is_contiguous():
        raise ValueError("kernel operands must be contiguous")
    return tensor.data_ptr()


def stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_NO_GUARD = contextlib.nullcontext()


def on_device(index: int):
    """Context in which ``index`` is the current CUDA device: nothing at all when it is so already."""
    return _NO_GUARD if torch.cuda.current_device() == index else torch.cuda.device(index)


def raw_stream(index: int) -> int:
    """The current stream's handle on device ``index`` without building a Stream object (a few microseconds less per
    library call, which counts for a layer that makes two of them per forward)."""
    if _raw_stream is not None:
        return _raw_stream(index)
    return torch.cuda.current_stream(index).cuda_stream


def raise_stream_error(code: int, what: str) -> None:
    if code:
        raise ValueError(f"{what}: {STREAM_ERRORS.get(int(code), f'device error {code}')}")
