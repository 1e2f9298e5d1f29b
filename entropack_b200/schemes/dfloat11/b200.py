"""DFloat11 lane over the sm_100a kernel library.

Entry points mirror the reference's lane (entropack/schemes/dfloat11/cuda.py:57,104,136):
``exponent_counter(flat, threads_per_block) -> dict``, ``encode(*, weight, codec, luts, bytes_per_thread,
threads_per_block)`` and ``decode(buffers)``. ``codec`` here is the pair ``(code_len int32[257],
code_val uint32[257])`` built by :func:`build_codec` (index 256 is the end-of-stream codeword).
"""
import ctypes

import numpy as np
import torch

from ... import _native
from .format import DFloat11Buffers, make_layout, parse_layout_cached

_MAX_LUT_ROWS = 65


def decode_tables(buffers: DFloat11Buffers) -> torch.Tensor:
    """The container's decode tables (fused level tables + an 11-bit multi-symbol table, 17 KB), built on the device by
    one small launch at the container's first decode and kept on the layout tensor. With them the decode runs the
    warp-per-run kernel, which copies them into shared memory; building them first and decoding with that kernel takes
    less time than one decode by the kernel that builds its own table in every CUDA block, so even a container that is
    decoded once gets them."""
    layout = buffers.layout
    device = buffers.luts.device
    cached = getattr(layout, "_dfloat11_decode_tables", None)
    if cached is not None and cached.device == device:
        return cached
    lib = _native.load()
    luts = buffers.luts.contiguous()
    nbytes = lib.ep_dfloat11_decode_tables_bytes(int(luts.shape[0]))
    if nbytes < 0:
        _native.check(int(nbytes), "dfloat11 decode tables")
    tables = torch.empty(nbytes, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        status = lib.ep_dfloat11_build_decode_tables(_native.ptr(luts), int(luts.shape[0]), _native.ptr(tables), nbytes,
                                                     _native.stream_handle(device))
    _native.check(status, "dfloat11 decode tables")
    layout._dfloat11_decode_tables = tables
    return tables


def decode(buffers: DFloat11Buffers, *, error: torch.Tensor | None = None, kept_tables: bool = True) -> torch.Tensor:
    """Decode to a flat bf16 tensor on the buffers' device (one launch, two at a container's first decode; no host sync).
    ``kept_tables=False`` decodes without the container's kept tables, by the kernel that builds a table in every CUDA
    block (what a caller of the C entry point gets who passes no tables)."""
    sign_mantissa = buffers.sign_mantissa
    _native.require_cuda(sign_mantissa)
    bpt, tpb, widest = parse_layout_cached(buffers.layout)
    n = sign_mantissa.numel()
    # the kernel indexes the position and region records by block: their lengths are checked here, on the host, for free
    blocks = -(-buffers.encoded_exponent.numel() // (bpt * tpb))
    if buffers.output_positions.numel() != blocks + 1:
        raise ValueError(f"dfloat11 output_positions hold {buffers.output_positions.numel()} entries, the layout needs {blocks + 1}")
    if buffers.thread_meta.numel() != blocks * tpb:
        raise ValueError(f"dfloat11 thread_meta holds {buffers.thread_meta.numel()} entries, the layout needs {blocks * tpb}")
    if buffers.luts.ndim != 2 or buffers.luts.shape[1] != 256 or buffers.luts.shape[0] < 2:
        raise ValueError(f"dfloat11 luts must be [levels + 1, 256], got {tuple(buffers.luts.shape)}")
    out = torch.empty(n, dtype=torch.bfloat16, device=sign_mantissa.device)
    tables = decode_tables(buffers) if kept_tables else None
    with torch.cuda.device(sign_mantissa.device):
        status = _native.load().ep_dfloat11_decode(
            _native.ptr(buffers.luts.contiguous()), int(buffers.luts.shape[0]), _native.ptr(buffers.encoded_exponent),
            buffers.encoded_exponent.numel(), _native.ptr(sign_mantissa), _native.ptr(buffers.output_positions),
            _native.ptr(buffers.thread_meta), _native.ptr(out), n, bpt, tpb, widest, _native.ptr(tables),
            0 if tables is None else tables.numel(), _native.ptr(error), _native.stream_handle(sign_mantissa.device))
    _native.check(status, "dfloat11 decode")
    return out


def exponent_counter(weight: torch.Tensor, threads_per_block: int | None = None) -> dict[int, int]:
    flat = weight.reshape(-1)
    _native.require_cuda(flat)
    if flat.numel() == 0:
        return {}
    histogram = torch.empty(256, dtype=torch.int64, device=flat.device)
    with torch.cuda.device(flat.device):
        _native.check(_native.load().ep_dfloat11_histogram(
            _native.ptr(flat), flat.numel(), _native.ptr(histogram), _native.stream_handle(flat.device)), "dfloat11 histogram")
    return {symbol: int(count) for symbol, count in enumerate(histogram.cpu().tolist()) if count > 0}


def build_codec(counter: dict[int, int]):
    """(code_len, code_val) for a histogram of exponent values."""
    histogram = np.zeros(256, dtype=np.uint64)
    for symbol, count in counter.items():
        histogram[int(symbol)] = int(count)
    code_len = np.zeros(257, dtype=np.int32)
    code_val = np.zeros(257, dtype=np.uint32)
    _native.check(_native.load().ep_dfloat11_build_code(histogram.ctypes.data, code_len.ctypes.data, code_val.ctypes.data),
                  "dfloat11 code construction")
    return code_len, code_val


def build_luts(codec) -> torch.Tensor:
    code_len, code_val = codec
    luts = np.zeros((_MAX_LUT_ROWS, 256), dtype=np.uint8)
    rows = ctypes.c_int(0)
    _native.check(_native.load().ep_dfloat11_build_luts(code_len.ctypes.data, code_val.ctypes.data, luts.ctypes.data, _MAX_LUT_ROWS,
                                                        ctypes.addressof(rows)), "dfloat11 look-up tables")
    return torch.from_numpy(luts[: rows.value].copy())


def encode(*, weight: torch.Tensor, codec, luts: torch.Tensor, bytes_per_thread: int, threads_per_block: int) -> DFloat11Buffers:
    flat = weight.reshape(-1).contiguous()
    _native.require_cuda(flat)
    n = flat.numel()
    if not 5 <= bytes_per_thread <= 255:
        raise ValueError(
            "dfloat11 bytes_per_thread must be in [5, 255]: the region must exceed the 32-bit maximum code length and its "
            "worst-case symbol count must fit the 11-bit thread_meta field")
    if n >= 1 << 32:
        raise ValueError("dfloat11 requires fewer than 2^32 elements per tensor")
    device = flat.device
    code_len, code_val = codec
    lib = _native.load()
    with torch.cuda.device(device):
        stream = _native.stream_handle(device)
        code_len_dev = torch.from_numpy(code_len[:256].copy()).to(device)
        code_val_dev = torch.from_numpy(code_val[:256].astype(np.int64).astype(np.int32, casting="unsafe").copy()).to(device)
        chunks = int(lib.ep_dfloat11_chunks(n))
        chunk_bits = torch.empty(chunks, dtype=torch.uint32, device=device)
        chunk_offsets = torch.empty(chunks + 1, dtype=torch.uint32, device=device)
        total = torch.empty(1, dtype=torch.int64, device=device)
        _native.check(lib.ep_dfloat11_chunk_bits(_native.ptr(flat), n, _native.ptr(code_len_dev), _native.ptr(chunk_bits), stream),
                      "dfloat11 code lengths")
        _native.check(lib.ep_exclusive_scan_u32(_native.ptr(chunk_bits), chunks, _native.ptr(chunk_offsets), _native.ptr(total), stream),
                      "dfloat11 bit offsets")
        total_bits = int(total.item())
        if total_bits >= 1 << 32:
            raise ValueError("dfloat11 bitstream exceeds 2^32 bits; split the tensor")
        n_bytes = (total_bits + 7) // 8
        blocks = -(-n_bytes // (bytes_per_thread * threads_per_block))
        regions = blocks * threads_per_block
        encoded = torch.empty((n_bytes + 3) // 4 * 4 + 4, dtype=torch.uint8, device=device)
        sign_mantissa = torch.empty(n, dtype=torch.uint8, device=device)
        thread_meta = torch.empty(regions, dtype=torch.uint16, device=device)
        output_positions = torch.empty(blocks + 1, dtype=torch.uint32, device=device)
        region_scratch = torch.empty(2 * regions, dtype=torch.uint32, device=device)
        _native.check(lib.ep_dfloat11_pack(
            _native.ptr(flat), n, _native.ptr(code_len_dev), _native.ptr(code_val_dev), _native.ptr(chunk_offsets), total_bits,
            bytes_per_thread, threads_per_block, int(code_len[256]), int(code_val[256]), _native.ptr(encoded),
            _native.ptr(sign_mantissa), _native.ptr(thread_meta), _native.ptr(output_positions), _native.ptr(region_scratch), stream),
            "dfloat11 pack")
        positions = output_positions.to(torch.int64)
        widest = int((positions[1:] - positions[:-1]).max().item()) if blocks else 0
    return DFloat11Buffers(
        encoded_exponent=encoded[:n_bytes], sign_mantissa=sign_mantissa, luts=luts.to(device), output_positions=output_positions,
        thread_meta=thread_meta, layout=make_layout(bytes_per_thread, threads_per_block, widest).to(device))
