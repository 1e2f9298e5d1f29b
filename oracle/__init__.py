"""CPU oracle for the entropack compression hot path -- TEST INFRASTRUCTURE ONLY.

ctypes front end of the plain-C restatement in this directory (``tile_ans_oracle.c``,
``lattice_oracle.c``, ``dfloat11_oracle.c``). Only the test suite, the smoke check and the
CPU-baseline leg of the benchmark may import this package; the shipped package never does.

Every function takes and returns numpy arrays laid out exactly as the reference's buffer tuples
(``TileBuffers``, ``LatticeBuffers``, ``DFloat11Buffers``), so results can be compared field by
field with the reference's eager lanes and with the CUDA product.
"""
import ctypes
import math
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libentropack_oracle.so"
_SOURCES = ("tile_ans_oracle.c", "lattice_oracle.c", "dfloat11_oracle.c", "oracle_common.h")

NUM_STATES = 32
N_TABLES = 17


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc if the shared object is missing or older than its sources."""
    newest = max((_HERE / name).stat().st_mtime for name in _SOURCES)
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < newest:
        subprocess.run(["make", "-C", str(_HERE)] + (["-B"] if force else []), check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.orc_tile_ans_encode.restype = ctypes.c_int64
        _lib.orc_lattice_encode.restype = ctypes.c_int64
        _lib.orc_lattice_histogram.restype = ctypes.c_int64
        _lib.orc_lattice_freq_tables.restype = ctypes.c_int64
        _lib.orc_lattice_coded_bytes.restype = ctypes.c_double
        _lib.orc_quantized_cross_entropy.restype = ctypes.c_double
        _lib.orc_dfloat11_total_bits.restype = ctypes.c_int64
        _lib.orc_dfloat11_encode.restype = ctypes.c_int64
        _lib.orc_row_rms.restype = None
        _lib.orc_refit_scales.restype = None
        _lib.orc_lattice_minmax.restype = None
        _lib.orc_tile_ans_tables.restype = None
        _lib.orc_f32_to_bf16.restype = None
        _lib.orc_dfloat11_decode_sequential.restype = None
    return _lib


def _p(array: np.ndarray):
    return array.ctypes.data_as(ctypes.c_void_p)


def _c(array, dtype) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=dtype)


_ERRORS = {
    -1: "invalid argument", -2: "unable to normalize rANS frequencies", -3: "payload is truncated",
    -4: "payload contains unread words", -5: "raw lane payload length is invalid", -6: "out of memory",
    -7: "alphabet exceeds the rANS table",
}


def _check(code: int, what: str) -> int:
    if code < 0:
        raise ValueError(f"oracle {what}: {_ERRORS.get(int(code), code)}")
    return int(code)


# ------------------------------------------------------------------------------------------------
# Tile-ANS
# ------------------------------------------------------------------------------------------------
def normalize_counts(counts, table_size: int) -> np.ndarray:
    counts = _c(counts, np.int64)
    freq = np.zeros(counts.size, dtype=np.uint16)
    _check(lib().orc_normalize_counts(_p(counts), ctypes.c_int(counts.size), ctypes.c_int(table_size), _p(freq)), "normalize")
    return freq


def lattice_normalize(counts, table_size: int) -> np.ndarray:
    counts = _c(counts, np.int64)
    freq = np.zeros(counts.size, dtype=np.uint16)
    _check(lib().orc_lattice_normalize(_p(counts), ctypes.c_int(counts.size), ctypes.c_int(table_size), _p(freq)), "normalize")
    return freq


def tile_ans_default_tile_elements(nbytes: int) -> int:
    """entropack/schemes/tile_ans/__init__.py:24-27"""
    return 4096 if nbytes <= 32 * 1024 * 1024 else 8192


def tile_ans_plan(lane_bytes: np.ndarray, tile_elements: int, probability_bits: int = 0, raw_lane_threshold: float = 7.9):
    """Histogram -> (probability_bits, frequencies[lanes,256], lane_modes[lanes])."""
    num_lanes = lane_bytes.shape[1]
    counts = np.stack([np.bincount(lane_bytes[:, lane], minlength=256) for lane in range(num_lanes)]).astype(np.int64)
    counts = np.ascontiguousarray(counts)
    pb = ctypes.c_int(0)
    freqs = np.zeros((num_lanes, 256), dtype=np.uint16)
    modes = np.zeros(num_lanes, dtype=np.uint8)
    _check(lib().orc_tile_ans_plan(
        _p(counts), ctypes.c_int(num_lanes), ctypes.c_int64(tile_elements), ctypes.c_double(raw_lane_threshold),
        ctypes.c_int(probability_bits), ctypes.byref(pb), _p(freqs), _p(modes)), "tile_ans plan")
    return pb.value, freqs, modes


def tile_ans_encode(data: np.ndarray, itemsize: int, tile_elements: int = 0, probability_bits: int = 0,
                    raw_lane_threshold: float = 7.9) -> dict:
    """Encode the raw little-endian bytes of a tensor (``data``: uint8, n * itemsize bytes)."""
    raw = _c(data, np.uint8).reshape(-1, itemsize)
    n = raw.shape[0]
    if n == 0:
        raise ValueError("tile_ans does not support empty tensors")
    if tile_elements == 0:
        tile_elements = tile_ans_default_tile_elements(raw.size)
    pb, freqs, modes = tile_ans_plan(raw, tile_elements, probability_bits, raw_lane_threshold)
    tiles = -(-n // tile_elements)
    streams = tiles * itemsize
    ans_lanes = int((modes == 0).sum())
    payload = np.zeros(streams * tile_elements, dtype=np.uint16)
    offsets = np.zeros(streams + 1, dtype=np.uint32)
    states = np.zeros((tiles * ans_lanes, NUM_STATES), dtype=np.uint32)
    words = _check(lib().orc_tile_ans_encode(
        _p(raw), ctypes.c_int64(n), ctypes.c_int(itemsize), ctypes.c_int64(tile_elements), ctypes.c_int(pb), _p(freqs),
        _p(modes), _p(payload), _p(offsets), _p(states)), "tile_ans encode")
    cdfs = np.zeros((itemsize, 256), dtype=np.uint16)
    tables = np.zeros((itemsize, 1 << pb), dtype=np.uint32)
    lib().orc_tile_ans_tables(_p(freqs), ctypes.c_int(itemsize), ctypes.c_int(pb), _p(cdfs), _p(tables))
    return {
        "payload": payload[:words].copy(), "offsets": offsets, "states": states, "decode_tables": tables,
        "lane_modes": modes, "layout": np.array([tile_elements, pb, itemsize, n], dtype=np.int64),
    }


def tile_ans_decode(buffers: dict) -> np.ndarray:
    """Decode to the tensor's raw bytes (uint8, n * itemsize)."""
    tile_elements, pb, lanes, n = (int(v) for v in np.asarray(buffers["layout"]).tolist())
    payload = _c(buffers["payload"], np.uint16)
    offsets = _c(buffers["offsets"], np.uint32)
    states = _c(buffers["states"], np.uint32)
    tables = _c(buffers["decode_tables"], np.uint32)
    modes = _c(buffers["lane_modes"], np.uint8)
    out = np.zeros(n * lanes, dtype=np.uint8)
    _check(lib().orc_tile_ans_decode(
        _p(payload), _p(offsets), _p(states), _p(tables), _p(modes), ctypes.c_int64(tile_elements), ctypes.c_int(pb),
        ctypes.c_int(lanes), ctypes.c_int64(n), _p(out)), "tile_ans decode")
    return out


# ------------------------------------------------------------------------------------------------
# EntroPack-Lossy (E8 + rANS)
# ------------------------------------------------------------------------------------------------
def recommended_tile_elements(target_bpp: float) -> int:
    """entropack/schemes/lattice_rans/format.py:104-111"""
    if target_bpp <= 2.0:
        return 32768
    if target_bpp <= 4.0:
        return 16384
    if target_bpp <= 7.0:
        return 8192
    return 4096


def vector_tile_elements(tile_elements: int) -> int:
    return max(32, tile_elements // 9)


def row_rms(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    rms = np.zeros(x.shape[0], dtype=np.float32)
    lib().orc_row_rms(_p(x), ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), _p(rms))
    return rms


def e8_quantize(x: np.ndarray, rms: np.ndarray, scale: float):
    x = _c(x, np.float32)
    rows, cols = x.shape
    vectors = rows * (cols // 8)
    fields = np.zeros((vectors, 8), dtype=np.int32)
    cosets = np.zeros(vectors, dtype=np.int32)
    _check(lib().orc_e8_quantize(_p(x), _p(_c(rms, np.float32)), ctypes.c_float(scale), ctypes.c_int64(rows),
                                 ctypes.c_int64(cols), _p(fields), _p(cosets)), "e8 quantize")
    return fields, cosets


def lattice_stats(fields: np.ndarray, cosets: np.ndarray):
    """(stream_meta int64[17,4], bins int64[sum alphabets]) for quantised symbols."""
    fields = _c(fields, np.int32)
    cosets = _c(cosets, np.int32)
    vectors = cosets.size
    minmax = np.zeros(33, dtype=np.int32)
    lib().orc_lattice_minmax(_p(fields), _p(cosets), ctypes.c_int64(vectors), _p(minmax))
    total = 2
    for st in range(16):
        if minmax[2 * st] != np.iinfo(np.int32).max:
            total += int(minmax[2 * st + 1]) - int(minmax[2 * st]) + 1
    meta = np.zeros((N_TABLES, 4), dtype=np.int64)
    bins = np.zeros(total, dtype=np.int64)
    used = lib().orc_lattice_histogram(_p(fields), _p(cosets), ctypes.c_int64(vectors), _p(minmax), _p(meta), _p(bins),
                                       ctypes.c_int64(total))
    _check(used, "histogram")
    return meta, bins[:used]


def lattice_coded_bytes(meta: np.ndarray, bins: np.ndarray, prob_bits: int, tile_elements: int) -> float:
    status = ctypes.c_int(0)
    value = lib().orc_lattice_coded_bytes(_p(_c(meta, np.int64)), _p(_c(bins, np.int64)), ctypes.c_int(prob_bits),
                                          ctypes.c_int64(tile_elements), ctypes.byref(status))
    _check(status.value, "coded_bytes")
    return float(value)


#: scale-independent terms of the eager lane's byte model, entropack/schemes/lattice_rans/eager.py:102-107
#: (MODEL_LAYOUT_BYTES 64 + MODEL_STREAM_META_BYTES 408 + 384).
EAGER_MODEL_FIXED_BYTES = 64 + 408 + 384


def subsample_rows(rows: int, cols: int, max_vectors: int):
    """Seeded row subsample of the rate search, entropack/schemes/lattice_rans/format.py:127-134 and
    eager.py:110-114. Returns None when every row is used."""
    import torch

    sub_rows = max(1, min(rows, max_vectors // (cols // 8)))
    if sub_rows >= rows:
        return None
    generator = torch.Generator().manual_seed(rows * 1000003 + cols)
    return torch.randperm(rows, generator=generator)[:sub_rows].numpy()


def lattice_bisect_scale(x, rms, target_bpp, prob_bits, tile_elements, iterations=12, max_vectors=262144) -> float:
    """entropack/schemes/lattice_rans/eager.py:110-136"""
    rows, cols = x.shape
    index = subsample_rows(rows, cols, max_vectors)
    x_sub = x if index is None else np.ascontiguousarray(x[index])
    rms_sub = rms if index is None else np.ascontiguousarray(rms[index])
    sub_rows = x_sub.shape[0]
    n_sub = sub_rows * cols
    lo, hi = 0.001, 8.0
    for _ in range(iterations):
        mid = math.sqrt(lo * hi)
        fields, cosets = e8_quantize(x_sub, rms_sub, mid)
        meta, bins = lattice_stats(fields, cosets)
        total = lattice_coded_bytes(meta, bins, prob_bits, tile_elements) + sub_rows * 4 + EAGER_MODEL_FIXED_BYTES
        if 8 * total / n_sub > target_bpp:
            lo = mid
        else:
            hi = mid
    return math.sqrt(lo * hi)


def refit_scales(x, fields, cosets, rms, scale) -> np.ndarray:
    x = _c(x, np.float32)
    rows, cols = x.shape
    scales = np.zeros(rows, dtype=np.float32)
    lib().orc_refit_scales(_p(x), _p(_c(fields, np.int32)), _p(_c(cosets, np.int32)), _p(_c(rms, np.float32)),
                           ctypes.c_float(scale), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(scales))
    return scales


def lattice_encode_symbols(fields, cosets, prob_bits: int, tile_elements: int):
    """Entropy-code quantised symbols: tables (eager.py:269-296) + rans.encode_vector_stream."""
    fields = _c(fields, np.int32)
    cosets = _c(cosets, np.int32)
    vectors = cosets.size
    meta, bins = lattice_stats(fields, cosets)
    freq_tables = np.zeros(int(meta[:, 3].sum()), dtype=np.uint16)
    _check(lib().orc_lattice_freq_tables(_p(meta), _p(bins), ctypes.c_int(prob_bits), _p(freq_tables)), "freq tables")
    tile_vectors = vector_tile_elements(tile_elements)
    tiles = max(1, -(-vectors // tile_vectors))
    payload = np.zeros(tiles * tile_vectors * 9, dtype=np.uint16)
    offsets = np.zeros(tiles + 1, dtype=np.uint32)
    states = np.zeros((tiles, NUM_STATES), dtype=np.uint32)
    words = _check(lib().orc_lattice_encode(
        _p(fields), _p(cosets), ctypes.c_int64(vectors), _p(meta), _p(freq_tables), ctypes.c_int(prob_bits),
        ctypes.c_int64(tile_elements), _p(payload), _p(offsets), _p(states)), "lattice encode")
    return payload[:words].copy(), offsets, states, meta.astype(np.int32), freq_tables


def lattice_encode(x: np.ndarray, target_bpp: float, prob_bits=None, tile_elements=None, iterations: int = 12,
                   max_vectors: int = 262144) -> dict:
    """Whole lossy encode of fp32 ``x`` [rows, cols] (cols % 8 == 0), eager.py:147-194, 308-341 with
    row_rdo_iterations = 0. ``target_bpp`` is already capped by the caller."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    if cols % 8:
        raise ValueError("cols must be a multiple of 8")
    if tile_elements is None:
        tile_elements = recommended_tile_elements(target_bpp)
    auto = prob_bits in (None, 0)
    pb = (11 if target_bpp <= 7.0 else 12) if auto else int(prob_bits)
    rms = row_rms(x)
    if not np.isfinite(rms).all():
        raise ValueError("row RMS overflowed")
    if float(np.abs(x).max()) == 0.0:
        scale = 1.0
        fields, cosets = e8_quantize(x, rms, scale)
    else:
        while True:
            escalate = False
            scale = lattice_bisect_scale(x, rms, target_bpp, pb, tile_elements, iterations, max_vectors)
            while True:
                fields, cosets = e8_quantize(x, rms, scale)
                meta, _bins = lattice_stats(fields, cosets)
                alpha = int(meta[:, 3].max())
                if alpha <= (1 << pb):
                    break
                if auto and pb < 15:
                    pb += 1
                    escalate = True
                    break
                scale *= alpha / (1 << pb) * 1.05
            if not escalate:
                break
    scales = refit_scales(x, fields, cosets, rms, scale)
    payload, offsets, states, meta, freq_tables = lattice_encode_symbols(fields, cosets, pb, tile_elements)
    return {
        "payload": payload, "offsets": offsets, "states": states, "stream_meta": meta, "freq_tables": freq_tables,
        "scales": scales, "layout": np.array([cols, pb, tile_elements], dtype=np.int64),
        "_search_scale": scale,
    }


def lattice_decode_f32(buffers: dict, rows: int, want_symbols: bool = False):
    """Decode + reconstruct to fp32 [rows, cols_padded] (before the container cast)."""
    cols, pb, tile_elements = (int(v) for v in np.asarray(buffers["layout"]).tolist())
    out = np.zeros((rows, cols), dtype=np.float32)
    vectors = rows * cols // 8
    fields = np.zeros((vectors, 8), dtype=np.int32) if want_symbols else None
    cosets = np.zeros(vectors, dtype=np.int32) if want_symbols else None
    _check(lib().orc_lattice_decode(
        _p(_c(buffers["payload"], np.uint16)), _p(_c(buffers["offsets"], np.uint32)), _p(_c(buffers["states"], np.uint32)),
        _p(_c(buffers["stream_meta"], np.int32)), _p(_c(buffers["freq_tables"], np.uint16)),
        _p(_c(buffers["scales"], np.float32)), ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int(pb),
        ctypes.c_int64(tile_elements), _p(out), _p(fields) if want_symbols else None,
        _p(cosets) if want_symbols else None), "lattice decode")
    return (out, fields, cosets) if want_symbols else out


def snap_to_container(values, dtype):
    """Container cast of decoded fp32 values, entropack/schemes/lattice_rans/format.py:153-168."""
    import torch

    values = torch.as_tensor(values)
    if dtype == torch.float32:
        return values
    if dtype == torch.bool:
        return values.round() != 0
    if not dtype.is_floating_point:
        edge = torch.tensor(float(torch.iinfo(dtype).max) + 1.0, dtype=values.dtype)
        high = float(torch.nextafter(edge, torch.full_like(edge, float("-inf"))))
        return values.round().clamp(float(torch.iinfo(dtype).min), high).to(dtype)
    limit = float(torch.finfo(dtype).max)
    return values.clamp(-limit, limit).to(dtype)


def lattice_decode(buffers: dict, shape, dtype):
    """Full decode to a torch tensor of ``shape`` / ``dtype`` (columns sliced back from the padding)."""
    out = snap_to_container(lattice_decode_f32(buffers, int(shape[0])), dtype)
    return out[:, : shape[1]]


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    values = _c(values, np.float32)
    out = np.zeros(values.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(values), ctypes.c_int64(values.size), _p(out))
    return out


# ------------------------------------------------------------------------------------------------
# DFloat11
# ------------------------------------------------------------------------------------------------
def dfloat11_code(counts) -> tuple[np.ndarray, np.ndarray]:
    """(code_len int32[257], code_val uint32[257]); index 256 is the end-of-stream codeword."""
    counts = _c(counts, np.int64)
    code_len = np.zeros(257, dtype=np.int32)
    code_val = np.zeros(257, dtype=np.uint32)
    _check(lib().orc_dfloat11_build_code(_p(counts), _p(code_len), _p(code_val)), "dfloat11 code")
    return code_len, code_val


def dfloat11_luts(code_len, code_val) -> np.ndarray:
    luts = np.zeros((65, 256), dtype=np.uint8)
    rows = _check(lib().orc_dfloat11_build_luts(_p(_c(code_len, np.int32)), _p(_c(code_val, np.uint32)), _p(luts)), "dfloat11 luts")
    return luts[:rows].copy()


def dfloat11_encode(bits: np.ndarray, bytes_per_thread: int = 16, threads_per_block: int = 128, code=None) -> dict:
    """Encode bf16 bit patterns (uint16, flat)."""
    bits = _c(bits, np.uint16).reshape(-1)
    n = bits.size
    if code is None:
        counts = np.bincount((bits >> 7) & 0xFF, minlength=256)
        code = dfloat11_code(counts)
    code_len, code_val = code
    luts = dfloat11_luts(code_len, code_val)
    total_bits = int(lib().orc_dfloat11_total_bits(_p(bits), ctypes.c_int64(n), _p(code_len)))
    n_bytes = (total_bits + 7) // 8
    blocks = -(-n_bytes // (bytes_per_thread * threads_per_block))
    encoded = np.zeros(n_bytes, dtype=np.uint8)
    sign_mantissa = np.zeros(n, dtype=np.uint8)
    thread_meta = np.zeros(blocks * threads_per_block, dtype=np.uint16)
    output_positions = np.zeros(blocks + 1, dtype=np.uint32)
    widest = _check(lib().orc_dfloat11_encode(
        _p(bits), ctypes.c_int64(n), _p(code_len), _p(code_val), ctypes.c_int(bytes_per_thread),
        ctypes.c_int(threads_per_block), _p(encoded), _p(sign_mantissa), _p(thread_meta), _p(output_positions)),
        "dfloat11 encode")
    return {
        "encoded_exponent": encoded, "sign_mantissa": sign_mantissa, "luts": luts, "output_positions": output_positions,
        "thread_meta": thread_meta, "layout": np.array([bytes_per_thread, threads_per_block, widest], dtype=np.int32),
    }


def dfloat11_decode(buffers: dict, use_regions: bool = False) -> np.ndarray:
    """Decode to bf16 bit patterns (uint16). ``use_regions`` walks thread_meta/output_positions the
    way a parallel decoder does; otherwise one cursor runs over the whole stream as the eager lane does."""
    luts = _c(buffers["luts"], np.uint8)
    encoded = _c(buffers["encoded_exponent"], np.uint8)
    sign_mantissa = _c(buffers["sign_mantissa"], np.uint8)
    n = sign_mantissa.size
    out = np.zeros(n, dtype=np.uint16)
    if use_regions:
        bpt, tpb, _ = (int(v) for v in np.asarray(buffers["layout"]).tolist())
        _check(lib().orc_dfloat11_decode_regions(
            _p(luts), ctypes.c_int(luts.shape[0]), _p(encoded), ctypes.c_int64(encoded.size), _p(sign_mantissa),
            ctypes.c_int64(n), _p(_c(buffers["output_positions"], np.uint32)), _p(_c(buffers["thread_meta"], np.uint16)),
            ctypes.c_int(bpt), ctypes.c_int(tpb), _p(out)), "dfloat11 decode")
    else:
        lib().orc_dfloat11_decode_sequential(_p(luts), ctypes.c_int(luts.shape[0]), _p(encoded),
                                             ctypes.c_int64(encoded.size), _p(sign_mantissa), ctypes.c_int64(n), _p(out))
    return out


def set_threads(n: int) -> None:
    """Cap the OpenMP threads the oracle uses (for the timed CPU baseline)."""
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(n))
    except OSError:
        pass
