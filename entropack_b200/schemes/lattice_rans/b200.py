"""EntroPack-Lossy lane over the sm_100a kernel library.

Entry points mirror the reference's lane (entropack/schemes/lattice_rans/cuda.py:561,781):
``encode(weight, *, target_bpp, prob_bits, tile_elements, row_rdo_iterations, row_rdo_candidates,
scale_search_iterations, scale_search_max_vectors)`` and ``decode(buffers, *, shape, dtype,
threads_per_block, l2_prefetch)``.
"""
import torch

from ... import _native
from .format import LATTICE_DIM, LatticeBuffers, decode_geometry, snap_to_container

STORE_KINDS = {
    torch.bfloat16: 0, torch.float16: 1, torch.float32: 2, torch.float8_e4m3fn: 3, torch.float8_e5m2: 4, torch.int8: 5,
    torch.uint8: 6, torch.int16: 7, torch.uint16: 8, torch.int32: 9, torch.uint32: 10, torch.int64: 11, torch.uint64: 12,
    torch.bool: 13,
}
#: no saturating device cast exists for these; they are decoded to fp32 and cast by torch, as in the reference
_VIA_FLOAT32 = frozenset({torch.float8_e4m3fnuz, torch.float8_e5m2fnuz})


def max_alphabet(buffers: LatticeBuffers) -> int:
    """Largest alphabet of the 17 tables; read from the device once per container and cached on the layout."""
    cached = getattr(buffers.layout, "_lattice_rans_max_alphabet", None)
    if cached is None:
        cached = int(buffers.stream_meta[:, 3].max().item())
        buffers.layout._lattice_rans_max_alphabet = cached
    return cached


def slot_tables(buffers: LatticeBuffers, prob_bits: int, alphabet: int, device: torch.device, *, build_now: bool = False) -> torch.Tensor | None:
    """The container's decode plan: its 17 slot tables, built on the device once and kept on the layout tensor (as the
    reference keeps its plan, entropack/schemes/lattice_rans/cuda.py:697-741) so that later decodes copy them into
    shared memory instead of rebuilding them from the stored frequencies at the head of every launch. A container
    that is decoded only once never gets one: the first decode builds its tables inside the kernel and this returns
    None; the second builds the kept copy (139 KB at prob_bits 11), and so does a call with ``build_now`` (what
    ``prepare_plan`` makes for every layer of a model before its first pass). Must not be first reached during a stream
    capture."""
    layout = buffers.layout
    cached = getattr(layout, "_lattice_rans_slot_tables", None)
    if cached is not None and cached.device == device:
        return cached
    seen = getattr(layout, "_lattice_rans_decodes", 0)
    layout._lattice_rans_decodes = seen + 1
    if seen == 0 and not build_now:
        return None
    lib = _native.load()
    nbytes = lib.ep_lattice_slot_tables_bytes(prob_bits, alphabet)
    if nbytes < 0:
        _native.check(int(nbytes), "lattice_rans slot tables")
    tables = torch.empty(nbytes, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        status = lib.ep_lattice_build_slot_tables(
            _native.ptr(buffers.stream_meta), _native.ptr(buffers.freq_tables), buffers.freq_tables.numel(), prob_bits, alphabet,
            _native.ptr(tables), nbytes, _native.stream_handle(device))
    _native.check(status, "lattice_rans slot tables")
    layout._lattice_rans_slot_tables = tables
    return tables


def prepare_plan(buffers: LatticeBuffers, *, shape) -> bool:
    """Builds the container's kept slot tables now (see ``slot_tables``). False when they were there already or the
    container's tables are of the kind that stays in global memory and is rebuilt per call."""
    _native.require_cuda(buffers.payload)
    if getattr(buffers.layout, "_lattice_rans_slot_tables", None) is not None:
        return False
    info = decode_geometry(buffers._asdict(), shape)
    _check_lengths(buffers, info)
    alphabet = max_alphabet(buffers)
    if _native.load().ep_lattice_slot_tables_bytes(info["prob_bits"], alphabet) <= 0:
        return False
    return slot_tables(buffers, info["prob_bits"], alphabet, buffers.payload.device, build_now=True) is not None


def _tables_or_scratch(buffers: LatticeBuffers, prob_bits: int, alphabet: int, device: torch.device, what: str):
    """(buffer, bytes, ready) for the decode entry points: the kept slot tables when there are any, else scratch for the
    kernels that keep their tables in global memory, else nothing."""
    tables = slot_tables(buffers, prob_bits, alphabet, device)
    if tables is not None:
        return tables, tables.numel(), 1
    scratch_bytes = _native.load().ep_lattice_decode_scratch_bytes(prob_bits, alphabet)
    if scratch_bytes < 0:
        _native.check(int(scratch_bytes), what)
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=device) if scratch_bytes else None
    return scratch, scratch_bytes, 0


def _check_lengths(buffers: LatticeBuffers, info: dict) -> None:
    """The kernels index offsets, states, scales and the table records by tile, row and table: their lengths are checked
    here, on the host, without reading anything back from the device."""
    tiles, rows = info["total_tiles"], info["rows"]
    if buffers.offsets.numel() != tiles + 1:
        raise ValueError(f"lattice_rans offsets hold {buffers.offsets.numel()} entries, the layout needs {tiles + 1}")
    if buffers.states.numel() != tiles * 32:
        raise ValueError(f"lattice_rans states hold {buffers.states.numel()} words, the layout needs {tiles * 32}")
    if buffers.scales.numel() != rows:
        raise ValueError(f"lattice_rans scales hold {buffers.scales.numel()} entries for {rows} rows")
    if buffers.stream_meta.numel() != 17 * 4:
        raise ValueError(f"lattice_rans stream_meta holds {buffers.stream_meta.numel()} entries instead of 17 x 4")


def decode(buffers: LatticeBuffers, *, shape, dtype: torch.dtype, threads_per_block=None, l2_prefetch=True,
           error: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Decode to ``[rows, cols_padded]`` of ``dtype`` on the buffers' device (one or two launches, no host sync
    after the first call on a container)."""
    payload = buffers.payload
    _native.require_cuda(payload)
    info = decode_geometry(buffers._asdict(), shape)
    rows, cols, prob_bits = info["rows"], info["cols"], info["prob_bits"]
    device = payload.device
    via_float = dtype in _VIA_FLOAT32
    out_dtype = torch.float32 if via_float else dtype
    if out is None:
        out = torch.empty((rows, cols), dtype=out_dtype, device=device)
    _check_lengths(buffers, info)
    alphabet = max_alphabet(buffers)
    lib = _native.load()
    scratch, scratch_bytes, ready = _tables_or_scratch(buffers, prob_bits, alphabet, device, "lattice_rans decode")
    with torch.cuda.device(device):
        status = lib.ep_lattice_decode(
            _native.ptr(payload), payload.numel(), _native.ptr(buffers.offsets), _native.ptr(buffers.states),
            _native.ptr(buffers.stream_meta), _native.ptr(buffers.freq_tables), buffers.freq_tables.numel(), _native.ptr(buffers.scales),
            _native.ptr(out),
            STORE_KINDS[out_dtype], rows, cols, prob_bits, info["tile_elements"], alphabet, _native.ptr(scratch),
            scratch_bytes, ready, _native.ptr(error), _native.stream_handle(device))
    _native.check(status, "lattice_rans decode")
    return snap_to_container(out, dtype) if via_float else out


class PreparedDecode:
    """One container's decode with the host's share done once: the geometry parsed, the lengths checked, the kept slot
    tables found, the sixteen pointers and sizes of the library call laid out. A call then allocates the output, reads
    the current stream and makes the library call, nothing else -- a layer that decodes its weight at every forward
    otherwise spends more time in Python than a 3840 x 3840 decode takes on the device. ``prepared_decode`` makes one
    only once the container's tables are kept; the object holds the buffers (and so keeps them alive) and is good for
    as long as the caller still holds the same ``payload`` tensor (``valid_for``)."""

    __slots__ = ("buffers", "tables", "rows", "cols", "dtype", "index", "_head", "_tail")

    def __init__(self, buffers: LatticeBuffers, tables: torch.Tensor, info: dict, dtype: torch.dtype, alphabet: int):
        self.buffers, self.tables, self.dtype = buffers, tables, dtype
        self.rows, self.cols = info["rows"], info["cols"]
        self.index = buffers.payload.device.index
        ptr = _native.ptr
        self._head = (ptr(buffers.payload), buffers.payload.numel(), ptr(buffers.offsets), ptr(buffers.states), ptr(buffers.stream_meta),
                      ptr(buffers.freq_tables), buffers.freq_tables.numel(), ptr(buffers.scales))
        self._tail = (STORE_KINDS[dtype], self.rows, self.cols, info["prob_bits"], info["tile_elements"], alphabet, ptr(tables),
                      tables.numel(), 1)

    def __reduce__(self):
        # a copied or unpickled layer makes its own (the pointers above belong to this container's storage)
        return (type(None), ())

    def valid_for(self, buffers: dict, device: torch.device) -> bool:
        return buffers.get("payload") is self.buffers.payload and device.type == "cuda" and device.index == self.index

    def __call__(self, out: torch.Tensor | None = None, error: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((self.rows, self.cols), dtype=self.dtype, device=self.buffers.payload.device)
        error_at = None if error is None else error.data_ptr()
        with _native.on_device(self.index):
            status = _native.load().ep_lattice_decode(*self._head, out.data_ptr(), *self._tail, error_at, _native.raw_stream(self.index))
        if status:
            _native.check(status, "lattice_rans decode")
        return out


def prepared_decode(buffers: LatticeBuffers, *, shape, dtype: torch.dtype) -> PreparedDecode | None:
    """A ``PreparedDecode`` for a container on a CUDA device whose slot tables are kept already (from its second decode
    on, or after ``prepare_plan``) and whose dtype the kernel stores directly; None otherwise."""
    if buffers.payload.device.type != "cuda" or dtype in _VIA_FLOAT32 or dtype not in STORE_KINDS:
        return None
    tables = getattr(buffers.layout, "_lattice_rans_slot_tables", None)
    if tables is None or tables.device != buffers.payload.device:
        return None
    if not all(getattr(buffers, name).is_contiguous() for name in LatticeBuffers._fields):
        return None
    info = decode_geometry(buffers._asdict(), shape)
    _check_lengths(buffers, info)
    return PreparedDecode(buffers, tables, info, dtype, max_alphabet(buffers))


MAX_FUSED_TOKENS = 4


def linear_forward(buffers: LatticeBuffers, *, shape, x: torch.Tensor, bias: torch.Tensor | None,
                   error: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ decode(W).T + bias`` for up to four rows of bf16 activations without materialising ``W``: the decode
    kernel multiplies every reconstructed vector (rounded to bf16, as the dense weight would be) into the tokens'
    dot products and adds them, per weight row, into fp32 accumulators; the block that finishes last adds the bias
    and rounds to bf16. ``x`` is ``[tokens, cols]`` with ``cols`` equal to the stored (multiple of 8) column count."""
    payload = buffers.payload
    _native.require_cuda(payload)
    info = decode_geometry(buffers._asdict(), shape)
    rows, cols, prob_bits = info["rows"], info["cols"], info["prob_bits"]
    tokens = x.shape[0]
    if x.dtype != torch.bfloat16 or x.ndim != 2 or x.shape[1] != cols or not 1 <= tokens <= MAX_FUSED_TOKENS:
        raise ValueError(f"fused forward takes bf16 activations [1..{MAX_FUSED_TOKENS}, {cols}], got {tuple(x.shape)} {x.dtype}")
    device = payload.device
    x = x.contiguous()
    bias = None if bias is None else bias.to(torch.bfloat16).contiguous()
    products = torch.empty(tokens * rows + 1, dtype=torch.float32, device=device)   # accumulators + the kernel's block counter
    out = torch.empty((tokens, rows), dtype=torch.bfloat16, device=device)
    _check_lengths(buffers, info)
    alphabet = max_alphabet(buffers)
    lib = _native.load()
    scratch, scratch_bytes, ready = _tables_or_scratch(buffers, prob_bits, alphabet, device, "lattice_rans fused forward")
    with torch.cuda.device(device):
        status = lib.ep_lattice_linear_forward(
            _native.ptr(payload), payload.numel(), _native.ptr(buffers.offsets), _native.ptr(buffers.states),
            _native.ptr(buffers.stream_meta), _native.ptr(buffers.freq_tables), buffers.freq_tables.numel(), _native.ptr(buffers.scales),
            rows, cols, prob_bits,
            info["tile_elements"], alphabet, _native.ptr(scratch), scratch_bytes, ready, _native.ptr(x), _native.ptr(bias), tokens,
            _native.ptr(products), _native.ptr(out), _native.ptr(error), _native.stream_handle(device))
    _native.check(status, "lattice_rans fused forward")
    return out


def encode(weight, *, target_bpp, prob_bits, tile_elements, row_rdo_iterations, row_rdo_candidates,
           scale_search_iterations, scale_search_max_vectors) -> LatticeBuffers:
    from . import encoder

    return encoder.encode(
        weight, target_bpp=float(target_bpp), prob_bits=prob_bits, tile_elements=int(tile_elements),
        row_rdo_iterations=int(row_rdo_iterations), row_rdo_candidates=int(row_rdo_candidates),
        scale_search_iterations=int(scale_search_iterations), scale_search_max_vectors=int(scale_search_max_vectors))
