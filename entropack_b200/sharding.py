"""Whole-model compression across the GPUs of one node, and a column-sharded compressed linear.

The reference has no multi-GPU code; every layer (and every tile inside a layer) is independent, so the
work shards without any exchange on the data path:

* :func:`partition_layers` assigns layers to ranks, largest first onto the lightest rank;
* :func:`compress_layers` compresses this rank's share (one process per GPU, ``torch.distributed`` only
  to learn rank and world size) and returns ``{layer index: CompressedTensor}``;
* :class:`ColumnShardedLinear` keeps rows ``[rank * N / G, (rank + 1) * N / G)`` of a weight on each rank
  (row scales and whole E8 vectors stay local) and exchanges only the ``[M, N / G]`` outputs -- the one
  exchange of the package. Above 128 tokens on GPUs with peer access the exchange is folded into the product: the
  tensor-core kernel's epilogue stores every finished tile into all ranks' ``[M, N]`` buffers (ordinary stores through
  peer mappings of symmetric memory), followed by one bounded flag barrier; otherwise it is an NCCL all-gather.
"""
import ctypes
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

#: The synthetic 276-linear DiT used as the whole-model workload: 30 blocks of 9 linears plus 6
#: embed/head linears, hidden 3840, MLP 10240. (out_features, in_features) per layer, in model order.
DIT_HIDDEN, DIT_MLP, DIT_BLOCKS = 3840, 10240, 30
_BLOCK_LAYERS = (
    (3 * DIT_HIDDEN, DIT_HIDDEN),   # fused qkv
    (DIT_HIDDEN, DIT_HIDDEN),       # attention output
    (DIT_MLP, DIT_HIDDEN),          # mlp up
    (DIT_HIDDEN, DIT_MLP),          # mlp down
    (DIT_HIDDEN, DIT_HIDDEN), (DIT_HIDDEN, DIT_HIDDEN), (DIT_HIDDEN, DIT_HIDDEN),   # modulation / projection layers
    (DIT_HIDDEN, DIT_HIDDEN), (DIT_HIDDEN, DIT_HIDDEN),
)


def dit_layer_shapes() -> list[tuple[int, int]]:
    shapes = [(DIT_HIDDEN, DIT_HIDDEN)] * 3
    for _ in range(DIT_BLOCKS):
        shapes.extend(_BLOCK_LAYERS)
    shapes.extend([(DIT_HIDDEN, DIT_HIDDEN)] * 3)
    return shapes


def mixed_bit_targets(shapes, mean_bpp: float = 2.3, seed: int = 0) -> list[float]:
    """Per-layer targets from a fixed seeded draw, rescaled so the element-weighted mean is ``mean_bpp``
    (the reference's sensitivity-based allocator is not public; this stands in for its output)."""
    generator = torch.Generator().manual_seed(seed)
    raw = 1.6 + 1.6 * torch.rand(len(shapes), generator=generator)
    weights = torch.tensor([float(r * c) for r, c in shapes])
    raw = raw * (mean_bpp / float((raw * weights).sum() / weights.sum()))
    return [round(float(v), 3) for v in raw]


def bind_host_thread_near(device: torch.device | int) -> list[int] | None:
    """Restrict the calling process to the CPUs that NVML reports as local to ``device`` (the cores of the socket its
    PCIe root hangs off), so that pinned staging buffers allocated afterwards sit in that socket's memory and uploads
    and downloads do not cross the inter-socket link. With one rank per GPU on a two-socket host this is what keeps
    the ranks' host traffic apart. Returns the CPUs now in use, or None when nothing was changed (no NVML, no
    affinity information, or none of the local CPUs is available to this process). Only the process's own CPU
    affinity is touched; no GPU setting is."""
    import os

    try:
        import pynvml
    except ImportError:
        return None
    index = device if isinstance(device, int) else (device.index if device.index is not None else torch.cuda.current_device())
    try:
        pynvml.nvmlInit()
        properties = torch.cuda.get_device_properties(index)
        bus = f"{properties.pci_domain_id:08x}:{properties.pci_bus_id:02x}:{properties.pci_device_id:02x}.0"
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
    except Exception:    # NVML missing on the host, an unknown bus id, an old driver: leave the process where it is
        return None
    local = {64 * word + bit for word, bits in enumerate(mask) for bit in range(64) if (bits >> bit) & 1}
    usable = sorted(local & os.sched_getaffinity(0))
    if not usable:
        return None
    os.sched_setaffinity(0, usable)
    return usable


def partition_layers(sizes, world_size: int) -> list[list[int]]:
    """Greedy longest-processing-time assignment: layers by decreasing size onto the least-loaded rank.
    Deterministic (ties go to the lower layer index, then the lower rank)."""
    if world_size < 1:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(sizes)), key=lambda i: (-sizes[i], i))
    load = [0] * world_size
    shares: list[list[int]] = [[] for _ in range(world_size)]
    for index in order:
        rank = min(range(world_size), key=lambda r: (load[r], r))
        shares[rank].append(index)
        load[rank] += sizes[index]
    return [sorted(share) for share in shares]


def _rank_and_world(group=None) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def compress_layers(weights, configs, group=None, compress_fn=None) -> dict:
    """Compress this rank's share of ``weights`` (a sequence of callables or tensors; callables are only
    invoked for layers this rank owns, so a rank never materialises the others' weights).
    ``configs`` is one config or one per layer. Returns ``{layer index: compressed}``."""
    from .compression import compress

    compress_fn = compress_fn or compress
    rank, world = _rank_and_world(group)
    sizes = [getattr(w, "numel", lambda: 0)() if isinstance(w, torch.Tensor) else int(getattr(w, "size_hint", 1)) for w in weights]
    mine = partition_layers(sizes, world)[rank]
    per_layer = configs if isinstance(configs, (list, tuple)) else [configs] * len(weights)
    result = {}
    for index in mine:
        weight = weights[index] if isinstance(weights[index], torch.Tensor) else weights[index]()
        result[index] = compress_fn(weight, per_layer[index])
    return result


def gather_columns(local: torch.Tensor, group=None, staging: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather ``[..., N / G]`` shards along the last dimension into ``[..., N]`` (rank order): one
    ``all_gather_into_tensor`` into a ``[G, ..., N / G]`` buffer (``staging``, when the caller keeps one) and one
    strided copy that interleaves the ranks' column blocks."""
    _rank, world = _rank_and_world(group)
    if world == 1:
        return local
    local = local.contiguous()
    shape = (world, *local.shape)
    if staging is None or tuple(staging.shape) != shape or staging.dtype != local.dtype or staging.device != local.device:
        staging = torch.empty(shape, dtype=local.dtype, device=local.device)
    # the collective wants the ranks' pieces stacked along the first dimension: [G * M, N / G] is the same memory
    dist.all_gather_into_tensor(staging.view(world * local.shape[0], *local.shape[1:]), local, group=group)
    return staging.movedim(0, -2).reshape(*local.shape[:-1], world * local.shape[-1])


@dataclass
class RowSlice:
    begin: int
    end: int


def row_slice(out_features: int, rank: int, world: int) -> RowSlice:
    if out_features % world:
        raise ValueError(f"out_features {out_features} is not divisible by the {world} ranks of the group")
    rows = out_features // world
    return RowSlice(rank * rows, (rank + 1) * rows)


#: how long a rank waits at the barrier behind a scattered product for a peer that does not arrive, in microseconds
PEER_BARRIER_TIMEOUT_US = 2_000_000


class _PeerOutputs:
    """Two ``[M, N]`` bf16 output buffers in symmetric memory (used alternately, so that a forward never writes into
    rows a peer may still be reading from the forward before) and one row of arrival flags per rank, with every
    rank's copies mapped into this process. Creating one is a collective over the group."""

    def __init__(self, rows: int, cols: int, device: torch.device, group, rank: int, world: int):
        # no multicast object is bound to these allocations: peers are reached with plain stores only
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symmetric_memory

        group = dist.group.WORLD if group is None else group
        self.rank, self.world = rank, world
        self.buffers, self.handles, self.peer_pointers = [], [], []
        for _ in range(2):
            buffer = symmetric_memory.empty((rows, cols), dtype=torch.bfloat16, device=device)
            handle = symmetric_memory.rendezvous(buffer, group)
            peers = [int(handle.buffer_ptrs[r]) for r in range(world) if r != rank]
            self.buffers.append(buffer)
            self.handles.append(handle)
            self.peer_pointers.append((ctypes.c_void_p * len(peers))(*peers))
        self.flags = symmetric_memory.empty((max(world, 4),), dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self.flag_handle = symmetric_memory.rendezvous(self.flags, group)
        self.flag_rows = (ctypes.c_void_p * world)(*[int(self.flag_handle.buffer_ptrs[r]) for r in range(world)])
        dist.barrier(group)      # every rank's flags are zero before anyone's first arrival is stored
        self.epoch = 0
        self.turn = 0


class ColumnShardedLinear(torch.nn.Module):
    """A compressed linear whose output features are split over the ranks of a process group.

    Each rank compresses and decodes only its own rows of the weight; activations are replicated; the forward
    computes ``x @ W_rank^T`` locally and the ranks exchange the outputs. ``exchange="scatter"`` (tried first under
    ``"auto"``) writes every output tile straight into all ranks' ``[M, N]`` buffers from the product's epilogue and
    ends with one bounded barrier; it needs bf16 activations of more than 128 rows, the plain :class:`CompressedLinear`
    and symmetric memory with peer access. ``exchange="gather"`` is the NCCL all-gather plus one interleaving copy.
    A scattered forward returns a view of one of two alternating buffers, valid until the layer's next forward but one
    (``copy_output=True`` returns a private copy instead). ``check()`` reads the layer's error word (a peer that did
    not arrive, a wait that ran out inside the product) and raises."""

    def __init__(self, linear: torch.nn.Linear, layer_cls=None, group=None, exchange: str = "auto", copy_output: bool = False,
                 **layer_kwargs):
        super().__init__()
        from .linear import CompressedLinear

        if exchange not in ("auto", "scatter", "gather"):
            raise ValueError(f"exchange must be 'auto', 'scatter' or 'gather', got {exchange!r}")
        layer_cls = layer_cls or CompressedLinear
        self.group = group
        self.exchange = exchange
        self.copy_output = copy_output
        self.scatter_unavailable = None if layer_cls is CompressedLinear else f"{layer_cls.__name__} has no scattered product"
        self._peer_outputs: dict[int, _PeerOutputs] = {}
        self._error = None
        rank, world = _rank_and_world(group)
        rows = row_slice(linear.out_features, rank, world)
        shard = torch.nn.Linear(linear.in_features, rows.end - rows.begin, bias=linear.bias is not None,
                                device=linear.weight.device, dtype=linear.weight.dtype)
        with torch.no_grad():
            shard.weight.copy_(linear.weight[rows.begin : rows.end])
            if linear.bias is not None:
                shard.bias.copy_(linear.bias[rows.begin : rows.end])
        self.rows = rows
        self.out_features = linear.out_features
        self.local = layer_cls.from_linear(shard, **layer_kwargs)
        self._staging = None      # the all-gather's landing buffer, kept between calls of the same shape

    def _scatter_applies(self, x: torch.Tensor, world: int) -> bool:
        return (self.exchange != "gather" and self.scatter_unavailable is None and world > 1 and world <= 8 and x.is_cuda
                and x.dtype == torch.bfloat16 and x.numel() // max(1, x.shape[-1]) > 128 and x.shape[-1] % 8 == 0
                and (self.out_features // world) % 8 == 0 and not (torch.is_grad_enabled() and x.requires_grad))

    def _scattered_forward(self, x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
        from . import _native

        flat = x.reshape(-1, x.shape[-1]).contiguous()
        tokens = flat.shape[0]
        outputs = self._peer_outputs.get(tokens)
        if outputs is None:
            outputs = self._peer_outputs[tokens] = _PeerOutputs(tokens, self.out_features, x.device, self.group, rank, world)
        if self._error is None:
            self._error = torch.zeros(1, dtype=torch.int32, device=x.device)
        weight = self.local.dequantize(x.device)
        bias = self.local._bias_on(x.device)
        target = outputs.buffers[outputs.turn]
        lib = _native.load()
        columns = self.out_features // world
        with torch.cuda.device(x.device):
            stream = _native.stream_handle(x.device)
            _native.check(lib.ep_linear_forward_scatter(
                _native.ptr(flat), _native.ptr(weight), _native.ptr(None if bias is None else bias.contiguous()), target.data_ptr(),
                outputs.peer_pointers[outputs.turn], world - 1, self.out_features, rank * columns, tokens, columns, flat.shape[1],
                _native.ptr(self._error), stream), "scattered linear forward")
            outputs.epoch += 1
            _native.check(lib.ep_peer_barrier(outputs.flag_rows, rank, world, outputs.epoch & 0xFFFFFFFF, PEER_BARRIER_TIMEOUT_US,
                                              _native.ptr(self._error), stream), "peer barrier")
        outputs.turn ^= 1
        result = target.clone() if self.copy_output else target
        return result.reshape(*x.shape[:-1], self.out_features)

    def check(self) -> None:
        """Raise if a scattered forward of this layer reported a failure on the device (synchronises)."""
        if self._error is not None:
            code = int(self._error.item())
            if code:
                from . import _native

                self._error.zero_()
                _native.raise_stream_error(code, "column-sharded linear forward")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rank, world = _rank_and_world(self.group)
        if self._scatter_applies(x, world):
            try:
                return self._scattered_forward(x, rank, world)
            except (RuntimeError, ImportError, AttributeError) as error:
                if self.exchange == "scatter":
                    raise
                # no symmetric memory or no peer access on this machine: every rank fails the same collective set-up the
                # same way, and the layer gathers from here on
                self.scatter_unavailable = f"{type(error).__name__}: {error}"
        local = self.local(x).contiguous()
        shape = (world, *local.shape)
        if world > 1 and (self._staging is None or tuple(self._staging.shape) != shape or self._staging.dtype != local.dtype
                          or self._staging.device != local.device):
            self._staging = torch.empty(shape, dtype=local.dtype, device=local.device)
        return gather_columns(local, self.group, self._staging)
