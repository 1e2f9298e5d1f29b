"""Decoding the next layer's weight while the current layer's product runs.

``CompressedLinear.forward`` decodes its weight and then multiplies: two kernels that cannot share an SM (each is
persistent and takes most of an SM's shared memory) and that leave half of the GPU idle each -- the decode is a set of
serial rANS chains that no number of SMs makes shorter than about 60 us, the product needs the tensor cores and none of
the integer pipes. Within one layer there is nothing to overlap (every tile's chain ends at the same moment, so no band
of the weight is ready early). Across layers there is: with the order of the layers known, the weight of the layer
that runs next is decoded on a second stream, on 52 of the 148 SMs, while the current product runs on the other 96
(``ep_set_sm_limits``). For two 3840 x 3840 layers at 4096 tokens that is 108 us a layer instead of 135 us (product
100 us on 96 SMs, decode 66 us on 52, both hidden behind each other). It pays only between two layers that are small
enough for their tiles to decode side by side on the decode's share; larger layers run as before.

The reference decodes and multiplies one after the other (entropack/linear/linear.py:163-165) and has nothing like it.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _native
from .compression import CompressedTensor

DECODE_SMS = 52            # SMs the decode ahead may fill while a product runs
PRODUCT_SMS = 96           # SMs the product keeps meanwhile
DECODE_WARPS_PER_SM = 24   # tiles the lossy decode kernel holds per SM
MIN_TOKENS = 129           # below this the product is not the two-block tensor-core kernel and is over before a decode is


class DecodeAhead:
    """Registers ``layers`` (``CompressedLinear`` modules in the order a forward pass calls them) for decode-ahead.

    While it is active, a registered layer whose successor is eligible launches its product on ``PRODUCT_SMS`` SMs and
    then, on a second stream, the decode of the successor's weight on ``DECODE_SMS`` SMs into one of two buffers that
    the layers share; the successor's forward finds its weight decoded. A layer called out of order simply decodes
    its own weight as usual. Results are bit for bit what the layers give without it. ``cyclic`` (default) makes the
    last layer's successor the first, for passes that repeat. Use as a context manager or call ``close()``.

    Not for training (it is skipped under autograd). To capture a pass into a CUDA graph: run one pass first (the second
    stream and the buffers are made at the first use), call ``drain()``, capture, and call ``drain()`` again before the
    capture ends, so that the decode started ahead of the pass's end is joined into the graph.
    """

    def __init__(self, layers: Sequence[torch.nn.Module], *, cyclic: bool = True):
        self.layers = list(layers)
        self.cyclic = cyclic
        self._position = {id(layer): index for index, layer in enumerate(self.layers)}
        if len(self._position) != len(self.layers):
            raise ValueError("a layer may be registered once in the order given")
        self._buffers: list[torch.Tensor] | None = None
        self._side: torch.cuda.Stream | None = None
        self._pending: tuple[int, int, torch.cuda.Event] | None = None   # (layer position, buffer, decode finished)
        self._known: dict[int, tuple] = {}                                # per layer: (container, geometry, packed buffers)
        self._latest = 1                                                  # buffer used last
        self.decoded_ahead = 0                                            # how many forwards found their weight ready
        for layer in self.layers:
            if getattr(layer, "_decode_ahead", None) is not None:
                raise ValueError("a layer belongs to one DecodeAhead at a time")
            layer._decode_ahead = self

    def close(self) -> None:
        for layer in self.layers:
            if getattr(layer, "_decode_ahead", None) is self:
                layer._decode_ahead = None
        self._pending = None

    def drain(self) -> None:
        """Makes the calling stream wait for the decode that was started ahead, if any, and forgets it (the layer it was
        for decodes its own weight when it runs). Call between passes where the streams have to meet: before a CUDA-graph
        capture begins and before it ends."""
        pending, self._pending = self._pending, None
        if pending is not None and self._buffers is not None:
            torch.cuda.current_stream(self._buffers[0].device).wait_event(pending[2])

    def __enter__(self) -> "DecodeAhead":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    # ------------------------------------------------------------------------------------------------------------
    def _geometry(self, layer) -> tuple[int, int, int] | None:
        """(rows, columns, tiles) of a layer whose weight this scheme can decode ahead, else None. Looked up once per
        container: a layer keeps its answer until its weight is replaced."""
        container = getattr(layer, "weight", None)
        known = self._known.get(id(layer))
        if known is not None and known[0] is container:
            return known[1]
        from .linear import CompressedLinear
        from .schemes.base import packed_buffers
        from .schemes.lattice_rans.format import LatticeBuffers, decode_geometry

        geometry, packed = None, None
        if (type(layer) is CompressedLinear and isinstance(container, CompressedTensor) and container.compress_method == "lattice_rans"
                and container.encoded_dtype == torch.bfloat16 and container.dtype == torch.bfloat16 and container.device.type == "cuda"
                and layer.in_features % 8 == 0):
            info = decode_geometry(container.buffers, tuple(container.shape))
            if info["cols"] == layer.in_features and info["rows"] == layer.out_features:
                geometry = (info["rows"], info["cols"], info["total_tiles"])
                packed = packed_buffers(container.buffers, LatticeBuffers)
        self._known[id(layer)] = (container, geometry, packed)
        return geometry

    def _small(self, geometry) -> bool:
        return geometry is not None and geometry[2] <= DECODE_SMS * DECODE_WARPS_PER_SM

    def _decode(self, layer, geometry, buffer: torch.Tensor) -> torch.Tensor:
        from .schemes.lattice_rans import b200

        rows, cols, _ = geometry
        out = buffer[: rows * cols].view(rows, cols)
        b200.decode(self._known[id(layer)][2], shape=(rows, cols), dtype=torch.bfloat16, out=out)
        return out

    def _ensure(self, device: torch.device) -> None:
        if self._buffers is not None and self._buffers[0].device == device:
            return
        largest = 0
        for layer in self.layers:
            geometry = self._geometry(layer)
            if geometry is not None and layer.weight.device == device:
                largest = max(largest, geometry[0] * geometry[1])
        self._buffers = [torch.empty(max(1, largest), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self._side = torch.cuda.Stream(device)
        self._pending = None

    def forward(self, layer, x: torch.Tensor) -> torch.Tensor | None:
        """The layer's output, or None when this call is not one for decode-ahead (the layer then runs as usual)."""
        from .linear import _native_gemm_applies, linear_forward

        geometry = self._geometry(layer)
        if (geometry is None or not x.is_cuda or x.dtype != torch.bfloat16 or x.device != layer.weight.device
                or (torch.is_grad_enabled() and x.requires_grad) or x.numel() == 0):
            return None
        tokens = x.numel() // x.shape[-1]
        if tokens < MIN_TOKENS:
            return None
        device = x.device
        self._ensure(device)
        if geometry[0] * geometry[1] > self._buffers[0].numel():
            return None
        rows, cols, _ = geometry
        bias = layer._bias_on(device)
        if not _native_gemm_applies(x, self._buffers[0][: rows * cols].view(rows, cols), bias):
            return None
        main = torch.cuda.current_stream(device)
        position = self._position[id(layer)]

        pending, self._pending = self._pending, None
        if pending is not None and pending[0] == position:
            slot = pending[1]
            main.wait_event(pending[2])
            weight = self._buffers[slot][: rows * cols].view(rows, cols)
            self.decoded_ahead += 1
        else:
            if pending is not None:
                main.wait_event(pending[2])    # a decode for a layer that did not come next: let it finish, drop it
            slot = 1 - self._latest
            weight = self._decode(layer, geometry, self._buffers[slot])
        self._latest = slot

        follower = None
        if position + 1 < len(self.layers) or self.cyclic:
            follower_position = (position + 1) % len(self.layers)
            follower = self.layers[follower_position]
            follower_geometry = self._geometry(follower)
            if not (self._small(geometry) and self._small(follower_geometry) and follower.weight.device == device
                    and follower_geometry[0] * follower_geometry[1] <= self._buffers[0].numel()):
                follower = None

        lib = _native.load()
        before_product = torch.cuda.Event()
        before_product.record(main)
        if follower is None:
            out = linear_forward(x, weight, bias)
        else:
            with torch.cuda.device(device):
                _native.check(lib.ep_set_sm_limits(0, PRODUCT_SMS), "sm limits")
                try:
                    out = linear_forward(x, weight, bias)
                finally:
                    lib.ep_set_sm_limits(0, 0)
        if follower is not None:
            # The decode ahead writes the other buffer, which the product before this one read last: it may start once
            # the calling stream has reached the point just before this product (the event was recorded there).
            side = self._side
            side.wait_event(before_product)
            with torch.cuda.stream(side), torch.cuda.device(device):
                _native.check(lib.ep_set_sm_limits(DECODE_SMS, 0), "sm limits")
                try:
                    self._decode(follower, follower_geometry, self._buffers[1 - slot])
                finally:
                    lib.ep_set_sm_limits(0, 0)
                done = torch.cuda.Event()
                done.record(side)
            self._pending = (follower_position, 1 - slot, done)
        return out
