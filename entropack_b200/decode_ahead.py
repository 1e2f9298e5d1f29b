"""Decoding the next layer's weight while the current layer's product runs.

``CompressedLinear.forward`` decodes its weight and then multiplies: two kernels that cannot share an SM (each is
persistent and takes most of an SM's shared memory) and that leave half of the GPU idle each -- the decode is a set of
serial rANS chains that no number of SMs makes shorter than about 60 us, the product needs the tensor cores and none of
the integer pipes. Within one layer there is nothing to overlap (every tile's chain ends at the same moment, so no band
of the weight is ready early). Across layers there is: with the order of the layers known, the weight of the layer
that runs next is decoded on a second stream, on 52 of the 148 SMs, while the current product runs on the other 96
(``ep_set_sm_limits``). For two 3840 x 3840 layers at 4096 tokens that is 105-108 us a layer instead of 135 us (product
100 us on 96 SMs, decode 66 us on 52, both hidden behind each other). It pays only where the next layer's tiles all
decode side by side on that share (at most 1248 tiles: 20 million weights in 16384-symbol tiles, 9 million in the
8192-symbol tiles of the FP8 layers' default -- four 3840 x 3840 FP8 layers at 5 bpp in a ring measured 122 us a layer
with a decode ahead that takes its tiles in two turns against 105 us without). Beside a long product (a 10240-wide
layer at 4096 tokens) the decode ahead gets 28 SMs and the product 120; other layers run as before.

The reference decodes and multiplies one after the other (entropack/linear/linear.py:163-165) and has nothing like it.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _native
from .compression import CompressedTensor

DECODE_SMS = 52            # SMs the decode ahead may fill while a product runs
PRODUCT_SMS = 96           # SMs the product keeps meanwhile
# beside a long product (of a layer past MAX_PRODUCT_WEIGHTS at thousands of tokens) the decode gets fewer SMs and takes
# its tiles in two turns, still well inside the product's time: measured at 4096 tokens with a 3840 x 3840 weight
# decoded ahead, 3840 -> 10240: 246 us together against 261 us in turn; 10240 -> 3840: 240 against 280; 3840 -> 11520: 265
# against 287
SLIM_DECODE_SMS = 28
WIDE_PRODUCT_SMS = 120
LONG_PRODUCT_WORK = 9e10   # tokens x weights from which a product outlasts a two-turn decode on SLIM_DECODE_SMS
DECODE_WARPS_PER_SM = 24   # tiles the lossy decode kernel holds per SM
MIN_TOKENS = 129           # from here on the product is the two-block tensor-core kernel that shares the GPU by SMs
FEW_TOKENS = 16            # up to here it is the streaming kernel, whose small blocks fit on an SM beside a decode block
ALL_SMS = 148
MAX_PRODUCT_WEIGHTS = 20 << 20   # a longer product loses more on 96 SMs than hiding a decode behind it gains


class _Plan:
    """What is known about a registered layer's weight: looked up once per container."""

    __slots__ = ("container", "payload", "rows", "cols", "dtype", "nbytes", "tiles", "packed", "prepared")

    def __init__(self, container):
        self.container = container
        self.payload = None
        self.rows = self.cols = self.nbytes = self.tiles = 0
        self.dtype = None
        self.packed = self.prepared = None


class DecodeAhead:
    """Registers ``layers`` (compressed linear modules in the order a forward pass calls them) for decode-ahead.

    While it is active, a registered layer whose successor is eligible launches its product on ``PRODUCT_SMS`` SMs and
    then, on a second stream, the decode of the successor's weight on ``DECODE_SMS`` SMs into one of two buffers that
    the layers share; the successor's forward finds its weight decoded. A layer called out of order simply decodes
    its own weight as usual. Results are bit for bit what the layers give without it. ``cyclic`` (default) makes the
    last layer's successor the first, for passes that repeat. Use as a context manager or call ``close()``.

    Handled: ``CompressedLinear`` with a lossy-coded bf16 weight (up to 16 tokens, where the product's small blocks run
    beside the decode's on every SM, and from 129 tokens up, where the two share the GPU by SMs and the successor may have
    at most 1248 tiles), ``CompressedFP8Linear`` / ``CompressedINT8Linear`` with lossy-coded codes (from 129 tokens up).
    Other layers in the list, and other token counts, run as they always do.

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
        self._buffers: list[torch.Tensor] | None = None                  # two byte buffers
        self._side: torch.cuda.Stream | None = None
        self._pending: tuple[int, int, torch.cuda.Event] | None = None   # (layer position, buffer, decode finished)
        self._plans: dict[int, _Plan] = {}
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
    def _plan(self, layer) -> _Plan:
        container = getattr(layer, "weight", None)
        plan = self._plans.get(id(layer))
        # module.to() swaps a container's contents in place: the payload tensor tells a moved container from the same one
        payload = container.buffers.get("payload") if isinstance(container, CompressedTensor) else None
        if plan is not None and plan.container is container and plan.payload is payload:
            return plan
        from .linear import CompressedLinear, QuantizedLinear
        from .schemes.base import packed_buffers
        from .schemes.lattice_rans.format import LatticeBuffers, decode_geometry

        plan = _Plan(container)
        plan.payload = payload
        if type(layer) is CompressedLinear:
            dtype = torch.bfloat16 if (isinstance(container, CompressedTensor) and container.dtype == torch.bfloat16
                                       and container.encoded_dtype == torch.bfloat16) else None
        elif isinstance(layer, QuantizedLinear):
            dtype = layer.code_dtype
        else:
            dtype = None
        if (dtype is not None and isinstance(container, CompressedTensor) and container.compress_method == "lattice_rans"
                and container.device.type == "cuda" and layer.in_features % 8 == 0):
            info = decode_geometry(container.buffers, tuple(container.shape))
            if info["cols"] == layer.in_features and info["rows"] == layer.out_features:
                plan.rows, plan.cols, plan.dtype = info["rows"], info["cols"], dtype
                plan.nbytes = plan.rows * plan.cols * torch.empty((), dtype=dtype).element_size()
                plan.tiles = info["total_tiles"]
                plan.packed = packed_buffers(container.buffers, LatticeBuffers)
        self._plans[id(layer)] = plan
        return plan

    def _view(self, plan: _Plan, slot: int) -> torch.Tensor:
        return self._buffers[slot][: plan.nbytes].view(plan.dtype).view(plan.rows, plan.cols)

    def _decode(self, plan: _Plan, slot: int) -> torch.Tensor:
        from .schemes.lattice_rans import b200

        out = self._view(plan, slot)
        if plan.prepared is None:          # there is none before the container's slot tables are kept
            plan.prepared = b200.prepared_decode(plan.packed, shape=(plan.rows, plan.cols), dtype=plan.dtype)
        if plan.prepared is not None:
            return plan.prepared(out=out)
        b200.decode(plan.packed, shape=(plan.rows, plan.cols), dtype=plan.dtype, out=out)
        return out

    def _ensure(self, device: torch.device) -> None:
        if self._buffers is not None and self._buffers[0].device == device:
            return
        largest = 0
        for layer in self.layers:
            plan = self._plan(layer)
            if plan.dtype is not None and layer.weight.device == device:
                largest = max(largest, plan.nbytes)
        self._buffers = [torch.empty(max(16, largest), dtype=torch.uint8, device=device) for _ in range(2)]
        self._side = torch.cuda.Stream(device)
        self._pending = None

    def forward(self, layer, x: torch.Tensor) -> torch.Tensor | None:
        """The layer's output, or None when this call is not one for decode-ahead (the layer then runs as usual)."""
        from .linear import CompressedLinear, _native_gemm_applies, linear_forward

        plan = self._plan(layer)
        if (plan.dtype is None or not x.is_cuda or x.device != layer.weight.device or x.numel() == 0
                or (torch.is_grad_enabled() and x.requires_grad)):
            return None
        tokens = x.numel() // x.shape[-1]
        plain = type(layer) is CompressedLinear
        # A few tokens: the product is the streaming kernel, whose blocks run on the same SMs as a decode's (and the weight
        # is decoded to memory instead of being multiplied inside the fused kernel); many: the GPU is shared by SMs.
        # In between the product's blocks need an SM's shared memory to themselves and would only queue behind a decode.
        few = plain and tokens <= FEW_TOKENS
        if not few and tokens < MIN_TOKENS:
            return None
        device = x.device
        self._ensure(device)
        if plan.nbytes > self._buffers[0].numel():
            return None
        bias = layer._bias_on(device) if plain else None
        if plain and not _native_gemm_applies(x, self._view(plan, 0), bias):
            return None
        main = torch.cuda.current_stream(device)
        position = self._position[id(layer)]

        pending, self._pending = self._pending, None
        if pending is not None and pending[0] == position:
            slot = pending[1]
            main.wait_event(pending[2])
            weight = self._view(plan, slot)
            self.decoded_ahead += 1
        else:
            if pending is not None:
                main.wait_event(pending[2])    # a decode for a layer that did not come next: let it finish, drop it
            slot = 1 - self._latest
            weight = self._decode(plan, slot)
        self._latest = slot

        follower_plan = None
        decode_sms, product_sms = (0, 0) if few else (DECODE_SMS, PRODUCT_SMS)
        if position + 1 < len(self.layers) or self.cyclic:
            follower_position = (position + 1) % len(self.layers)
            follower = self.layers[follower_position]
            candidate = self._plan(follower)
            # the successor's tiles have to decode side by side (tiles that wait for a second turn double the decode): on the
            # whole GPU beside a streaming product, on the decode's share beside a tensor-core one, which moreover must
            # not be so long that running it on 96 SMs costs more than the hidden decode saves
            if candidate.dtype is not None and follower.weight.device == device and candidate.nbytes <= self._buffers[0].numel():
                if few:
                    eligible = candidate.tiles <= ALL_SMS * DECODE_WARPS_PER_SM
                elif candidate.tiles > DECODE_SMS * DECODE_WARPS_PER_SM:
                    eligible = False
                elif plan.rows * plan.cols <= MAX_PRODUCT_WEIGHTS:
                    eligible = True
                else:
                    eligible = float(tokens) * plan.rows * plan.cols >= LONG_PRODUCT_WORK
                    decode_sms, product_sms = SLIM_DECODE_SMS, WIDE_PRODUCT_SMS
                if eligible:
                    follower_plan = candidate

        def product():
            return linear_forward(x, weight, bias) if plain else layer._forward8(x, codes=weight)

        lib = _native.load()
        before_product = torch.cuda.Event()
        before_product.record(main)
        if follower_plan is None:
            return product()
        with torch.cuda.device(device):
            _native.check(lib.ep_set_sm_limits(0, product_sms), "sm limits")
            try:
                out = product()
            finally:
                lib.ep_set_sm_limits(0, 0)
        # The decode ahead writes the other buffer, which the product before this one read last: it may start once the
        # calling stream has reached the point just before this product (the event was recorded there).
        side = self._side
        side.wait_event(before_product)
        with torch.cuda.stream(side), torch.cuda.device(device):
            _native.check(lib.ep_set_sm_limits(decode_sms, 0), "sm limits")
            try:
                self._decode(follower_plan, 1 - slot)
            finally:
                lib.ep_set_sm_limits(0, 0)
            done = torch.cuda.Event()
            done.record(side)
        self._pending = (follower_position, 1 - slot, done)
        return out
