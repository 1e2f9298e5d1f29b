"""Linear layers that keep their weight compressed and decode it on every forward.

Stands in for entropack/linear/linear.py:18-490: same class names, constructor arguments, properties
(``qweight``, ``stored_nbytes``, ``compressed_bits``, ``container_dtype``), ``from_linear`` /
``compress_weight`` / ``dequantize`` / ``codes`` and the same checkpoint keys
(``<prefix>weight.entropack_quant_state``, ``<prefix>weight_quant_scale``, ``<prefix>bias``), so a
state_dict written by either implementation loads into the other.

Forward: the weight is decoded by the fused sm_100a decode kernel (entropy decode, dequantisation and
the container cast in one pass, straight from the packed blob) into a dense operand that a GEMM consumes
while it is still resident in the 126 MB L2. The INT8 layer's optional ConvRot rotation runs on the
library's butterfly kernel (``convrot.py``). Activations that are not bf16, and calls that need gradients,
fall back to ``torch.nn.functional.linear`` on the decoded weight.
"""
import dataclasses
from numbers import Real
from typing import ClassVar

import torch
from torch.nn import functional as F

from . import _native
from .compression import CompressedTensor, compress, decompress
from .convrot import choose_convrot_group, rotate_activation, rotate_weight
from .registry import default_config, get_scheme, name_for_config, require_dtype
from .schemes import EntroPackLossyConfig, RawConfig

_EPS = torch.finfo(torch.float32).eps
_SOURCE_KINDS = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _native_gemm_applies(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> bool:
    """The library GEMM takes bf16 operands on one CUDA device with K a multiple of 8; gradients, other dtypes
    and odd shapes go through torch."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.device == x.device
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.device == x.device))
            and x.shape[-1] % 8 == 0 and x.numel() > 0 and not (torch.is_grad_enabled() and x.requires_grad))


#: one int32 error word per device, zeroed when it is made and handed to every product this module launches: a bounded
#: wait that runs out inside a tensor-core kernel leaves its code there instead of passing unnoticed
_error_words: dict[torch.device, torch.Tensor] = {}


def kernel_error_word(device: torch.device) -> torch.Tensor:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _error_words.get(device)
    if word is None:
        word = _error_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def check_kernel_errors(device: torch.device | None = None) -> None:
    """Read the error words of the products launched so far (``device``, or every device used) and raise if a kernel
    reported a failure -- a wait inside a tensor-core product that ran out leaves an incomplete output. Reading the
    word waits for the device, so this is for the end of a step or a test, not for every forward."""
    for where, word in list(_error_words.items()):
        if device is not None and torch.device(device) != where:
            continue
        code = int(word.item())
        if code:
            word.zero_()
            _native.raise_stream_error(code, f"a product on {where}")


def prepare_decode_plans(module: torch.nn.Module) -> int:
    """Builds the per-container decode plans (kept decode tables) of every compressed layer under ``module`` whose
    container is on a CUDA device, and returns how many were built.

    A layer otherwise gets its plan along the way (the lossy scheme at a container's second decode), with an allocation
    and an extra launch in the middle of an early forward pass. Calling this once after a model is loaded and moved to
    its device makes the first pass as fast as the later ones and leaves no allocation for a pass that is being
    captured into a CUDA graph. The reference builds its plan per container at the first decode
    (entropack/schemes/lattice_rans/cuda.py:697-741) and has no call for a whole model."""
    built = 0
    for layer in module.modules():
        container = getattr(layer, "weight", None)
        if isinstance(layer, CompressedLinear) and isinstance(container, CompressedTensor) and container.device.type == "cuda":
            built += bool(container.scheme.prepare_decode_plan(container.buffers, shape=tuple(container.shape)))
    return built


def linear_forward(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                   error: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T + bias`` in bf16 through ``ep_linear_forward`` (streaming mma.sync kernel for up to 16 tokens,
    tcgen05 tensor-core kernel above). ``error`` defaults to the device's shared error word (``check_kernel_errors``)."""
    flat = x.reshape(-1, x.shape[-1]).contiguous()
    weight = weight.contiguous()
    if error is None:
        error = kernel_error_word(x.device)
    out = torch.empty((flat.shape[0], weight.shape[0]), dtype=torch.bfloat16, device=x.device)
    index = x.device.index
    with _native.on_device(index):
        status = _native.load().ep_linear_forward(
            _native.ptr(flat), _native.ptr(weight), _native.ptr(bias.contiguous() if bias is not None else None), _native.ptr(out),
            flat.shape[0], weight.shape[0], flat.shape[1], _native.ptr(error), _native.raw_stream(index))
    _native.check(status, "linear forward")
    return out.reshape(*x.shape[:-1], weight.shape[0])


def _pad_to(tensor: torch.Tensor, dim: int, size: int) -> torch.Tensor:
    missing = size - tensor.shape[dim]
    if missing <= 0:
        return tensor
    shape = list(tensor.shape)
    shape[dim] = missing
    return torch.cat([tensor, tensor.new_zeros(shape)], dim=dim)


_SIDE_STREAMS: dict[int, "torch.cuda.Stream"] = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """One extra stream per device for work that runs beside a layer's weight decode."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    stream = _SIDE_STREAMS.get(index)
    if stream is None:
        stream = _SIDE_STREAMS[index] = torch.cuda.Stream(device=index)
    return stream


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class CompressedLinear(torch.nn.Linear):
    """``torch.nn.Linear`` whose frozen weight is a :class:`CompressedTensor` parameter.

    Args:
        in_features, out_features, bias: as for ``torch.nn.Linear``; the bias is stored uncompressed.
        config: compression configuration; ``None`` picks the lossless scheme for ``dtype``.
        device: device of the bias (compressed buffers stay where the source weight was).
        dtype: container dtype the weight is compressed in.
    """

    state_buffer_names: ClassVar[tuple[str, ...]] = ()
    state_buffer_dtypes: ClassVar[dict[str, torch.dtype]] = {}
    #: When ``forward`` multiplies inside the decode kernel (``_fused_forward``: no dense weight is ever written) instead
    #: of decoding and then multiplying: up to this many tokens and from this many weights on. The fused kernel's steps
    #: carry the product's instructions, so it only wins where the dense weight it avoids would leave L2 on its way to
    #: the product -- measured at 4 bpp: 87 against 91 us for one token on 3840 -> 10240 and 83 against 89 us on
    #: 10240 -> 3840, but 69 against 62 us on 3840 x 3840 and 83 against 65 us there at four tokens. A caller that wants
    #: the weight never materialised sets ``fused_max_tokens = 4`` and ``fused_min_weights = 0`` on the layer or the class.
    fused_max_tokens: ClassVar[int] = 1
    fused_min_weights: ClassVar[int] = 32 << 20

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, config=None,
                 device: str | torch.device | None = None, dtype: torch.dtype = torch.bfloat16):
        with torch.device("meta"):
            super().__init__(in_features, out_features, bias=False, dtype=dtype)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False)
        self.config = config
        self._init_dtype = require_dtype(dtype)
        if config is not None:
            scheme = get_scheme(name_for_config(config))
            if not scheme.supports(self.container_dtype):
                raise ValueError(f"'{scheme.name}' does not support format {self.container_dtype}")
        self.weight = torch.nn.Parameter(torch.zeros(0, dtype=self._init_dtype, device=device), requires_grad=False)
        for name in self.state_buffer_names:
            self.register_buffer(name, torch.zeros(out_features, dtype=self.state_buffer_dtypes[name], device=device), persistent=True)

    # ---- configuration -------------------------------------------------------------------------
    @property
    def _encode_config(self):
        return default_config(self.container_dtype) if self.config is None else dataclasses.replace(self.config)

    @property
    def _decode_config(self):
        return self.weight.scheme.make_config({}) if self.config is None else dataclasses.replace(self.config)

    @property
    def container_dtype(self) -> torch.dtype:
        """The dtype the weight is compressed in; layer casts (``.to(dtype)``) do not change it."""
        return self._init_dtype

    @property
    def qweight(self) -> torch.Tensor:
        """The packed blob, under the attribute name quantisation frameworks look for."""
        return self.weight.entropack_quant_state if isinstance(self.weight, CompressedTensor) else self.bias

    @property
    def stored_nbytes(self) -> int:
        total = self.weight.storage_nbytes()
        for name in self.state_buffer_names:
            buffer = self._buffers.get(name)
            if buffer is not None:
                total += buffer.numel() * buffer.element_size()
        return total

    @property
    def compressed_bits(self) -> float:
        rows, cols = self.weight.shape
        return self.stored_nbytes * 8 / (rows * cols)

    @property
    def device(self) -> torch.device:
        if self.weight is not None:
            return self.weight.device
        return self.bias.device if self.bias is not None else torch.device("meta")

    # ---- compression ---------------------------------------------------------------------------
    def _check_weight_shape(self, shape) -> None:
        expected = (self.out_features, self.in_features)
        if tuple(shape) != expected:
            raise ValueError(f"weight has shape {tuple(shape)}, but the layer expects {expected}")

    def _compress_tensor(self, tensor: torch.Tensor) -> CompressedTensor:
        compressed = compress(tensor.to(self.container_dtype), self._encode_config)
        if compressed.compress_method == "raw" and "reason" in compressed.header:
            raise RuntimeError(
                f"{compressed.header['requested']} cannot store a {tuple(tensor.shape)} {self.container_dtype} weight for "
                f"{type(self).__name__}: {compressed.header['reason']}")
        return compressed

    def compress_weight(self, weight: torch.Tensor) -> None:
        """Compress ``weight`` and make it this layer's weight."""
        self._check_weight_shape(weight.shape)
        self.weight = torch.nn.Parameter(self._compress_tensor(weight.detach()), requires_grad=False)

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, **kwargs) -> "CompressedLinear":
        """A layer of this class holding ``linear``'s weight compressed and a copy of its bias."""
        weight = linear.weight
        if weight is None or weight.device.type == "meta":
            raise ValueError("cannot compress a Linear whose weight is not materialized")
        kwargs.setdefault("dtype", weight.dtype)
        layer = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, device=weight.device, **kwargs)
        layer.compress_weight(weight.data)
        if linear.bias is not None:
            layer.bias = torch.nn.Parameter(linear.bias.data.clone(), requires_grad=False)
        return layer

    # ---- decode and forward ----------------------------------------------------------------------
    def _container(self) -> CompressedTensor:
        if not isinstance(self.weight, CompressedTensor):
            raise RuntimeError(f"{type(self).__name__}({self.in_features}, {self.out_features}) has nothing to decode: "
                               "the weight was not correctly loaded")
        return self.weight

    def dequantize(self, device: str | torch.device | None = None) -> torch.Tensor:
        """The dense weight, decoded on ``device`` (default: where the blob lives)."""
        return decompress(self._container().to(device=device), self._decode_config)

    def _decoded_for_product(self, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
        """What ``decompress`` gives for the container as ``dtype`` on ``device``, for the forward pass: from the third
        call on through a prepared decode (``schemes/lattice_rans/b200.py``), which skips the per-call validation, lane
        look-up and layout parsing of the general path -- they cost more host time than the decode takes on the device.
        The prepared decode is dropped as soon as the layer's container, its storage, its device or its config object
        is another one."""
        held = self.__dict__.get("_prepared")
        container = self.weight
        if held is not None:
            config, prepared = held
            if (prepared is not None and config is self.config and prepared.dtype == dtype and isinstance(container, CompressedTensor)
                    and prepared.valid_for(container.buffers, device)):
                return prepared()
            del self.__dict__["_prepared"]
        dense = decompress(self._container().to(device=device, dtype=dtype), self._decode_config)
        prepared = self._prepare_decode(device, dtype, dense)
        if prepared is not None:
            self.__dict__["_prepared"] = (self.config, prepared)
        return dense

    def _prepare_decode(self, device: torch.device, dtype: torch.dtype, dense: torch.Tensor):
        container = self.weight
        if (container.compress_method != "lattice_rans" or container.device != device or device.type != "cuda"
                or container.encoded_dtype != dtype or tuple(dense.shape) != tuple(container.shape) or not dense.is_contiguous()):
            return None
        from .schemes.base import packed_buffers
        from .schemes.lattice_rans import b200
        from .schemes.lattice_rans.format import LatticeBuffers

        config = self._decode_config
        packed = packed_buffers(container.buffers, LatticeBuffers)
        lane, run_on = container.scheme.lane_for(packed.layout, config.execution_backend, gate_dtype=False)
        if lane is not b200 or run_on != device:
            return None
        prepared = b200.prepared_decode(packed, shape=tuple(container.shape), dtype=dtype)
        if prepared is None or (prepared.rows, prepared.cols) != tuple(container.shape):
            return None
        return prepared

    def _bias_on(self, device: torch.device) -> torch.Tensor | None:
        return None if self.bias is None else self.bias.to(device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ahead = getattr(self, "_decode_ahead", None)
        if ahead is not None:
            pipelined = ahead.forward(self, x)
            if pipelined is not None:
                return pipelined
        if (x.shape[-1] and x.numel() // x.shape[-1] <= self.fused_max_tokens
                and self.in_features * self.out_features >= self.fused_min_weights):
            fused = self._fused_forward(x)
            if fused is not None:
                return fused
        weight = self._decoded_for_product(x.device, self.weight.dtype)
        bias = self._bias_on(x.device)
        if _native_gemm_applies(x, weight, bias):
            return linear_forward(x, weight, bias)
        return F.linear(x, weight.to(x.dtype), bias)

    def _fused_forward(self, x: torch.Tensor) -> torch.Tensor | None:
        """At decode-time batch sizes (up to 4 tokens) a lossy-coded bf16 weight is multiplied while it is being
        decoded, without ever being written out; None when that path does not apply. ``forward`` takes it where it is
        the faster one (``fused_max_tokens``, ``fused_min_weights``)."""
        container = self.weight
        if (type(self) is not CompressedLinear or not isinstance(container, CompressedTensor) or container.compress_method != "lattice_rans"
                or container.encoded_dtype != torch.bfloat16 or container.dtype != torch.bfloat16 or x.dtype != torch.bfloat16
                or not x.is_cuda or container.device != x.device or self.in_features % 8 != 0 or x.numel() == 0
                or (torch.is_grad_enabled() and x.requires_grad)):
            return None
        flat = x.reshape(-1, x.shape[-1])
        lane = container.scheme.lane()
        if flat.shape[0] > lane.MAX_FUSED_TOKENS:
            return None
        from .schemes.base import packed_buffers
        from .schemes.lattice_rans.format import LatticeBuffers

        out = lane.linear_forward(packed_buffers(container.buffers, LatticeBuffers), shape=tuple(container.shape), x=flat,
                                  bias=self._bias_on(x.device))
        return out.reshape(*x.shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        scheme = "auto" if self.config is None else name_for_config(self.config)
        parts = [f"scheme={scheme}", f"container={str(self.container_dtype).removeprefix('torch.')}"]
        if isinstance(self.weight, CompressedTensor):
            parts.append(f"bits={self.compressed_bits:.3f}")
        if self.config is not None:
            parts.append(f"config={type(self.config).__name__}")
        return ", ".join(parts)

    # ---- module plumbing -------------------------------------------------------------------------
    def _apply(self, fn, recurse=True):
        # auxiliary scale buffers keep their dtype when the module is cast
        held = {name: self._buffers.pop(name) for name in self.state_buffer_names if name in self._buffers}
        try:
            super()._apply(fn, recurse=recurse)
        finally:
            for name, buffer in held.items():
                if buffer is None:
                    self._buffers[name] = None
                    continue
                moved = fn(buffer)
                self._buffers[name] = moved if moved.dtype == buffer.dtype else buffer.to(device=moved.device)
        return self

    def _save_to_state_dict(self, destination: dict, prefix: str, keep_vars: bool) -> None:
        super()._save_to_state_dict(destination, prefix, keep_vars)
        if isinstance(self.weight, CompressedTensor):
            destination.pop(prefix + "weight")
            blob = self.weight.entropack_quant_state
            destination[prefix + "weight.entropack_quant_state"] = blob if keep_vars else blob.detach()

    def _load_from_state_dict(self, state_dict: dict, prefix: str, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        key = prefix + "weight.entropack_quant_state"
        if key in state_dict:
            try:
                blob = state_dict[key]
                assign = local_metadata.get("assign_to_params_buffers", False)
                current = self._parameters.get("weight")
                if not assign:
                    if current is not None and current.device.type != "meta":
                        device = current.device
                    elif self.bias is not None and self.bias.device.type != "meta":
                        device = self.bias.device
                    else:
                        device = blob.device
                    blob = blob.to(device=device, copy=True)
                container = CompressedTensor.unpack(blob)
                self._check_weight_shape(container.shape)
                loaded = torch.nn.Parameter(container, requires_grad=False)
                if not assign and isinstance(current, CompressedTensor):
                    torch.utils.swap_tensors(current, loaded)
                else:
                    self._parameters["weight"] = loaded
            except (TypeError, ValueError) as error:
                error_msgs.append(f"{prefix[:-1]}: {error}")
            state_dict.pop(key)
        elif strict:
            missing_keys.append(key)
        weight = self._parameters.pop("weight")
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        self._parameters["weight"] = weight


class _W8A8Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        ctx.layer, ctx.x_shape = layer, x.shape
        return layer._forward8(x.detach())

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_output):
        grad = grad_output.reshape(-1, grad_output.shape[-1])
        weight = ctx.layer.dequantize(grad.device).to(grad.dtype)
        return torch.mm(grad, weight).reshape(ctx.x_shape), None


class QuantizedLinear(CompressedLinear):
    """Base of the 8-bit layers: per-row scaled codes, optionally lattice-coded, 8-bit GEMM at run time."""

    code_dtype: ClassVar[torch.dtype]
    code_max: ClassVar[float]
    rounds_to_integer: ClassVar[bool]
    code_alignment: ClassVar[int]
    min_tokens: ClassVar[int]
    min_capability: ClassVar[tuple[int, int]]
    state_buffer_names = ("weight_quant_scale",)
    state_buffer_dtypes = {"weight_quant_scale": torch.float32}

    def __init__(self, in_features, out_features, bias=True, *, config=None, device=None, dtype=torch.bfloat16):
        super().__init__(in_features, out_features, bias=bias, config=self._coded(config), device=device, dtype=dtype)

    @property
    def container_dtype(self) -> torch.dtype:
        return self.code_dtype

    @classmethod
    def _coded(cls, config):
        if config is None:
            return RawConfig()
        if isinstance(config, RawConfig):
            return config
        if not isinstance(config, EntroPackLossyConfig):
            raise TypeError(f"{cls.__name__} stores {cls.code_dtype} codes: either uncoded (RawConfig) or lattice-coded "
                            f"(EntroPackLossyConfig), got {type(config).__name__}")
        rate = config.target_bpp
        if isinstance(rate, bool) or not isinstance(rate, Real) or not 0.0 < float(rate) < 8.0:
            raise ValueError(f"{cls.__name__} stores {cls.code_dtype} codes, 8 bits wide, so a target_bpp only pays below 8; "
                             f"got {rate!r}. Pass RawConfig to store the codes uncoded.")
        return config

    def _quantize_rows(self, tensor: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        flat = tensor.reshape(-1, tensor.shape[-1]).float()
        scale = (flat.abs().amax(dim=1) / self.code_max).clamp(min=_EPS)
        scaled = flat / scale.unsqueeze(1)
        if self.rounds_to_integer:
            scaled = scaled.round()
        return scaled.clamp(-self.code_max, self.code_max).to(self.code_dtype), scale

    def _prepare_activation(self, flat: torch.Tensor) -> torch.Tensor:
        return flat

    def _prepare_weight_source(self, weight: torch.Tensor) -> torch.Tensor:
        return weight

    def _restore_weight_basis(self, weight: torch.Tensor) -> torch.Tensor:
        return weight

    def compress_weight(self, weight: torch.Tensor) -> None:
        self._check_weight_shape(weight.shape)
        codes, scale = self._quantize_rows(self._prepare_weight_source(weight.detach()))
        self.weight = torch.nn.Parameter(self._compress_tensor(codes), requires_grad=False)
        self.weight_quant_scale = scale

    def codes(self, device: str | torch.device | None = None) -> torch.Tensor:
        """The weight codes in ``code_dtype``, decoded for the 8-bit GEMM."""
        return decompress(self._container().to(device=device, dtype=self.code_dtype), self._decode_config)

    def _scale(self, device: torch.device) -> torch.Tensor:
        return self.weight_quant_scale.to(device=device, dtype=torch.float32)

    def dequantize(self, device: str | torch.device | None = None) -> torch.Tensor:
        codes = self.codes(device)
        return self._restore_weight_basis(codes.float() * self._scale(codes.device).unsqueeze(1)).to(self._init_dtype)

    def _require_8bit_gemm(self, device: torch.device) -> None:
        if device.type != "cuda":
            raise RuntimeError(f"{type(self).__name__} needs a CUDA device with an 8-bit tensor core, compute capability "
                               f"{self.min_capability} or later; got {device}.")
        capability = torch.cuda.get_device_capability(device)
        if capability < self.min_capability:
            raise RuntimeError(f"{type(self).__name__} needs compute capability {self.min_capability} or later and "
                               f"{torch.cuda.get_device_name(device)} reports {capability}.")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._require_8bit_gemm(x.device)
        if x.requires_grad:
            return _W8A8Function.apply(x, self)
        ahead = getattr(self, "_decode_ahead", None)
        if ahead is not None:
            pipelined = ahead.forward(self, x)
            if pipelined is not None:
                return pipelined
        return self._forward8(x)

    def _forward8(self, x: torch.Tensor, codes: torch.Tensor | None = None) -> torch.Tensor:
        """``codes``: the weight codes where the caller has decoded them already (decode-ahead)."""
        flat = self._prepare_activation(x.reshape(-1, x.shape[-1]))
        beside = (codes is None and flat.is_cuda and flat.shape[0] >= self.beside_decode_tokens
                  and not isinstance(self.config, RawConfig))
        if beside:
            # the activations are quantised on a second stream while the weight codes are decoded on this one: the
            # decode is a latency-bound chain that leaves most of an SM's issue slots and all of its memory bandwidth idle
            flat = flat.contiguous()       # a copy, if one is needed, is made before the second stream is let go
            current, side = torch.cuda.current_stream(flat.device), _side_stream(flat.device)
            side.wait_stream(current)
            activation, scale = self._quantize_activations(flat.detach(), stream=side)
            codes = self._decoded_for_product(x.device, self.code_dtype)
            current.wait_stream(side)
        else:
            activation, scale = self._quantize_activations(flat.detach())
        if codes is None:
            codes = self._decoded_for_product(x.device, self.code_dtype)
        weight_scale = self._scale(codes.device)
        tokens = activation.shape[0]
        rows = max(tokens, self.min_tokens)
        outs = _round_up(self.out_features, self.code_alignment)
        cols = _round_up(self.in_features, self.code_alignment)
        out = self._gemm(_pad_to(_pad_to(activation, 0, rows), 1, cols), _pad_to(_pad_to(codes, 0, outs), 1, cols),
                         _pad_to(scale, 0, rows), _pad_to(weight_scale, 0, outs), x.dtype)
        return out[:tokens, : self.out_features].reshape(*x.shape[:-1], self.out_features)

    def _bias_padded(self, device: torch.device, columns: int) -> torch.Tensor | None:
        bias = self._bias_on(device)
        return None if bias is None else _pad_to(bias, 0, columns)

    #: names of the library's activation quantiser and scaled 8-bit product for this code type
    quantize_entry: ClassVar[str]
    gemm_entry: ClassVar[str]

    #: from this many tokens on, a coded layer quantises its activations beside the weight decode (below it the host's
    #: two extra event hand-overs cost more than the few microseconds the quantiser takes)
    beside_decode_tokens: ClassVar[int] = 1024

    def _quantize_activations(self, tensor: torch.Tensor, stream: "torch.cuda.Stream | None" = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Weights (once, at compression time) go through the torch expression of ``_quantize_rows``; activations on a
        GPU, every forward, through one kernel that computes the same scale and the same codes. ``stream``: where the
        kernel is launched (the caller orders it against the current stream, on which the results are allocated)."""
        kind = _SOURCE_KINDS.get(tensor.dtype)
        if not tensor.is_cuda or kind is None or tensor.numel() == 0:
            return self._quantize_rows(tensor)
        flat = tensor.reshape(-1, tensor.shape[-1]).contiguous()
        codes = torch.empty(flat.shape, dtype=self.code_dtype, device=flat.device)
        scale = torch.empty(flat.shape[0], dtype=torch.float32, device=flat.device)
        with torch.cuda.device(flat.device):
            status = getattr(_native.load(), self.quantize_entry)(
                _native.ptr(flat), kind, flat.shape[0], flat.shape[1], _native.ptr(codes), _native.ptr(scale),
                stream.cuda_stream if stream is not None else _native.stream_handle(flat.device))
        _native.check(status, "8-bit activation quantisation")
        return codes, scale

    def _gemm(self, activation, codes, activation_scale, weight_scale, out_dtype):
        """Scaled 8-bit product on the library's tcgen05 kernel (bf16 or fp32 results; fp16 goes through fp32)."""
        bias = self._bias_padded(codes.device, weight_scale.shape[0])
        direct = out_dtype in (torch.bfloat16, torch.float32)
        out = torch.empty((activation.shape[0], codes.shape[0]), dtype=out_dtype if direct else torch.float32, device=codes.device)
        activation, codes = activation.contiguous(), codes.contiguous()
        activation_scale, weight_scale = activation_scale.contiguous(), weight_scale.contiguous()
        bias32 = None if bias is None else bias.float().contiguous()   # held until after the launch
        with torch.cuda.device(codes.device):
            status = getattr(_native.load(), self.gemm_entry)(
                _native.ptr(activation), _native.ptr(codes), _native.ptr(activation_scale), _native.ptr(weight_scale),
                _native.ptr(bias32), _native.ptr(out), int(out.dtype == torch.float32), activation.shape[0], codes.shape[0],
                activation.shape[1], _native.ptr(kernel_error_word(codes.device)), _native.stream_handle(codes.device))
        _native.check(status, "8-bit linear forward")
        return out if direct else out.to(out_dtype)


class CompressedFP8Linear(QuantizedLinear):
    """FP8 E4M3 weights and activations with per-row scales; codes stored raw or lattice-coded below 8 bpp."""

    code_dtype = torch.float8_e4m3fn
    code_max = float(torch.finfo(torch.float8_e4m3fn).max)
    rounds_to_integer = False
    code_alignment = 16
    min_tokens = 1
    min_capability = (10, 0)

    quantize_entry = "ep_quantize_rows_fp8"
    gemm_entry = "ep_linear_forward_fp8"


class CompressedINT8Linear(QuantizedLinear):
    """Symmetric INT8 weights and activations with per-row scales, multiplied on the library's ``kind::i8`` tensor-core
    kernel. ``use_convrot`` rotates the weight before quantisation and the activations before theirs (the flag is not
    stored in the checkpoint, as in the reference)."""

    code_dtype = torch.int8
    code_max = 127.0
    rounds_to_integer = True
    code_alignment = 16     # the tensor-core kernel takes K in multiples of 16 bytes
    min_tokens = 1          # (the reference pads to 17 rows for torch._int_mm; this kernel has no such floor)
    min_capability = (10, 0)

    def __init__(self, in_features, out_features, bias=True, *, config=None, device=None, dtype=torch.bfloat16,
                 use_convrot: bool = False, convrot_groupsize: int = 256):
        self.use_convrot = bool(use_convrot)
        self._convrot_group = choose_convrot_group(in_features, convrot_groupsize) if self.use_convrot else None
        if self.use_convrot and self._convrot_group is None:
            raise ValueError(f"use_convrot requires in_features {in_features} to contain a power-of-four group; "
                             f"got convrot_groupsize={convrot_groupsize}")
        super().__init__(in_features, out_features, bias=bias, config=config, device=device, dtype=dtype)

    def _prepare_activation(self, flat: torch.Tensor) -> torch.Tensor:
        return rotate_activation(flat, self._convrot_group) if self.use_convrot else flat

    def _prepare_weight_source(self, weight: torch.Tensor) -> torch.Tensor:
        return rotate_weight(weight, self._convrot_group) if self.use_convrot else weight

    def _restore_weight_basis(self, weight: torch.Tensor) -> torch.Tensor:
        return rotate_weight(weight, self._convrot_group, inverse=True) if self.use_convrot else weight

    quantize_entry = "ep_quantize_rows_int8"
    gemm_entry = "ep_linear_forward_int8"


__all__ = ["CompressedFP8Linear", "CompressedINT8Linear", "CompressedLinear", "QuantizedLinear", "check_kernel_errors"]
