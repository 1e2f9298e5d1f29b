"""Compressed linear layers: API, checkpoint format, forward numerics (GEMM outputs within bf16 tolerance)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import buffers_of, load_golden

pytestmark = pytest.mark.gpu


def _relative(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


@pytest.mark.parametrize("tokens", [1, 16, 256])
def test_compressed_linear_forward_matches_dense_on_decoded_weight(tokens):
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(6)
    dense = torch.nn.Linear(3840, 1536, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(1536, 3840, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    layer = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0))
    assert abs(layer.compressed_bits - 4.0) < 0.05
    x = torch.randn(tokens, 3840, generator=g, device="cuda").to(torch.bfloat16)
    weight = layer.dequantize()
    assert weight.shape == dense.weight.shape and weight.dtype == torch.bfloat16
    expected = torch.nn.functional.linear(x.float(), weight.float(), dense.bias.float())
    assert _relative(layer(x), expected) <= 1e-2
    # and the lossy weight is close to the original (about 7 % relative L2 at 4 bpp)
    assert float((weight.float() - dense.weight.float()).norm() / dense.weight.float().norm()) < 0.09


def test_decode_plans_of_a_model_are_built_up_front():
    """``prepare_decode_plans`` gives every compressed layer of a module its kept decode tables before the first pass;
    a pass with them gives what a pass of freshly compressed layers gives, which build their tables on the way."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(8)

    def make():
        layers = []
        for index, (out_features, in_features, config) in enumerate((
                (512, 1024, ep.EntroPackLossyConfig(target_bpp=4.0)), (768, 512, ep.EntroPackLossyConfig(target_bpp=6.0)),
                (256, 768, ep.DFloat11Config()), (512, 256, ep.TileANSConfig()))):
            dense = torch.nn.Linear(in_features, out_features, bias=index % 2 == 0, device="cuda", dtype=torch.bfloat16)
            with torch.no_grad():
                dense.weight.copy_((torch.randn(out_features, in_features, generator=torch.Generator(device="cuda").manual_seed(index),
                                                device="cuda") * 0.02).to(torch.bfloat16))
                if dense.bias is not None:
                    dense.bias.zero_()
            layers.append(ep.CompressedLinear.from_linear(dense, config=config))
        return torch.nn.Sequential(*layers)

    prepared, plain = make(), make()
    assert ep.prepare_decode_plans(prepared) == 3          # two lossy containers and the DFloat11 one; Tile-ANS keeps no plan
    assert ep.prepare_decode_plans(prepared) == 0          # nothing left to build
    for layer in list(prepared)[:2]:
        assert getattr(layer.weight.buffers["layout"], "_lattice_rans_slot_tables", None) is not None
    assert getattr(prepared[2].weight.buffers["layout"], "_dfloat11_decode_tables", None) is not None
    for tokens in (2, 300):
        x = torch.randn(tokens, 1024, generator=g, device="cuda").to(torch.bfloat16)
        assert torch.equal(prepared(x), plain(x))
    ep.check_kernel_errors()


def test_decode_ahead_gives_the_layers_own_outputs():
    """With ``DecodeAhead`` a layer's weight is decoded on a second stream while the layer before it multiplies (on a
    share of the SMs each); outputs are bit for bit those of the plain layers, in order, out of order, with layers in
    the list that it does not handle, and from a CUDA graph captured after a first pass."""
    import entropack_b200 as ep

    def make(out_features, in_features, config, bias, seed):
        dense = torch.nn.Linear(in_features, out_features, bias=bias, device="cuda", dtype=torch.bfloat16)
        with torch.no_grad():
            dense.weight.copy_((torch.randn(out_features, in_features, generator=torch.Generator(device="cuda").manual_seed(seed),
                                            device="cuda") * 0.02).to(torch.bfloat16))
        return ep.CompressedLinear.from_linear(dense, config=config)

    def make8(cls, seed):
        dense = torch.nn.Linear(1024, 1024, bias=seed % 2 == 0, device="cuda", dtype=torch.bfloat16)
        with torch.no_grad():
            dense.weight.copy_((torch.randn(1024, 1024, generator=torch.Generator(device="cuda").manual_seed(seed), device="cuda")
                                * 0.02).to(torch.bfloat16))
        return cls.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=5.0))

    lossy = ep.EntroPackLossyConfig(target_bpp=4.0)
    layers = [make(1024, 1024, lossy, True, 0), make(1536, 1024, lossy, False, 1), make(1024, 1536, lossy, True, 2),
              make(1024, 1024, ep.DFloat11Config(), False, 3), make(1024, 1024, ep.EntroPackLossyConfig.low_latency(4.0), True, 4),
              make8(ep.CompressedFP8Linear, 5), make8(ep.CompressedINT8Linear, 6), make8(ep.CompressedFP8Linear, 7)]
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(300, 1024, generator=g, device="cuda").to(torch.bfloat16)

    def run(order=range(len(layers))):
        outputs, h = [], x
        for index in order:
            h = layers[index](h)
            outputs.append(h)
        return outputs

    with torch.no_grad():
        expected = run()
        expected_few = {}
        for tokens in (8, 2):
            h = x[:tokens]
            for index in range(3):
                h = layers[index](h)
            expected_few[tokens] = h
        with ep.DecodeAhead(layers) as ahead:
            for _ in range(3):
                for got, want in zip(run(), expected):
                    assert torch.equal(got, want)
            assert ahead.decoded_ahead >= 15        # every pass: layers 1, 2, 5, 6 and 7; the later ones: layer 0 as well
            # a few tokens: the product's blocks share the SMs with the next layer's decode; eight tokens take the same
            # kernels with and without (bit-equal), and so do two (layers of this size no longer take the fused kernel)
            h8, h2 = x[:8], x[:2]
            for index in range(3):
                h8, h2 = layers[index](h8), layers[index](h2)
            assert torch.equal(h8, expected_few[8]) and _relative(h2, expected_few[2]) < 1e-2
            # out of order: a layer whose weight was not the one decoded ahead decodes it itself
            h = layers[2](expected[1])
            assert torch.equal(h, expected[2])
            h = layers[0](x)
            assert torch.equal(h, expected[0])
            # a captured pass
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                run()
                ahead.drain()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    captured = run()
                    ahead.drain()
            torch.cuda.current_stream().wait_stream(stream)
            for _ in range(2):
                graph.replay()
                torch.cuda.synchronize()
                for got, want in zip(captured, expected):
                    assert torch.equal(got, want)
        assert all(getattr(layer, "_decode_ahead", None) is None for layer in layers)
        for got, want in zip(run(), expected):
            assert torch.equal(got, want)
    ep.check_kernel_errors()


def test_lossless_default_config_round_trips_exactly():
    import entropack_b200 as ep

    dense = torch.nn.Linear(512, 384, bias=False, device="cuda", dtype=torch.bfloat16)
    layer = ep.CompressedLinear.from_linear(dense)
    assert layer.weight.compress_method == "dfloat11"
    assert torch.equal(layer.dequantize().view(torch.int16), dense.weight.view(torch.int16))
    # The weights are bit-exact; the product is not compared bit for bit with cuBLAS, whose summation order differs:
    # both must sit within one bf16 rounding step (2^-8 relative, 2^-7 allowed) of the fp32 product.
    x = torch.randn(8, 512, device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(5))
    exact = torch.nn.functional.linear(x.float(), dense.weight.float())
    for produced in (layer(x), dense(x)):
        assert produced.dtype == torch.bfloat16
        assert bool(((produced.float() - exact).abs() <= 2.0 ** -7 * exact.abs() + 1e-3).all())


def test_state_dict_round_trip_and_reference_checkpoint_loads():
    import entropack_b200 as ep

    dense = torch.nn.Linear(256, 64, bias=True, device="cuda", dtype=torch.bfloat16)
    layer = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0))
    state = layer.state_dict()
    assert set(state) == {"weight.entropack_quant_state", "bias"}
    fresh = ep.CompressedLinear(256, 64, bias=True, config=ep.EntroPackLossyConfig(target_bpp=4.0), device="cuda")
    fresh.load_state_dict(state)
    assert torch.equal(fresh.dequantize().view(torch.int16), layer.dequantize().view(torch.int16))
    # a blob written by the reference (golden fixture, 64 x 256 bf16 at 4 bpp) loads and decodes to its bytes
    record = load_golden("lattice_bf16_4p0")
    reference_state = {"weight.entropack_quant_state": torch.from_numpy(record["blob"].copy()), "bias": torch.zeros(64, dtype=torch.bfloat16)}
    fresh.load_state_dict(reference_state)
    decoded = fresh.dequantize()
    assert decoded.cpu().contiguous().view(torch.uint8).numpy().tobytes() == record["decoded_bytes"].tobytes()


@pytest.mark.parametrize("tokens", [1, 16, 256, 2048])      # 2048: activations quantised beside the weight decode
def test_fp8_linear_forward(tokens):
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(7)
    dense = torch.nn.Linear(1024, 768, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(768, 1024, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    layer = ep.CompressedFP8Linear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=5.0))
    assert set(layer.state_dict()) == {"weight.entropack_quant_state", "bias", "weight_quant_scale"}
    assert layer.codes().dtype == torch.float8_e4m3fn
    x = torch.randn(tokens, 1024, generator=g, device="cuda").to(torch.bfloat16)
    out = layer(x)
    # reference formula on the decoded codes: per-token fp8 activations, fp32 accumulate, row/col scales, bias
    codes = layer.codes().float()
    a_scale = (x.float().abs().amax(dim=1) / 448.0).clamp(min=torch.finfo(torch.float32).eps)
    a_codes = (x.float() / a_scale.unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    expected = (a_codes @ codes.t()) * a_scale.unsqueeze(1) * layer.weight_quant_scale.unsqueeze(0) + dense.bias.float()
    assert _relative(out, expected) <= 1e-2
    assert _relative(out, dense(x)) < 0.08


def test_int8_linear_forward_and_unsupported_rotation():
    import entropack_b200 as ep

    dense = torch.nn.Linear(512, 256, bias=False, device="cuda", dtype=torch.bfloat16)
    layer = ep.CompressedINT8Linear.from_linear(dense)
    x = torch.randn(32, 512, device="cuda", dtype=torch.bfloat16)
    assert _relative(layer(x), dense(x)) < 0.05


@pytest.mark.parametrize("features,group", [(512, 256), (320, 64), (48, 16), (12, 4)])
def test_convrot_kernel_is_the_reference_rotation(features, group):
    """The butterfly passes against the dense Kronecker matrix (fp32: 1e-5 of the largest value), its self-inverse
    property, and the group chosen for each width."""
    from entropack_b200 import convrot

    assert convrot.choose_convrot_group(features) == group
    generator = torch.Generator(device="cuda").manual_seed(8)
    x = torch.randn(37, features, generator=generator, device="cuda")
    matrix = convrot.build_convrot_matrix(group, device="cuda")
    expected = (x.reshape(37, features // group, group) @ matrix).reshape(37, features)
    rotated = convrot.rotate_activation(x, group)
    assert float((rotated - expected).abs().max()) <= 1e-5 * float(expected.abs().max())
    assert float((convrot.rotate_weight(rotated, group, inverse=True) - x).abs().max()) <= 1e-5 * float(x.abs().max())
    half = convrot.rotate_activation(x.to(torch.bfloat16), group)
    assert half.dtype == torch.bfloat16 and float((half.float() - expected).abs().max()) <= 2.0 ** -7 * float(expected.abs().max())


def test_int8_linear_with_convrot_tames_outlier_channels():
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(9)
    dense = torch.nn.Linear(1024, 256, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        weight = torch.randn(256, 1024, generator=g, device="cuda") * 0.02
        weight[:, 7] *= 40.0          # one input channel dominates every row's scale
        dense.weight.copy_(weight.to(torch.bfloat16))
    x = torch.randn(64, 1024, generator=g, device="cuda").to(torch.bfloat16)
    plain = ep.CompressedINT8Linear.from_linear(dense)
    rotated = ep.CompressedINT8Linear.from_linear(dense, use_convrot=True)
    assert rotated._convrot_group == 256 and set(rotated.state_dict()) == set(plain.state_dict())
    exact = dense(x)
    # the rotation spreads the outlier channel over its group: finer weight codes, smaller error
    assert _relative(rotated(x), exact) < _relative(plain(x), exact) < 0.2
    assert _relative(rotated.dequantize(), dense.weight) < 0.02
    with pytest.raises(ValueError):
        ep.CompressedINT8Linear(514, 256, use_convrot=True)


@pytest.mark.parametrize("tokens,features,bias", [(1, 3840, True), (3, 1536, False), (4, 264, True), (2, 1024, True)])
def test_fused_small_batch_forward_matches_product_with_decoded_weight(tokens, features, bias):
    """Up to 4 tokens the lossy-coded layer multiplies while it decodes (no dense weight is written). The result must
    be the product with the decoded bf16 weight: fp32 sums in another order, then one bf16 rounding, 2^-7 relative to
    the largest output."""
    import entropack_b200 as ep
    from entropack_b200.schemes.base import packed_buffers
    from entropack_b200.schemes.lattice_rans.format import LatticeBuffers

    g = torch.Generator(device="cuda").manual_seed(21)
    dense = torch.nn.Linear(features, 520, bias=bias, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(520, features, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    layer = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0))
    x = torch.randn(2, tokens // 2 if tokens % 2 == 0 else tokens, features, generator=g, device="cuda").to(torch.bfloat16)
    x = x[:1] if tokens % 2 else x        # [1, tokens, K] or [2, tokens / 2, K]: leading dimensions are flattened
    weight = layer.dequantize()
    expected = torch.nn.functional.linear(x.float(), weight.float(), None if not bias else dense.bias.float())
    # the kernel itself, then the layer's own choice (a layer this small decodes and multiplies in turn), then the layer
    # told to multiply while it decodes whatever its size
    for out in (layer._fused_forward(x), layer(x)):
        assert out is not None and out.shape == expected.shape and out.dtype == torch.bfloat16
        assert float((out.float() - expected).abs().max() / expected.abs().max()) <= 2.0 ** -7
    layer.fused_max_tokens, layer.fused_min_weights = 4, 0
    assert torch.equal(layer(x), layer._fused_forward(x))
    # the error word stays clear and five tokens take the two-kernel path
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    lane = layer.weight.scheme.lane()
    lane.linear_forward(packed_buffers(layer.weight.buffers, LatticeBuffers), shape=tuple(layer.weight.shape), x=x.reshape(-1, features),
                        bias=None, error=error)
    assert int(error.item()) == 0
    assert layer._fused_forward(torch.zeros(5, features, device="cuda", dtype=torch.bfloat16)) is None


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
def test_prepared_decode_follows_the_layers_container(kind):
    """From a container's third decode on, a layer's forward decodes through a prepared call (pointers and sizes kept
    from the general path). It must give the same bytes, and must be dropped when the layer gets another weight, is
    copied, or has its state loaded."""
    import copy

    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(31)
    cls = ep.CompressedLinear if kind == "bf16" else ep.CompressedFP8Linear
    config = ep.EntroPackLossyConfig(target_bpp=4.0 if kind == "bf16" else 5.0)

    def dense_layer():
        dense = torch.nn.Linear(1024, 768, bias=True, device="cuda", dtype=torch.bfloat16)
        with torch.no_grad():
            dense.weight.copy_((torch.randn(768, 1024, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
        return dense

    first, second = dense_layer(), dense_layer()
    layer = cls.from_linear(first, config=config)
    x = torch.randn(48, 1024, generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        outputs = [layer(x) for _ in range(4)]
        assert layer.__dict__.get("_prepared") is not None          # the last calls went through it
        assert all(torch.equal(outputs[0], later) for later in outputs[1:])
        assert _relative(outputs[0], first(x)) < 0.08
        state = copy.deepcopy(layer.state_dict())
        twin = copy.deepcopy(layer)
        assert torch.equal(twin(x), outputs[0])
        layer.compress_weight(second.weight.data)
        replaced = [layer(x) for _ in range(4)]
        assert all(torch.equal(replaced[0], later) for later in replaced[1:])
        assert not torch.equal(replaced[0], outputs[0]) and _relative(replaced[0], F.linear(x, second.weight, first.bias)) < 0.08
        layer.load_state_dict(state)
        assert all(torch.equal(layer(x), outputs[0]) for _ in range(4))
        assert torch.equal(twin(x), outputs[0])


def test_fp8_layer_with_activations_quantised_beside_the_decode_captures_into_a_graph():
    """From 1024 tokens on the 8-bit layers quantise their activations on a second stream while the weight codes are
    decoded. Captured into a CUDA graph the second stream must fork from and join the capturing one: the replay gives
    the eager call's bytes."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(17)
    dense = torch.nn.Linear(1024, 768, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(768, 1024, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    layer = ep.CompressedFP8Linear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=5.0))
    x = torch.randn(1536, 1024, generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        eager = [layer(x) for _ in range(3)][-1]          # the container's decode plan and prepared decode exist now
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                captured = layer(x)
        torch.cuda.current_stream().wait_stream(stream)
        captured.zero_()
        graph.replay()
        torch.cuda.synchronize()
    assert torch.equal(captured, eager)
    ep.check_kernel_errors()
