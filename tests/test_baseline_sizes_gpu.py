"""Parity at the benchmark sizes: the GPU kernels against the CPU oracle on the very tensors the benchmark
configurations name, through the C ABI (lanes) and the public API.

* lossy 4096 x 11008 bf16 with 41 heavy-tailed rows at 2.3 / 3.5 / 4.0 / 6.0 bpp: the GPU container equals the
  oracle's buffer for buffer, the GPU decode equals the oracle's bytes, and the stored rate sits within 0.01 bpp of
  what the reference's own encoder stored for that tensor (``golden/baseline_lossy_scalars.json``, written by
  ``golden/make_golden.py --only baseline`` from the imported reference);
* DFloat11 4096 x 4096 bf16 and Tile-ANS 8192 x 8192 fp8 / fp32: containers equal the oracle's, and each side
  decodes the other's;
* the compressed layers at 4096 tokens on the benchmark's layer shapes, against the fp32 product.
"""
import hashlib
import json

import numpy as np
import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


def _bytes(tensor: torch.Tensor) -> bytes:
    return tensor.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes()


def baseline_lossy_weight(rows, cols, seed, outliers):
    """Same construction as ``golden/make_golden.py:baseline_lossy_weight`` (checked through the input checksum)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    if outliers:
        picks = torch.randperm(rows, generator=g)[:outliers]
        heavy = torch.randn(outliers, cols, generator=g) / torch.sqrt(torch.randn(outliers, cols, 3, generator=g).square().mean(-1))
        w[picks] = heavy * 0.02
    return w.to(torch.bfloat16)


@pytest.fixture(scope="module")
def lossy_case():
    record = json.loads((GOLDEN / "baseline_lossy_scalars.json").read_text())
    weight = baseline_lossy_weight(record["rows"], record["cols"], record["seed"], record["outliers"])
    digest = hashlib.sha256(weight.view(torch.uint8).numpy().tobytes()).hexdigest()
    assert digest == record["input_sha256"], "this machine's seeded tensor is not the one the reference's scalars were taken on"
    return record, weight


@pytest.mark.parametrize("bpp", [2.3, 3.5, 4.0, 6.0])
def test_lossy_full_size_container_and_decode_equal_the_oracle(oracle_module, lossy_case, bpp):
    import entropack_b200 as ep
    from entropack_b200.schemes.lattice_rans import b200
    from entropack_b200.schemes.lattice_rans.format import LatticeBuffers

    record, weight = lossy_case
    reference = record["rates"][str(bpp)]
    config = ep.EntroPackLossyConfig(target_bpp=bpp)
    compressed = ep.compress(weight.cuda(), config)
    assert compressed.compress_method == "lattice_rans"
    ours = {key: value.cpu().numpy() for key, value in compressed.buffers.items()}
    expected = oracle_module.lattice_encode(weight.float().numpy(), bpp)
    expected.pop("_search_scale")
    for key in LatticeBuffers._fields:
        assert np.array_equal(ours[key], expected[key]), f"{bpp} bpp: buffer {key} differs from the oracle's"
    # the reference's own numbers for this tensor: same table width and tiling, rate within 0.01 bpp (no slack)
    assert int(ours["layout"][1]) == reference["prob_bits"] and int(ours["layout"][2]) == reference["tile_elements"]
    assert abs(compressed.actual_bpp - reference["actual_bpp"]) <= 0.01
    restored = ep.decompress(compressed, config)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    lane_out = b200.decode(LatticeBuffers(**compressed.buffers), shape=tuple(weight.shape), dtype=torch.bfloat16, error=error)
    assert int(error.item()) == 0 and torch.equal(lane_out.view(torch.int16), restored.view(torch.int16))
    decoded = oracle_module.lattice_decode(ours, tuple(weight.shape), torch.bfloat16)
    assert _bytes(restored) == _bytes(decoded), f"{bpp} bpp: GPU decode differs from the oracle's"
    relative = float((restored.float().cpu() - weight.float()).norm() / weight.float().norm())
    assert relative <= reference["rel_l2"] * 1.002


def test_dfloat11_full_size_against_the_oracle(oracle_module):
    import entropack_b200 as ep
    from entropack_b200.schemes.dfloat11 import b200
    from entropack_b200.schemes.dfloat11.format import DFloat11Buffers

    weight = (torch.randn(4096, 4096, generator=torch.Generator().manual_seed(0)) * 0.02).to(torch.bfloat16)
    bits = weight.reshape(-1).view(torch.int16).numpy().view(np.uint16)
    config = ep.DFloat11Config()
    compressed = ep.compress(weight.cuda(), config)
    assert compressed.compress_method == "dfloat11"
    ours = {key: value.cpu().numpy() for key, value in compressed.buffers.items()}
    expected = oracle_module.dfloat11_encode(bits)
    for key in DFloat11Buffers._fields:
        assert np.array_equal(ours[key], expected[key]), f"buffer {key} differs from the oracle's"
    assert np.array_equal(oracle_module.dfloat11_decode(ours), bits)
    assert np.array_equal(oracle_module.dfloat11_decode(ours, use_regions=True), bits)
    restored = ep.decompress(compressed, config)
    assert torch.equal(restored.view(torch.int16).cpu(), weight.view(torch.int16))
    theirs = DFloat11Buffers(**{key: torch.from_numpy(np.ascontiguousarray(expected[key])).cuda() for key in DFloat11Buffers._fields})
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    decoded = b200.decode(theirs, error=error)
    assert int(error.item()) == 0
    assert np.array_equal(decoded.view(torch.int16).cpu().numpy().view(np.uint16), bits), "GPU decode of the oracle's container differs"


def _lossless_tensor(kind):
    seeds = {"fp8_e4m3": 1, "fp32": 4}
    x = torch.randn(8192, 8192, generator=torch.Generator().manual_seed(seeds[kind]))
    if kind == "fp8_e4m3":
        return (x * (448.0 / x.abs().max())).to(torch.float8_e4m3fn)
    return x * 0.02


@pytest.mark.parametrize("kind", ["fp8_e4m3", "fp32"])
def test_tile_ans_full_size_against_the_oracle(oracle_module, kind):
    import entropack_b200 as ep
    from entropack_b200.schemes.tile_ans import b200
    from entropack_b200.schemes.tile_ans.format import TileBuffers

    tensor = _lossless_tensor(kind)
    raw = tensor.view(torch.uint8).numpy().reshape(-1)
    config = ep.TileANSConfig()
    compressed = ep.compress(tensor.cuda(), config)
    assert compressed.compress_method == "tile_ans"
    ours = {key: value.cpu().numpy() for key, value in compressed.buffers.items()}
    expected = oracle_module.tile_ans_encode(raw, tensor.element_size(), int(ours["layout"][0]))
    for key in TileBuffers._fields:
        assert np.array_equal(ours[key], expected[key]), f"{kind}: buffer {key} differs from the oracle's"
    assert np.array_equal(oracle_module.tile_ans_decode(ours), raw), f"{kind}: the oracle cannot decode the GPU container"
    theirs = TileBuffers(**{key: torch.from_numpy(np.ascontiguousarray(expected[key])).cuda() for key in TileBuffers._fields})
    decoded = b200.decode(theirs, dtype=tensor.dtype, threads_per_block=None)
    assert np.array_equal(decoded.cpu().view(torch.uint8).numpy().reshape(-1), raw), f"{kind}: GPU decode of the oracle's container differs"
    assert torch.equal(ep.decompress(compressed, config).view(torch.uint8).cpu().reshape(-1), torch.from_numpy(raw))


def _relative(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


@pytest.mark.parametrize("out_features,in_features", [(3840, 3840), (10240, 3840)])
def test_compressed_linear_at_4096_tokens_on_the_benchmark_shapes(out_features, in_features):
    """bf16 layer at 4 bpp: decode + tensor-core product against the fp32 product with the decoded weight, 1e-2 of the
    largest output (the benchmark's GEMM tolerance)."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(6)
    dense = torch.nn.Linear(in_features, out_features, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(out_features, in_features, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    layer = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0))
    x = torch.randn(4096, in_features, generator=g, device="cuda").to(torch.bfloat16)
    weight = layer.dequantize()
    expected = torch.nn.functional.linear(x.float(), weight.float(), dense.bias.float())
    out = layer(x)
    assert out.shape == (4096, out_features) and out.dtype == torch.bfloat16
    assert _relative(out, expected) <= 1e-2


@pytest.mark.parametrize("out_features,in_features", [(3840, 3840), (10240, 3840)])
def test_fp8_linear_at_4096_tokens_on_the_benchmark_shapes(out_features, in_features):
    """FP8 codes lattice-coded at 5 bpp: quantised activations x decoded codes with row and column scales, against
    the same formula in fp32, 1e-2 of the largest output."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(7)
    dense = torch.nn.Linear(in_features, out_features, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(out_features, in_features, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    layer = ep.CompressedFP8Linear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=5.0))
    assert abs(layer.weight.actual_bpp - 5.0) < 0.06
    x = torch.randn(4096, in_features, generator=g, device="cuda").to(torch.bfloat16)
    out = layer(x)
    codes = layer.codes().float()
    a_scale = (x.float().abs().amax(dim=1) / 448.0).clamp(min=torch.finfo(torch.float32).eps)
    a_codes = (x.float() / a_scale.unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    expected = (a_codes @ codes.t()) * a_scale.unsqueeze(1) * layer.weight_quant_scale.unsqueeze(0) + dense.bias.float()
    assert out.shape == (4096, out_features)
    assert _relative(out, expected) <= 1e-2
    assert _relative(out, dense(x)) < 0.08
