"""EntroPack-Lossy kernels against the golden fixtures and the CPU oracle (bit-exact), through the C ABI."""
import ast

import numpy as np
import pytest
import torch

from conftest import buffers_of, golden_names, load_golden

pytestmark = pytest.mark.gpu


def _to_device(buffers: dict):
    from entropack_b200.schemes.lattice_rans.format import LatticeBuffers

    keys = LatticeBuffers._fields
    return LatticeBuffers(**{key: torch.from_numpy(np.ascontiguousarray(buffers[key])).cuda() for key in keys})


def _bytes(tensor: torch.Tensor) -> bytes:
    return tensor.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes()


def _gpu_decode(buffers: dict, shape, dtype) -> torch.Tensor:
    from entropack_b200.schemes.lattice_rans import b200

    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = b200.decode(_to_device(buffers), shape=shape, dtype=dtype, error=error)
    assert int(error.item()) == 0
    return out[:, : shape[1]]


@pytest.mark.parametrize("name", golden_names("lattice_"))
def test_decode_reference_bitstreams(name):
    record = load_golden(f"lattice_{name}")
    dtype = getattr(torch, str(record["dtype"]))
    shape = tuple(int(v) for v in record["shape"])
    decoded = _gpu_decode(buffers_of(record), shape, dtype)
    assert _bytes(decoded) == record["decoded_bytes"].tobytes()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float8_e4m3fn, torch.float8_e5m2, torch.int8, torch.uint8,
                                   torch.int16, torch.int32, torch.int64, torch.bool, torch.float8_e4m3fnuz])
def test_every_container_cast_matches_oracle(oracle_module, dtype):
    """One reference bitstream decoded into every container dtype, with scales blown up so the
    saturating casts are exercised."""
    record = load_golden("lattice_bf16_6p0_outliers")
    buffers = buffers_of(record)
    buffers["scales"] = (buffers["scales"] * np.float32(3000.0 if dtype not in (torch.bool,) else 30.0)).astype(np.float32)
    shape = tuple(int(v) for v in record["shape"])
    expected = oracle_module.lattice_decode(buffers, shape, dtype)
    decoded = _gpu_decode(buffers, shape, dtype)
    assert _bytes(decoded) == _bytes(expected)


@pytest.mark.parametrize("name", golden_names("lattice_"))
def test_encode_matches_oracle_bit_for_bit(oracle_module, name):
    """Same input -> the GPU encoder and the CPU oracle produce identical containers (every buffer)."""
    from entropack_b200.schemes.lattice_rans import b200
    from entropack_b200.schemes.lattice_rans.format import recommended_tile_elements

    record = load_golden(f"lattice_{name}")
    dtype = getattr(torch, str(record["dtype"]))
    shape = tuple(int(v) for v in record["shape"])
    options = ast.literal_eval(str(record["options"]))
    source = torch.from_numpy(record["input_bytes"].copy()).view(dtype).reshape(shape)
    pad = -shape[1] % 8
    if pad:
        source = torch.cat([source, source.new_zeros(shape[0], pad)], dim=1)
    target = min(float(record["target_bpp"]), source.element_size() * 8.0)
    tile_elements = options.get("tile_elements") or recommended_tile_elements(target)
    max_vectors = options.get("scale_search_max_vectors", 262144)
    expected = oracle_module.lattice_encode(source.float().numpy(), target, tile_elements=tile_elements, max_vectors=max_vectors)
    ours = b200.encode(source.cuda(), target_bpp=target, prob_bits=None, tile_elements=tile_elements, row_rdo_iterations=0,
                       row_rdo_candidates=5, scale_search_iterations=12, scale_search_max_vectors=max_vectors)
    assert float(ours.layout._lattice_rans_search_scale) == float(expected["_search_scale"])
    for key in ("layout", "stream_meta", "freq_tables", "scales", "offsets", "states", "payload"):
        assert np.array_equal(getattr(ours, key).cpu().numpy(), expected[key]), key
    # and the reference's numbers for the same input: rate within 0.01 bpp, distortion no worse
    reference = buffers_of(record)
    elements = shape[0] * shape[1]
    size = lambda b: sum(np.asarray(b[k]).nbytes for k in reference)  # noqa: E731
    assert abs(size({k: getattr(ours, k).cpu().numpy() for k in reference}) - size(reference)) * 8 / elements <= 0.01 + 512 / elements


def _weights(rows, cols, seed, outliers):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    if outliers:
        picks = torch.randperm(rows, generator=g)[:outliers]
        heavy = torch.randn(outliers, cols, generator=g) / torch.sqrt(torch.randn(outliers, cols, 3, generator=g).square().mean(-1))
        w[picks] = heavy * 0.02
    return w.to(torch.bfloat16)


@pytest.mark.parametrize("bpp", [2.3, 3.5, 4.0, 6.0])
def test_public_api_round_trip_against_oracle(oracle_module, bpp):
    """512 x 2048 bf16 with Student-t(3) outlier rows through compress/decompress: stored rate near the
    target, the oracle decodes our container to the same bits, and we decode the oracle's."""
    import entropack_b200 as ep

    weight = _weights(512, 2048, 5, 5)
    config = ep.EntroPackLossyConfig(target_bpp=bpp)
    compressed = ep.compress(weight.cuda(), config)
    assert compressed.compress_method == "lattice_rans"
    compressed.scheme.validate_buffers(compressed.buffers, tuple(weight.shape), weight.dtype)
    assert abs(compressed.actual_bpp - bpp) < 0.06
    restored = ep.decompress(compressed, config)
    assert restored.shape == weight.shape and restored.dtype == weight.dtype
    ours = {key: value.cpu().numpy() for key, value in compressed.buffers.items()}
    expected = oracle_module.lattice_decode(ours, tuple(weight.shape), weight.dtype)
    assert _bytes(restored) == _bytes(expected)
    theirs = oracle_module.lattice_encode(weight.float().numpy(), bpp)
    theirs.pop("_search_scale")
    assert _bytes(_gpu_decode(theirs, tuple(weight.shape), weight.dtype)) == _bytes(oracle_module.lattice_decode(theirs, tuple(weight.shape), weight.dtype))
    relative = ((restored.float().cpu() - weight.float()).norm() / weight.float().norm()).item()
    assert relative < {2.3: 0.30, 3.5: 0.13, 4.0: 0.09, 6.0: 0.03}[bpp]


def test_full_size_lossy_round_trip():
    """4096 x 11008 bf16 at 4 bpp: encode and decode on the GPU; re-encoding the decoded symbols is not
    possible without the oracle at this size, so check rate, distortion and a second decode's determinism."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(5)
    weight = (torch.randn(4096, 11008, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    config = ep.EntroPackLossyConfig(target_bpp=4.0)
    compressed = ep.compress(weight, config)
    assert abs(compressed.actual_bpp - 4.0) < 0.03
    first = ep.decompress(compressed, config)
    second = ep.decompress(compressed, config)
    assert torch.equal(first.view(torch.int16), second.view(torch.int16))
    relative = ((first.float() - weight.float()).norm() / weight.float().norm()).item()
    assert 0.05 < relative < 0.09


def test_malformed_lossy_stream_is_reported():
    record = load_golden("lattice_bf16_6p0_outliers")
    buffers = buffers_of(record)
    from entropack_b200.schemes.lattice_rans import b200

    bad = dict(buffers)
    bad["states"] = (buffers["states"] ^ np.uint32(0x00001234)).astype(np.uint32)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    b200.decode(_to_device(bad), shape=tuple(int(v) for v in record["shape"]), dtype=torch.bfloat16, error=error)
    torch.cuda.synchronize()
    assert int(error.item()) in (2, 3)
