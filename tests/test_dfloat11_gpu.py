"""DFloat11 kernels against the golden fixtures and the CPU oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import buffers_of, golden_names, load_golden

pytestmark = pytest.mark.gpu


def _to_device(buffers: dict):
    from entropack_b200.schemes.dfloat11.format import DFloat11Buffers

    return DFloat11Buffers(**{key: torch.from_numpy(np.ascontiguousarray(value)).cuda() for key, value in buffers.items()})


def _gpu_decode(buffers: dict) -> np.ndarray:
    """Three decodes of one container: by the kernel that builds its table in every CUDA block, then with the kept
    tables made and used (warp-per-run kernel where the layout allows it), then with them found again. All must agree."""
    from entropack_b200.schemes.dfloat11 import b200

    device_buffers = _to_device(buffers)
    results = []
    for call in range(3):
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = b200.decode(device_buffers, error=error, kept_tables=call > 0)
        assert int(error.item()) == 0
        results.append(out.view(torch.int16).cpu().numpy().view(np.uint16))
    assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])
    return results[0]


@pytest.mark.parametrize("name", golden_names("dfloat11_"))
def test_kept_decode_tables_decode_like_tables_built_in_the_kernel(name):
    """Without kept tables: a 10-bit multi-symbol table built by every CUDA block. With them: the 11-bit tables built at
    the container's first decode, kept on it and copied in by every decode. All give the source bits."""
    from entropack_b200.schemes.dfloat11 import b200

    record = load_golden(f"dfloat11_{name}")
    device_buffers = _to_device(buffers_of(record))
    for call, kept in enumerate((False, True, True, False)):
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = b200.decode(device_buffers, error=error, kept_tables=kept)
        assert int(error.item()) == 0
        assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), record["input_bits"]), f"decode {call + 1} differs"
        assert (getattr(device_buffers.layout, "_dfloat11_decode_tables", None) is not None) == (call >= 1)


def _gpu_encode(bits: np.ndarray, bytes_per_thread=16, threads_per_block=128) -> dict:
    from entropack_b200.schemes.dfloat11 import b200

    weight = torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)
    codec = b200.build_codec(b200.exponent_counter(weight, threads_per_block))
    buffers = b200.encode(weight=weight, codec=codec, luts=b200.build_luts(codec), bytes_per_thread=bytes_per_thread,
                          threads_per_block=threads_per_block)
    return {key: value.cpu().numpy() for key, value in buffers._asdict().items()}


@pytest.mark.parametrize("name", golden_names("dfloat11_"))
def test_decode_reference_bitstreams(name):
    record = load_golden(f"dfloat11_{name}")
    assert np.array_equal(_gpu_decode(buffers_of(record)), record["input_bits"])


@pytest.mark.parametrize("name", golden_names("dfloat11_"))
def test_encode_reproduces_reference_bitstreams(name):
    """With the same code table the reference's encoder was given, every buffer is byte-identical."""
    record = load_golden(f"dfloat11_{name}")
    reference = buffers_of(record)
    ours = _gpu_encode(record["input_bits"])
    for key in ("layout", "luts", "sign_mantissa", "encoded_exponent", "thread_meta", "output_positions"):
        assert np.array_equal(ours[key], reference[key]), key


@pytest.mark.parametrize("n,bpt,tpb", [(1 << 20, 16, 128), (700001, 16, 128), (50000, 5, 32), (123457, 37, 96), (33, 16, 128), (1, 16, 128),
                                      (300000, 255, 64), (400000, 8, 256), (250000, 12, 100), (600000, 64, 64), (90000, 8, 32),
                                      (5000, 16, 1024), (60000, 8, 20), (60000, 16, 48), (3000000, 16, 128)])
def test_against_oracle_both_directions(oracle_module, n, bpt, tpb):
    g = torch.Generator().manual_seed(n)
    values = torch.randn(n, generator=g) * torch.exp(torch.randn(n, generator=g) * (3.0 if n % 2 else 0.3)) * 0.02
    bits = values.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    expected = oracle_module.dfloat11_encode(bits, bpt, tpb)
    ours = _gpu_encode(bits, bpt, tpb)
    for key in ("layout", "luts", "sign_mantissa", "encoded_exponent", "thread_meta", "output_positions"):
        assert np.array_equal(ours[key], expected[key]), key
    assert np.array_equal(_gpu_decode(expected), bits)
    assert np.array_equal(oracle_module.dfloat11_decode(ours, use_regions=True), bits)


def test_runs_of_equal_exponents_beside_wide_ones(oracle_module):
    """Half the tensor zeros (one-bit codewords, 128 to a region), half values of every magnitude: the zero half's
    runs of 32 regions decode to far more elements than the mean run, which the warp kernel's shared slices are sized
    from, so they take its path without staging."""
    n = 1 << 20
    g = torch.Generator().manual_seed(11)
    values = torch.randn(n, generator=g) * torch.exp(torch.randn(n, generator=g) * 4.0)
    values[n // 3: n // 3 + n // 2] = 0.0
    bits = values.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    expected = oracle_module.dfloat11_encode(bits, 16, 128)
    counts = expected["thread_meta"].astype(np.int64) & 2047
    per_run = counts.reshape(-1, 32).sum(axis=1)
    assert per_run.max() > 1.25 * per_run.mean() + 64     # the case is what it claims to be
    assert np.array_equal(_gpu_decode(expected), bits)


def test_full_size_round_trip_public_api():
    """BF16 4096 x 4096, N(0, 0.02^2): compress and decompress through the public API, bit-exact, ~11 bpp."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed(0)
    weight = (torch.randn(4096, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    compressed = ep.compress(weight, ep.DFloat11Config())
    assert compressed.compress_method == "dfloat11"
    compressed.scheme.validate_buffers(compressed.buffers, tuple(weight.shape), weight.dtype)
    assert 10.5 < compressed.actual_bpp < 11.2
    restored = ep.decompress(compressed, ep.DFloat11Config())
    assert torch.equal(restored.view(torch.int16), weight.view(torch.int16))


def test_malformed_metadata_is_reported_not_faulted():
    from entropack_b200.schemes.dfloat11 import b200

    record = load_golden("dfloat11_wide")
    buffers = buffers_of(record)
    bad = dict(buffers)
    positions = buffers["output_positions"].copy()
    positions[1] = positions[-1] + 1000
    bad["output_positions"] = positions
    device_bad = _to_device(bad)
    for call in range(3):   # both decode kernels
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        b200.decode(device_bad, error=error, kept_tables=call > 0)
        torch.cuda.synchronize()
        assert int(error.item()) != 0
    bad = dict(buffers)
    meta = buffers["thread_meta"].copy()
    meta[: meta.size // 2] |= 2047   # more codewords than any region can hold
    bad["thread_meta"] = meta
    device_bad = _to_device(bad)
    for call in range(3):
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        b200.decode(device_bad, error=error, kept_tables=call > 0)
        torch.cuda.synchronize()
        assert int(error.item()) != 0
    bad = dict(buffers)
    luts = buffers["luts"].copy()
    luts[0, :] = 255  # every byte of level 0 points at a child level that may not exist
    bad["luts"] = luts
    device_bad = _to_device(bad)
    for call in range(3):
        b200.decode(device_bad, kept_tables=call > 0)
        torch.cuda.synchronize()
