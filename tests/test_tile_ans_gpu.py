"""Tile-ANS kernels against the golden fixtures and the CPU oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import buffers_of, golden_names, load_golden

pytestmark = pytest.mark.gpu

DTYPES = {
    1: torch.uint8, 2: torch.uint16, 4: torch.uint32, 8: torch.uint64,
}


def _to_device(buffers: dict):
    from entropack_b200.schemes.tile_ans.format import TileBuffers

    return TileBuffers(**{key: torch.from_numpy(np.ascontiguousarray(value)).cuda() for key, value in buffers.items()})


def _gpu_decode(buffers: dict, itemsize: int) -> np.ndarray:
    from entropack_b200.schemes.tile_ans import b200

    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = b200.decode(_to_device(buffers), dtype=DTYPES[itemsize], error=error)
    assert int(error.item()) == 0
    return out.view(torch.uint8).cpu().numpy()


def _gpu_encode(data: np.ndarray, itemsize: int, tile_elements: int, probability_bits: int = 0) -> dict:
    from entropack_b200.schemes.tile_ans import b200

    weight = torch.from_numpy(data.copy()).cuda().view(DTYPES[itemsize])
    buffers = b200.encode(weight=weight, tile_elements=tile_elements, probability_bits=probability_bits,
                          raw_lane_threshold=7.9, threads_per_block=None)
    return {key: value.cpu().numpy() for key, value in buffers._asdict().items()}


@pytest.mark.parametrize("name", golden_names("tile_ans_"))
def test_decode_reference_bitstreams(name):
    record = load_golden(f"tile_ans_{name}")
    decoded = _gpu_decode(buffers_of(record), int(record["itemsize"]))
    assert np.array_equal(decoded, record["input_bytes"])


@pytest.mark.parametrize("name", golden_names("tile_ans_"))
def test_reference_bitstreams_decode_in_runs_of_tiles(name):
    """ep_tile_ans_decode_tiles over three runs (a first tile alone, a middle run, the rest) writes the bytes of the
    whole-tensor decode; with only the payload words of each run's streams present in the payload buffer."""
    from entropack_b200.schemes.tile_ans import b200
    from entropack_b200.schemes.tile_ans.format import num_tiles, parse_layout

    record = load_golden(f"tile_ans_{name}")
    host = buffers_of(record)
    itemsize = int(record["itemsize"])
    buffers = _to_device(host)
    tile_elements, _, lanes, elements = parse_layout(buffers.layout)
    tiles = num_tiles(elements, tile_elements)
    cuts = sorted({0, min(1, tiles), (tiles + 1) // 2, tiles})
    out = torch.full((elements * lanes,), 0xA5, dtype=torch.uint8, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    offsets = host["offsets"].astype(np.int64)
    whole_payload = np.ascontiguousarray(host["payload"])
    for first, last in zip(cuts, cuts[1:]):
        # a payload buffer that holds this run's words only; everything else is poison
        partial = np.full_like(whole_payload, 0xDEAD)
        for lane in range(lanes):
            begin, end = int(offsets[lane * tiles + first]), int(offsets[lane * tiles + last])
            partial[begin:end] = whole_payload[begin:end]
        b200.decode(buffers._replace(payload=torch.from_numpy(partial).cuda()), dtype=DTYPES[itemsize], error=error, out=out,
                    tiles=(first, last - first))
    assert int(error.item()) == 0
    assert np.array_equal(out.cpu().numpy(), record["input_bytes"])


@pytest.mark.parametrize("name", golden_names("tile_ans_"))
def test_encode_reproduces_reference_bitstreams(name):
    record = load_golden(f"tile_ans_{name}")
    reference = buffers_of(record)
    ours = _gpu_encode(record["input_bytes"], int(record["itemsize"]), int(reference["layout"][0]),
                       int(record["probability_bits_arg"]))
    for key in ("layout", "lane_modes", "decode_tables", "offsets", "states", "payload"):
        assert np.array_equal(ours[key], reference[key]), key


def _seeded(kind: str, n: int, seed: int) -> tuple[np.ndarray, int]:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g)
    if kind == "fp8":
        t = (x * (448.0 / x.abs().max())).to(torch.float8_e4m3fn)
    elif kind == "int8":
        t = (x * 20).round().clamp(-127, 127).to(torch.int8)
    elif kind == "fp16":
        t = (x * 0.02).to(torch.float16)
    elif kind == "bf16":
        t = (x * 0.02).to(torch.bfloat16)
    elif kind == "fp32":
        t = x * 0.02
    elif kind == "int64":
        t = (x * 3000).round().to(torch.int64)
    else:
        raise AssertionError(kind)
    return t.view(torch.uint8).numpy().copy(), t.element_size()


@pytest.mark.parametrize("kind,n,tile", [
    ("fp8", 1 << 20, 8192), ("int8", (1 << 20) + 13, 4096), ("fp16", 700001, 8192), ("bf16", 1 << 19, 4096),
    ("fp32", 300007, 8192), ("int64", 100003, 8192), ("fp8", 31, 4096), ("fp16", 33, 32), ("bf16", 1, 4096),
])
def test_against_oracle_both_directions(oracle_module, kind, n, tile):
    data, itemsize = _seeded(kind, n, seed=n % 97)
    expected = oracle_module.tile_ans_encode(data, itemsize, tile)
    ours = _gpu_encode(data, itemsize, tile)
    for key in ("layout", "lane_modes", "decode_tables", "offsets", "states", "payload"):
        assert np.array_equal(ours[key], expected[key]), key
    assert np.array_equal(_gpu_decode(expected, itemsize), data)
    assert np.array_equal(oracle_module.tile_ans_decode(ours), data)


@pytest.mark.parametrize("kind", ["fp8", "int8", "fp16", "fp32"])
def test_full_size_round_trip(kind):
    """8192 x 8192 of each benchmark dtype: encode and decode on the GPU, bit-exact restore, and the
    public API agrees with the lane."""
    import entropack_b200 as ep

    g = torch.Generator(device="cuda").manual_seed({"fp8": 1, "int8": 2, "fp16": 3, "fp32": 4}[kind])
    x = torch.randn(8192, 8192, generator=g, device="cuda")
    if kind == "fp8":
        t = (x * (448.0 / x.abs().max())).to(torch.float8_e4m3fn)
    elif kind == "int8":
        t = (x * 20).round().clamp(-127, 127).to(torch.int8)
    elif kind == "fp16":
        t = (x * 0.02).to(torch.float16)
    else:
        t = x * 0.02
    del x
    compressed = ep.compress(t, ep.TileANSConfig())
    assert compressed.compress_method == "tile_ans"
    compressed.scheme.validate_buffers(compressed.buffers, tuple(t.shape), t.dtype)
    restored = ep.decompress(compressed, ep.TileANSConfig())
    assert restored.dtype == t.dtype and restored.shape == t.shape
    assert torch.equal(restored.view(torch.uint8), t.view(torch.uint8))
    assert compressed.actual_bpp < t.element_size() * 8


def test_malformed_streams_are_reported_not_faulted():
    from entropack_b200.schemes.tile_ans import b200

    record = load_golden("tile_ans_fp8_e4m3_large")
    buffers = buffers_of(record)
    # truncated payload: offsets now point past the end
    bad = dict(buffers)
    bad["payload"] = buffers["payload"][: buffers["payload"].size // 2].copy()
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    b200.decode(_to_device(bad), dtype=torch.uint8, error=error)
    assert int(error.item()) == 1
    # corrupted states: streams are no longer consumed exactly
    bad = dict(buffers)
    bad["states"] = (buffers["states"] ^ np.uint32(0x00013570)).astype(np.uint32)
    error.zero_()
    b200.decode(_to_device(bad), dtype=torch.uint8, error=error)
    assert int(error.item()) in (2, 3)
    torch.cuda.synchronize()


def test_decompress_many_matches_decompress_and_fills_pinned_outputs():
    """The pipelined bulk decode (three streams) returns what per-tensor decompress returns, for mixed schemes,
    and leaves the same bytes in the pinned host outputs."""
    import entropack_b200 as ep

    generator = torch.Generator(device="cuda").manual_seed(11)
    tensors = [
        (torch.randn(300, 257, generator=generator, device="cuda") * 0.02).to(torch.bfloat16),
        (torch.randn(64, 4096, generator=generator, device="cuda") * 20).round().clamp(-127, 127).to(torch.int8),
        torch.randn(129, 512, generator=generator, device="cuda"),
        (torch.randn(256, 512, generator=generator, device="cuda") * 0.02).to(torch.bfloat16),
    ]
    configs = [ep.TileANSConfig(), ep.TileANSConfig(), ep.TileANSConfig(), ep.DFloat11Config()]
    containers = [ep.compress(t, c) for t, c in zip(tensors, configs)]
    expected = [ep.decompress(c, cfg) for c, cfg in zip(containers, configs)]
    blobs = [c.entropack_quant_state.cpu().pin_memory() for c in containers]
    outputs = [torch.empty(t.numel() * t.element_size(), dtype=torch.uint8).pin_memory() for t in tensors]
    for _ in range(2):   # the second pass reuses the streams
        decoded = ep.decompress_many(blobs, configs, device="cuda", out=outputs)
        for want, got, source, host in zip(expected, decoded, tensors, outputs):
            assert got.dtype == want.dtype and got.shape == want.shape
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
            assert torch.equal(got.view(torch.uint8), source.view(torch.uint8))
            assert torch.equal(host, want.reshape(-1).view(torch.uint8).cpu())


@pytest.mark.parametrize("piece_bytes,first_piece_bytes", [(64 << 10, 16 << 10), (1 << 20, 1 << 20)])
def test_decompress_many_streams_tile_ans_containers_in_pieces(monkeypatch, piece_bytes, first_piece_bytes):
    """A Tile-ANS container in host memory is uploaded, decoded and sent back in runs of tiles
    (ep_tile_ans_decode_tiles); the bytes must be those of the whole-tensor decode. Piece sizes are turned down so
    that small tensors take the path: ragged last tile, raw and coded byte lanes, 1/2/4-byte elements, a tile count
    that is no multiple of the block's 8."""
    import entropack_b200 as ep
    from entropack_b200.compression import pipeline

    monkeypatch.setattr(pipeline, "PIECE_BYTES", piece_bytes)
    monkeypatch.setattr(pipeline, "FIRST_PIECE_BYTES", first_piece_bytes)
    taken = []
    inner = pipeline._decode_streamed
    monkeypatch.setattr(pipeline, "_decode_streamed", lambda *a, **k: (taken.append(a[1].units), inner(*a, **k))[1])

    generator = torch.Generator(device="cuda").manual_seed(12)
    tensors = [
        (torch.randn(531, 4099, generator=generator, device="cuda") * 20).round().clamp(-127, 127).to(torch.int8),
        (torch.randn(1100, 1111, generator=generator, device="cuda") * 0.02).to(torch.float16),
        torch.randn(1023, 999, generator=generator, device="cuda") * 0.02,
        (torch.randn(2048, 1024, generator=generator, device="cuda") * 0.02).to(torch.bfloat16),
        torch.randn(9, 100, generator=generator, device="cuda"),            # too small to stream
    ]
    config = ep.TileANSConfig()
    containers = [ep.compress(t, config) for t in tensors]
    blobs = [c.entropack_quant_state.cpu().pin_memory() for c in containers]
    outputs = [torch.empty_like(t, device="cpu").pin_memory() for t in tensors]
    for _ in range(2):
        for host in outputs:
            host.view(torch.uint8).fill_(0xA5)
        decoded = ep.decompress_many(blobs, config, device="cuda", out=outputs)
        for got, source, host in zip(decoded, tensors, outputs):
            assert got.dtype == source.dtype and got.shape == source.shape
            assert torch.equal(got.view(torch.uint8), source.view(torch.uint8))
            assert torch.equal(host.view(torch.uint8), source.cpu().view(torch.uint8))
    assert len(taken) == 8 and all(units > 8 for units in taken)


def test_decode_tiles_rejects_ranges_outside_the_tensor():
    import entropack_b200 as ep
    from entropack_b200.schemes.base import packed_buffers
    from entropack_b200.schemes.tile_ans import b200
    from entropack_b200.schemes.tile_ans.format import TileBuffers

    tensor = torch.randn(64, 4096, device="cuda").to(torch.bfloat16)
    container = ep.compress(tensor, ep.TileANSConfig(tile_elements=4096))
    buffers = packed_buffers(container.buffers, TileBuffers)
    out = torch.zeros(tensor.numel() * 2, dtype=torch.uint8, device="cuda")
    b200.decode(buffers, dtype=torch.bfloat16, out=out, tiles=(8, 16))
    torch.cuda.synchronize()
    whole = tensor.reshape(-1).view(torch.uint8)
    span = slice(8 * 4096 * 2, 24 * 4096 * 2)
    assert torch.equal(out[span], whole[span]) and int(out[: span.start].max()) == 0 and int(out[span.stop :].max()) == 0
    b200.decode(buffers, dtype=torch.bfloat16, out=out, tiles=(64, 0))     # an empty run at the end is fine
    for bad in [(-1, 4), (60, 5), (65, 0), (0, -1)]:
        with pytest.raises(ValueError):
            b200.decode(buffers, dtype=torch.bfloat16, out=out, tiles=bad)
