"""Host-side logic that needs no GPU: the C-ABI library loads and exports what the header declares,
the table planner matches the oracle, configs validate like the reference's, the container is
byte-compatible."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import ROOT, buffers_of, golden_names, load_golden


def test_library_exports_every_declared_symbol():
    from entropack_b200 import _native, build

    build.build()
    lib = ctypes.CDLL(str(_native.library_path()))
    declared = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        declared += re.findall(r"\b(ep_[a-z0-9_]+)\s*\(", text)
    assert declared, "no declarations found"
    for name in sorted(set(declared)):
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert _native.load().ep_abi_version() >= 1


@pytest.mark.parametrize("name", golden_names("tile_ans_"))
def test_table_planner_matches_reference(name):
    from entropack_b200.schemes.tile_ans import b200

    record = load_golden(f"tile_ans_{name}")
    reference = buffers_of(record)
    itemsize = int(record["itemsize"])
    lanes = record["input_bytes"].reshape(-1, itemsize)
    counts = np.stack([np.bincount(lanes[:, b], minlength=256) for b in range(itemsize)]).astype(np.uint64)
    pb, _freq, _cdf, tables, modes = b200.plan_tables(
        np.ascontiguousarray(counts), int(reference["layout"][0]), int(record["probability_bits_arg"]), 7.9)
    assert pb == int(reference["layout"][1])
    assert np.array_equal(modes, reference["lane_modes"])
    assert np.array_equal(tables, reference["decode_tables"])


def test_config_validation_matches_reference_rules():
    import entropack_b200 as ep
    from entropack_b200.schemes.config import validate_config

    validate_config(ep.TileANSConfig())
    with pytest.raises(ValueError):
        validate_config(ep.TileANSConfig(probability_bits=8))
    with pytest.raises(ValueError):
        validate_config(ep.TileANSConfig(tile_elements=-1))
    with pytest.raises(TypeError):
        validate_config(ep.TileANSConfig(tile_elements=1.5))
    with pytest.raises(TypeError):
        validate_config(ep.TileANSConfig(raw_lane_threshold=None))
    with pytest.raises(ValueError):
        validate_config(ep.TileANSConfig(raw_lane_threshold=8.5))


@pytest.mark.parametrize("stem", ["tile_ans_bf16", "tile_ans_int64_mixed", "tile_ans_int8_single"])
def test_container_is_byte_compatible(stem):
    import entropack_b200 as ep

    record = load_golden(stem)
    blob = torch.from_numpy(record["blob"].copy())
    container = ep.CompressedTensor.unpack(blob)
    assert tuple(container.shape) == tuple(int(v) for v in record["shape"])
    for key, value in buffers_of(record).items():
        assert np.array_equal(container.buffers[key].numpy(), value), key
    rebuilt = ep.CompressedTensor(header=container.header, buffers=container.buffers, shape=container.shape, dtype=container.dtype)
    assert torch.equal(rebuilt.entropack_quant_state, blob)
    assert container.actual_bpp == blob.numel() * 8 / container.numel()
    state = container.state_dict()
    again = ep.CompressedTensor.from_state_dict(state)
    assert torch.equal(again.entropack_quant_state, blob)
    with pytest.raises(ValueError):
        ep.CompressedTensor.unpack(blob[:-16])
    container.scheme.validate_buffers(container.buffers, tuple(container.shape), container.encoded_dtype)



def test_moved_container_keeps_parsed_header_and_host_metadata(monkeypatch):
    """clone / detach / to reuse the parsed header (no second read of the blob) and carry the metadata a scheme
    cached on the small buffers, so a container primed in host memory decodes without device-to-host reads."""
    import entropack_b200 as ep
    from entropack_b200.compression import compressed_tensor

    record = load_golden("tile_ans_bf16")
    container = ep.CompressedTensor.unpack(torch.from_numpy(record["blob"].copy()))
    container.scheme.prime_host_metadata(container.buffers)
    layout = container.buffers["layout"]
    assert layout._tile_ans_layout[0] > 0 and layout._tile_ans_lane_modes.dtype == np.uint8

    calls = []
    original = compressed_tensor.parse_blob
    monkeypatch.setattr(compressed_tensor, "parse_blob", lambda blob: calls.append(1) or original(blob))
    for moved in (container.clone(), container.detach(), container.to("cpu", copy=True)):
        assert moved.header == container.header and tuple(moved.shape) == tuple(container.shape)
        assert torch.equal(moved.entropack_quant_state, container.entropack_quant_state)
        assert moved.buffers["layout"]._tile_ans_layout == layout._tile_ans_layout
        assert moved.buffers["layout"]._tile_ans_lane_modes is layout._tile_ans_lane_modes
    assert not calls



def test_ratio_ladder_matches_the_reference():
    from entropack_b200.schemes.lattice_rans.encoder import ratio_ladder

    ladders = load_golden("rdo_ratio_ladders")
    for count, expected in ladders.items():
        assert list(ratio_ladder(int(count))) == expected.tolist()


def test_rate_tradeoff_keeps_the_rate_budget():
    from entropack_b200.schemes.lattice_rans.encoder import _choose_rate_tradeoff

    rng = np.random.default_rng(4)
    rates = np.sort(rng.uniform(500.0, 900.0, size=(200, 5)).astype(np.float32), axis=1)        # finer candidates cost more
    distortion = np.sort(rng.uniform(1.0, 2.0, size=(200, 5)).astype(np.float32), axis=1)[:, ::-1].copy()  # and err less
    row = np.arange(200)
    unconstrained = _choose_rate_tradeoff(distortion, rates, 1e9)
    assert np.array_equal(unconstrained, distortion.argmin(1))
    budget = float(rates[:, 2].sum())
    choice = _choose_rate_tradeoff(distortion, rates, budget)
    assert rates[row, choice].sum(dtype=np.float32) <= budget
    # spending the budget on finer candidates must beat giving every row the middle one
    assert distortion[row, choice].sum() <= distortion[:, 2].sum()



def test_convrot_group_rules():
    from entropack_b200 import convrot

    assert [convrot.is_convrot_group(v) for v in (4, 16, 64, 256, 1024, 8, 2, 0, 12, 4.0, True)] == [True] * 5 + [False] * 6
    assert convrot.choose_convrot_group(3840) == 256 and convrot.choose_convrot_group(320) == 64
    assert convrot.choose_convrot_group(3840, 16) == 16 and convrot.choose_convrot_group(6) is None
    with pytest.raises(ValueError):
        convrot.choose_convrot_group(3840, 32)
    matrix = convrot.build_convrot_matrix(64)
    assert torch.equal(matrix, matrix.t()) and torch.allclose(matrix @ matrix, torch.eye(64), atol=1e-6)


def test_no_cpu_fallback():
    import entropack_b200 as ep

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ep.DispatchError):
        ep.compress(torch.zeros(64, 64), ep.TileANSConfig())
    with pytest.raises(ep.DispatchError):
        ep.compress(torch.zeros(64, 64), ep.TileANSConfig(execution_backend="eager"))


def test_product_never_imports_the_oracle():
    offenders = []
    for path in (ROOT / "entropack_b200").rglob("*.py"):
        text = path.read_text()
        if re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M):
            offenders.append(str(path))
    assert not offenders, offenders


@pytest.mark.parametrize("name", golden_names("dfloat11_"))
def test_dfloat11_code_and_luts_match_reference(oracle_module, name):
    from entropack_b200.schemes.dfloat11 import b200

    record = load_golden(f"dfloat11_{name}")
    counts = np.bincount((record["input_bits"] >> 7) & 0xFF, minlength=256)
    codec = b200.build_codec({i: int(c) for i, c in enumerate(counts) if c})
    expected_len, expected_val = oracle_module.dfloat11_code(counts)
    assert np.array_equal(codec[0], expected_len) and np.array_equal(codec[1], expected_val)
    assert np.array_equal(b200.build_luts(codec).numpy(), buffers_of(record)["luts"])


def test_lattice_host_model_matches_reference():
    """ep_lattice_coded_bytes / ep_lattice_tables on the unit fixture's symbols (min/max record and compact
    bins rebuilt with numpy the way the device kernels lay them out)."""
    import ctypes

    from entropack_b200 import _native

    units = load_golden("lattice_units")
    fields = np.concatenate([units["z0_6"], units["m"][:, None]], axis=1).astype(np.int64)
    cosets = units["c"].astype(np.int64)
    vectors = cosets.size
    minmax = np.zeros(34, dtype=np.int32)
    bins = [np.bincount(cosets, minlength=2)]
    for st in range(16):
        values = fields[cosets == (st & 1), st >> 1]
        if values.size:
            minmax[2 * st], minmax[2 * st + 1] = values.min(), values.max()
            bins.append(np.bincount(values - values.min()))
        else:
            minmax[2 * st], minmax[2 * st + 1] = np.iinfo(np.int32).max, np.iinfo(np.int32).min
    minmax[32] = cosets.max()
    bins = np.ascontiguousarray(np.concatenate(bins).astype(np.int32))
    lib = _native.load()
    assert lib.ep_lattice_bins_needed(minmax.ctypes.data) == bins.size
    for (pb, tile_elements), expected in zip(units["coded_args"], units["coded_bytes"]):
        value = ctypes.c_double()
        assert lib.ep_lattice_coded_bytes(minmax.ctypes.data, bins.ctypes.data, vectors, int(pb), int(tile_elements),
                                          ctypes.addressof(value)) == 0
        assert value.value == expected
    meta = np.zeros((17, 4), dtype=np.int32)
    freq = np.zeros(bins.size, dtype=np.uint16)
    entries = ctypes.c_int64()
    assert lib.ep_lattice_tables(minmax.ctypes.data, bins.ctypes.data, vectors, 11, meta.ctypes.data, freq.ctypes.data, freq.size,
                                 ctypes.addressof(entries)) == 0
    assert np.array_equal(meta, units["enc_meta"])
    assert np.array_equal(freq[: entries.value], units["enc_freq"])


def test_streamed_pieces_cover_every_unit_once_and_ramp_up():
    """Piece runs of the streamed bulk decode: contiguous, on granule boundaries, doubling from the first piece's size
    to the target, the last one ragged."""
    from types import SimpleNamespace

    from entropack_b200.compression.pipeline import _piece_runs

    plan = SimpleNamespace(units=8192 + 5, unit_output_bytes=8192, granule=8)
    runs = _piece_runs(plan, 16 << 20, 2 << 20)
    assert runs[0] == (0, 256) and runs[1] == (256, 512) and runs[2] == (768, 1024) and runs[3][1] == 2048 and runs[4][1] == 2048
    assert all(first % 8 == 0 for first, _ in runs)
    assert [first for first, _ in runs[1:]] == [first + count for first, count in runs[:-1]]
    assert runs[-1][0] + runs[-1][1] == plan.units
    # units larger than a piece: one granule at a time
    big = SimpleNamespace(units=20, unit_output_bytes=1 << 20, granule=8)
    assert _piece_runs(big, 1 << 20, 1 << 10) == [(0, 8), (8, 8), (16, 4)]


def test_reference_arm_of_the_bench_prints_its_line_without_a_gpu():
    """`bench.py --impl reference` times the CPU oracle on the host cores and needs no GPU: one JSON line with the
    headline metric's name and unit, the CPU baseline's description and an end-to-end entry without transfers."""
    import json
    import subprocess
    import sys

    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"].startswith("decode GB/s") and line["config"]["workload"] == "c2_tile_ans_decode"
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["steps"] == 1
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["value"] == line["value"] and baseline["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_decode_ahead_registration_rules():
    """A layer is registered once and with one DecodeAhead at a time; closing unhooks every layer (no GPU involved:
    modules that it does not handle are carried in the list and run as they always do)."""
    import entropack_b200 as ep

    first, second = torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)
    with pytest.raises(ValueError):
        ep.DecodeAhead([first, first])
    assert getattr(first, "_decode_ahead", None) is None       # a refused list leaves no hook behind
    ahead = ep.DecodeAhead([first, second])
    assert first._decode_ahead is ahead and second._decode_ahead is ahead
    with pytest.raises(ValueError):
        ep.DecodeAhead([second])
    ahead.drain()          # nothing pending, nothing allocated: a no-op
    ahead.close()
    assert first._decode_ahead is None and second._decode_ahead is None
    with ep.DecodeAhead([second, first]) as again:
        assert second._decode_ahead is again
    assert second._decode_ahead is None
    x = torch.randn(3, 8)
    assert torch.equal(first(x), torch.nn.functional.linear(x, first.weight, first.bias))


def test_forward_asks_for_the_fused_kernel_only_where_it_pays(monkeypatch):
    """The layer multiplies inside the decode kernel for one token on a large layer, and decodes and multiplies in turn
    otherwise; the two thresholds are plain attributes a caller may change. (The kernels themselves need a GPU: here
    the decode is replaced by a dense weight and the fused kernel by a recorder.)"""
    import entropack_b200 as ep

    layer = ep.CompressedLinear(64, 48, bias=False, config=ep.EntroPackLossyConfig(target_bpp=4.0), device="cpu")
    dense = torch.randn(48, 64).to(torch.bfloat16)
    asked = []
    monkeypatch.setattr(layer, "_decoded_for_product", lambda device, dtype: dense)
    monkeypatch.setattr(layer, "_fused_forward", lambda x: asked.append(tuple(x.shape)) or None)
    one, four = torch.randn(1, 64).to(torch.bfloat16), torch.randn(2, 2, 64).to(torch.bfloat16)
    assert (type(layer).fused_max_tokens, type(layer).fused_min_weights) == (1, 32 << 20)
    assert torch.equal(layer(one), torch.nn.functional.linear(one, dense)) and asked == []      # a small layer: never
    layer.fused_min_weights = 64 * 48
    layer(one), layer(four)
    assert asked == [(1, 64)]                                                                    # large enough: one token only
    layer.fused_max_tokens = 4
    layer(four)
    assert asked == [(1, 64), (2, 2, 64)]


def test_transfer_order_keeps_both_directions_busy():
    """Containers that upload faster than they download go first, smallest upload first; the rest follow, largest
    download first (Johnson's rule for upload -> download); without a download the given order stands."""
    from types import SimpleNamespace

    from entropack_b200.compression.pipeline import _transfer_order

    def container(upload_bytes, elements, element_size):
        return SimpleNamespace(entropack_quant_state=torch.empty(upload_bytes, dtype=torch.uint8),
                               numel=lambda: elements, element_size=lambda: element_size)

    # uploads / downloads in bytes: 0: 60/64, 1: 30/32, 2: 200/128 (uploads more than it downloads), 3: 300/256, 4: 10/64
    items = [container(60, 64, 1), container(30, 16, 2), container(200, 32, 4), container(300, 128, 2), container(10, 64, 1)]
    assert _transfer_order(items, with_download=True) == [4, 1, 0, 3, 2]
    assert _transfer_order(items, with_download=False) == [0, 1, 2, 3, 4]


def test_low_latency_preset_is_an_ordinary_tile_setting():
    """The preset only shortens the tiles (8192 symbols: 910 vectors, 257 chain steps instead of 513); every other field
    keeps its default or the caller's value, and the tile rule for plain configs is the reference's."""
    import entropack_b200 as ep
    from entropack_b200.schemes.lattice_rans.format import recommended_tile_elements

    preset, plain = ep.EntroPackLossyConfig.low_latency(4.0), ep.EntroPackLossyConfig(target_bpp=4.0)
    assert preset.tile_elements == 8192 and preset.target_bpp == 4.0
    assert {k: v for k, v in vars(preset).items() if k != "tile_elements"} == {k: v for k, v in vars(plain).items() if k != "tile_elements"}
    assert ep.EntroPackLossyConfig.low_latency(3.5, tile_elements=4096, row_rdo_iterations=2).tile_elements == 4096
    assert [recommended_tile_elements(b) for b in (1.5, 2.0, 2.3, 4.0, 4.5, 7.0, 7.5)] == [32768, 32768, 16384, 16384, 8192, 8192, 4096]
