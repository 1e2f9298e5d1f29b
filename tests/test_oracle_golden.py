"""The CPU oracle against the golden fixtures produced by the reference's eager lanes."""
import ast

import numpy as np
import pytest
import torch

from conftest import buffers_of, golden_names, load_golden


@pytest.mark.parametrize("name", golden_names("tile_ans_"))
def test_tile_ans_decode_matches_reference(oracle_module, name):
    record = load_golden(f"tile_ans_{name}")
    decoded = oracle_module.tile_ans_decode(buffers_of(record))
    assert np.array_equal(decoded, record["input_bytes"])


@pytest.mark.parametrize("name", golden_names("tile_ans_"))
def test_tile_ans_encode_matches_reference(oracle_module, name):
    record = load_golden(f"tile_ans_{name}")
    reference = buffers_of(record)
    itemsize = int(record["itemsize"])
    tile_elements = int(record["tile_elements_arg"])
    if tile_elements == 0:
        tile_elements = int(reference["layout"][0])
    ours = oracle_module.tile_ans_encode(
        record["input_bytes"], itemsize, tile_elements, int(record["probability_bits_arg"]))
    for key in ("layout", "lane_modes", "decode_tables", "offsets", "states", "payload"):
        assert np.array_equal(ours[key], reference[key]), key


@pytest.mark.parametrize("name", golden_names("lattice_"))
def test_lattice_decode_matches_reference(oracle_module, name):
    record = load_golden(f"lattice_{name}")
    dtype = getattr(torch, str(record["dtype"]))
    shape = tuple(int(v) for v in record["shape"])
    decoded = oracle_module.lattice_decode(buffers_of(record), shape, dtype)
    assert decoded.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes() == record["decoded_bytes"].tobytes()


def test_lattice_quantiser_matches_reference(oracle_module):
    units = load_golden("lattice_units")
    y = units["y"]
    fields, cosets = oracle_module.e8_quantize(y.reshape(1, -1), np.ones(1, np.float32), 1.0)
    assert np.array_equal(cosets, units["c"])
    assert np.array_equal(fields[:, :7], units["z0_6"])
    assert np.array_equal(fields[:, 7], units["m"])


def test_lattice_normaliser_matches_reference(oracle_module):
    units = load_golden("lattice_units")
    inputs, outputs = units["normalize_inputs"], units["normalize_outputs"]
    cursor_in = cursor_out = 0
    trials = 0
    while cursor_in < inputs.size:
        table_bits, alphabet = int(inputs[cursor_in]), int(inputs[cursor_in + 1])
        counts = inputs[cursor_in + 2 : cursor_in + 2 + alphabet]
        expected = outputs[cursor_out : cursor_out + alphabet]
        assert np.array_equal(oracle_module.lattice_normalize(counts, 1 << table_bits), expected)
        if alphabet <= 256:
            assert np.array_equal(oracle_module.normalize_counts(counts, 1 << table_bits), expected)
        cursor_in += 2 + alphabet
        cursor_out += alphabet
        trials += 1
    assert trials == 60


def test_lattice_size_model_and_stream_encoder_match_reference(oracle_module):
    units = load_golden("lattice_units")
    fields = np.concatenate([units["z0_6"], units["m"][:, None]], axis=1).astype(np.int32)
    cosets = units["c"].astype(np.int32)
    meta, bins = oracle_module.lattice_stats(fields, cosets)
    for (pb, tile_elements), expected in zip(units["coded_args"], units["coded_bytes"]):
        assert oracle_module.lattice_coded_bytes(meta, bins, int(pb), int(tile_elements)) == expected
    payload, offsets, states, meta32, freq = oracle_module.lattice_encode_symbols(fields, cosets, 11, 2000)
    assert np.array_equal(meta32, units["enc_meta"])
    assert np.array_equal(freq, units["enc_freq"])
    assert np.array_equal(offsets, units["enc_offsets"])
    assert np.array_equal(states, units["enc_states"])
    assert np.array_equal(payload, units["enc_payload"])


@pytest.mark.parametrize("name", golden_names("lattice_"))
def test_lattice_encode_tracks_reference(oracle_module, name):
    """Whole-encode parity is statistical (the row reductions are ordered differently, see
    oracle/lattice_oracle.c): same rate within 0.01 bpp of payload and a bitstream the decoder accepts."""
    record = load_golden(f"lattice_{name}")
    dtype = getattr(torch, str(record["dtype"]))
    shape = tuple(int(v) for v in record["shape"])
    options = ast.literal_eval(str(record["options"]))
    source = torch.from_numpy(record["input_bytes"].copy()).view(dtype).reshape(shape).float()
    pad = -shape[1] % 8
    if pad:
        source = torch.cat([source, source.new_zeros(shape[0], pad)], dim=1)
    itemsize = torch.empty((), dtype=dtype).element_size()
    target = min(float(record["target_bpp"]), itemsize * 8.0)
    reference = buffers_of(record)
    ours = oracle_module.lattice_encode(
        source.numpy(), target, tile_elements=options.get("tile_elements"),
        max_vectors=options.get("scale_search_max_vectors", 262144))
    assert np.array_equal(ours["layout"], reference["layout"])
    elements = shape[0] * shape[1]
    size = lambda b: sum(np.asarray(b[k]).nbytes for k in reference)  # noqa: E731
    assert abs(size(ours) - size(reference)) * 8 / elements <= 0.01 + 8 * 64 / elements
    restored = oracle_module.lattice_decode(ours, shape, dtype)
    expected = torch.from_numpy(record["decoded_bytes"].copy()).view(dtype).reshape(shape)
    ref_err = (expected.float() - source[:, : shape[1]]).norm()
    our_err = (restored.float() - source[:, : shape[1]]).norm()
    assert float(our_err) <= float(ref_err) * 1.02 + 1e-12


@pytest.mark.parametrize("name", golden_names("dfloat11_"))
def test_dfloat11_matches_reference(oracle_module, name):
    record = load_golden(f"dfloat11_{name}")
    reference = buffers_of(record)
    for use_regions in (False, True):
        assert np.array_equal(oracle_module.dfloat11_decode(reference, use_regions=use_regions), record["input_bits"])
    ours = oracle_module.dfloat11_encode(record["input_bits"])
    for key in ("layout", "luts", "sign_mantissa", "encoded_exponent", "thread_meta", "output_positions"):
        assert np.array_equal(ours[key], reference[key]), key


def test_lattice_full_size_rates_match_the_reference(oracle_module):
    """The lossy benchmark tensor (4096 x 11008 bf16, 41 heavy-tailed rows) at the four benchmark rates: the oracle's
    whole encode lands on the table width, tiling, largest alphabet, payload length (to a few words: the row RMS sums
    run in another order, which moves a handful of ties) and relative error that the reference's own encoder produced
    (``golden/baseline_lossy_scalars.json``), and its stored rate is within 0.0001 bpp of the reference's."""
    import hashlib
    import json

    from conftest import GOLDEN

    record = json.loads((GOLDEN / "baseline_lossy_scalars.json").read_text())
    g = torch.Generator().manual_seed(record["seed"])
    weight = torch.randn(record["rows"], record["cols"], generator=g) * 0.02
    picks = torch.randperm(record["rows"], generator=g)[: record["outliers"]]
    heavy = torch.randn(record["outliers"], record["cols"], generator=g) / torch.sqrt(
        torch.randn(record["outliers"], record["cols"], 3, generator=g).square().mean(-1))
    weight[picks] = heavy * 0.02
    weight = weight.to(torch.bfloat16)
    assert hashlib.sha256(weight.view(torch.uint8).numpy().tobytes()).hexdigest() == record["input_sha256"]
    source = weight.float().numpy()
    shape = (record["rows"], record["cols"])
    for bpp, reference in record["rates"].items():
        ours = oracle_module.lattice_encode(source, float(bpp))
        ours.pop("_search_scale")
        assert int(ours["layout"][1]) == reference["prob_bits"] and int(ours["layout"][2]) == reference["tile_elements"]
        assert int(ours["stream_meta"][:, 3].max()) == reference["max_alphabet"]
        assert abs(int(ours["payload"].size) - reference["payload_words"]) <= 8
        stored = sum(int(np.asarray(v).nbytes) for v in ours.values())
        # the reference's figure counts the blob header and alignment padding (a few hundred bytes of 22 MB)
        assert abs(stored * 8 / weight.numel() - reference["actual_bpp"]) <= 1e-4
        decoded = oracle_module.lattice_decode(ours, shape, torch.bfloat16)
        relative = float((decoded.float() - weight.float()).norm() / weight.float().norm())
        assert abs(relative - reference["rel_l2"]) <= 1e-6
