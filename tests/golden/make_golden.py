"""Regenerates the golden fixtures in this directory from the reference's own eager (CPU) lanes.

Run from the repository root in a container that has the reference checked out:

    python tests/golden/make_golden.py [--reference /path/to/entropack-checkout]

The reference ships no golden vectors, so its eager lanes are the executable specification: every
fixture holds a seeded input and the exact buffers / outputs the reference produced for it. The
fixtures are what travels; the reference itself is never needed to run the tests.

DFloat11 encode in the reference needs the third-party ``dahuffman`` package, which is not
installed. A stand-in module exposing the four members the reference touches
(``HuffmanCodec.from_frequencies``, ``get_code_table``, ``_table``, ``_eof``) is installed into
``sys.modules``; its code table comes from the oracle's own Huffman builder, so codeword values are
ours while every downstream byte (LUTs, bitstream, metadata) is produced by reference code.
"""
import argparse
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402


def install_huffman_stand_in():
    class _EOF:
        def __repr__(self):
            return "_EOF"

    eof = _EOF()

    class HuffmanCodec:
        def __init__(self, table):
            self._table = table
            self._eof = eof

        @classmethod
        def from_frequencies(cls, frequencies):
            counts = np.zeros(256, dtype=np.int64)
            for symbol, count in frequencies.items():
                counts[int(symbol)] = int(count)
            code_len, code_val = oracle.dfloat11_code(counts)
            order = sorted((int(code_len[s]), int(code_val[s]), s) for s in range(257) if code_len[s] > 0)
            table = {}
            for bits, value, symbol in order:
                table[eof if symbol == 256 else symbol] = (bits, value)
            return cls(table)

        def get_code_table(self):
            return self._table

    module = types.ModuleType("dahuffman")
    module.HuffmanCodec = HuffmanCodec
    sys.modules["dahuffman"] = module


def as_numpy(buffers: dict) -> dict:
    out = {}
    for key, value in buffers.items():
        tensor = value.detach().cpu().contiguous()
        if tensor.dtype == torch.bfloat16:
            tensor = tensor.view(torch.int16)
        out[key] = tensor.numpy()
    return out


def raw_bytes(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().contiguous().reshape(-1).view(torch.uint8).numpy().copy()


def tile_ans_cases():
    g = torch.Generator().manual_seed(1234)
    randn = lambda *shape: torch.randn(*shape, generator=g)  # noqa: E731
    cases = {}
    base = randn(96, 130) * 0.02
    cases["bf16"] = (base.to(torch.bfloat16), {})
    cases["fp16"] = (base.to(torch.float16), {})
    cases["fp32"] = (base.clone(), {})
    x = randn(75, 129)
    cases["fp8_e4m3"] = ((x * (448.0 / x.abs().max())).to(torch.float8_e4m3fn), {})
    cases["int8"] = ((randn(64, 200) * 20).round().clamp(-127, 127).to(torch.int8), {})
    cases["int32_small"] = ((randn(5000) * 40).round().to(torch.int32), {})
    cases["uint8_noise"] = (torch.randint(0, 256, (9000,), generator=g, dtype=torch.uint8), {})
    cases["int16_const_lane_pb12"] = (torch.randint(0, 200, (7001,), generator=g, dtype=torch.int16), {"probability_bits": 12})
    cases["bf16_ragged_tile100"] = ((randn(1237) * 0.02).to(torch.bfloat16), {"tile_elements": 100, "probability_bits": 10})
    cases["fp32_tile33"] = (randn(700) * 0.02, {"tile_elements": 33})
    cases["int8_single"] = (torch.tensor([5], dtype=torch.int8), {})
    cases["fp16_31"] = ((randn(31) * 0.02).to(torch.float16), {"tile_elements": 64})
    cases["int64_mixed"] = ((randn(3000) * 1000).round().to(torch.int64), {})
    big = randn(256, 1024)
    cases["bf16_large"] = ((big * 0.02).to(torch.bfloat16), {})
    cases["fp8_e4m3_large"] = ((big * (448.0 / big.abs().max())).to(torch.float8_e4m3fn), {})
    return cases


def make_tile_ans(ep, out_dir: Path):
    for name, (tensor, options) in tile_ans_cases().items():
        config = ep.TileANSConfig(execution_backend="eager", **options)
        compressed = ep.compress(tensor, config)
        assert compressed.compress_method == "tile_ans", (name, compressed.header)
        restored = ep.decompress(compressed, config)
        assert torch.equal(restored.view(torch.uint8), tensor.view(torch.uint8)), name
        record = {f"buf_{k}": v for k, v in as_numpy(compressed.buffers).items()}
        record["input_bytes"] = raw_bytes(tensor)
        record["itemsize"] = np.array(tensor.element_size())
        record["dtype"] = np.array(str(tensor.dtype).removeprefix("torch."))
        record["shape"] = np.array(tensor.shape, dtype=np.int64)
        record["tile_elements_arg"] = np.array(options.get("tile_elements", 0))
        record["probability_bits_arg"] = np.array(options.get("probability_bits", 0))
        if tensor.numel() < 50000:
            record["blob"] = compressed.entropack_quant_state.numpy()
        np.savez_compressed(out_dir / f"tile_ans_{name}.npz", **record)
        print(f"tile_ans {name}: {compressed.actual_bpp:.3f} bpp, pb={int(compressed.buffers['layout'][1])}, "
              f"modes={compressed.buffers['lane_modes'].tolist()}")


def lattice_weight(rows, cols, seed, outlier_rows=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    if outlier_rows:
        picks = torch.randperm(rows, generator=g)[:outlier_rows]
        w[picks] = torch.distributions.StudentT(3.0).sample((outlier_rows, cols)).to(torch.float32) * 0.02
    return w


def make_lattice(ep, out_dir: Path):
    from entropack.schemes.lattice_rans import eager, rans

    torch.manual_seed(99)  # StudentT sampling uses the global generator
    cases = {
        "bf16_2p3": (lattice_weight(64, 256, 5, 1).to(torch.bfloat16), 2.3, {}),
        "bf16_3p5": (lattice_weight(64, 256, 5, 1).to(torch.bfloat16), 3.5, {}),
        "bf16_4p0": (lattice_weight(64, 256, 5, 1).to(torch.bfloat16), 4.0, {}),
        "bf16_6p0": (lattice_weight(64, 256, 5, 1).to(torch.bfloat16), 6.0, {}),
        "bf16_4p0_pad": (lattice_weight(50, 203, 6).to(torch.bfloat16), 4.0, {"tile_elements": 2000}),
        "bf16_subsample": (lattice_weight(300, 64, 7).to(torch.bfloat16), 4.0, {"scale_search_max_vectors": 800}),
        "fp16_4p0": (lattice_weight(40, 128, 8).to(torch.float16), 4.0, {}),
        "fp32_5p0": (lattice_weight(40, 128, 9), 5.0, {}),
        "bf16_9p0_pb12": (lattice_weight(32, 128, 10).to(torch.bfloat16), 9.0, {}),
        "bf16_6p0_outliers": (lattice_weight(128, 512, 12, 6).to(torch.bfloat16), 6.0, {}),
        "bf16_10p5_wide": (lattice_weight(64, 512, 13, 4).to(torch.bfloat16), 10.5, {}),
    }
    w = lattice_weight(48, 128, 11)
    scale = (w.abs().amax(dim=1) / 448.0).clamp(min=torch.finfo(torch.float32).eps)
    cases["fp8_codes_5p0"] = ((w / scale.unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn), 5.0, {})
    cases["int8_codes_5p0"] = ((w / (w.abs().amax(dim=1, keepdim=True) / 127)).round().clamp(-127, 127).to(torch.int8), 5.0, {})
    for name, (tensor, bpp, options) in cases.items():
        config = ep.EntroPackLossyConfig(target_bpp=bpp, execution_backend="eager", **options)
        compressed = ep.compress(tensor, config)
        assert compressed.compress_method == "lattice_rans", (name, compressed.header)
        restored = ep.decompress(compressed, config)
        record = {f"buf_{k}": v for k, v in as_numpy(compressed.buffers).items()}
        record["input_bytes"] = raw_bytes(tensor)
        record["decoded_bytes"] = raw_bytes(restored)
        record["dtype"] = np.array(str(tensor.dtype).removeprefix("torch."))
        record["shape"] = np.array(tensor.shape, dtype=np.int64)
        record["target_bpp"] = np.array(bpp)
        record["actual_bpp"] = np.array(compressed.actual_bpp)
        record["options"] = np.array(repr(options))
        record["blob"] = compressed.entropack_quant_state.numpy()
        rel = ((restored.float() - tensor.float()).norm() / tensor.float().norm()).item()
        record["rel_l2"] = np.array(rel)
        np.savez_compressed(out_dir / f"lattice_{name}.npz", **record)
        print(f"lattice {name}: target {bpp} actual {compressed.actual_bpp:.4f} rel_l2 {rel:.4f} "
              f"pb={int(compressed.buffers['layout'][1])} alpha_max={int(compressed.buffers['stream_meta'][:, 3].max())}")

    # Sub-function pins: quantiser, normaliser, size model, stream encoder.
    g = torch.Generator().manual_seed(4321)
    y = torch.randn(4000, 8, generator=g) * 1.7
    y[:500] = (torch.randint(-6, 7, (500, 8), generator=g).float() * 0.5)      # exact ties on the half-integer grid
    y[500:700] = (torch.randint(-8, 9, (200, 8), generator=g).float() * 0.25)
    point = eager.nearest_e8(y)
    c, z0_6, m = eager.point_to_fields(point)
    counts_list, freq_list = [], []
    rng = np.random.default_rng(7)
    for trial in range(60):
        alphabet = int(rng.integers(1, 300))
        table_bits = int(rng.integers(9, 13))
        if trial % 3 == 0:
            counts = rng.integers(0, 5, alphabet)
        elif trial % 3 == 1:
            counts = (rng.pareto(1.2, alphabet) * 50).astype(np.int64)
        else:
            counts = rng.integers(0, 100000, alphabet)
        counts = counts.astype(np.int64)
        if counts.sum() == 0:
            counts[0] = 3
        counts_list.append(np.concatenate([[table_bits, alphabet], counts]))
        freq_list.append(rans.normalize_freq(counts, 1 << table_bits).astype(np.int64))
    c_np, z_np, m_np = c.numpy(), z0_6.numpy(), m.numpy()
    stats = eager._stream_stats(eager._coord_streams(c_np, z_np, m_np))
    coded = [rans.coded_bytes(stats[0], stats[1], pb, te) for pb, te in ((11, 16384), (9, 4096), (12, 288))]
    payload, states, offsets, meta, freq_tables = eager._encode_streams(c_np, z_np, m_np, 11, 2000)
    np.savez_compressed(
        out_dir / "lattice_units.npz", y=y.numpy(), c=c_np.astype(np.int32), z0_6=z_np.astype(np.int32),
        m=m_np.astype(np.int32), normalize_inputs=np.concatenate(counts_list), normalize_outputs=np.concatenate(freq_list),
        coded_bytes=np.array(coded), coded_args=np.array([[11, 16384], [9, 4096], [12, 288]]),
        enc_payload=payload.astype(np.uint16), enc_states=states.astype(np.uint32), enc_offsets=offsets.astype(np.uint32),
        enc_meta=meta.astype(np.int32), enc_freq=freq_tables.astype(np.uint16),
    )
    print("lattice units: coded_bytes", coded)


def make_rdo(ep, out_dir: Path):
    """Per-row rate-distortion refinement (row_rdo_iterations > 0). Row choices hang on float32 sums whose order is
    torch's, so these records pin what the refinement achieves (size, error, valid bitstream), not its exact picks."""
    from entropack.schemes.lattice_rans import rdo

    torch.manual_seed(123)
    cases = {
        "bf16_4p0": (lattice_weight(192, 512, 21, 8).to(torch.bfloat16), 4.0, {"row_rdo_iterations": 2}),
        "bf16_3p0_k7": (lattice_weight(128, 384, 22, 5).to(torch.bfloat16), 3.0, {"row_rdo_iterations": 3, "row_rdo_candidates": 7}),
    }
    for name, (tensor, bpp, options) in cases.items():
        plain = ep.EntroPackLossyConfig(target_bpp=bpp, execution_backend="eager")
        refined = ep.EntroPackLossyConfig(target_bpp=bpp, execution_backend="eager", **options)
        record = {"input_bytes": raw_bytes(tensor), "dtype": np.array(str(tensor.dtype).removeprefix("torch.")),
                  "shape": np.array(tensor.shape, dtype=np.int64), "target_bpp": np.array(bpp), "options": np.array(repr(options))}
        for label, config in (("plain", plain), ("rdo", refined)):
            compressed = ep.compress(tensor, config)
            assert compressed.compress_method == "lattice_rans", (name, compressed.header)
            restored = ep.decompress(compressed, config)
            record[f"{label}_actual_bpp"] = np.array(compressed.actual_bpp)
            record[f"{label}_rel_l2"] = np.array(((restored.float() - tensor.float()).norm() / tensor.float().norm()).item())
            if label == "rdo":
                for key, value in as_numpy(compressed.buffers).items():
                    record[f"buf_{key}"] = value
                record["decoded_bytes"] = raw_bytes(restored)
        np.savez_compressed(out_dir / f"rdo_{name}.npz", **record)
        print(f"rdo {name}: plain {float(record['plain_actual_bpp']):.4f} bpp / {float(record['plain_rel_l2']):.5f}, "
              f"refined {float(record['rdo_actual_bpp']):.4f} bpp / {float(record['rdo_rel_l2']):.5f}")
    ladders = {str(count): np.array(rdo.ratio_ladder(count)) for count in range(1, 10)}
    np.savez_compressed(out_dir / "rdo_ratio_ladders.npz", **ladders)


def baseline_lossy_weight(rows, cols, seed, outliers):
    """The lossy benchmark tensor: bf16 N(0, 0.02^2) rows, `outliers` of them (seeded pick) Student-t(3) x 0.02 built
    from the same CPU generator. tests/test_baseline_sizes_gpu.py builds the same tensor; the record's checksum ties
    the two together."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    if outliers:
        picks = torch.randperm(rows, generator=g)[:outliers]
        heavy = torch.randn(outliers, cols, generator=g) / torch.sqrt(torch.randn(outliers, cols, 3, generator=g).square().mean(-1))
        w[picks] = heavy * 0.02
    return w.to(torch.bfloat16)


def make_baseline_scalars(ep, out_dir: Path):
    """The reference's stored rate and relative error on the full-size lossy benchmark tensor (4096 x 11008 bf16, 41
    heavy-tailed rows) at the four benchmark rates: scalars only, the containers are tens of megabytes."""
    import hashlib
    import json

    tensor = baseline_lossy_weight(4096, 11008, 5, 41)
    record = {"rows": 4096, "cols": 11008, "seed": 5, "outliers": 41,
              "input_sha256": hashlib.sha256(raw_bytes(tensor).tobytes()).hexdigest(), "rates": {}}
    for bpp in (2.3, 3.5, 4.0, 6.0):
        config = ep.EntroPackLossyConfig(target_bpp=bpp, execution_backend="eager")
        compressed = ep.compress(tensor, config)
        assert compressed.compress_method == "lattice_rans", compressed.header
        restored = ep.decompress(compressed, config)
        rel = ((restored.float() - tensor.float()).norm() / tensor.float().norm()).item()
        buffers = as_numpy(compressed.buffers)
        record["rates"][str(bpp)] = {
            "actual_bpp": compressed.actual_bpp, "rel_l2": rel, "prob_bits": int(buffers["layout"][1]),
            "tile_elements": int(buffers["layout"][2]), "max_alphabet": int(buffers["stream_meta"][:, 3].max()),
            "payload_words": int(buffers["payload"].size),
            "decoded_sha256": hashlib.sha256(raw_bytes(restored).tobytes()).hexdigest(),
        }
        print(f"baseline lossy {bpp}: {record['rates'][str(bpp)]}", flush=True)
        (out_dir / "baseline_lossy_scalars.json").write_text(json.dumps(record, indent=1, sort_keys=True) + "\n")


def make_dfloat11(ep, out_dir: Path):
    g = torch.Generator().manual_seed(77)
    cases = {
        "normal": (torch.randn(120, 173, generator=g) * 0.02).to(torch.bfloat16),
        "wide": (torch.randn(30000, generator=g) * torch.exp(torch.randn(30000, generator=g) * 6)).to(torch.bfloat16),
        "tiny": (torch.randn(7, generator=g)).to(torch.bfloat16),
        "constant": torch.full((5000,), 0.5, dtype=torch.bfloat16),
    }
    for name, tensor in cases.items():
        config = ep.DFloat11Config(execution_backend="eager")
        compressed = ep.compress(tensor, config)
        assert compressed.compress_method == "dfloat11", (name, compressed.header)
        restored = ep.decompress(compressed, config)
        assert torch.equal(restored.view(torch.int16), tensor.view(torch.int16)), name
        record = {f"buf_{k}": v for k, v in as_numpy(compressed.buffers).items()}
        record["input_bits"] = tensor.reshape(-1).view(torch.int16).numpy().view(np.uint16)
        record["shape"] = np.array(tensor.shape, dtype=np.int64)
        record["blob"] = compressed.entropack_quant_state.numpy()
        np.savez_compressed(out_dir / f"dfloat11_{name}.npz", **record)
        print(f"dfloat11 {name}: {compressed.actual_bpp:.3f} bpp, luts {tuple(compressed.buffers['luts'].shape)}")


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of modelscope/entropack to import the eager lane from")
    parser.add_argument("--only", default="all", choices=("all", "tile_ans", "lattice", "rdo", "dfloat11", "baseline"))
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    install_huffman_stand_in()
    import entropack as ep

    if args.only in ("all", "tile_ans"):
        make_tile_ans(ep, HERE)
    if args.only in ("all", "lattice"):
        make_lattice(ep, HERE)
    if args.only in ("all", "rdo"):
        make_rdo(ep, HERE)
    if args.only in ("all", "dfloat11"):
        make_dfloat11(ep, HERE)
    if args.only == "baseline":      # minutes of single-threaded reference code: only on request
        make_baseline_scalars(ep, HERE)


if __name__ == "__main__":
    main()
