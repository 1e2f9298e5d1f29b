"""The allocation-free lossy decode (``ep_lattice_decode_static``) against the regular entry point.

Some callers cannot allocate device memory at the time they decode (all of HBM already belongs to
their own pool, or they run inside an allocator callback), so this variant keeps its table scratch in
a fixed array inside the library. Here it is called straight through the C ABI, twice in a row, on a
container that needs that scratch, and must reproduce the regular entry point's output bit for bit;
a container above the fixed array's limit must be refused. This file sorts last on purpose.
"""
import numpy as np
import pytest
import torch

from conftest import buffers_of, load_golden

pytestmark = pytest.mark.gpu


def _device_buffers(record):
    return {key: torch.from_numpy(np.ascontiguousarray(value)).cuda() for key, value in buffers_of(record).items()}


def _call(lib, name, buffers, out, rows, cols, prob_bits, tile_elements, alphabet, extra):
    stream = torch.cuda.current_stream().cuda_stream
    head = (buffers["payload"].data_ptr(), buffers["payload"].numel(), buffers["offsets"].data_ptr(), buffers["states"].data_ptr(),
            buffers["stream_meta"].data_ptr(), buffers["freq_tables"].data_ptr(), buffers["freq_tables"].numel(),
            buffers["scales"].data_ptr(), out.data_ptr(), 0, rows, cols, prob_bits, tile_elements, alphabet)
    return getattr(lib, name)(*head, *extra, None, stream)


def test_static_scratch_decode_matches_regular_decode():
    from entropack_b200 import _native

    lib = _native.load()
    record = load_golden("lattice_bf16_10p5_wide")  # prob_bits 12, alphabet 613: needs the 64-bit global tables
    buffers = _device_buffers(record)
    rows = int(record["shape"][0])
    cols, prob_bits, tile_elements = (int(v) for v in buffers_of(record)["layout"])
    alphabet = int(buffers_of(record)["stream_meta"][:, 3].max())
    scratch_bytes = lib.ep_lattice_decode_scratch_bytes(prob_bits, alphabet)
    assert scratch_bytes > 0 and prob_bits <= lib.ep_lattice_decode_static_max_prob_bits()
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device="cuda")
    expected = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
    assert _call(lib, "ep_lattice_decode", buffers, expected, rows, cols, prob_bits, tile_elements, alphabet,
                 (scratch.data_ptr(), scratch_bytes, 0)) == 0
    torch.cuda.synchronize()
    assert expected[:, : int(record["shape"][1])].contiguous().cpu().view(torch.uint8).numpy().tobytes() == record["decoded_bytes"].tobytes()

    # a shared-memory-path container in between leaves different state behind on the device
    other = load_golden("lattice_bf16_4p0")
    other_buffers = _device_buffers(other)
    other_cols, other_pb, other_tile = (int(v) for v in buffers_of(other)["layout"])
    other_out = torch.zeros((int(other["shape"][0]), other_cols), dtype=torch.bfloat16, device="cuda")
    for attempt in range(2):
        out = torch.full((rows, cols), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        # free device memory as the driver counts it (cudaMemGetInfo): it sees any allocation, by anyone, torch's
        # allocator or not. The first call on a device may still load the library's code and its fixed array, so the
        # claim is checked on the second.
        before_driver, before_torch = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        status = _call(lib, "ep_lattice_decode_static", buffers, out, rows, cols, prob_bits, tile_elements, alphabet, ())
        assert status == 0, _native.load().ep_status_string(status)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before_torch
        if attempt > 0:
            assert torch.cuda.mem_get_info()[0] == before_driver
        assert torch.equal(out.view(torch.int16), expected.view(torch.int16)), f"call {attempt + 1} differs"
        assert _call(lib, "ep_lattice_decode_static", other_buffers, other_out, int(other["shape"][0]), other_cols, other_pb,
                     other_tile, int(buffers_of(other)["stream_meta"][:, 3].max()), ()) == 0
        torch.cuda.synchronize()
        assert other_out[:, : int(other["shape"][1])].contiguous().cpu().view(torch.uint8).numpy().tobytes() == other["decoded_bytes"].tobytes()


def test_static_scratch_decode_refuses_oversized_tables():
    from entropack_b200 import _native

    lib = _native.load()
    record = load_golden("lattice_bf16_10p5_wide")
    buffers = _device_buffers(record)
    rows = int(record["shape"][0])
    cols, _prob_bits, tile_elements = (int(v) for v in buffers_of(record)["layout"])
    out = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
    too_wide = lib.ep_lattice_decode_static_max_prob_bits() + 1
    status = _call(lib, "ep_lattice_decode_static", buffers, out, rows, cols, too_wide, tile_elements, 600, ())
    assert status == -6  # EP_ERR_TOO_LARGE
    assert b"too large" in lib.ep_status_string(status)
