"""The library's bf16 GEMM (streaming mma.sync kernel for up to 16 rows, tcgen05/TMEM kernel above) against an fp32 torch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,bias", [
    (1, 512, 1024, True), (4, 384, 3840, False), (16, 1000, 264, True),          # few tokens: the streaming kernel,
    (16, 3840, 3840, True), (3, 1001, 1000, False), (9, 3840, 10240, True),       # with ragged features and a ragged last slice,
    (16, 5000, 512, True), (16, 10240, 3840, False), (3, 10250, 264, True), (5, 11520, 264, False),   # 2, 3, 3 and 4 feature sets a block
    (17, 128, 64, False), (128, 128, 128, True), (256, 384, 1024, True),         # tensor-core kernel
    (300, 1000, 264, True), (130, 136, 3840, False), (1024, 3840, 3840, True),
    (4096, 3840, 3840, True), (1500, 10000, 1088, True), (2100, 4600, 1152, False),   # two-block tiles, whole and ragged
])
def test_matches_fp32_reference(m, n, k, bias):
    from entropack_b200.linear import linear_forward

    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = torch.randn(n, generator=g, device="cuda").to(torch.bfloat16) if bias else None
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = linear_forward(x, w, b, error=error)
    torch.cuda.synchronize()
    assert int(error.item()) == 0
    expected = x.float() @ w.float().t() + (b.float() if bias else 0.0)
    # tolerance from the metric definition: max |y - y_ref| / max |y_ref| <= 1e-2 (bf16 output rounding is ~4e-3)
    assert float((out.float() - expected).abs().max() / expected.abs().max()) <= 1e-2


# 16-byte row reads, element-wise fallback, two and four register-held reads per thread, rows too long to hold
@pytest.mark.parametrize("cols", [1000, 1001, 3840, 8192, 10240])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_fp8_row_quantisation_matches_the_torch_expression(dtype, cols):
    """Same scale and the same e4m3 codes, bit for bit, as QuantizedLinear._quantize_rows computes with torch ops."""
    from entropack_b200 import _native

    generator = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(37, cols, generator=generator, device="cuda") * 3).to(dtype)
    x[5] = 0          # an all-zero row takes the epsilon scale
    x[6, 10] = 7e4 if dtype is not torch.float16 else 6e4
    codes = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device="cuda")
    scales = torch.empty(x.shape[0], dtype=torch.float32, device="cuda")
    kind = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[dtype]
    _native.check(_native.load().ep_quantize_rows_fp8(_native.ptr(x), kind, x.shape[0], x.shape[1], _native.ptr(codes), _native.ptr(scales),
                                                      _native.stream_handle(x.device)), "quantise")
    flat = x.float()
    expected_scale = (flat.abs().amax(dim=1) / 448.0).clamp(min=torch.finfo(torch.float32).eps)
    expected_codes = (flat / expected_scale.unsqueeze(1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    assert torch.equal(scales, expected_scale)
    assert torch.equal(codes.view(torch.uint8), expected_codes.view(torch.uint8))


@pytest.mark.parametrize("m,n,k,out_dtype,with_bias", [
    (1, 768, 1024, torch.bfloat16, True), (16, 3840, 3840, torch.bfloat16, False), (200, 1000, 2048, torch.float32, True),
    (4096, 3840, 3840, torch.bfloat16, True), (300, 520, 4096, torch.bfloat16, False), (1500, 10000, 1152, torch.float32, True),
])
def test_fp8_gemm_matches_scaled_mm(m, n, k, out_dtype, with_bias):
    """tcgen05 kind::f8f6f4 kernel against torch._scaled_mm on the same codes and scales. Products of e4m3 values are
    exact in fp32, so only the summation order differs: 1e-4 of the largest output for fp32 results; bf16 results add
    their own rounding, half a unit in the 8th bit, 2^-8 relative."""
    from entropack_b200 import _native

    generator = torch.Generator(device="cuda").manual_seed(11)
    a = (torch.randn(m, k, generator=generator, device="cuda") * 50).clamp(-448, 448).to(torch.float8_e4m3fn)
    b = (torch.randn(n, k, generator=generator, device="cuda") * 50).clamp(-448, 448).to(torch.float8_e4m3fn)
    a_scale = torch.rand(m, generator=generator, device="cuda") * 0.01 + 0.001
    b_scale = torch.rand(n, generator=generator, device="cuda") * 0.01 + 0.001
    bias = torch.randn(n, generator=generator, device="cuda") if with_bias else None
    out = torch.empty((m, n), dtype=out_dtype, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    _native.check(_native.load().ep_linear_forward_fp8(
        _native.ptr(a), _native.ptr(b), _native.ptr(a_scale), _native.ptr(b_scale), _native.ptr(bias), _native.ptr(out),
        int(out_dtype == torch.float32), m, n, k, _native.ptr(error), _native.stream_handle(out.device)), "fp8 gemm")
    assert int(error.item()) == 0
    expected = (a.float() @ b.float().t()) * a_scale.unsqueeze(1) * b_scale.unsqueeze(0)
    if bias is not None:
        expected = expected + bias
    assert float((out.float() - expected).abs().max() / expected.abs().max()) <= (1e-4 if out_dtype is torch.float32 else 2.0 ** -8)
    if n % 16 == 0 and k % 16 == 0 and out_dtype is torch.bfloat16:
        library = torch._scaled_mm(a, b.t(), scale_a=a_scale.unsqueeze(1), scale_b=b_scale.unsqueeze(0),
                                   bias=None if bias is None else bias.to(torch.bfloat16), out_dtype=torch.bfloat16)
        assert float((out.float() - library.float()).abs().max() / expected.abs().max()) <= 1e-2


@pytest.mark.parametrize("cols", [777, 2048, 3840, 8192, 10240])
def test_int8_row_quantisation_matches_the_torch_expression(cols):
    from entropack_b200 import _native

    generator = torch.Generator(device="cuda").manual_seed(4)
    x = (torch.randn(33, cols, generator=generator, device="cuda") * 3).to(torch.bfloat16)
    x[2] = 0
    x[3, :8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 127.0, -127.0], device="cuda").to(torch.bfloat16) * (x[3].abs().max() / 127)
    codes = torch.empty(x.shape, dtype=torch.int8, device="cuda")
    scales = torch.empty(x.shape[0], dtype=torch.float32, device="cuda")
    _native.check(_native.load().ep_quantize_rows_int8(_native.ptr(x), 0, x.shape[0], x.shape[1], _native.ptr(codes), _native.ptr(scales),
                                                       _native.stream_handle(x.device)), "quantise")
    flat = x.float()
    expected_scale = (flat.abs().amax(dim=1) / 127.0).clamp(min=torch.finfo(torch.float32).eps)
    expected_codes = (flat / expected_scale.unsqueeze(1)).round().clamp(-127.0, 127.0).to(torch.int8)
    assert torch.equal(scales, expected_scale)
    assert torch.equal(codes, expected_codes)


@pytest.mark.parametrize("m,n,k,out_dtype,with_bias", [
    (1, 768, 1024, torch.float32, True), (40, 1000, 2048, torch.float32, False), (4096, 3840, 3840, torch.bfloat16, True),
    (2100, 4600, 1152, torch.float32, False),
])
def test_int8_gemm_is_the_exact_integer_product_scaled(m, n, k, out_dtype, with_bias):
    """kind::i8 accumulates in 32-bit integers, so the product itself is exact; what remains is one fp32 multiply-add
    per output (1e-6 relative to the largest output) and, for bf16 results, their rounding (2^-8)."""
    from entropack_b200 import _native

    generator = torch.Generator(device="cuda").manual_seed(12)
    a = torch.randint(-127, 128, (m, k), generator=generator, device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (n, k), generator=generator, device="cuda", dtype=torch.int8)
    a_scale = torch.rand(m, generator=generator, device="cuda") * 0.01 + 0.001
    b_scale = torch.rand(n, generator=generator, device="cuda") * 0.01 + 0.001
    bias = torch.randn(n, generator=generator, device="cuda") if with_bias else None
    out = torch.empty((m, n), dtype=out_dtype, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    _native.check(_native.load().ep_linear_forward_int8(
        _native.ptr(a), _native.ptr(b), _native.ptr(a_scale), _native.ptr(b_scale), _native.ptr(bias), _native.ptr(out),
        int(out_dtype == torch.float32), m, n, k, _native.ptr(error), _native.stream_handle(out.device)), "int8 gemm")
    assert int(error.item()) == 0
    exact = (a.double() @ b.double().t()) * a_scale.double().unsqueeze(1) * b_scale.double().unsqueeze(0)
    if bias is not None:
        exact = exact + bias.double()
    tolerance = 1e-6 if out_dtype is torch.float32 else 2.0 ** -8
    assert float((out.double() - exact).abs().max() / exact.abs().max()) <= tolerance


def test_scattered_product_writes_its_columns_into_every_destination():
    """ep_linear_forward_scatter on one GPU: the product lands in columns [col0, col0 + n) of rows that are ld elements
    long, in the local destination and in a second one standing in for a peer's buffer; everything else stays as it was,
    and the values equal ep_linear_forward's."""
    import ctypes

    from entropack_b200 import _native
    from entropack_b200.linear import linear_forward

    lib = _native.load()
    generator = torch.Generator(device="cuda").manual_seed(17)
    stream = torch.cuda.current_stream().cuda_stream
    for tokens, columns, inner, ld, col0 in ((300, 480, 1024, 3840, 960), (4096, 256, 512, 1032, 8), (129, 72, 64, 100, 20), (1000, 200, 256, 404, 4)):
        x = torch.randn(tokens, inner, generator=generator, device="cuda").to(torch.bfloat16)
        w = (torch.randn(columns, inner, generator=generator, device="cuda") * 0.05).to(torch.bfloat16)
        bias = torch.randn(columns, generator=generator, device="cuda").to(torch.bfloat16)
        expected = linear_forward(x, w, bias)
        local = torch.full((tokens, ld), 7.0, dtype=torch.bfloat16, device="cuda")
        peer = torch.full((tokens, ld), 7.0, dtype=torch.bfloat16, device="cuda")
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        peers = (ctypes.c_void_p * 1)(peer.data_ptr())
        status = lib.ep_linear_forward_scatter(x.data_ptr(), w.data_ptr(), bias.data_ptr(), local.data_ptr(), peers, 1, ld, col0, tokens,
                                               columns, inner, error.data_ptr(), stream)
        assert status == 0, lib.ep_status_string(status)
        torch.cuda.synchronize()
        assert int(error.item()) == 0
        for destination in (local, peer):
            assert torch.equal(destination[:, col0:col0 + columns].view(torch.int16), expected.view(torch.int16))
            untouched = torch.cat([destination[:, :col0], destination[:, col0 + columns:]], dim=1)
            assert bool((untouched == 7.0).all())
    few = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    assert lib.ep_linear_forward_scatter(few.data_ptr(), few.data_ptr(), None, out.data_ptr(), None, 0, 64, 0, 128, 64, 64, None, stream) == -2


def test_peer_barrier_passes_on_arrival_and_gives_up_on_a_peer_that_never_arrives():
    """The barrier's wait is bounded: with the peer's arrival already in this rank's flag row it returns at once and
    leaves its own arrival in the peer's row; with a flag that nothing sets it gives up after the time limit, records
    the timeout in the error word and returns -- the context stays usable."""
    import ctypes
    import time

    from entropack_b200 import _native

    lib = _native.load()
    stream = torch.cuda.current_stream().cuda_stream
    mine = torch.zeros(4, dtype=torch.int32, device="cuda")      # rank 0's row
    theirs = torch.zeros(4, dtype=torch.int32, device="cuda")    # rank 1's row, standing in for a peer mapping
    rows = (ctypes.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    mine[1] = 5                                                   # the peer arrived at epoch 5 already
    assert lib.ep_peer_barrier(rows, 0, 2, 5, 50_000, error.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(error.item()) == 0 and int(theirs[0].item()) == 5
    begin = time.perf_counter()
    assert lib.ep_peer_barrier(rows, 0, 2, 6, 20_000, error.data_ptr(), stream) == 0    # epoch 6 never comes: 20 ms limit
    torch.cuda.synchronize()
    assert time.perf_counter() - begin < 2.0
    assert int(error.item()) == 9 and int(theirs[0].item()) == 6
    assert torch.equal(mine.cpu(), torch.tensor([0, 5, 0, 0], dtype=torch.int32))
    assert lib.ep_peer_barrier(rows, 0, 9, 1, 1000, None, stream) == -1 and lib.ep_peer_barrier(rows, 2, 2, 1, 1000, None, stream) == -1
