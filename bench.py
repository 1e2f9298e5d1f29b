#!/usr/bin/env python
"""Benchmark of the compression hot path: lossless Tile-ANS decode throughput.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python bench.py --only <kernel> [--kind ...] [--rows R] [--cols C] [--bpp B] [--reps N]     (see run_only)

Workload ("c2_tile_ans_decode"): the four 8192 x 8192 tensors of the lossless benchmark config --
fp8 e4m3 (N(0,1) scaled to amax 448), int8 (round(N(0,20^2)) clipped to +-127), fp16 and fp32
(N(0,0.02^2)) -- seeded synthetic data, compressed once at set-up. One step decodes all four
containers. Bytes per step = container bytes (header excluded) read once + dense bytes written once.

  value      device-resident throughput: containers already in HBM, K steps timed with CUDA events
             (one region per step, a 512 MB L2 flush between steps outside the timed regions).
  e2e        the same decode through the public API starting from pinned HOST blobs: host->device
             copy of each blob, decode, device->host copy of each dense result, all inside the timed
             region. `to_device_only_per_gpu_GBps_rank0` beside it: the same call leaving the results on
             the device (a checkpoint load), one byte read back.
  roofline   per-launch CUDA-event timing of the decode kernel (the only kernel in the step):
             algorithmic bytes / average launch time against the measured HBM copy bandwidth.
  cpu_baseline / --impl reference
             the CPU oracle (a C port of the reference's eager lane, OpenMP over tiles) decoding a
             quarter-height sample of the same four tensors on the host cores.

With N > 1 (torchrun, one rank per GPU) every rank decodes its own copy of the workload (weak
scaling, no collective on the data path); the time is the max over ranks. The one collective of the
package, the output all-gather of the column-sharded linear, is timed beside it ("sharded_linear").
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

KINDS = ("fp8_e4m3", "int8", "fp16", "fp32")
SEEDS = {"fp8_e4m3": 1, "int8": 2, "fp16": 3, "fp32": 4}
ROWS, COLS = 8192, 8192
METRIC = "decode GB/s/GPU (HBM frac)"


# dram__bytes_read.sum + dram__bytes_write.sum of the four decode launches of one step, one ncu capture per tensor
# kind (`ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none -k regex:tile_ans_decode
# -s 1 -c 1 python bench.py --only tile_ans_decode --kind <kind> --reps 2`). A capture, not a live measurement: it is
# dated, and goes stale when the decode kernel's memory behaviour changes.
DRAM_TRAFFIC = {"captured": "2026-11-25", "bytes": {"fp8_e4m3": 86.55e6, "int8": 85.29e6, "fp16": 220.24e6, "fp32": 468.38e6}}
DRAM_TRAFFIC_BYTES = float(sum(DRAM_TRAFFIC["bytes"].values()))


def make_tensor(kind: str, rows: int, cols: int, device) -> torch.Tensor:
    generator = torch.Generator(device=device).manual_seed(SEEDS[kind])
    x = torch.randn(rows, cols, generator=generator, device=device)
    if kind == "fp8_e4m3":
        return (x * (448.0 / x.abs().max())).to(torch.float8_e4m3fn)
    if kind == "int8":
        return (x * 20).round().clamp(-127, 127).to(torch.int8)
    if kind == "fp16":
        return (x * 0.02).to(torch.float16)
    return x * 0.02


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class L2Flush:
    """Writes a 512 MB buffer (four times the L2), then reads it back: the write throws everything else out of
    L2, the read leaves L2 holding clean lines, so the kernel timed next does not pay for writing back the
    flush's own dirty lines."""

    def __init__(self, device):
        self.buffer = torch.empty(128 * 1024 * 1024, dtype=torch.int32, device=device)

    def __call__(self):
        self.buffer.zero_()
        self.buffer.sum()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines: list[str] = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._drain, daemon=True)
        self.thread.start()

    def _drain(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(clocks)[len(clocks) // 2:] if clocks else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max_clock, "reasons": sorted(reasons),
                "samples": len(clocks)}


# ------------------------------------------------------------------------------------------------
# --only: one kernel of the hot path, a few launches on a seeded synthetic case (the command that
# goes under a profiler: `ncu -k regex:<kernel> -c <reps> ... python bench.py --only <op> ...`)
# ------------------------------------------------------------------------------------------------
ONLY_OPS = ("tile_ans_decode", "tile_ans_encode", "lattice_decode", "lattice_encode", "dfloat11_decode", "dfloat11_encode",
            "linear", "layer_forward")


def make_case(kind: str, rows: int, cols: int, device, seed: int = 1) -> torch.Tensor:
    generator = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(rows, cols, generator=generator, device=device)
    if kind == "fp8_e4m3":
        return (x * (448.0 / x.abs().max())).to(torch.float8_e4m3fn)
    if kind == "int8":
        return (x * 20).round().clamp(-127, 127).to(torch.int8)
    if kind == "int8_narrow":
        return (x * 2).round().clamp(-127, 127).to(torch.int8)
    if kind == "fp16":
        return (x * 0.02).to(torch.float16)
    if kind == "bf16":
        return (x * 0.02).to(torch.bfloat16)
    if kind == "fp32":
        return x * 0.02
    if kind == "bf16_outliers":
        # 1 % of the rows heavy-tailed (Student-t, 3 degrees of freedom): the lossy benchmark tensor
        picks = torch.randperm(rows, generator=generator, device=device)[: max(1, rows // 100)]
        student = torch.randn(picks.numel(), cols, generator=generator, device=device) / \
            torch.randn(picks.numel(), cols, 3, generator=generator, device=device).square().mean(-1).sqrt()
        x[picks] = student
        return (x * 0.02).to(torch.bfloat16)
    if kind == "int16_pair":
        # two independent small-valued bytes per element: both byte lanes are entropy coded
        low = (x * 20).round().clamp(-127, 127).to(torch.int16) & 0xFF
        high = (torch.randn(rows, cols, generator=generator, device=device) * 20).round().clamp(-127, 127).to(torch.int16)
        return low | (high << 8)
    raise ValueError(kind)


def run_only(args) -> None:
    """Set-up (tensor generation, encoding) first; then the chosen kernel runs ``--reps`` times back to back, each launch
    timed with CUDA events after a 512 MB L2 flush (a profiler's `-k regex:<kernel> -c <reps>` captures exactly those)."""
    import entropack_b200 as ep

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    stream = torch.cuda.current_stream(device)
    flush = L2Flush(device)
    rows, cols = args.rows, args.cols

    def repeat(fn):
        times = []
        for _ in range(args.reps):
            flush()
            torch.cuda._sleep(1_000_000)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            out = fn()
            end.record(stream)
            end.synchronize()
            times.append(begin.elapsed_time(end) * 1e3)
        return out, times

    report = {"op": args.only, "kind": args.kind, "rows": rows, "cols": cols, "reps": args.reps}
    if args.only == "linear":
        from entropack_b200 import _native
        from entropack_b200.linear import linear_forward

        weight = make_case("bf16", cols, args.inner, device)
        tokens = make_case("bf16", rows, args.inner, device, seed=2) * 50
        if args.operand == "bf16":
            _, times = repeat(lambda: linear_forward(tokens, weight))
        else:
            # 8-bit codes with per-row scales, as the quantised layers hand them to the kernel
            lib = _native.load()
            if args.operand == "fp8":
                entry, codes_x, codes_w = lib.ep_linear_forward_fp8, tokens.to(torch.float8_e4m3fn), (weight * 50).to(torch.float8_e4m3fn)
            else:
                entry, codes_x, codes_w = (lib.ep_linear_forward_int8, tokens.round().clamp(-127, 127).to(torch.int8),
                                           (weight * 2000).round().clamp(-127, 127).to(torch.int8))
            scale_x = torch.full((rows,), 0.02, device=device)
            scale_w = torch.full((cols,), 0.01, device=device)
            out = torch.empty((rows, cols), dtype=torch.bfloat16, device=device)
            _, times = repeat(lambda: _native.check(entry(
                _native.ptr(codes_x), _native.ptr(codes_w), _native.ptr(scale_x), _native.ptr(scale_w), None, _native.ptr(out), 0, rows,
                cols, args.inner, None, _native.stream_handle(device)), "8-bit linear forward"))
        report.update(operand=args.operand, inner=args.inner, us=times)
    elif args.only == "layer_forward":
        # CompressedLinear.forward (decode + product, or the fused kernel for one token on a large layer): rows = tokens, cols = out features
        dense = torch.nn.Linear(args.inner, cols, bias=False, device=device, dtype=torch.bfloat16)
        with torch.no_grad():
            dense.weight.copy_(make_case("bf16", cols, args.inner, device))
        options = {"tile_elements": args.tile_elements} if args.tile_elements else {}
        layer = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=args.bpp, **options))
        x = make_case("bf16", rows, args.inner, device, seed=2) * 50
        with torch.no_grad():
            _, times = repeat(lambda: layer(x))
        report.update(inner=args.inner, bits=layer.compressed_bits, us=times)
    else:
        tensor = make_case(args.kind, rows, cols, device)
        if args.only.startswith("lattice"):
            options = {"tile_elements": args.tile_elements} if args.tile_elements else {}
            config = ep.EntroPackLossyConfig(target_bpp=args.bpp, **options)
        elif args.only.startswith("dfloat11"):
            config = ep.DFloat11Config()
        else:
            config = ep.TileANSConfig(tile_elements=args.tile_elements)
        if args.only.endswith("_decode"):
            container = ep.compress(tensor, config)
            torch.cuda.synchronize(device)
            out, times = repeat(lambda: ep.decompress(container, config))
            if container.lossless:
                assert torch.equal(out.view(torch.uint8), tensor.view(torch.uint8))
            nbytes = container.storage_nbytes(include_header=False) + tensor.numel() * tensor.element_size()
        else:
            container, times = repeat(lambda: ep.compress(tensor, config))
            nbytes = container.storage_nbytes(include_header=False) + tensor.numel() * tensor.element_size()
        report.update(bpp=container.actual_bpp, algorithmic_bytes=nbytes, us=times,
                      GBps=[nbytes / (t * 1e-6) / 1e9 for t in times])
    torch.cuda.synchronize(device)
    print(json.dumps(report))


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle port on host cores
# ------------------------------------------------------------------------------------------------
def cpu_workload(sample_rows: int):
    import oracle

    oracle.build()
    work = []
    for kind in KINDS:
        tensor = make_tensor(kind, sample_rows, COLS, "cpu")
        raw = tensor.view(torch.uint8).numpy().reshape(-1)
        buffers = oracle.tile_ans_encode(raw, tensor.element_size(), 8192)
        nbytes = sum(int(np.asarray(v).nbytes) for v in buffers.values()) + raw.nbytes
        work.append((buffers, raw, nbytes))
    return oracle, work


def time_cpu(steps: int, warmup: int, sample_rows: int) -> dict:
    oracle, work = cpu_workload(sample_rows)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    # torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm is meant to use every host thread it may run on
    oracle.set_threads(cores)
    total_bytes = sum(nbytes for _, _, nbytes in work)
    for _ in range(warmup):
        for buffers, _, _ in work:
            oracle.tile_ans_decode(buffers)
    begin = time.perf_counter()
    for _ in range(steps):
        for buffers, raw, _ in work:
            out = oracle.tile_ans_decode(buffers)
    elapsed = time.perf_counter() - begin
    assert np.array_equal(out, work[-1][1])
    return {
        "value": total_bytes * steps / elapsed / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
        "sample": f"rows 0..{sample_rows - 1} of each of the four 8192x8192 tensors ({sample_rows}x{COLS} per dtype), "
                  f"{steps} passes, OpenMP over tiles",
        "ms_per_step": elapsed / steps * 1e3, "bytes_per_step": total_bytes,
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    result = time_cpu(args.steps, args.warmup, sample_rows=2048)
    line = {
        "impl": "reference", "metric": METRIC, "value": result["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": result["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "c2_tile_ans_decode", "tensors": list(KINDS), "shape": [ROWS, COLS],
                   "note": "reference is Python; its eager lane is timed through the C oracle port on host cores"},
        "cpu_baseline": {k: result[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": result["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# B200 arm
# ------------------------------------------------------------------------------------------------
def run_b200(args) -> None:
    import entropack_b200 as ep
    from entropack_b200 import _native
    from entropack_b200.schemes.tile_ans import b200 as lane
    from entropack_b200.schemes.tile_ans.format import TileBuffers, parse_layout_cached

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    # keep this rank's host thread, and the pinned buffers it allocates, on the socket its GPU hangs off (undone before the
    # CPU baseline, which uses every host thread)
    from entropack_b200 import sharding

    original_cpus = os.sched_getaffinity(0)
    bound_cpus = sharding.bind_host_thread_near(device)
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    config = ep.TileANSConfig()
    containers, launches, dense_bytes, stored_bytes = [], [], 0, 0
    lib = _native.load()
    stream = torch.cuda.current_stream(device)
    for kind in KINDS:
        tensor = make_tensor(kind, ROWS, COLS, device)
        container = ep.compress(tensor, config)
        assert container.compress_method == "tile_ans"
        check = ep.decompress(container, config)
        assert torch.equal(check.view(torch.uint8), tensor.view(torch.uint8)), f"{kind}: round trip is not bit-exact"
        del check
        buffers = TileBuffers(**container.buffers)
        tile_elements, prob_bits, lanes, elements = parse_layout_cached(buffers.layout)
        modes = np.ascontiguousarray(buffers.lane_modes.cpu().numpy())
        output = torch.empty(elements * lanes, dtype=torch.uint8, device=device)
        arguments = (
            buffers.payload.data_ptr(), buffers.payload.numel(), buffers.offsets.data_ptr(), buffers.states.data_ptr(),
            buffers.decode_tables.data_ptr(), modes.ctypes.data, output.data_ptr(), elements, tile_elements, prob_bits, lanes,
            None, stream.cuda_stream)
        launches.append((kind, arguments, modes, output, tensor))
        containers.append(container)
        dense_bytes += elements * lanes
        stored_bytes += container.storage_nbytes(include_header=False)
    bytes_per_step = dense_bytes + stored_bytes
    per_kind_bytes = [c.storage_nbytes(include_header=False) + c.numel() * c.element_size() for c in containers]

    flush = L2Flush(device)

    def step():
        for _, arguments, *_ in launches:
            status = lib.ep_tile_ans_decode(*arguments)
            if status != 0:
                _native.check(status, "tile_ans decode")

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(device)
    for kind, _, _, output, tensor in launches:
        assert torch.equal(output, tensor.view(torch.uint8).reshape(-1)), f"{kind}: decode differs from the source"

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for index in range(args.steps):
        flush()
        starts[index].record(stream)
        step()
        stops[index].record(stream)
    barrier()
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = float(sum(step_ms))

    # per-launch timing of the decode kernel for the roofline
    kernel_ms = [0.0] * len(launches)
    for _ in range(args.steps):
        flush()
        for index, (_, arguments, *_rest) in enumerate(launches):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            lib.ep_tile_ans_decode(*arguments)
            end.record(stream)
            end.synchronize()
            kernel_ms[index] += begin.elapsed_time(end)
    kernel_ms = [v / args.steps for v in kernel_ms]

    # the other decoders and the encoders of the hot path, timed the same way (L2 flushed before every launch);
    # reported for context under "others", not part of the headline value
    others = measure_others(ep, device, flush, args.steps) if not args.headline_only else {}

    # whole-model encode: this rank's share of the synthetic 276-linear DiT at 4 bpp (layers sharded, no collectives)
    model = measure_model_encode(ep, device, rank, world) if not args.headline_only else {
        "seconds": 0.0, "layers": 0, "bpp": 0.0, "decode_seconds": 0.0, "forward_seconds": 0.0, "forward_graph_seconds": None,
        "plans": 0, "plans_seconds": 0.0, "forward_ahead_seconds": 0.0, "forward_ahead_graph_seconds": None,
        "mixed_seconds": 0.0, "mixed_bpp": 0.0}

    # the package's one collective: the output all-gather of a column-sharded layer (every rank takes part)
    sharded = measure_sharded_linear(ep, device, rank, world, args.steps) if distributed and not args.headline_only else {}

    # end to end through the public API from pinned host blobs
    host_blobs = [c.entropack_quant_state.cpu().pin_memory() for c in containers]
    host_outputs = [torch.empty(c.numel() * c.element_size(), dtype=torch.uint8).pin_memory() for c in containers]
    h2d_bytes = sum(b.numel() for b in host_blobs)
    d2h_bytes = sum(o.numel() for o in host_outputs)

    def e2e_step():
        # the public bulk call: upload, decode and download of successive tensors overlap on three streams
        ep.decompress_many(host_blobs, config, device=device, out=host_outputs)
        torch.cuda.synchronize(device)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(2, min(args.steps, 5))
    barrier()
    e2e_begin = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_seconds = time.perf_counter() - e2e_begin
    clocks = sampler.stop() if rank == 0 else None
    assert torch.equal(host_outputs[0], launches[0][4].view(torch.uint8).reshape(-1).cpu())

    # For context, what loading a checkpoint costs: the same call without host outputs leaves the dense tensors on the
    # device (what a model wants), and the step reads one byte of the last one back. Not the headline: the reference arm
    # decodes into host memory, so the number compared with it keeps the full download.
    def load_step():
        dense = ep.decompress_many(host_blobs, config, device=device)
        return int(dense[-1].view(torch.uint8).reshape(-1)[-1].item())

    load_step()
    barrier()
    load_begin = time.perf_counter()
    for _ in range(e2e_steps):
        load_step()
    barrier()
    load_seconds = time.perf_counter() - load_begin

    if distributed:
        timed_keys = ("seconds", "decode_seconds", "forward_seconds", "mixed_seconds")
        times = torch.tensor([total_ms, e2e_seconds] + [model[key] for key in timed_keys], dtype=torch.float64, device=device)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        total_ms, e2e_seconds = float(times[0]), float(times[1])
        for position, key in enumerate(timed_keys):
            model[key] = float(times[2 + position])
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    ms_per_step = total_ms / args.steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    kernel_seconds = sum(kernel_ms) * 1e-3
    achieved = bytes_per_step / kernel_seconds / 1e9
    os.sched_setaffinity(0, original_cpus)
    if args.headline_only:
        cpu = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": "skipped (--headline-only)"}
    else:
        cpu = time_cpu(steps=3, warmup=1, sample_rows=2048)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": "c2_tile_ans_decode", "tensors": list(KINDS), "shape": [ROWS, COLS],
                   "bytes_per_step": bytes_per_step, "stored_bpp": {k: round(c.actual_bpp, 4) for k, c in zip(KINDS, containers)},
                   "l2": "inputs larger than L2, plus a 512 MB write-then-read flush between timed steps", "per_gpu_GBps": value / world,
                   "hbm_frac_of_" + peak_kind: value / world / peak},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_kind, "traffic": DRAM_TRAFFIC_BYTES, "traffic_captured": DRAM_TRAFFIC["captured"],
                     "kernel": "tile_ans_decode_kernel",
                     "per_launch_ms": dict(zip(KINDS, kernel_ms)),
                     "per_launch_GBps": {k: b / (ms * 1e-3) / 1e9 for k, b, ms in zip(KINDS, per_kind_bytes, kernel_ms)}},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": world * bytes_per_step * e2e_steps / e2e_seconds / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps,
                "per_gpu_GBps": bytes_per_step * e2e_steps / e2e_seconds / 1e9,
                "host_cpus_near_gpu": None if bound_cpus is None else len(bound_cpus),
                "to_device_only_per_gpu_GBps_rank0": bytes_per_step * e2e_steps / load_seconds / 1e9},
        "others": others,
        "sharded_linear": sharded,
        "model_encode": {"workload": "synthetic DiT, 276 linears (hidden 3840, mlp 10240), bf16 N(0,0.02^2), 4 bpp, layers sharded "
                                     "largest-first over the ranks", "seconds": model["seconds"], "layers_on_rank0": model["layers"],
                         "mean_bpp_rank0": model["bpp"], "decode_all_seconds": model["decode_seconds"],
                         "decode_plans_built_rank0": model["plans"], "decode_plans_seconds_rank0": model["plans_seconds"],
                         "forward_4096_tokens_seconds": model["forward_seconds"],
                         "forward_4096_tokens_decode_ahead_seconds_rank0": model["forward_ahead_seconds"],
                         "forward_4096_tokens_three_runs_rank0": model.get("forward_runs"),
                         "forward_4096_tokens_decode_ahead_three_runs_rank0": model.get("forward_ahead_runs"),
                         "forward_4096_tokens_decode_ahead_cuda_graph_seconds_rank0": model["forward_ahead_graph_seconds"],
                         "forward_4096_tokens_cuda_graph_seconds_rank0": model["forward_graph_seconds"], "mixed_2p3_bpp_encode_seconds": model["mixed_seconds"],
                         "mixed_mean_bpp_rank0": model["mixed_bpp"]},
        "gpu_launches": len(launches) * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


def measure_sharded_linear(ep, device, rank: int, world: int, reps: int) -> dict:
    """Column-sharded CompressedLinear at 4096 tokens on two of the model's layer shapes: each rank holds N / G rows of
    the weight at 4 bpp, runs decode + product on its slice and the ranks all-gather the [M, N / G] outputs (the
    package's one collective). Device times (CUDA events, max over ranks) of the local forward, of the gather alone and
    of both; the gathered output is checked, bit for bit, against the same shards computed on one GPU."""
    import torch.distributed as dist

    from entropack_b200 import sharding

    stream = torch.cuda.current_stream(device)
    reps = max(3, min(reps, 10))
    results = {}

    def timed(fn):
        fn()
        total = 0.0
        for _ in range(reps):
            dist.barrier()
            torch.cuda.synchronize(device)
            # a spin of about a millisecond lets the host queue the whole call behind it, so that the events bracket
            # device work only and not the Python time between the two records
            torch.cuda._sleep(2_000_000)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            fn()
            end.record(stream)
            end.synchronize()
            total += begin.elapsed_time(end)
        worst = torch.tensor([total / reps], dtype=torch.float64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        return float(worst[0]) * 1e3

    config = ep.EntroPackLossyConfig(target_bpp=4.0)
    tokens = 4096
    for out_features, in_features in ((3840, 3840), (10240, 3840)):
        if out_features % world:
            continue
        generator = torch.Generator(device=device).manual_seed(77)       # the same weight and activations on every rank
        dense = torch.nn.Linear(in_features, out_features, bias=False, device=device, dtype=torch.bfloat16)
        with torch.no_grad():
            dense.weight.copy_((torch.randn(out_features, in_features, generator=generator, device=device) * 0.02).to(torch.bfloat16))
        x = torch.randn(tokens, in_features, generator=generator, device=device).to(torch.bfloat16)
        layer = sharding.ColumnShardedLinear(dense, config=config, exchange="gather")
        fused = sharding.ColumnShardedLinear(dense, config=config, exchange="auto")
        fused.local = layer.local          # one compressed shard serves both
        with torch.no_grad():
            out = layer(x)
            local = layer.local(x).contiguous()
            staging = torch.empty((world, *local.shape), dtype=local.dtype, device=device)
            entry = {
                "local_forward_us": timed(lambda: layer.local(x)),
                "all_gather_us": timed(lambda: dist.all_gather_into_tensor(staging.view(world * local.shape[0], local.shape[1]), local)),
                "all_gather_and_interleave_us": timed(lambda: sharding.gather_columns(local, None, staging)),
                "forward_gather_us": timed(lambda: layer(x)),
            }
            # the exchange folded into the product's epilogue: peer stores over NVLink + one bounded flag barrier
            scattered = fused(x).clone()
            fused.check()
            entry["scatter_unavailable"] = fused.scatter_unavailable
            if fused.scatter_unavailable is None:
                entry["forward_scatter_us"] = timed(lambda: fused(x))
                fused.check()
                entry["scatter_matches_gather"] = bool(torch.equal(scattered.view(torch.int16), out.view(torch.int16)))
            # the same row shards, compressed and multiplied one after the other on this GPU
            pieces = []
            for r in range(world):
                rows = sharding.row_slice(out_features, r, world)
                shard = torch.nn.Linear(in_features, rows.end - rows.begin, bias=False, device=device, dtype=torch.bfloat16)
                shard.weight.copy_(dense.weight[rows.begin:rows.end])
                pieces.append(ep.CompressedLinear.from_linear(shard, config=config)(x))
            identical = bool(torch.equal(out.view(torch.int16), torch.cat(pieces, dim=-1).view(torch.int16)))
        agree = torch.tensor([int(identical)], device=device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        received = (world - 1) * tokens * (out_features // world) * 2          # bytes each GPU receives = (G-1)/G * M * N * 2
        entry.update(matches_single_gpu=bool(int(agree[0])), bytes_received_per_gpu=received,
                     all_gather_GBps_per_gpu=received / entry["all_gather_us"] / 1e3,
                     nvlink_frac_of_770=received / entry["all_gather_us"] / 1e3 / 770.0)
        results[f"{in_features}x{out_features}_M{tokens}"] = entry
        del layer, fused, dense, pieces, staging
    return results


def measure_model_encode(ep, device, rank: int, world: int) -> dict:
    """This rank's share of the synthetic 276-linear DiT: every layer compressed at 4 bpp, then decoded, then run on
    4096 tokens (decode + product per layer, every layer fed its own width of seeded activations), then compressed
    again at the mixed per-layer targets that average 2.3 bpp. Wall-clock seconds around device-synchronised loops."""
    from entropack_b200 import sharding

    shapes = sharding.dit_layer_shapes()
    mine = sharding.partition_layers([r * c for r, c in shapes], world)[rank]
    targets = sharding.mixed_bit_targets(shapes)
    config = ep.EntroPackLossyConfig(target_bpp=4.0)
    warm = (torch.randn(3840, 3840, generator=torch.Generator(device=device).manual_seed(999), device=device) * 0.02).to(torch.bfloat16)
    ep.compress(warm, config)

    def layer_weights():
        generator = torch.Generator(device=device).manual_seed(1000 + rank)
        for index in mine:
            rows, cols = shapes[index]
            yield index, (torch.randn(rows, cols, generator=generator, device=device) * 0.02).to(torch.bfloat16)

    seconds, stored, elements, layers = 0.0, 0, 0, []
    for index, weight in layer_weights():
        torch.cuda.synchronize(device)
        begin = time.perf_counter()
        container = ep.compress(weight, config)
        torch.cuda.synchronize(device)
        seconds += time.perf_counter() - begin
        stored += container.storage_nbytes()
        elements += weight.numel()
        layer = ep.CompressedLinear(weight.shape[1], weight.shape[0], bias=False, config=config, device=device)
        layer.load_state_dict({"weight.entropack_quant_state": container.entropack_quant_state})
        layers.append(layer)

    # every layer's kept decode tables, built once as a serving process would after loading the checkpoint
    torch.cuda.synchronize(device)
    begin = time.perf_counter()
    plans = ep.prepare_decode_plans(torch.nn.ModuleList(layers))
    torch.cuda.synchronize(device)
    plans_seconds = time.perf_counter() - begin

    for layer in layers[:4]:
        layer.dequantize()
    torch.cuda.synchronize(device)
    begin = time.perf_counter()
    for layer in layers:
        layer.dequantize()
    torch.cuda.synchronize(device)
    decode_seconds = time.perf_counter() - begin

    generator = torch.Generator(device=device).manual_seed(2000 + rank)
    tokens = {width: torch.randn(4096, width, generator=generator, device=device).to(torch.bfloat16)
              for width in sorted({layer.in_features for layer in layers})}
    with torch.no_grad():
        for layer in layers[:4]:
            layer(tokens[layer.in_features])
        torch.cuda.synchronize(device)
        forward_runs = []
        for _ in range(3):          # wall-clock around one eager pass: the fastest of three is quoted, all three are reported
            begin = time.perf_counter()
            for layer in layers:
                layer(tokens[layer.in_features])
            torch.cuda.synchronize(device)
            forward_runs.append(time.perf_counter() - begin)
    forward_seconds = min(forward_runs)

    # the same pass with every layer's weight decoded ahead where that pays (two small layers in a row)
    with torch.no_grad(), ep.DecodeAhead(layers) as ahead:
        for layer in layers[:12]:
            layer(tokens[layer.in_features])
        ahead.drain()
        torch.cuda.synchronize(device)
        ahead_runs = []
        for _ in range(3):
            begin = time.perf_counter()
            for layer in layers:
                layer(tokens[layer.in_features])
            ahead.drain()
            torch.cuda.synchronize(device)
            ahead_runs.append(time.perf_counter() - begin)
        ahead_seconds = min(ahead_runs)

    # the same pass replayed from a CUDA graph: one submission for all the layers' kernels, no host work between them
    graph_seconds = None
    try:
        capture_stream = torch.cuda.Stream(device)
        capture_stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(capture_stream), torch.no_grad():
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=capture_stream):
                for layer in layers:
                    layer(tokens[layer.in_features])
        torch.cuda.current_stream(device).wait_stream(capture_stream)
        graph.replay()
        torch.cuda.synchronize(device)
        begin = time.perf_counter()
        graph.replay()
        torch.cuda.synchronize(device)
        graph_seconds = time.perf_counter() - begin
        del graph
    except Exception as error:      # capture is an optimisation of the host side only; report why it was not available
        graph_seconds = f"unavailable: {type(error).__name__}: {error}"[:200]

    # and the decode-ahead pass from a graph: the two streams' kernels become branches of the graph, with no host in between
    ahead_graph_seconds = None
    try:
        capture_stream = torch.cuda.Stream(device)
        capture_stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(capture_stream), torch.no_grad(), ep.DecodeAhead(layers, cyclic=False) as ahead:
            for layer in layers[:12]:
                layer(tokens[layer.in_features])
            ahead.drain()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=capture_stream):
                for layer in layers:
                    layer(tokens[layer.in_features])
                ahead.drain()
        torch.cuda.current_stream(device).wait_stream(capture_stream)
        graph.replay()
        torch.cuda.synchronize(device)
        begin = time.perf_counter()
        graph.replay()
        torch.cuda.synchronize(device)
        ahead_graph_seconds = time.perf_counter() - begin
        del graph
    except Exception as error:
        ahead_graph_seconds = f"unavailable: {type(error).__name__}: {error}"[:200]
    del layers, tokens

    mixed_seconds, mixed_stored = 0.0, 0
    for index, weight in layer_weights():
        mixed = ep.EntroPackLossyConfig(target_bpp=targets[index])
        torch.cuda.synchronize(device)
        begin = time.perf_counter()
        container = ep.compress(weight, mixed)
        torch.cuda.synchronize(device)
        mixed_seconds += time.perf_counter() - begin
        mixed_stored += container.storage_nbytes()
    return {"seconds": seconds, "layers": len(mine), "bpp": stored * 8 / max(1, elements), "decode_seconds": decode_seconds,
            "plans": plans, "plans_seconds": plans_seconds, "forward_ahead_seconds": ahead_seconds,
            "forward_runs": forward_runs, "forward_ahead_runs": ahead_runs,
            "forward_ahead_graph_seconds": ahead_graph_seconds,
            "forward_seconds": forward_seconds, "forward_graph_seconds": graph_seconds, "mixed_seconds": mixed_seconds, "mixed_bpp": mixed_stored * 8 / max(1, elements)}


def measure_others(ep, device, flush, reps: int) -> dict:
    """Device-resident timings of the remaining hot-path kernels on their benchmark configurations:
    DFloat11 on bf16 4096x4096, EntroPack-Lossy at 4 bpp on bf16 4096x11008 (1 % heavy-tailed rows)."""
    stream = torch.cuda.current_stream(device)
    reps = max(3, min(reps, 10))

    def timed(fn):
        fn()
        torch.cuda.synchronize(device)
        total = 0.0
        for _ in range(reps):
            flush()
            # a spin of about a millisecond lets the host queue the whole call behind it, so that the events
            # bracket device work only and not the Python time between the two records
            torch.cuda._sleep(2_000_000)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            fn()
            end.record(stream)
            end.synchronize()
            total += begin.elapsed_time(end)
        return total / reps

    results = {}
    generator = torch.Generator(device=device).manual_seed(0)
    weight = (torch.randn(4096, 4096, generator=generator, device=device) * 0.02).to(torch.bfloat16)
    config = ep.DFloat11Config()
    container = ep.compress(weight, config)
    assert torch.equal(ep.decompress(container, config).view(torch.int16), weight.view(torch.int16))
    nbytes = container.storage_nbytes(include_header=False) + weight.numel() * 2
    ms = timed(lambda: ep.decompress(container, config))
    results["dfloat11_decode_bf16_4096x4096"] = {"ms": ms, "GBps": nbytes / ms / 1e6, "bpp": container.actual_bpp}
    ms = timed(lambda: ep.compress(weight, config))
    results["dfloat11_encode_bf16_4096x4096"] = {"ms": ms, "GBps": nbytes / ms / 1e6}

    generator = torch.Generator(device=device).manual_seed(5)
    weight = torch.randn(4096, 11008, generator=generator, device=device) * 0.02
    heavy = torch.randperm(4096, generator=generator, device=device)[:41]
    student = torch.randn(41, 11008, generator=generator, device=device) / torch.randn(41, 11008, 3, generator=generator, device=device).square().mean(-1).sqrt()
    weight[heavy] = student * 0.02
    weight = weight.to(torch.bfloat16)
    for bpp in (2.3, 3.5, 4.0, 6.0):
        config = ep.EntroPackLossyConfig(target_bpp=bpp)
        container = ep.compress(weight, config)
        restored = ep.decompress(container, config)
        relative = float((restored.float() - weight.float()).norm() / weight.float().norm())
        nbytes = container.storage_nbytes(include_header=False) + weight.numel() * 2
        ms = timed(lambda: ep.decompress(container, config))
        results[f"lossy_decode_bf16_4096x11008_{bpp}bpp"] = {"ms": ms, "GBps": nbytes / ms / 1e6, "actual_bpp": container.actual_bpp,
                                                             "rel_l2": relative}
        ms = timed(lambda: ep.compress(weight, config))
        results[f"lossy_encode_bf16_4096x11008_{bpp}bpp"] = {"ms": ms, "GBps": nbytes / ms / 1e6}
    tensor = make_tensor("fp8_e4m3", ROWS, COLS, device)
    config = ep.TileANSConfig()
    ms = timed(lambda: ep.compress(tensor, config))
    results["tile_ans_encode_fp8_8192x8192"] = {"ms": ms}
    del tensor, weight, container

    # CompressedLinear forward (decode every call + library GEMM) against bf16 cuBLAS on the dense weight, L2 cold
    from entropack_b200.linear import linear_forward

    generator = torch.Generator(device=device).manual_seed(6)
    for out_features, in_features in ((3840, 3840), (10240, 3840)):
        dense = torch.nn.Linear(in_features, out_features, bias=False, device=device, dtype=torch.bfloat16)
        with torch.no_grad():
            dense.weight.copy_((torch.randn(out_features, in_features, generator=generator, device=device) * 0.02).to(torch.bfloat16))
        layer = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=4.0))
        decoded = layer.dequantize()
        # the same layer with the low-latency preset: half-length tiles halve the serial decode chain (reference-decodable)
        preset = ep.CompressedLinear.from_linear(dense, config=ep.EntroPackLossyConfig.low_latency(target_bpp=4.0))
        norm = dense.weight.float().norm()
        rel_l2 = float((decoded.float() - dense.weight.float()).norm() / norm)
        preset_rel_l2 = float((preset.dequantize().float() - dense.weight.float()).norm() / norm)
        for tokens in (1, 16, 256, 4096):
            x = torch.randn(tokens, in_features, generator=generator, device=device).to(torch.bfloat16)
            reference = torch.nn.functional.linear(x.float(), decoded.float())
            ours = layer(x)
            error = float((ours.float() - reference).abs().max() / reference.abs().max())
            entry = {
                "compressed_forward_us": timed(lambda: layer(x)) * 1e3,
                "library_gemm_us": timed(lambda: linear_forward(x, decoded)) * 1e3,
                "cublas_dense_us": timed(lambda: torch.nn.functional.linear(x, dense.weight)) * 1e3,
                "max_rel_err": error, "bits": layer.compressed_bits, "rel_l2": rel_l2,
                "low_latency_forward_us": timed(lambda: preset(x)) * 1e3, "low_latency_bits": preset.compressed_bits,
                "low_latency_rel_l2": preset_rel_l2,
            }
            if tokens == 4096:
                entry["library_gemm_tflops"] = 2.0 * tokens * out_features * in_features / entry["library_gemm_us"] / 1e6
                entry["cublas_tflops"] = 2.0 * tokens * out_features * in_features / entry["cublas_dense_us"] / 1e6
            if out_features == 3840:
                # what a call costs the host (Python + launches), taken while the device is kept busy by a spin, and the
                # wall-clock time per call of a plain loop of eager calls (the larger of host and device time)
                torch.cuda.synchronize(device)
                torch.cuda._sleep(200_000_000)
                begin = time.perf_counter()
                for _ in range(100):
                    layer(x)
                entry["host_us_per_call"] = (time.perf_counter() - begin) / 100 * 1e6
                torch.cuda.synchronize(device)
                begin = time.perf_counter()
                for _ in range(100):
                    layer(x)
                torch.cuda.synchronize(device)
                entry["eager_loop_us_per_call"] = (time.perf_counter() - begin) / 100 * 1e6
            results[f"linear_{in_features}x{out_features}_M{tokens}"] = entry

    # Decode-ahead: four different 3840 x 3840 layers called in a ring at 4096 tokens, each decoding its weight on every
    # call; plain (decode, then product) against DecodeAhead (the next layer's weight decoded on a second stream on 52
    # SMs while the current product runs on 96). Per-layer time over 16 calls inside one pair of events.
    x = torch.randn(4096, 3840, generator=generator, device=device).to(torch.bfloat16)
    for name, layer_cls, bpp in (("linear_ring_4x3840x3840_M4096", ep.CompressedLinear, 4.0),):
        ring = []
        for _ in range(4):
            dense = torch.nn.Linear(3840, 3840, bias=False, device=device, dtype=torch.bfloat16)
            with torch.no_grad():
                dense.weight.copy_((torch.randn(3840, 3840, generator=generator, device=device) * 0.02).to(torch.bfloat16))
            ring.append(layer_cls.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=bpp)))
        ep.prepare_decode_plans(torch.nn.ModuleList(ring))

        def ring_pass(calls=16):
            h = None
            for index in range(calls):
                h = ring[index % 4](x)
            return h

        plain_out = ring_pass(4)
        plain_us = timed(ring_pass) * 1e3 / 16
        with ep.DecodeAhead(ring) as ahead:
            ahead_out = ring_pass(4)
            ahead_us = timed(ring_pass) * 1e3 / 16
            found_ready = ahead.decoded_ahead
        results[name] = {"forward_us_per_layer": plain_us, "decode_ahead_forward_us_per_layer": ahead_us,
                         "weights_found_decoded": found_ready, "same_output": bool(torch.equal(plain_out, ahead_out))}
        # one token through the same ring: plain = decode, then the streaming product; decode-ahead = the next layer's
        # weight decoded while the streaming product of the current one runs on the same SMs
        one = x[:1].contiguous()

        def ring_pass_one(calls=16):
            h = None
            for index in range(calls):
                h = ring[index % 4](one)
            return h

        plain_one = ring_pass_one(4)
        plain_one_us = timed(ring_pass_one) * 1e3 / 16
        with ep.DecodeAhead(ring):
            ahead_one = ring_pass_one(4)
            ahead_one_us = timed(ring_pass_one) * 1e3 / 16
        results[name.replace("M4096", "M1")] = {
            "forward_us_per_layer": plain_one_us, "decode_ahead_forward_us_per_layer": ahead_one_us,
            "max_rel_difference": float((plain_one.float() - ahead_one.float()).abs().max() / plain_one.float().abs().max())}
        del ring
    del x

    # FP8 layer (codes lattice-coded at 5 bpp): activation quantisation + scaled fp8 product on the library's
    # tcgen05 kernel, against torch._scaled_mm on the same codes
    dense = torch.nn.Linear(3840, 3840, bias=False, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((torch.randn(3840, 3840, generator=generator, device=device) * 0.02).to(torch.bfloat16))
    layer = ep.CompressedFP8Linear.from_linear(dense, config=ep.EntroPackLossyConfig(target_bpp=5.0))
    codes, weight_scale = layer.codes(device), layer.weight_quant_scale.to(device)
    for tokens in (16, 4096):
        x = torch.randn(tokens, 3840, generator=generator, device=device).to(torch.bfloat16)
        a_codes, a_scale = layer._quantize_activations(x)
        expected = (a_codes.float() @ codes.float().t()) * a_scale.unsqueeze(1) * weight_scale.unsqueeze(0)
        produced = layer(x)
        entry = {
            "max_rel_err": float((produced.float() - expected).abs().max() / expected.abs().max()),
            "compressed_forward_us": timed(lambda: layer(x)) * 1e3,
            "quantize_activations_us": timed(lambda: layer._quantize_activations(x)) * 1e3,
            "library_fp8_gemm_us": timed(lambda: layer._gemm(a_codes, codes, a_scale, weight_scale, torch.bfloat16)) * 1e3,
            "scaled_mm_us": timed(lambda: torch._scaled_mm(a_codes, codes.t(), scale_a=a_scale.unsqueeze(1),
                                                           scale_b=weight_scale.unsqueeze(0), out_dtype=torch.bfloat16)) * 1e3,
            "bits": layer.compressed_bits,
        }
        if tokens == 4096:
            entry["library_fp8_gemm_tflops"] = 2.0 * tokens * 3840 * 3840 / entry["library_fp8_gemm_us"] / 1e6
            entry["scaled_mm_tflops"] = 2.0 * tokens * 3840 * 3840 / entry["scaled_mm_us"] / 1e6
        results[f"fp8_linear_3840x3840_M{tokens}"] = entry
    return results


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--headline-only", action="store_true",
                        help="time the headline workload and e2e only (no secondary kernels, model encode or CPU baseline): "
                             "the short command whose launch list goes under a profiler")
    parser.add_argument("--only", choices=ONLY_OPS, default=None, help="run one kernel a few times and print its timings (see run_only)")
    parser.add_argument("--kind", default="fp8_e4m3", help="--only: tensor kind (fp8_e4m3, int8, fp16, bf16, fp32, bf16_outliers, int16_pair)")
    parser.add_argument("--rows", type=int, default=8192, help="--only: rows (linear / layer_forward: tokens)")
    parser.add_argument("--cols", type=int, default=8192, help="--only: columns (linear / layer_forward: output features)")
    parser.add_argument("--inner", type=int, default=3840, help="--only linear / layer_forward: input features")
    parser.add_argument("--operand", default="bf16", choices=("bf16", "fp8", "int8"), help="--only linear: operand type")
    parser.add_argument("--bpp", type=float, default=4.0, help="--only lattice_* / layer_forward: target rate")
    parser.add_argument("--tile-elements", type=int, default=0, help="--only: tile size of the encoder (0 = automatic)")
    parser.add_argument("--reps", type=int, default=3, help="--only: timed launches")
    args = parser.parse_args()
    if args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
