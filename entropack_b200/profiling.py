"""Runs one kernel of the hot path a few times on a seeded synthetic case, for use under a profiler.

    python -m entropack_b200.profiling --op tile_ans_decode --kind fp8_e4m3 --rows 8192 --cols 8192 --reps 3

Set-up (tensor generation, encoding) happens first; the profiled kernel then runs ``--reps`` times
back to back, so ``ncu -k regex:<kernel> -c <reps>`` captures exactly those launches.
"""
import argparse

import torch


def make_tensor(kind: str, rows: int, cols: int, device, seed: int = 1) -> torch.Tensor:
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


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--op", default="tile_ans_decode",
                        choices=("tile_ans_decode", "tile_ans_encode", "lattice_decode", "lattice_encode", "dfloat11_decode",
                                 "dfloat11_encode", "linear"))
    parser.add_argument("--bpp", type=float, default=4.0)
    parser.add_argument("--kind", default="fp8_e4m3")
    parser.add_argument("--rows", type=int, default=8192)
    parser.add_argument("--cols", type=int, default=8192)
    parser.add_argument("--reps", type=int, default=3)
    parser.add_argument("--tile-elements", type=int, default=0, help="tile-ANS tile size (0 = automatic)")
    parser.add_argument("--inner", type=int, default=3840, help="linear: K (rows = tokens M, cols = features N)")
    parser.add_argument("--operand", default="bf16", choices=("bf16", "fp8", "int8"), help="linear: operand type of the product")
    args = parser.parse_args()

    import entropack_b200 as ep

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.op == "linear":
        from entropack_b200.linear import linear_forward

        weight = make_tensor("bf16", args.cols, args.inner, device)
        tokens = make_tensor("bf16", args.rows, args.inner, device, seed=2) * 50
        if args.operand == "bf16":
            for _ in range(args.reps):
                out = linear_forward(tokens, weight)
        else:
            # 8-bit codes with per-row scales, as the quantised layers hand them to the kernel
            from entropack_b200 import _native

            lib = _native.load()
            if args.operand == "fp8":
                entry, codes_x, codes_w = lib.ep_linear_forward_fp8, tokens.to(torch.float8_e4m3fn), (weight * 50).to(torch.float8_e4m3fn)
            else:
                entry, codes_x, codes_w = lib.ep_linear_forward_int8, tokens.round().clamp(-127, 127).to(torch.int8), (weight * 2000).round().clamp(-127, 127).to(torch.int8)
            scale_x = torch.full((args.rows,), 0.02, device=device)
            scale_w = torch.full((args.cols,), 0.01, device=device)
            out = torch.empty((args.rows, args.cols), dtype=torch.bfloat16, device=device)
            for _ in range(args.reps):
                _native.check(entry(_native.ptr(codes_x), _native.ptr(codes_w), _native.ptr(scale_x), _native.ptr(scale_w), None,
                                    _native.ptr(out), 0, args.rows, args.cols, args.inner, None, _native.stream_handle(device)),
                              "8-bit linear forward")
        torch.cuda.synchronize()
        print(f"linear {args.operand} M={args.rows} N={args.cols} K={args.inner}: {args.reps} launches")
        return
    tensor = make_tensor(args.kind, args.rows, args.cols, device)
    config = ep.TileANSConfig(tile_elements=args.tile_elements)
    if args.op.startswith("lattice"):
        config = ep.EntroPackLossyConfig(target_bpp=args.bpp)
    elif args.op.startswith("dfloat11"):
        config = ep.DFloat11Config()
    if args.op.endswith("_decode") and not args.op.startswith("tile_ans"):
        container = ep.compress(tensor, config)
        torch.cuda.synchronize()
        for _ in range(args.reps):
            out = ep.decompress(container, config)
        torch.cuda.synchronize()
        print(f"{args.op} {args.kind} {args.rows}x{args.cols}: {container.actual_bpp:.4f} bpp, {args.reps} launches")
    elif args.op == "tile_ans_decode":
        container = ep.compress(tensor, config)
        torch.cuda.synchronize()
        for _ in range(args.reps):
            out = ep.decompress(container, config)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.uint8), tensor.view(torch.uint8))
        print(f"{args.op} {args.kind} {args.rows}x{args.cols}: {container.actual_bpp:.4f} bpp, {args.reps} launches")
    else:
        for _ in range(args.reps):
            container = ep.compress(tensor, config)
        torch.cuda.synchronize()
        print(f"{args.op} {args.kind} {args.rows}x{args.cols}: {container.actual_bpp:.4f} bpp, {args.reps} launches")


if __name__ == "__main__":
    main()
