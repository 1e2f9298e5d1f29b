"""Builds ``libentropack_b200.so`` (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python -m entropack_b200.build [--force] [--verbose]

Each source under ``csrc/`` is compiled to an object under ``build/`` (skipped when newer than its
inputs) and linked into ``entropack_b200/lib/libentropack_b200.so``. nvcc cross-compiles, so this
works on a machine without a GPU.
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
INCLUDE = ROOT / "include"
OBJECTS = ROOT / "build" / "obj"
LIBRARY = PACKAGE / "lib" / "libentropack_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the entropack_b200 kernels cannot be built")
    return nvcc


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers() -> list[Path]:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h")))


def _stale(target: Path, inputs) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(path.stat().st_mtime > stamp for path in inputs)


def _compile(source: Path, force: bool, verbose: bool) -> Path:
    obj = OBJECTS / (source.name + ".o")
    if force or _stale(obj, [source, *_headers(), Path(__file__)]):
        command = [_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, "-I", str(INCLUDE), "-c", str(source), "-o", str(obj)]
        if source.suffix == ".cpp":
            command = [c for c in command if c not in ("--expt-relaxed-constexpr",)]
        result = subprocess.run(command, capture_output=True, text=True)
        log = OBJECTS / (source.name + ".log")
        log.write_text(" ".join(command) + "\n" + result.stdout + result.stderr)
        if verbose or result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source.name} (see {log})")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJECTS.mkdir(parents=True, exist_ok=True)
    LIBRARY.parent.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(lambda src: _compile(src, force, verbose), sources()))
    if force or _stale(LIBRARY, objects):
        command = [_nvcc(), "-shared", *ARCH_FLAGS, "-o", str(LIBRARY), *map(str, objects)]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError("linking libentropack_b200.so failed")
    return LIBRARY


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
