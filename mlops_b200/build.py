"""Build recipe of the native library: every `.cu` under `csrc/` is compiled by nvcc for
sm_100a only and linked into `mlops_b200/libb200moe.so` (in-tree, so the same file is
what the tests and the bench load).

    python -m mlops_b200.build [--force] [--verbose]
    python -m mlops_b200.build --define B200_GEMM_TRACE=1 --output /some/where/libb200moe_trace.so

The second form builds a variant with extra preprocessor definitions (the in-kernel cycle
counters, an experimental switch) into a file of its own, leaving the shipped library alone;
`B200MOE_LIBRARY=<that file>` makes the package load it.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
BUILD_DIR = PACKAGE_DIR / "build"
LIBRARY = PACKAGE_DIR / "libb200moe.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for path in sorted(paths):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def sources():
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False, defines=(), output: Path | None = None) -> Path:
    """Compile and link the library when a source changed; return its path. `defines`
    (`NAME=VALUE` strings) and `output` build a variant beside the shipped library."""
    srcs = sources()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    variant = bool(defines) or output is not None
    library = Path(output) if output is not None else LIBRARY
    build_dir = BUILD_DIR / ("variant_" + hashlib.sha256(" ".join(defines).encode()).hexdigest()[:8]) if variant \
        else BUILD_DIR
    stamp = build_dir / "stamp"
    digest = _digest(srcs + headers) + " " + " ".join(defines)
    if not force and library.exists() and stamp.exists() and stamp.read_text() == digest:
        return library
    build_dir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    extra = (["-Xptxas", "-v"] if verbose else []) + [f"-D{d}" for d in defines]

    def compile_one(src: Path) -> Path:
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or done.returncode != 0:
            sys.stderr.write(done.stdout + done.stderr)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objects = list(pool.map(compile_one, srcs))
    link = [nvcc, "-shared", "-o", str(library), *map(str, objects), "-cudart", "static"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        sys.stderr.write(done.stdout + done.stderr)
        raise RuntimeError("link failed")
    stamp.write_text(digest)
    return library


if __name__ == "__main__":
    argv = sys.argv[1:]
    defines = [argv[i + 1] for i, a in enumerate(argv) if a == "--define" and i + 1 < len(argv)]
    output = next((Path(argv[i + 1]) for i, a in enumerate(argv) if a == "--output" and i + 1 < len(argv)), None)
    if defines and output is None:
        raise SystemExit("--define builds a variant: name its file with --output")
    path = build(force="--force" in argv, verbose="--verbose" in argv, defines=defines, output=output)
    print(path)
