"""Stand-alone device probes kept beside the kernels they explain (`csrc/probes/*.cu`): small CUDA
programs that measure one hardware behaviour the design depends on. They are not part of the
library; this module compiles one with nvcc for sm_100a into the build folder and runs it.

    python -m mlops_b200.probes handshake    # tcgen05 issue rate, commit latency, the accumulator ring
"""

from __future__ import annotations

import argparse
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PROBES = ROOT / "csrc" / "probes"


def build(name: str) -> Path:
    source = PROBES / f"{name}.cu"
    if not source.exists():
        raise FileNotFoundError(f"no probe {name!r}; have: {sorted(p.stem for p in PROBES.glob('*.cu'))}")
    out = ROOT.parent / "build" / "probes" / name
    out.parent.mkdir(parents=True, exist_ok=True)
    if not out.exists() or out.stat().st_mtime < max(source.stat().st_mtime, (ROOT / "csrc" / "common.cuh").stat().st_mtime):
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-o", str(out),
                        str(source)], check=True)
    return out


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("name", nargs="?", default="handshake")
    parser.add_argument("--build-only", action="store_true")
    args = parser.parse_args()
    binary = build(args.name)
    if args.build_only:
        print(binary)
        return
    sys.exit(subprocess.run([str(binary)]).returncode)


if __name__ == "__main__":
    main()
