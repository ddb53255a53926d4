"""Per-role cycle counters of the FP8 grouped GEMM, read from a trace build of the library.

    python -m mlops_b200.build --define B200_GEMM_TRACE=1 --output build/libb200moe_trace.so
    B200MOE_LIBRARY=build/libb200moe_trace.so python -m mlops_b200.gemm_trace

With `B200_GEMM_TRACE` the kernel's roles of CTA 0 (the two UMMA issuers, the two epilogue
halves, the TMA producer) write `clock64()` at fixed points of a window of K blocks into a
buffer handed over with `b200moe_debug_set_gemm_trace`; this module runs one launch of a
DeepSeek-V3-shaped projection with the buffer attached and prints the mean distances between
those points. The counters perturb the kernel (about +30% run time): the figures say where the
roles wait for one another, not how fast the untraced kernel is. The shipped library has none
of this code.
"""

from __future__ import annotations

import argparse
import ctypes

import torch

from . import _lib, ops


def _trace_shape(lib):
    values = [ctypes.c_int() for _ in range(4)]
    if not hasattr(lib, "b200moe_debug_gemm_trace_shape"):
        raise RuntimeError("this library was built without -DB200_GEMM_TRACE=1 (see the module docstring)")
    lib.b200moe_debug_gemm_trace_shape(*(ctypes.byref(v) for v in values))
    return tuple(v.value for v in values)


def trace(rows, experts, n, k, *, b_mn_major=False, pair=0, device="cuda:0"):
    """One traced launch; returns `(table [slots, K blocks, fields] float64, first K block)`."""
    lib = ctypes.CDLL(str(_lib.LIBRARY_PATH))
    slots, its, fields, first = _trace_shape(lib)
    lib.b200moe_debug_set_gemm_trace.argtypes = [ctypes.c_void_p]
    g = torch.Generator(device=device).manual_seed(0)
    a = torch.randn(rows, k, device=device, generator=g).bfloat16()
    a_q, a_s = ops.quantize_rows(a)
    del a
    w = torch.randn(experts, k if b_mn_major else n, n if b_mn_major else k, device=device, generator=g).bfloat16()
    b_q, b_s = ops.quantize_blocks(w)
    del w
    offsets = torch.arange(experts + 1, device=device, dtype=torch.int32) * (rows // experts)
    ops.set_gemm_pair(pair)
    for _ in range(2):
        ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets, b_mn_major=b_mn_major)
    buffer = torch.zeros(slots * its * fields, dtype=torch.int64, device=device)
    lib.b200moe_debug_set_gemm_trace(ctypes.c_void_p(buffer.data_ptr()))
    try:
        ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets, b_mn_major=b_mn_major)
        torch.cuda.synchronize(device)
    finally:
        lib.b200moe_debug_set_gemm_trace(None)
        ops.set_gemm_pair(-1)
    return buffer.cpu().view(slots, its, fields).double(), first


def report(table, first):
    """Text summary: slot 0/1 = issuer of even/odd K blocks (fields: loop top, operands landed,
    slab 0 free, slab 0 issued, slab 1 free, slab 1 issued), slot 2/3 = epilogue half 0/1
    (fields: wait begins, slab complete, loads done, slab released), slot 4 = producer (fields:
    wait begins, stage free)."""
    its = table.shape[1]
    lines = [f"K blocks {first}..{first + its - 1} of CTA 0, SM cycles"]

    def mean(x):
        return float(x.mean())

    issued = torch.stack([table[i % 2, i, 5] for i in range(its)])
    lines.append(f"period per K block (slab 1 issued -> next K block's slab 1 issued): {mean((issued[1:] - issued[:-1])[8:]):.0f}")
    for slot, name in ((0, "issuer, even K blocks"), (1, "issuer, odd K blocks")):
        rows = table[slot, slot::2][4:]
        lines.append(
            f"{name}: loop top -> operands {mean(rows[:, 1] - rows[:, 0]):.0f} | -> slab 0 free {mean(rows[:, 2] - rows[:, 1]):.0f}"
            f" | issue slab 0 {mean(rows[:, 3] - rows[:, 2]):.0f} | -> slab 1 free {mean(rows[:, 4] - rows[:, 3]):.0f}"
            f" | issue slab 1 {mean(rows[:, 5] - rows[:, 4]):.0f} | to next loop top {mean(rows[1:, 0] - rows[:-1, 5]):.0f}")
    for slot, name in ((2, "epilogue half 0"), (3, "epilogue half 1")):
        rows = table[slot][8:]
        lines.append(
            f"{name}: wait for slab {mean(rows[:, 1] - rows[:, 0]):.0f} | tcgen05.ld {mean(rows[:, 2] - rows[:, 1]):.0f}"
            f" | promote + release {mean(rows[:, 3] - rows[:, 2]):.0f} | per K block {mean(rows[1:, 1] - rows[:-1, 1]):.0f}")
    for half, slot in ((0, 2), (1, 3)):
        seen = [float(table[slot, i, 1] - table[i % 2, i, 3 + 2 * half]) for i in range(8, its)]
        back = [float(table[i % 2, i + 2, 2 + 2 * half] - table[slot, i, 3]) for i in range(8, its - 2)]
        lines.append(f"slab {half}: issued -> epilogue sees it complete {sum(seen) / len(seen):.0f}"
                     f" | released -> issuer (two K blocks later) has it {sum(back) / len(back):.0f}")
    producer = table[4][8:]
    lines.append(f"producer: wait for stage {mean(producer[:, 1] - producer[:, 0]):.0f}"
                 f" | per K block {mean(producer[1:, 1] - producer[:-1, 1]):.0f}")
    return "\n".join(lines)


ISSUER_FIELDS = ("loop top", "operands landed", "slab 0 free", "slab 0 issued", "slab 1 free", "slab 1 issued")
EPILOGUE_FIELDS = ("wait begins", "slab complete", "loads done", "slab released", "tile boundary: store begins",
                   "tile boundary: store issued", "tile boundary: next tile's number read", "tile boundary: next tile located")


def timeline(table, first, start, count):
    """The stamps of K blocks `start .. start + count - 1` (relative to the window) of all roles,
    merged and ordered by time; times relative to the earliest of them."""
    events = []
    for i in range(start, start + count):
        for f, name in enumerate(ISSUER_FIELDS):
            events.append((float(table[i % 2, i, f]), f"issuer {i % 2}", first + i, name))
        for half, slot in ((0, 2), (1, 3)):
            for f, name in enumerate(EPILOGUE_FIELDS):
                events.append((float(table[slot, i, f]), f"epilogue {half}", first + i, name))
        for f, name in enumerate(("wait begins", "stage free")):
            events.append((float(table[4, i, f]), "producer", first + i, name))
    events = [e for e in events if e[0] > 0]
    events.sort()
    base = events[0][0]
    return "\n".join(f"{t - base:8.0f}  {role:<11} K block {kb:<4} {name}" for t, role, kb, name in events)


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--timeline", type=int, default=0, help="also print the ordered stamps of this many K blocks")
    parser.add_argument("--timeline-start", type=int, default=24, help="... from this K block of the window on")
    parser.add_argument("--rows", type=int, default=32768)
    parser.add_argument("--experts", type=int, default=32)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=7168)
    parser.add_argument("--mn-major", action="store_true", help="input-gradient form (weights read MN-major)")
    parser.add_argument("--pair", type=int, default=0, help="1: CTA-pair form")
    args = parser.parse_args()
    table, first = trace(args.rows, args.experts, args.n, args.k, b_mn_major=args.mn_major, pair=args.pair)
    print(f"rows {args.rows} experts {args.experts} N {args.n} K {args.k} mn_major {args.mn_major} pair {args.pair}")
    print(report(table, first))
    if args.timeline:
        print(timeline(table, first, args.timeline_start, args.timeline))


if __name__ == "__main__":
    main()
