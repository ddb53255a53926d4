"""Sustained timing of the FP8 grouped GEMM at the four shapes of a DeepSeek-V3-sized expert
layer, with the SM clock and board power sampled while it runs.

    python -m mlops_b200.gemm_probe                      # the shipped library
    python -m mlops_b200.build --define B200_GEMM_ABLATE=1 --output build/libb200moe_abl1.so
    B200MOE_LIBRARY=build/libb200moe_abl1.so python -m mlops_b200.gemm_probe --label no-epilogue-reads

A B200 under this kernel sits at its power limit, so the clock it settles at is part of the
result: the table gives TFLOP/s over a few seconds, the median clock and power, and the cycles
per K block (128 x 256 x 128 E4M3 multiply-adds on one SM; 512 at the tensor cores' rate)
computed from the MEASURED clock. Ablation builds (`B200_GEMM_ABLATE`: bit 0 no accumulator
reads, bit 1 reads without multiply-adds, bit 2 no TMA traffic after the first fill) give wrong
results on purpose; this module only times them.
"""

from __future__ import annotations

import argparse
import statistics
import subprocess
import threading
import time

import torch

from . import ops

SHAPES = (  # name, N, K, weights read MN-major (input gradients)
    ("up", 4096, 7168, False),
    ("down", 7168, 2048, False),
    ("dgrad_down", 2048, 7168, True),
    ("dgrad_up", 7168, 4096, True),
)


def _sample(stop, out, index):
    query = ["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-i", str(index)]
    while not stop.is_set():
        try:
            mhz, watts = subprocess.run(query, capture_output=True, text=True).stdout.strip().split(",")
            out.append((float(mhz), float(watts)))
        except ValueError:
            pass
        time.sleep(0.05)


def probe(rows, experts, n, k, b_mn_major, *, seconds=2.5, pair=0, device="cuda:0"):
    """`(ms per launch, TFLOP/s, median SM MHz, median W)` over about `seconds` of back-to-back launches."""
    g = torch.Generator(device=device).manual_seed(0)
    a = torch.randn(rows, k, device=device, generator=g).bfloat16()
    a_q, a_s = ops.quantize_rows(a)
    del a
    w = torch.randn(experts, k if b_mn_major else n, n if b_mn_major else k, device=device, generator=g).bfloat16()
    b_q, b_s = ops.quantize_blocks(w)
    del w
    offsets = torch.arange(experts + 1, device=device, dtype=torch.int32) * (rows // experts)
    ops.set_gemm_pair(pair)
    try:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets, b_mn_major=b_mn_major)
        start.record()
        for _ in range(5):
            ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets, b_mn_major=b_mn_major)
        end.record()
        torch.cuda.synchronize(device)
        reps = max(10, int(seconds * 1e3 / (start.elapsed_time(end) / 5)))
        stop, samples = threading.Event(), []
        sampler = threading.Thread(target=_sample, args=(stop, samples, torch.device(device).index or 0))
        sampler.start()
        time.sleep(0.1)
        start.record()
        for _ in range(reps):
            ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets, b_mn_major=b_mn_major)
        end.record()
        torch.cuda.synchronize(device)
        stop.set()
        sampler.join()
    finally:
        ops.set_gemm_pair(-1)
    ms = start.elapsed_time(end) / reps
    settled = samples[len(samples) // 3:] or [(float("nan"), float("nan"))]
    return (ms, 2.0 * rows * n * k / ms / 1e9, statistics.median(s[0] for s in settled),
            statistics.median(s[1] for s in settled))


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--rows", type=int, default=32768)
    parser.add_argument("--experts", type=int, default=32)
    parser.add_argument("--seconds", type=float, default=2.5)
    parser.add_argument("--pair", type=int, default=0, help="1: CTA-pair form")
    parser.add_argument("--label", default="shipped")
    parser.add_argument("--shapes", default="up,down,dgrad_down,dgrad_up")
    args = parser.parse_args()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    print(f"| build | shape | ms | TFLOP/s | SM MHz | W | cycles per K block |")
    print("|---|---|---|---|---|---|---|")
    for name, n, k, mn in SHAPES:
        if name not in args.shapes.split(","):
            continue
        ms, tflops, mhz, watts = probe(args.rows, args.experts, n, k, mn, seconds=args.seconds, pair=args.pair)
        k_blocks_per_sm = (args.rows // 128) * (n // 256) * (k // 128) / sms
        print(f"| {args.label} | {name} {args.rows}x{n}x{k} | {ms:.3f} | {tflops:.0f} | {mhz:.0f} | {watts:.0f} | "
              f"{ms * 1e-3 * mhz * 1e6 / k_blocks_per_sm:.0f} |", flush=True)


if __name__ == "__main__":
    main()
