"""Seeded input factories shared by `make_golden.py` (which feeds them to the reference)
and by the tests (which feed them to the oracle and to the CUDA path). Each fixture stores
`checksum(...)` of the inputs it was made from, so a generator that ever produced different
numbers would be noticed instead of silently comparing unrelated data."""

from __future__ import annotations

import torch


def checksum(*tensors) -> torch.Tensor:
    """Order-sensitive 64-bit sums of the raw bytes of every tensor."""
    sums = []
    for t in tensors:
        raw = t.detach().contiguous().view(torch.uint8).reshape(-1).to(torch.int64)
        weights = (torch.arange(raw.numel(), dtype=torch.int64) % 251) + 1
        sums.append(int((raw * weights).sum()))
    return torch.tensor(sums, dtype=torch.int64)


def config1():
    """Benchmark configuration 1 (the CPU-runnable case): T=512, D=256, 8 experts, top-2 softmax routing, F=512, seed 0."""
    torch.manual_seed(0)
    T, D, E, K, F = 512, 256, 8, 2, 512
    x = torch.randn(T, D).bfloat16()
    residual = torch.zeros_like(x)
    router = torch.randn(E, D) * 0.02
    w13 = (torch.randn(E, 2 * F, D) * 0.02).bfloat16()
    w2 = (torch.randn(E, D, F) * 0.02).bfloat16()
    dy = torch.randn(T, D).bfloat16()
    return dict(x=x, residual=residual, router=router, w13=w13, w2=w2, dy=dy, top_k=K,
                routing_mode="softmax_then_topk")


def block_weight():
    """A [3, 200, 192] weight with partial 128-blocks on both axes, an all-zero block and
    block scales spread over 2^+-14 (the shapes the reference's FP8 tests exercise:
    tests/test_sonicmoe_block_fp8.py:31-76, tests/test_block_fp8_transpose_gemm.py:431-444)."""
    g = torch.Generator().manual_seed(7)
    w = torch.randn(3, 200, 192, generator=g) * 0.02
    w[0, :128, :128] = 0
    w[1, 128:, :128] *= 2.0 ** 14
    w[2, :128, 128:] *= 2.0 ** -14
    return w


def activation_rows():
    g = torch.Generator().manual_seed(8)
    x = torch.randn(40, 192, generator=g).bfloat16()
    x[0] = 0
    x[1] *= 1000
    gather = torch.randint(0, 40, (70,), generator=g).to(torch.int32)
    return x, gather


def ep_case():
    """Fixed routes with a globally empty expert (expert 5), as in the reference's
    tests/expert_parallel/test_reference.py:14-44."""
    torch.manual_seed(17)
    T, D, E, K, F = 48, 128, 6, 2, 128
    x = torch.randn(T, D).bfloat16()
    gate = torch.randn(E, F, D) * 0.05
    up = torch.randn(E, F, D) * 0.05
    down = torch.randn(E, D, F) * 0.05
    ids = torch.stack([torch.randperm(E - 1)[:K] for _ in range(T)]).to(torch.int32)
    p = torch.rand(T, K)
    return dict(x=x, gate=gate, up=up, down=down, ids=ids, p=p)


def lora_case(rank=16):
    """A small expert-LoRA layer: T=96, D=128, 4 experts, top-2, F=128; factors as in
    benchmark configuration 5 (A ~ N(0, 0.02), B = 0.01 N(0, 1), bf16), alpha = rank (scale 1)."""
    torch.manual_seed(23)
    T, D, E, K, F = 96, 128, 4, 2, 128
    x = torch.randn(T, D).bfloat16()
    residual = torch.randn(T, D).bfloat16()
    router = torch.randn(E, D) * 0.1
    w13 = (torch.randn(E, 2 * F, D) * 0.05).bfloat16()
    w2 = (torch.randn(E, D, F) * 0.05).bfloat16()
    a13 = (torch.randn(E, rank, D) * 0.02).bfloat16()
    b13 = (torch.randn(E, 2 * F, rank) * 0.01).bfloat16()
    a2 = (torch.randn(E, rank, F) * 0.02).bfloat16()
    b2 = (torch.randn(E, D, rank) * 0.01).bfloat16()
    dy = torch.randn(T, D).bfloat16()
    return dict(x=x, residual=residual, router=router, w13=w13, w2=w2, a13=a13, b13=b13, a2=a2, b2=b2, dy=dy,
                top_k=K, routing_mode="softmax_then_topk", scale=4.0)
