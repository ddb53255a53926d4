"""Worker of tests/test_gpu_ep.py for expert LoRA under expert parallelism: every rank holds
the same global experts and factors, keeps its shard, runs the expert-parallel layer with a
frozen base on its own tokens and checks output, input gradient and factor gradients against
the single-GPU `mlops_b200.lora.expert_lora` run on the full set (factor gradients: every
rank's tokens contribute, so the single-GPU ones are all-reduced and sliced to the shard)."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from mlops_b200 import ep, ops  # noqa: E402
from mlops_b200.lora import expert_lora  # noqa: E402
from mlops_b200.weights import BlockFP8Weight  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    experts, top_k, width, inner, tokens, lora_rank, scale = 8, 2, 256, 256, 280 + 24 * rank, 12, 0.5
    mode = "softmax_then_topk"

    g = torch.Generator().manual_seed(9)  # global parameters: identical on every rank
    router = (torch.randn(experts, width, generator=g) * 0.05).to(device)
    w13_full = (torch.randn(experts, 2 * inner, width, generator=g) * 0.05).bfloat16().to(device)
    w2_full = (torch.randn(experts, width, inner, generator=g) * 0.05).bfloat16().to(device)
    factors = dict(
        a13=(torch.randn(experts, lora_rank, width, generator=g) * 0.05).bfloat16().to(device),
        b13=(torch.randn(experts, 2 * inner, lora_rank, generator=g) * 0.05).bfloat16().to(device),
        a2=(torch.randn(experts, lora_rank, inner, generator=g) * 0.05).bfloat16().to(device),
        b2=(torch.randn(experts, width, lora_rank, generator=g) * 0.05).bfloat16().to(device),
    )
    gl = torch.Generator().manual_seed(200 + rank)  # this rank's tokens
    x = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    residual = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    dy = torch.randn(tokens, width, generator=gl).bfloat16().to(device)

    config = ep.ExpertParallelConfig(hidden=width, experts=experts, intermediate=inner, top_k=top_k,
                                     routing_mode=mode, expert_map="contiguous")
    local = experts // world
    pick = torch.arange(rank * local, (rank + 1) * local, device=device)
    w13, w2 = ops.quantize_blocks(w13_full), ops.quantize_blocks(w2_full)
    module = ep.ExpertParallelMoE(
        config, dist.group.WORLD, router_weight=router, w13=(w13[0][pick].contiguous(), w13[1][pick].contiguous()),
        w2=(w2[0][pick].contiguous(), w2[1][pick].contiguous()), device=device, chunks=2,
        lora=dict({k: v[pick].contiguous() for k, v in factors.items()}, scale=scale))
    output, aux, counts, psum, saved = module.forward(x, residual)
    grads = module.backward(saved, dy, need_experts=False)  # frozen base
    torch.cuda.synchronize()
    ops.check_status(device)
    assert grads["grad_w13"] is None and grads["grad_w2"] is None

    # single-GPU expectation on the full experts and factors
    xs = x.clone().requires_grad_(True)
    leaves = {k: v.clone().requires_grad_(True) for k, v in factors.items()}
    ref = expert_lora(xs, residual, router, BlockFP8Weight.quantize(w13_full), BlockFP8Weight.quantize(w2_full),
                      leaves["a13"], leaves["b13"], leaves["a2"], leaves["b2"], top_k=top_k, routing_mode=mode,
                      scale=scale)
    ref[0].backward(dy)
    assert torch.equal(output, ref[0].detach()), "output differs from the single-GPU layer"
    mx, mean = O.rel_errors(grads["grad_x"].float().cpu(), xs.grad.float().cpu())
    assert mx <= 2e-2 and mean <= 2e-3, ("grad_x", mx, mean)
    for name in ("a13", "b13", "a2", "b2"):
        total = leaves[name].grad.float().clone()
        dist.all_reduce(total)
        got = grads["grad_" + name].float()
        assert got.shape == total[pick].shape, (name, got.shape, total[pick].shape)
        mx, mean = O.rel_errors(got.cpu(), total[pick].cpu())
        assert mx <= 2e-2 and mean <= 2e-3, (name, mx, mean)
    dist.barrier()
    if rank == 0:
        print(f"ep lora worker ok: world={world}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
