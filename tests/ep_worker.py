"""Worker of tests/test_gpu_ep.py: one process per GPU (torch.distributed.run). Every rank
builds the same global experts, keeps its shard, runs the expert-parallel layer on its own
tokens and checks it against the single-GPU layer run on the full weights (the method of the
reference's tests/expert_parallel/gpu/reference_quack.py:14-69: expected expert gradients
are all-reduced, then sliced to the local shard)."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from mlops_b200 import ep, layer, ops  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    expert_map, mode = sys.argv[1], sys.argv[2]
    experts, top_k, width, inner, tokens = 8, 2, 256, 256, 300 + 17 * rank
    shared_on = mode == "sigmoid_noaux_tc"

    g = torch.Generator().manual_seed(5)  # global parameters: identical on every rank
    router = (torch.randn(experts, width, generator=g) * 0.05).to(device)
    bias = (torch.randn(experts, generator=g) * 0.1).to(device) if mode == "sigmoid_noaux_tc" else None
    w13 = ops.quantize_blocks((torch.randn(experts, 2 * inner, width, generator=g) * 0.05).bfloat16().to(device))
    w2 = ops.quantize_blocks((torch.randn(experts, width, inner, generator=g) * 0.05).bfloat16().to(device))
    shared = None
    if shared_on:
        shared = ((torch.randn(2 * inner, width, generator=g) * 0.05).bfloat16().to(device),
                  (torch.randn(width, inner, generator=g) * 0.05).bfloat16().to(device))
    gl = torch.Generator().manual_seed(100 + rank)  # this rank's tokens
    x = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    residual = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    dy = torch.randn(tokens, width, generator=gl).bfloat16().to(device)

    config = ep.ExpertParallelConfig(hidden=width, experts=experts, intermediate=inner, top_k=top_k,
                                     routing_mode=mode, n_group=4 if shared_on else 1,
                                     topk_group=2 if shared_on else 1, routed_scaling=2.5 if shared_on else 1.0,
                                     expert_map=expert_map,
                                     dedup=expert_map == "contiguous")  # one case each way
    local = experts // world
    mine = [e for e in range(experts) if int(ep.placement(config, world)[e]) // local == rank]
    mine.sort(key=lambda e: int(ep.placement(config, world)[e]))
    pick = torch.tensor(mine, device=device)
    module = ep.ExpertParallelMoE(config, dist.group.WORLD, router_weight=router, router_bias=bias,
                                  w13=(w13[0][pick].contiguous(), w13[1][pick].contiguous()),
                                  w2=(w2[0][pick].contiguous(), w2[1][pick].contiguous()), shared=shared,
                                  device=device, weight_grad_dtype=torch.float32,
                                  chunks=3 if expert_map == "strided" else 1)
    output, aux, counts, psum, saved = module.forward(x, residual)
    grads = module.backward(saved, dy)
    torch.cuda.synchronize()
    ops.check_status(device)

    # single-GPU expectation on the full weights
    base, shared_h13 = residual, None
    if shared_on:
        y_shared, shared_h13 = layer.shared_expert_forward(x, *shared)
        base = residual + y_shared
    kwargs = dict(top_k=top_k, routing_mode=mode, router_bias=bias, n_group=config.n_group,
                  topk_group=config.topk_group, routed_scaling=config.routed_scaling)
    ref = layer.forward_routed(x, base, router, w13, w2, **kwargs)
    ref_grads = layer.backward_routed(dy, None, None, x, router, w13, w2, *ref[4:], top_k=top_k,
                                      routing_mode=mode, weight_grad_dtype=torch.float32)
    expected_x = ref_grads[0]
    if shared_on:
        expected_x = expected_x + layer.shared_expert_backward(dy, x, *shared, shared_h13)[0]
    assert torch.equal(counts, ref[2]), "counts differ"
    assert torch.equal(output, ref[0]), "output differs from the single-GPU layer"  # row-wise identical math
    torch.testing.assert_close(aux, ref[1])
    mx, mean = O.rel_errors(grads["grad_x"].float().cpu(), expected_x.float().cpu())
    assert mx <= 2e-2 and mean <= 2e-3, ("grad_x", mx, mean)
    mx, mean = O.rel_errors(grads["grad_router"].float().cpu(), ref_grads[2].float().cpu())
    assert mx <= 1e-3, ("grad_router", mx)
    for name, full in (("grad_w13", ref_grads[3]), ("grad_w2", ref_grads[4])):
        total = full.clone()
        dist.all_reduce(total)  # every rank's tokens contribute to an expert's gradient
        mx, mean = O.rel_errors(grads[name].float().cpu(), total[pick].float().cpu())
        assert mx <= 1e-3, (name, mx)
    report = module.report()
    assert report["bytes_moved"] > 0
    dist.barrier()
    if rank == 0:
        print(f"ep worker ok: world={world} map={expert_map} mode={mode}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
