"""Worker of tests/test_gpu_ep.py: the expert-parallel layer as an `nn.Module` with ordinary
autograd (`ExpertParallelLayer`), against the runtime's explicit forward / backward."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from mlops_b200 import ep, ops  # noqa: E402
from mlops_b200.weights import BlockFP8Weight  # noqa: E402


def main():
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    world, rank = dist.get_world_size(), dist.get_rank()
    experts, width, inner, top_k, tokens = 4 * world, 256, 256, 2, 200
    g = torch.Generator().manual_seed(3 + rank)
    router = (torch.randn(experts, width, generator=g) * 0.05).to(device)  # differs per rank on purpose
    w13 = BlockFP8Weight.quantize((torch.randn(4, 2 * inner, width, generator=g) * 0.05).bfloat16().to(device))
    w2 = BlockFP8Weight.quantize((torch.randn(4, width, inner, generator=g) * 0.05).bfloat16().to(device))
    shared = ((torch.randn(2 * inner, width, generator=g) * 0.05).bfloat16().to(device).requires_grad_(True),
              (torch.randn(width, inner, generator=g) * 0.05).bfloat16().to(device).requires_grad_(True))
    config = ep.ExpertParallelConfig(hidden=width, experts=experts, intermediate=inner, top_k=top_k)
    module = ep.ExpertParallelLayer(config, dist.group.WORLD, gate_up_weight=w13.requires_grad_(True),
                                    down_weight=w2.requires_grad_(True), router_weight=router.requires_grad_(True),
                                    shared=shared, device=device, chunks=2)
    # construction broadcast rank 0's replicated parameters
    reference_router = module.router_weight.detach().clone()
    dist.broadcast(reference_router, src=0)
    assert torch.equal(reference_router, module.router_weight.detach())
    assert [tuple(p.shape) for p in module.expert_parameters()] == [(4, 2 * inner, width), (4, width, inner)]

    x = torch.randn(tokens, width, generator=g).bfloat16().to(device).requires_grad_(True)
    dy = torch.randn(tokens, width, generator=g).bfloat16().to(device)
    out = module(x)
    aux, counts, psum = module.last_statistics
    (out.float() * dy.float()).sum().add(aux * 0.5).backward()
    torch.cuda.synchronize()
    ops.check_status(device)
    assert counts.dtype == torch.int64 and int(counts.sum()) == tokens * top_k
    for parameter in (*module.expert_parameters(), *module.replicated_parameters()):
        assert parameter.grad is not None and parameter.grad.shape == parameter.shape
    assert x.grad.shape == x.shape

    # the same step through the runtime's explicit calls
    runtime = module._runtime
    output2, aux2, counts2, psum2, saved = runtime.forward(x.detach(), torch.zeros_like(x))
    grads = runtime.backward(saved, dy, torch.tensor(0.5, device=device), None)
    assert torch.equal(out.detach(), output2) and torch.equal(counts, counts2)
    assert torch.equal(x.grad, grads["grad_x"])
    assert torch.equal(module.gate_up_weight.grad, grads["grad_w13"])
    assert torch.equal(module.router_weight.grad, grads["grad_router"])

    # externally supplied routes bypass the router; replicated gradients are summed on request
    ids = torch.randint(0, experts, (tokens, 1), generator=g).expand(-1, top_k).clone()
    ids[:, 1] = (ids[:, 0] + 1) % experts
    weights = torch.full((tokens, top_k), 0.5)
    routed = module(x.detach(), ids.to(device).to(torch.int32), weights.to(device))
    assert routed.shape == x.shape
    before = module.router_weight.grad.clone()
    module.synchronize_replicated_gradients()
    total = before.clone()
    dist.all_reduce(total)
    assert torch.equal(module.router_weight.grad, total)
    module.close()
    try:
        module(x.detach())
        raise SystemExit("a closed layer accepted a call")
    except RuntimeError:
        pass
    dist.barrier()
    if rank == 0:
        print("ep module worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
