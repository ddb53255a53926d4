"""Worker of tests/test_gpu_ep.py: `mlops_b200.ep.parity_check` (the expert-parallel layer
against the single-GPU layer on the gathered weights) for the routing modes and return forms,
one rank per GPU under torch.distributed.run."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from mlops_b200 import ep  # noqa: E402


def main():
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    cases = (
        dict(routing_mode="sigmoid_noaux_tc", n_group=2, topk_group=1, routed_scaling=2.5, shared=True, presum=True),
        dict(routing_mode="sigmoid_noaux_tc", n_group=2, topk_group=1, routed_scaling=2.5, shared=True, presum=False),
        dict(routing_mode="softmax_then_topk", shared=False),
        # the token rows written straight into the peers' arenas by this library's kernel (NVLink
        # peer memory) instead of the library all-to-all: the same results, bit for bit without presum
        dict(routing_mode="sigmoid_noaux_tc", n_group=2, topk_group=1, routed_scaling=2.5, shared=True, presum=False,
             transport="peer"),
        dict(routing_mode="sigmoid_noaux_tc", n_group=2, topk_group=1, routed_scaling=2.5, shared=True, presum=True,
             transport="peer"),
    )
    for case in cases:
        result = ep.parity_check(dist.group.WORLD, device, **case)
        if dist.get_rank() == 0:
            print("ep check ok:", result)
        assert result["presum_return"] == bool(case.get("presum")) and (result["output_bit_equal"] or case.get("presum"))
        assert result["transport"] == case.get("transport", "nccl")
    dist.barrier()
    if dist.get_rank() == 0:
        print("ep check worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
