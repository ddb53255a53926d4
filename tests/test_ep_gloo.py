"""Host-side logic of the expert-parallel exchange on CPU: two gloo ranks plan and move rows
with the package's own `make_plan` / `exchange`, and failures are raised on the host (a
mismatched configuration) before anything is launched. No GPU is involved."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, world=2, **kwargs):
    port = _free_port()
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, rank, world, port, queue, kwargs)) for rank in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    errors = [r for r in results if isinstance(r, str)]
    assert not errors, errors
    return sorted(results, key=lambda r: r["rank"])


def _entry(fn, rank, world, port, queue, kwargs):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, **kwargs)
        out["rank"] = rank
        queue.put(out)
    except Exception as error:  # noqa: BLE001 - reported to the parent
        queue.put(f"rank {rank}: {type(error).__name__}: {error}")
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _exchange_case(rank, world, expert_map):
    from mlops_b200 import ep
    from oracle import moe_oracle as O

    config = ep.ExpertParallelConfig(hidden=128, experts=6, intermediate=128, top_k=2, expert_map=expert_map)
    ep.handshake(config, dist.group.WORLD)
    keys = ep.placement(config, world)
    local = config.experts // world
    g = torch.Generator().manual_seed(100 + rank)
    tokens = 37 + 5 * rank
    ids = torch.stack([torch.randperm(config.experts, generator=g)[:2] for _ in range(tokens)]).to(torch.int32)
    x = torch.randn(tokens, 8, generator=g)
    order, offsets, slots = O.sort_assignments(keys[ids.long()], config.experts)
    counts = offsets[1:] - offsets[:-1]
    plan = ep.make_plan(counts, dist.group.WORLD)
    rows = x[order.long() // 2]
    # tag every row with (source rank, expert) so the receiver can check what it got
    expert_of_row = ids.reshape(-1)[order.long()].float()
    tagged = torch.cat([rows, torch.full((rows.shape[0], 1), float(rank)), expert_of_row[:, None]], dim=1)
    received, _ = ep.exchange(tagged, plan, dist.group.WORLD)
    seg = plan.segment_offsets.tolist()
    assert received.shape[0] == plan.recv_rows == seg[-1]
    for source in range(world):
        for j in range(local):
            lo, hi = seg[source * local + j], seg[source * local + j + 1]
            block = received[lo:hi]
            assert bool((block[:, -2] == source).all())
            expert = block[:, -1].long()
            assert bool((keys[expert].long() == rank * local + j).all())  # my j-th local expert
    back, _ = ep.exchange(received, plan, dist.group.WORLD, back=True)
    assert torch.equal(back, tagged)  # the return trip restores the sender's order
    return dict(sent=plan.send_rows, received=plan.recv_rows, splits=plan.send_splits)


@pytest.mark.parametrize("expert_map", ["contiguous", "strided"])
def test_two_ranks_exchange_rows_by_expert_owner(expert_map):
    results = _run(_exchange_case, expert_map=expert_map)
    assert sum(r["sent"] for r in results) == sum(r["received"] for r in results) == 2 * (37 + 42)
    assert len(results[0]["splits"]) == 2


def _mismatch_case(rank, world):
    from mlops_b200 import ep

    config = ep.ExpertParallelConfig(hidden=128, experts=8, intermediate=128, top_k=2 + rank)
    try:
        ep.handshake(config, dist.group.WORLD)
    except RuntimeError as error:
        return dict(raised="differ" in str(error))
    return dict(raised=False)


def test_mismatched_configuration_raises_on_every_rank():
    assert all(r["raised"] for r in _run(_mismatch_case))


def test_configuration_validation():
    from mlops_b200 import ep

    with pytest.raises(ValueError):
        ep.ExpertParallelConfig(hidden=128, experts=6, intermediate=128, top_k=2).validate(4)
    with pytest.raises(ValueError):
        ep.ExpertParallelConfig(hidden=100, experts=8, intermediate=128, top_k=2).validate(2)
    with pytest.raises(ValueError):
        ep.ExpertParallelConfig(hidden=128, experts=8, intermediate=128, top_k=2, expert_map="x").validate(2)
    keys = ep.placement(ep.ExpertParallelConfig(hidden=128, experts=8, intermediate=128, top_k=2,
                                                expert_map="strided"), 4)
    assert keys.tolist() == [0, 2, 4, 6, 1, 3, 5, 7]  # expert e -> rank e % 4, slot e // 4
