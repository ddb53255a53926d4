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


def _dedup_case(rank, world):
    """De-duplicated dispatch over real collectives: copies and their expert lists travel, the
    receiver expands them, and what it ends up with equals what the row-per-assignment dispatch
    of the same tokens delivers (rows and order)."""
    from mlops_b200 import ep
    from oracle import moe_oracle as O

    config = ep.ExpertParallelConfig(hidden=128, experts=8, intermediate=128, top_k=3, dedup=True)
    ep.handshake(config, dist.group.WORLD)
    local = config.experts // world
    g = torch.Generator().manual_seed(300 + rank)
    tokens = 29 + 7 * rank
    ids = torch.stack([torch.randperm(config.experts, generator=g)[:3] for _ in range(tokens)]).to(torch.int32)
    weights = torch.rand(tokens, 3, generator=g)
    x = torch.randn(tokens, 8, generator=g)
    order, offsets, _slots = O.sort_assignments(ids, config.experts)
    mask = ep.copy_mask(ids, world, local)
    plan = ep.make_plans((offsets[1:] - offsets[:-1]).reshape(1, -1), dist.group.WORLD,
                         copy_counts=mask.sum(0).reshape(1, -1))[0]
    assert plan.send_copies == mask.sum(0).tolist()
    # reference: one row per assignment
    rows = x[order.long() // 3]
    row_w = weights.reshape(-1)[order.long()]
    expected_rows, _ = ep.exchange(rows, plan, dist.group.WORLD)
    expected_w, _ = ep.exchange(row_w, plan, dist.group.WORLD)
    # de-duplicated
    token, copy_ids, copy_w, token_copies = ep.build_copies(mask, ids, weights, local, sum(plan.send_copies))
    # every token finds its copy for every rank that holds one of its experts, and only there
    for t in range(mask.shape[0]):
        for r in range(mask.shape[1]):
            position = int(token_copies[t, r])
            assert (position >= 0) == bool(mask[t, r])
            if position >= 0:
                assert int(token[position]) == t
    got_rows, _ = ep.exchange(x[token.long()], plan, dist.group.WORLD, copies=True)
    got_meta, _ = ep.exchange(torch.cat([copy_ids, copy_w.view(torch.int32)], dim=1), plan, dist.group.WORLD,
                              copies=True)

    def cpu_sort(keys, groups):
        flat = keys.reshape(-1).long()
        offs = torch.zeros(groups + 1, dtype=torch.int32)
        offs[1:] = torch.bincount(flat, minlength=groups).cumsum(0).to(torch.int32)
        return torch.sort(flat, stable=True).indices.to(torch.int32), offs, None, None

    assignment, segments = ep.expand_copies(got_meta[:, :3].contiguous(), plan.recv_copies, local, plan.recv_rows,
                                            sort=cpu_sort)
    assert torch.equal(segments, plan.segment_offsets)
    assert torch.equal(got_rows[assignment.long() // 3], expected_rows)
    assert torch.equal(got_meta[:, 3:].contiguous().view(torch.float32).reshape(-1)[assignment.long()], expected_w)
    return dict(copies=sum(plan.send_copies), rows=plan.send_rows)


@pytest.mark.parametrize("world", [2, 4])
def test_deduplicated_dispatch_equals_row_per_assignment(world):
    results = _run(_dedup_case, world=world)
    assert all(r["copies"] <= r["rows"] for r in results)
    assert sum(r["copies"] for r in results) < sum(r["rows"] for r in results)  # fewer rows travel


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
