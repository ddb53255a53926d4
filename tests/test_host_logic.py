"""Host-side logic that needs no GPU: the oracle's routing VJP against the reference's fixture
(the kernels are compared with it on the GPU in test_gpu_routing.py), argument validation, the
expert-parallel index arithmetic."""

import pytest
import torch

from mlops_b200 import layer
from oracle import moe_oracle as O


def test_oracle_routing_gradient_matches_reference(golden):
    for case in golden("routing.pt"):
        grad = O.routing_gradient(
            case["grad_aux"], case["grad_psum"], case["grad_w"], case["weights"], case["ids"],
            case["logits"], case["counts"], routing_mode=case["mode"], lengths=case["lengths"],
        )
        torch.testing.assert_close(grad, case["grad_logits"], rtol=1e-5, atol=1e-6)


def test_lengths_must_cover_every_row():
    with pytest.raises(ValueError):
        layer._normalized_lengths((3, 4), 8)
    with pytest.raises(ValueError):
        layer._normalized_lengths((0, 8), 8)
    assert layer._normalized_lengths(None, 8) == (8,)


@pytest.mark.parametrize("world,local,seed", [(2, 3, 0), (4, 2, 1), (8, 4, 2), (1, 5, 3)])
def test_regroup_index_orders_received_rows_by_expert(world, local, seed):
    """Rows received as [source rank][local expert] segments are renumbered by expert, the
    sources in rank order inside an expert; the index is a permutation and empty segments are
    fine."""
    from mlops_b200.ep import regroup_index

    g = torch.Generator().manual_seed(seed)
    counts = torch.randint(0, 6, (world, local), generator=g)
    counts[0, 0] = 0
    offsets = torch.zeros(world * local + 1, dtype=torch.int32)
    offsets[1:] = counts.reshape(-1).cumsum(0).to(torch.int32)
    rows = int(counts.sum())
    by_expert, source = regroup_index(offsets, world, local, rows)
    # brute force: walk experts, then sources, and list the arrival positions
    expected, expected_offsets = [], [0]
    for e in range(local):
        for s in range(world):
            lo = int(offsets[s * local + e])
            expected.extend(range(lo, lo + int(counts[s, e])))
        expected_offsets.append(len(expected))
    assert by_expert.tolist() == expected_offsets
    assert source.tolist() == expected
    assert sorted(source.tolist()) == list(range(rows))


def _cpu_sort(keys, groups):
    flat = keys.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices.to(torch.int32)
    offsets = torch.zeros(groups + 1, dtype=torch.int32)
    offsets[1:] = torch.bincount(flat, minlength=groups).cumsum(0).to(torch.int32)
    return order, offsets, None, None


@pytest.mark.parametrize("world,local,top_k,seed", [(2, 4, 2, 0), (4, 2, 3, 1), (8, 4, 8, 2)])
def test_deduplicated_dispatch_reproduces_the_row_per_assignment_layout(world, local, top_k, seed):
    """Copies (one per token and destination rank, with the list of local experts) expand on the
    receiver into exactly the rows, in exactly the order, that sending one row per assignment
    sorted by (rank, expert, token) delivers."""
    from mlops_b200.ep import build_copies, copy_mask, expand_copies

    g = torch.Generator().manual_seed(seed)
    experts = world * local
    tokens = [11 + 3 * r for r in range(world)]
    keys = [torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(t)]).to(torch.int32)
            for t in tokens]
    weights = [torch.rand(t, top_k, generator=g) for t in tokens]
    sent = []  # per source: (token, ids, weight) of its copies and the copy counts per destination
    for s in range(world):
        mask = copy_mask(keys[s], world, local)
        counts = mask.sum(0)
        token, ids, weight, token_copies = build_copies(mask, keys[s], weights[s], local, int(counts.sum()))
        assert torch.equal(token_copies >= 0, mask)
        assert torch.equal(token[token_copies[mask].long()].long(), mask.nonzero()[:, 0])
        sent.append((token, ids, weight, counts.tolist()))
        assert all(int(n) <= tokens[s] for n in counts)
    for d in range(world):
        # what arrives at rank d: from every source its copies for d, in the order they were built
        ids, weight, origin, recv_copies = [], [], [], []
        for s in range(world):
            token, all_ids, all_weight, counts = sent[s]
            lo = sum(counts[:d])
            ids.append(all_ids[lo:lo + counts[d]])
            weight.append(all_weight[lo:lo + counts[d]])
            origin += [(s, int(t)) for t in token[lo:lo + counts[d]]]
            recv_copies.append(counts[d])
        ids, weight = torch.cat(ids), torch.cat(weight)
        # the row-per-assignment dispatch: every source sorts its assignments by (rank, expert, token)
        expected = []
        for s in range(world):
            rows = [(int(keys[s][t, k]) - d * local, t, float(weights[s][t, k]))
                    for t in range(tokens[s]) for k in range(top_k) if int(keys[s][t, k]) // local == d]
            expected += [(s, e, t, w) for e, t, w in sorted(rows)]
        assignment, offsets = expand_copies(ids, recv_copies, local, len(expected), sort=_cpu_sort)
        got = []
        for a in assignment.tolist():
            copy, slot = divmod(a, top_k)
            got.append((origin[copy][0], int(ids[copy, slot]), origin[copy][1], float(weight[copy, slot])))
        assert got == expected
        segment_rows = [sum(1 for row in expected if row[0] == s and row[1] == e)
                        for s in range(world) for e in range(local)]
        assert (offsets[1:] - offsets[:-1]).tolist() == segment_rows
