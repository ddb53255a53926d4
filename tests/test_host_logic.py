"""Host-side logic of the package that needs no GPU: the routing statistics and the routing
VJP (plain PyTorch) against the reference's fixtures, argument validation, scale layout."""

import pytest
import torch

from mlops_b200 import layer


def test_routing_statistics_match_reference(golden):
    for case in golden("routing.pt"):
        experts = case["logits"].shape[1]
        aux, counts, psum = layer.routing_statistics(
            case["logits"], case["ids"], case["counts"], routing_mode=case["mode"],
            lengths=case["lengths"], experts=experts,
        )
        torch.testing.assert_close(aux, case["aux"], rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(psum, case["psum"], rtol=1e-6, atol=1e-6)
        assert counts.dtype == torch.int64


def test_routing_gradient_matches_reference(golden):
    for case in golden("routing.pt"):
        grad = layer.routing_gradient(
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
