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
