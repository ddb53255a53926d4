"""Parity of the routing / permutation kernels, called through the C ABI on a B200:
expert ids, order, offsets, slots and counts bit-exact; route weights within fp32 rounding."""

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from mlops_b200 import ops

    return ops


def test_route_matches_reference_fixtures(golden):
    ops = _ops()
    for case in golden("routing.pt"):
        bias = None if case["bias"] is None else case["bias"].to(DEV)
        weights, ids = ops.route_topk(
            case["logits"].to(DEV), case["top_k"], case["mode"], bias=bias, n_group=case["n_group"],
            topk_group=case["topk_group"], routed_scaling=case["scaling"],
        )
        assert torch.equal(ids.cpu(), case["ids"]), case["mode"]
        torch.testing.assert_close(weights.cpu(), case["weights"], rtol=2e-6, atol=1e-7)
        order, offsets, slots, counts = ops.sort_assignments(case["ids"].to(DEV), case["logits"].shape[1])
        assert torch.equal(order.cpu(), case["order"])
        assert torch.equal(offsets.cpu(), case["offsets"])
        assert torch.equal(slots.cpu(), case["slots"])
        assert torch.equal(counts.cpu(), case["counts"])
    ops.check_status(DEV)


@pytest.mark.parametrize(
    "tokens,experts,top_k,mode,n_group,topk_group",
    [
        (4096, 8, 2, "softmax_then_topk", 1, 1),
        (4096, 128, 8, "softmax_then_topk", 1, 1),
        (4096, 256, 8, "sigmoid_noaux_tc", 8, 4),
        (2048, 256, 8, "topk_then_softmax", 1, 1),
        (1000, 96, 4, "sigmoid_noaux_tc", 8, 3),
        (1, 8, 8, "softmax_then_topk", 1, 1),
    ],
)
def test_route_ids_bit_exact_on_seeded_logits(tokens, experts, top_k, mode, n_group, topk_group):
    """Seeded fp32 logits fed to both sides; a row whose ids differ must be a genuine
    near-tie (counted and reported), and none is tolerated on these seeds."""
    ops = _ops()
    g = torch.Generator().manual_seed(tokens + experts)
    logits = torch.randn(tokens, experts, generator=g)
    bias = torch.randn(experts, generator=g) * 0.1 if mode == "sigmoid_noaux_tc" else None
    w_ref, id_ref = O.route(logits, top_k, mode, bias=bias, n_group=n_group, topk_group=topk_group,
                            routed_scaling=2.5)
    w, ids = ops.route_topk(logits.to(DEV), top_k, mode, bias=None if bias is None else bias.to(DEV),
                            n_group=n_group, topk_group=topk_group, routed_scaling=2.5)
    flipped = (ids.cpu() != id_ref).any(1).sum().item()
    assert flipped == 0, f"{flipped} of {tokens} rows selected different experts"
    torch.testing.assert_close(w.cpu(), w_ref, rtol=2e-6, atol=1e-7)


def test_sort_at_full_size_is_a_stable_permutation():
    """Config 5 size (T*K = 524288, E = 128, Zipf-skewed ids): bit-exact against the oracle and
    the size-independent properties (permutation, sortedness, stability, inverse)."""
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    experts = 128
    p = torch.arange(1, experts + 1).float().pow(-1.2)
    ids = torch.multinomial(p / p.sum(), 65536 * 8, replacement=True, generator=g).to(torch.int32).view(65536, 8)
    order, offsets, slots, counts = ops.sort_assignments(ids.to(DEV), experts)
    o_ref, f_ref, s_ref = O.sort_assignments(ids, experts)
    assert torch.equal(order.cpu(), o_ref) and torch.equal(offsets.cpu(), f_ref) and torch.equal(slots.cpu(), s_ref)
    order_l = order.long()
    flat = ids.reshape(-1).to(DEV)
    sorted_ids = flat[order_l]
    assert bool((sorted_ids[1:] >= sorted_ids[:-1]).all())                         # sortedness
    same = sorted_ids[1:] == sorted_ids[:-1]
    assert bool((order_l[1:][same] > order_l[:-1][same]).all())                    # stability
    assert torch.equal(torch.sort(order_l).values, torch.arange(flat.numel(), device=DEV))  # permutation
    assert torch.equal(slots.reshape(-1).long()[order_l], torch.arange(flat.numel(), device=DEV))  # inverse
    assert int(counts.sum()) == flat.numel()
    ops.check_status(DEV)


def test_sort_edge_cases():
    ops = _ops()
    # every assignment on one expert; experts without rows; a single assignment
    for ids, experts in (
        (torch.full((300, 2), 3, dtype=torch.int32), 8),
        (torch.tensor([[0, 7]], dtype=torch.int32), 8),
        (torch.tensor([[5]], dtype=torch.int32), 6),
    ):
        order, offsets, slots, counts = ops.sort_assignments(ids.to(DEV), experts)
        o_ref, f_ref, s_ref = O.sort_assignments(ids, experts)
        assert torch.equal(order.cpu(), o_ref) and torch.equal(offsets.cpu(), f_ref)
        assert torch.equal(slots.cpu(), s_ref)
    ops.check_status(DEV)


def test_out_of_range_expert_id_is_reported_and_sorted_as_the_nearest_expert():
    """A bad id must not leave holes in `order` / `slots` (later kernels index with them): it is
    reported in the status block and sorted as the nearest valid expert."""
    ops = _ops()
    from mlops_b200._lib import NativeError

    ids = torch.tensor([[0, 9], [-3, 2]], dtype=torch.int32, device=DEV)  # 9 >= experts, -3 < 0
    order, offsets, slots, counts = ops.sort_assignments(ids, 8)
    with pytest.raises(NativeError):
        ops.check_status(DEV)
    ops.check_status(DEV)  # the block was cleared
    clamped = ids.cpu().clamp(0, 7)
    o_ref, f_ref, s_ref = O.sort_assignments(clamped, 8)
    assert torch.equal(order.cpu(), o_ref) and torch.equal(offsets.cpu(), f_ref) and torch.equal(slots.cpu(), s_ref)
    assert int(counts.sum()) == 4


@pytest.mark.parametrize("mode", ["softmax_then_topk", "topk_then_softmax", "sigmoid_noaux_tc"])
def test_nan_and_infinite_logits_still_give_valid_ids(mode):
    """The reference selects with stable descending sorts, where NaN ranks first: ids stay K
    distinct experts in range and the NaN surfaces in the weights, never in an index."""
    ops = _ops()
    g = torch.Generator().manual_seed(17)
    experts, top_k = 64, 6
    logits = torch.randn(40, experts, generator=g)
    logits[0] = float("nan")                     # a diverged token: every logit NaN
    logits[1, 5] = float("nan")                  # one NaN
    logits[2, :60] = float("nan")                # fewer than K numbers left
    logits[3, 7] = float("inf")
    logits[4] = float("-inf")
    logits[5, 9] = float("-inf")
    kwargs = dict(bias=torch.randn(experts, generator=g) * 0.1, n_group=8, topk_group=4, routed_scaling=2.5) \
        if mode == "sigmoid_noaux_tc" else {}
    w_ref, ids_ref = O.route(logits, top_k, mode, **kwargs)
    dev_kwargs = dict(kwargs)
    if "bias" in dev_kwargs:
        dev_kwargs["bias"] = dev_kwargs["bias"].to(DEV)
    w, ids = ops.route_topk(logits.to(DEV), top_k, mode, **dev_kwargs)
    ids_c = ids.cpu()
    assert bool(((ids_c >= 0) & (ids_c < experts)).all())
    assert all(len(set(row.tolist())) == top_k for row in ids_c)
    assert torch.equal(ids_c, ids_ref), (ids_c[:6], ids_ref[:6])
    finite = torch.isfinite(w_ref).all(-1)
    torch.testing.assert_close(w.cpu()[finite], w_ref[finite], rtol=2e-6, atol=1e-7)
    assert torch.equal(torch.isnan(w.cpu()), torch.isnan(w_ref))


def test_routing_statistics_and_gradient_kernels_match_the_reference_fixture(golden):
    """`probability_sum`, `aux` and the gradient of the logits for every routing mode, with and
    without the auxiliary-loss and probability-sum cotangents and with several sequences:
    against the reference's own `routing_statistics` / `routing_gradient` outputs (fixture)."""
    from mlops_b200 import layer

    for case in golden("routing.pt"):
        experts = case["logits"].shape[1]
        dev = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
        aux, counts, psum = layer.routing_statistics(dev["logits"], dev["ids"], dev["counts"],
                                                     routing_mode=case["mode"], lengths=case["lengths"],
                                                     experts=experts)
        torch.testing.assert_close(aux.cpu(), case["aux"], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(psum.cpu(), case["psum"], rtol=1e-5, atol=1e-5)
        assert counts.dtype == torch.int64
        again = layer.routing_statistics(dev["logits"], dev["ids"], dev["counts"], routing_mode=case["mode"],
                                         lengths=case["lengths"], experts=experts)
        assert torch.equal(again[2], psum)  # a fixed summation order: bitwise repeatable
        grad = layer.routing_gradient(dev["grad_aux"], dev["grad_psum"], dev["grad_w"], dev["weights"], dev["ids"],
                                      dev["logits"], dev["counts"], routing_mode=case["mode"],
                                      lengths=case["lengths"])
        torch.testing.assert_close(grad.cpu(), case["grad_logits"], rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("mode,experts,top_k", [("sigmoid_noaux_tc", 256, 8), ("softmax_then_topk", 128, 8),
                                                 ("topk_then_softmax", 40, 3)])
def test_routing_gradient_kernel_against_the_oracle_at_size(mode, experts, top_k):
    from mlops_b200 import layer

    g = torch.Generator().manual_seed(experts)
    tokens = 3000
    logits = torch.randn(tokens, experts, generator=g) * 2
    kwargs = dict(bias=torch.randn(experts, generator=g) * 0.1, n_group=8, topk_group=4, routed_scaling=2.5) \
        if mode == "sigmoid_noaux_tc" else {}
    weights, ids = O.route(logits, top_k, mode, **kwargs)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=experts)
    grad_w = torch.randn(tokens, top_k, generator=g)
    grad_aux, grad_psum = torch.tensor(0.7), torch.randn(experts, generator=g)
    lengths = (1000, 1500, 500)
    for ga, gp, ln in ((None, None, (tokens,)), (grad_aux, grad_psum, (tokens,)), (grad_aux, grad_psum, lengths)):
        ref = O.routing_gradient(ga, gp, grad_w, weights, ids, logits, counts, routing_mode=mode, lengths=ln)
        dev = lambda t: None if t is None else t.to(DEV)  # noqa: E731
        out = layer.routing_gradient(dev(ga), dev(gp), dev(grad_w), dev(weights), dev(ids), dev(logits), dev(counts),
                                     routing_mode=mode, lengths=ln)
        torch.testing.assert_close(out.cpu(), ref, rtol=2e-5, atol=2e-6)
        aux_ref, _, psum_ref = O.routing_statistics(logits, ids, routing_mode=mode, lengths=ln, experts=experts)
        aux, _, psum = layer.routing_statistics(dev(logits), dev(ids), dev(counts), routing_mode=mode, lengths=ln,
                                                experts=experts)
        torch.testing.assert_close(aux.cpu(), aux_ref, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(psum.cpu(), psum_ref, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("world,local,top_k,tokens", [(2, 4, 4, 700), (8, 32, 8, 3000), (4, 1, 2, 33)])
def test_build_copies_kernel_matches_the_host_logic(world, local, top_k, tokens):
    """The sender's plan of a de-duplicated dispatch as one kernel against the tensor-op form that
    the CPU (gloo) tests of the expert-parallel layer pin: identical copies, metadata and positions."""
    from mlops_b200 import ep, ops

    g = torch.Generator().manual_seed(world * 100 + tokens)
    experts = world * local
    keys = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).to(torch.int32)
    weights = torch.rand(tokens, top_k, generator=g)
    mask = ep.copy_mask(keys, world, local)
    send_copies = mask.sum(0).tolist()
    token_ref, ids_ref, w_ref, tc_ref = ep.build_copies(mask, keys, weights, local, int(sum(send_copies)))
    token, meta, token_copies = ops.build_copies(keys.to(DEV), weights.to(DEV), world, local, send_copies)
    ops.check_status(DEV)
    assert torch.equal(token.cpu(), token_ref)
    assert torch.equal(meta[:, :top_k].cpu(), ids_ref)
    assert torch.equal(meta[:, top_k:].contiguous().view(torch.float32).cpu(), w_ref)
    assert torch.equal(token_copies.cpu(), tc_ref)
