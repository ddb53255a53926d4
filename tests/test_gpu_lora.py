"""Expert LoRA on a B200 through `mlops_b200.lora.expert_lora` against the CPU oracle
(identical FP8 operands: max rel <= 2e-2, mean <= 2e-3) and the reference's builtin
composition (fixture, 8e-2). Contracts from the reference's tests/test_sonicmoe_lora.py:
zero B factors equal `moe` (:159-193), a frozen base launches no base weight gradient
(:209-233), ranks that are not multiples of 8 are accepted (:446-451)."""

import pytest
import torch

import inputs
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FACTORS = ("a13", "b13", "a2", "b2")


def _setup(rank=16, base_grad=False):
    from mlops_b200.weights import BlockFP8Weight

    lc = inputs.lora_case(rank)
    dev = {k: v.to(DEV) if isinstance(v, torch.Tensor) else v for k, v in lc.items()}
    dev["x"].requires_grad_(True)
    dev["router"].requires_grad_(True)
    for name in FACTORS:
        dev[name].requires_grad_(True)
    g13 = BlockFP8Weight.quantize(dev["w13"]).requires_grad_(base_grad)
    g2 = BlockFP8Weight.quantize(dev["w2"]).requires_grad_(base_grad)
    return lc, dev, g13, g2


def _call(dev, g13, g2, **override):
    from mlops_b200.lora import expert_lora

    args = dict(dev, **override)
    return expert_lora(args["x"], args["residual"], args["router"], g13, g2, args["a13"], args["b13"], args["a2"],
                       args["b2"], top_k=dev["top_k"], routing_mode=dev["routing_mode"], scale=dev["scale"])


def test_rank_kernels_against_float64():
    from mlops_b200 import ops

    g = torch.Generator().manual_seed(2)
    counts = [0, 70, 131, 15, 260]
    offs = torch.zeros(6, dtype=torch.int32)
    offs[1:] = torch.tensor(counts).cumsum(0)
    rows = sum(counts)
    for rank, wide in ((16, 1280), (24, 384), (64, 2048)):
        x = torch.randn(rows, wide, generator=g).bfloat16()
        rank_major = torch.randn(5, rank, wide, generator=g).bfloat16()
        wide_major = torch.randn(5, wide, rank, generator=g).bfloat16()
        for factor, flag in ((rank_major, True), (wide_major, False)):
            t = ops.lora_project(x.to(DEV), factor.to(DEV), offs.to(DEV), rank_major=flag)
            ref = O._factor_rows(x, factor, offs, flag)
            mx, mean = O.rel_errors(t.float().cpu(), ref)
            assert mx <= 2e-2 and mean <= 2e-3, ("project", rank, wide, flag, mx, mean)
        t = torch.randn(rows, rank, generator=g).bfloat16()
        for factor, flag in ((wide_major, True), (rank_major, False)):
            c = ops.lora_expand(t.to(DEV), factor.to(DEV), offs.to(DEV), wide_major=flag, scale=0.5)
            ref = 0.5 * O._factor_rows(t, factor, offs, flag)
            mx, mean = O.rel_errors(c.float().cpu(), ref)
            assert mx <= 2e-2 and mean <= 2e-3, ("expand", rank, wide, flag, mx, mean)


def test_gemm_addend_is_added_before_the_rounding():
    from mlops_b200 import ops

    g = torch.Generator().manual_seed(4)
    a = torch.randn(200, 256, generator=g)
    a_q, a_s = O.quantize_rows(a)
    b_q, b_s = O.quantize_blocks(torch.randn(2, 384, 256, generator=g))
    offs = torch.tensor([0, 70, 200], dtype=torch.int32)
    addend = torch.randn(200, 384, generator=g).bfloat16()
    out = ops.grouped_gemm_fp8(a_q.to(DEV), a_s.to(DEV), b_q.to(DEV), b_s.to(DEV), offs.to(DEV),
                               addend=addend.to(DEV))
    ref = O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs) + addend.double()
    mx, mean = O.rel_errors(out.float().cpu(), ref)
    assert mx <= 2e-2 and mean <= 2e-3


@pytest.mark.parametrize("rank", [16, 12])
def test_layer_against_oracle(rank):
    from mlops_b200 import layer, ops

    lc, dev, g13, g2 = _setup(rank)
    out, aux, counts, psum = _call(dev, g13, g2)
    grads = torch.autograd.grad(out, [dev["x"], *(dev[n] for n in FACTORS)], dev["dy"])
    ops.check_status(DEV)
    w13, w2 = O.quantize_blocks(lc["w13"]), O.quantize_blocks(lc["w2"])
    logits = layer.router_logits(dev["x"].detach(), dev["router"].detach()).cpu()
    fwd = O.forward_lora_block_fp8(lc["x"], lc["residual"], logits, *w13, *w2, lc["a13"], lc["b13"], lc["a2"],
                                   lc["b2"], top_k=lc["top_k"], routing_mode=lc["routing_mode"], scale=lc["scale"])
    assert torch.equal(counts.cpu(), torch.bincount(fwd["ids"].reshape(-1).long(), minlength=4))
    mx, mean = O.rel_errors(out.float().cpu(), fwd["output"].float())
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    bwd = O.backward_lora_block_fp8(lc["dy"], fwd, *w13, *w2, lc["a13"], lc["b13"], lc["a2"], lc["b2"],
                                    top_k=lc["top_k"], scale=lc["scale"])
    for name, grad in zip(FACTORS, grads[1:]):
        assert grad.shape == lc[name].shape and grad.dtype == torch.bfloat16
        mx, mean = O.rel_errors(grad.float().cpu(), bwd["grad_" + name])
        assert mx <= 3e-2 and mean <= 3e-3, (name, mx, mean)
    grad_logits = O.routing_gradient(None, None, bwd["grad_route_weights"], fwd["weights"], fwd["ids"], logits,
                                         counts.cpu(), routing_mode=lc["routing_mode"], lengths=(96,))
    expected_x = bwd["grad_h2"].float() + grad_logits.bfloat16().float() @ lc["router"].bfloat16().float()
    mx, mean = O.rel_errors(grads[0].float().cpu(), expected_x)
    assert mx <= 3e-2 and mean <= 3e-3, ("grad_x", mx, mean)


def test_against_reference_builtin_fixture(golden):
    fixture = golden("lora_builtin.pt")
    lc, dev, g13, g2 = _setup()
    out, aux, counts, psum = _call(dev, g13, g2)
    grads = torch.autograd.grad(out, [dev["x"], dev["router"], *(dev[n] for n in FACTORS)], dev["dy"])

    def frob(a, e):
        return ((a.double().cpu() - e.double()).norm() / e.double().norm()).item()

    assert torch.equal(counts.cpu(), fixture["counts"])
    assert frob(out.float().cpu() - lc["residual"].float(), fixture["output"].float() - lc["residual"].float()) < 8e-2
    for name, grad in zip(("x", "router", *FACTORS), grads):
        assert frob(grad, fixture["grad_" + name]) < 8e-2, name


def test_zero_b_factors_equal_the_plain_layer_and_frozen_base_launches_no_base_wgrad():
    from mlops_b200 import ops, provider

    lc, dev, g13, g2 = _setup()
    zeros = dict(b13=torch.zeros_like(dev["b13"]), b2=torch.zeros_like(dev["b2"]))
    out, *_ = _call(dev, g13, g2, **zeros)
    plain, *_ = provider.apply(dev["x"], dev["residual"], dev["router"], g13, g2, top_k=dev["top_k"],
                               routing_mode=dev["routing_mode"])
    assert torch.equal(out, plain)
    # frozen base: gradients for the containers are None and their two GEMMs are not launched
    out, *_ = _call(dev, g13, g2)
    before = ops.LAUNCHES
    torch.autograd.grad(out, [dev["x"], *(dev[n] for n in FACTORS)], dev["dy"])
    frozen = ops.LAUNCHES - before
    lc, dev2, t13, t2 = _setup(base_grad=True)
    out2, *_ = _call(dev2, t13, t2)
    before = ops.LAUNCHES
    grads = torch.autograd.grad(out2, [dev2["x"], t13, t2, *(dev2[n] for n in FACTORS)], dev2["dy"])
    assert ops.LAUNCHES - before == frozen + 2
    assert grads[1].shape == t13.shape and grads[2].shape == t2.shape


def test_gradient_destinations_accumulate_in_the_gemm_store():
    """Two micro-batches with explicit destinations: each factor's buffer ends up holding
    `start + scale * (g1 + g2)` (the sums formed in fp32 inside the weight-gradient GEMMs'
    stores), the factors' own `.grad` stays empty, and the input gradient is unchanged
    (reference contract: src/mlops/providers/sonicmoe/lora_destinations.py:1-16)."""
    from mlops_b200 import ops
    from mlops_b200.lora import expert_lora

    lc, dev, g13, g2 = _setup(16)
    expected, grad_x = None, []
    for seed in (1, 2):
        x = (dev["x"].detach() * (1.0 + 0.25 * seed)).requires_grad_(True)
        out, *_ = _call(dict(dev, x=x), g13, g2)
        grads = torch.autograd.grad(out, [x, *(dev[n] for n in FACTORS)], dev["dy"])
        grad_x.append(grads[0])
        expected = [g.float() for g in grads[1:]] if expected is None else [e + g.float() for e, g in zip(expected, grads[1:])]
    start = {name: torch.randn(dev[name].shape, device=DEV) for name in FACTORS}
    buffers = {name: value.clone() for name, value in start.items()}
    for i, seed in enumerate((1, 2)):
        x = (dev["x"].detach() * (1.0 + 0.25 * seed)).requires_grad_(True)
        out, *_ = expert_lora(x, dev["residual"], dev["router"], g13, g2, *(dev[n] for n in FACTORS),
                              top_k=dev["top_k"], routing_mode=dev["routing_mode"], scale=dev["scale"],
                              gradient_destinations=buffers, gradient_scale=0.5)
        (gx,) = torch.autograd.grad(out, [x], dev["dy"], allow_unused=False)
        assert torch.equal(gx, grad_x[i])
    ops.check_status(DEV)
    for name, total in zip(FACTORS, expected):
        assert dev[name].grad is None
        want = start[name] + 0.5 * total
        torch.testing.assert_close(buffers[name], want, rtol=2e-2, atol=2e-2 * float(total.abs().mean()))
        assert not torch.equal(buffers[name], start[name])
    with pytest.raises(ValueError):
        expert_lora(dev["x"], dev["residual"], dev["router"], g13, g2, *(dev[n] for n in FACTORS),
                    top_k=dev["top_k"], routing_mode=dev["routing_mode"], scale=dev["scale"],
                    gradient_destinations={"a13": buffers["a13"]})
