"""Parity of the whole routed layer (forward and VJP) through the package's host mirror of
the reference's `forward_routed` / `backward_routed`, against (a) the CPU oracle on
identical block-FP8 operands (max relative error <= 2e-2, mean <= 2e-3; integers exact) and
(b) the reference's own native-PyTorch provider on config 1 (fixture) at the reference's
FP8-vs-bf16 bounds."""

import pytest
import torch

import inputs
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_REL, MEAN_REL = 2e-2, 2e-3


def _layer():
    from mlops_b200 import layer, ops

    return layer, ops


def _check(actual, expected, what):
    mx, mean = O.rel_errors(actual.float().cpu(), expected)
    assert mx <= MAX_REL and mean <= MEAN_REL, (what, mx, mean)


def _run_case(x, residual, router, w13, w2, dy, *, top_k, mode, bias=None, n_group=1, topk_group=1,
              scaling=1.0, limit=None):
    layer, ops = _layer()
    experts = router.shape[0]
    w13_q, w13_s = O.quantize_blocks(w13)
    w2_q, w2_s = O.quantize_blocks(w2)
    dev = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    result = layer.forward_routed(
        dev(x), dev(residual), dev(router), (dev(w13_q), dev(w13_s)), (dev(w2_q), dev(w2_s)), top_k=top_k,
        routing_mode=mode, router_bias=dev(bias), n_group=n_group, topk_group=topk_group,
        routed_scaling=scaling, swiglu_limit=limit,
    )
    output, aux, counts, psum, logits, route_weights, route_ids, order, offsets, slots, h13 = result
    ops.check_status(DEV)
    # the oracle takes the logits the device formed (bf16 operands, fp32 sums), so both sides
    # route from identical numbers
    fwd = O.forward_block_fp8(x, residual, logits.cpu(), w13_q, w13_s, w2_q, w2_s, top_k=top_k,
                              routing_mode=mode, router_bias=bias, n_group=n_group,
                              topk_group=topk_group, routed_scaling=scaling, swiglu_limit=limit)
    assert torch.equal(route_ids.cpu(), fwd["ids"])
    assert torch.equal(order.cpu(), fwd["order"]) and torch.equal(offsets.cpu(), fwd["offsets"])
    assert torch.equal(slots.cpu(), fwd["slots"])
    assert torch.equal(counts.cpu(), torch.bincount(fwd["ids"].reshape(-1).long(), minlength=experts))
    torch.testing.assert_close(route_weights.cpu(), fwd["weights"], rtol=2e-6, atol=1e-7)
    torch.testing.assert_close(logits.cpu(), O.router_logits(x, router), rtol=1e-4, atol=1e-4)
    _check(h13, fwd["h13"].float(), "h13")
    _check(output, fwd["output"].float(), "output")
    aux_ref, _, psum_ref = O.routing_statistics(logits.cpu(), fwd["ids"], routing_mode=mode,
                                                lengths=(x.shape[0],), experts=experts)
    torch.testing.assert_close(aux.cpu(), aux_ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(psum.cpu(), psum_ref, rtol=1e-5, atol=1e-5)

    grads = layer.backward_routed(
        dev(dy), None, None, dev(x), dev(router), (dev(w13_q), dev(w13_s)), (dev(w2_q), dev(w2_s)),
        logits, route_weights, route_ids, order, offsets, slots, h13, top_k=top_k, routing_mode=mode,
        swiglu_limit=limit, weight_grad_dtype=torch.float32,
    )
    ops.check_status(DEV)
    grad_h2, grad_residual, grad_router, grad_w13, grad_w2 = grads
    # oracle backward from the DEVICE's saved h13 so the two sides differentiate the same point
    fwd_dev = dict(fwd, h13=h13.cpu())
    bwd = O.backward_block_fp8(dy, x, fwd_dev, w13_q, w13_s, w2_q, w2_s, top_k=top_k, swiglu_limit=limit)
    assert torch.equal(grad_residual.cpu(), dy)
    grad_logits = O.routing_gradient(None, None, bwd["grad_route_weights"], fwd["weights"], fwd["ids"],
                                         logits.cpu(), counts.cpu(), routing_mode=mode, lengths=(x.shape[0],))
    expected_h2 = bwd["grad_h2"].float() + grad_logits.bfloat16().float() @ router.bfloat16().float()
    _check(grad_h2, expected_h2, "grad_h2")
    _check(grad_router, grad_logits.t() @ x.float(), "grad_router")
    for e in range(experts):
        if int(counts[e]) == 0:
            assert int(torch.count_nonzero(grad_w13[e])) == 0 and int(torch.count_nonzero(grad_w2[e])) == 0
    _check(grad_w13, bwd["grad_w13"], "grad_w13")
    _check(grad_w2, bwd["grad_w2"], "grad_w2")
    return result, grads


@pytest.mark.parametrize("case", ["config1", "groups"])
def test_bf16_compute_path_against_the_oracle_and_the_reference(case, golden):
    """Plain bf16 expert weights select the bf16 path (bf16 grouped GEMMs, nothing quantised):
    every output and gradient against the CPU restatement on the same bf16 weights, and on
    configuration 1 against the stored outputs of the reference's own bf16 provider
    (`native_torch.moe` on the dequantised block-FP8 weights: the same weight values)."""
    layer, ops = _layer()
    if case == "config1":
        c = inputs.config1()
        x, residual, router, dy = c["x"], c["residual"], c["router"], c["dy"]
        w13_q, w13_s = O.quantize_blocks(c["w13"])
        w2_q, w2_s = O.quantize_blocks(c["w2"])
        w13 = O.dequantize_blocks(w13_q, w13_s, torch.bfloat16)   # what the reference multiplies
        w2 = O.dequantize_blocks(w2_q, w2_s, torch.bfloat16)
        kwargs = dict(top_k=c["top_k"], routing_mode=c["routing_mode"])
        bias = None
    else:
        g = torch.Generator().manual_seed(31)
        tokens, width, inner, experts = 192, 192, 80, 16   # partial tiles everywhere
        x = torch.randn(tokens, width, generator=g).bfloat16()
        residual = torch.randn(tokens, width, generator=g).bfloat16()
        dy = torch.randn(tokens, width, generator=g).bfloat16()
        router = torch.randn(experts, width, generator=g) * 0.05
        w13 = (torch.randn(experts, 2 * inner, width, generator=g) * 0.05).bfloat16()
        w2 = (torch.randn(experts, width, inner, generator=g) * 0.05).bfloat16()
        bias = torch.randn(experts, generator=g) * 0.1
        kwargs = dict(top_k=4, routing_mode="sigmoid_noaux_tc", n_group=4, topk_group=2, routed_scaling=2.5)
    dev = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    result = layer.forward_routed(dev(x), dev(residual), dev(router), dev(w13), dev(w2), router_bias=dev(bias),
                                  swiglu_limit=7.0 if case == "groups" else None, **kwargs)
    output, aux, counts, psum, logits, route_weights, route_ids, order, offsets, slots, h13 = result
    ops.check_status(DEV)
    fwd = O.forward_bf16(x, residual, logits.cpu(), w13, w2, router_bias=bias,
                         swiglu_limit=7.0 if case == "groups" else None, **kwargs)
    assert torch.equal(route_ids.cpu(), fwd["ids"]) and torch.equal(order.cpu(), fwd["order"])
    _check(h13, fwd["h13"].float(), "h13")
    _check(output, fwd["output"].float(), "output")
    back_kwargs = {k: v for k, v in kwargs.items() if k in ("top_k", "routing_mode")}
    grads = layer.backward_routed(dev(dy), None, None, dev(x), dev(router), dev(w13), dev(w2), logits,
                                  route_weights, route_ids, order, offsets, slots, h13,
                                  swiglu_limit=7.0 if case == "groups" else None,
                                  weight_grad_dtype=torch.float32, **back_kwargs)
    ops.check_status(DEV)
    bwd = O.backward_bf16(dy, x, dict(fwd, h13=h13.cpu()), w13, w2, top_k=kwargs["top_k"],
                          swiglu_limit=7.0 if case == "groups" else None)
    grad_logits = O.routing_gradient(None, None, bwd["grad_route_weights"], fwd["weights"], fwd["ids"],
                                     logits.cpu(), counts.cpu(), routing_mode=kwargs["routing_mode"],
                                     lengths=(x.shape[0],))
    _check(grads[0], bwd["grad_h2"].float() + grad_logits.bfloat16().float() @ router.bfloat16().float(), "grad_h2")
    assert torch.equal(grads[1].cpu(), dy)
    _check(grads[2], grad_logits.t() @ x.float(), "grad_router")
    _check(grads[3], bwd["grad_w13"], "grad_w13")
    _check(grads[4], bwd["grad_w2"], "grad_w2")
    if case == "config1":
        fixture = golden("config1_native_torch.pt")

        def frob(a, e):
            return ((a.double().cpu() - e.double()).norm() / e.double().norm()).item()

        # bf16 against bf16 on the same weight values: rounding-order differences only
        assert frob(output, fixture["output"]) < 1e-2
        assert frob(grads[0], fixture["grad_x"]) < 1e-2
        assert frob(grads[2], fixture["grad_router"]) < 2e-2
        assert frob(grads[3][:, ::16, ::8], fixture["grad_w13_sample"]) < 1e-2
        assert frob(grads[4][:, ::8, ::16], fixture["grad_w2_sample"]) < 1e-2


def test_fp8_weight_gradients_stay_within_the_reference_bound_of_that_recipe():
    """`weight_grad_operands="fp8"`: the other gradients do not change at all, and the expert
    weight gradients stay within the relative-Frobenius bound the reference sets for its FP8
    weight-gradient recipe (6e-2, tests/test_sonicmoe_fp8.py:114-124) of the bf16-operand ones."""
    layer, ops = _layer()
    c1 = inputs.config1()
    w13_q, w13_s = O.quantize_blocks(c1["w13"])
    w2_q, w2_s = O.quantize_blocks(c1["w2"])
    dev = lambda t: t.to(DEV)  # noqa: E731
    w13, w2 = (dev(w13_q), dev(w13_s)), (dev(w2_q), dev(w2_s))
    result = layer.forward_routed(dev(c1["x"]), dev(c1["residual"]), dev(c1["router"]), w13, w2,
                                  top_k=c1["top_k"], routing_mode=c1["routing_mode"])
    saved = result[4:]
    grads = {}
    for operands in ("bf16", "fp8"):
        grads[operands] = layer.backward_routed(
            dev(c1["dy"]), None, None, dev(c1["x"]), dev(c1["router"]), w13, w2, *saved, top_k=c1["top_k"],
            routing_mode=c1["routing_mode"], weight_grad_dtype=torch.float32, weight_grad_operands=operands)
    ops.check_status(DEV)
    for i in (0, 1, 2):
        assert torch.equal(grads["fp8"][i], grads["bf16"][i])
    for i in (3, 4):
        exact, fp8 = grads["bf16"][i].double(), grads["fp8"][i].double()
        assert ((fp8 - exact).norm() / exact.norm()).item() < 6e-2
    with pytest.raises(ValueError):
        layer.backward_routed(dev(c1["dy"]), None, None, dev(c1["x"]), dev(c1["router"]), w13, w2, *saved,
                              top_k=c1["top_k"], routing_mode=c1["routing_mode"], weight_grad_operands="fp4")


def test_config1_against_oracle_and_reference_fixture(golden):
    c1 = inputs.config1()
    result, grads = _run_case(c1["x"], c1["residual"], c1["router"], c1["w13"], c1["w2"], c1["dy"],
                              top_k=c1["top_k"], mode=c1["routing_mode"])
    fixture = golden("config1_native_torch.pt")

    def frob(a, e):
        return ((a.double().cpu() - e.double()).norm() / e.double().norm()).item()

    # vs the reference's bf16-on-dequantised-weights provider: its FP8 tests' bounds
    # (output 4e-2 [4.5e-2 here, see tests/test_oracle_golden.py], dh2 8e-2, drouter 8e-2, dw 6e-2)
    assert frob(result[0], fixture["output"]) < 4.5e-2
    assert frob(grads[0], fixture["grad_x"]) < 8e-2
    assert frob(grads[2], fixture["grad_router"]) < 8e-2
    assert frob(grads[3][:, ::16, ::8], fixture["grad_w13_sample"]) < 6e-2
    assert frob(grads[4][:, ::8, ::16], fixture["grad_w2_sample"]) < 6e-2
    torch.testing.assert_close(result[1].cpu(), fixture["aux"], rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(result[3].cpu(), fixture["psum"], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize(
    "mode,experts,top_k,n_group,topk_group,scaling,limit",
    [
        ("topk_then_softmax", 8, 2, 1, 1, 1.0, None),
        ("sigmoid_noaux_tc", 16, 4, 4, 2, 2.5, None),
        ("softmax_then_topk", 5, 2, 1, 1, 1.0, 0.5),   # odd expert count, SwiGLU clamp
    ],
)
def test_routing_modes_against_oracle(mode, experts, top_k, n_group, topk_group, scaling, limit):
    g = torch.Generator().manual_seed(experts)
    tokens, width, inner = 300, 256, 384
    x = torch.randn(tokens, width, generator=g).bfloat16()
    residual = torch.randn(tokens, width, generator=g).bfloat16()
    router = torch.randn(experts, width, generator=g) * 0.05
    if mode == "sigmoid_noaux_tc":
        router[-1] = 0  # an expert no token prefers; bias below keeps it out of every top-k
    w13 = (torch.randn(experts, 2 * inner, width, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(experts, width, inner, generator=g) * 0.05).bfloat16()
    dy = torch.randn(tokens, width, generator=g).bfloat16()
    bias = None
    if mode == "sigmoid_noaux_tc":
        bias = torch.randn(experts, generator=g) * 0.1
        bias[-1] = -10.0
    _run_case(x, residual, router, w13, w2, dy, top_k=top_k, mode=mode, bias=bias, n_group=n_group,
              topk_group=topk_group, scaling=scaling, limit=limit)


def test_frozen_gradients_skip_their_gemms_and_leave_the_rest_bit_identical():
    """Reference contract (tests/test_moe_frozen_gradients.py:74-116): a gradient nobody asked
    for is an empty placeholder; the others are bit-identical to the all-trainable step."""
    layer, ops = _layer()
    c1 = inputs.config1()
    w13 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w13"]))
    w2 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w2"]))
    x, router, dy = c1["x"].to(DEV), c1["router"].to(DEV), c1["dy"].to(DEV)
    res = layer.forward_routed(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    saved = res[4:]
    full = layer.backward_routed(dy, None, None, x, router, w13, w2, *saved, top_k=2,
                                 routing_mode="softmax_then_topk")
    frozen = layer.backward_routed(dy, None, None, x, router, w13, w2, *saved, top_k=2,
                                   routing_mode="softmax_then_topk", need_router=False, need_w13=False,
                                   need_w2=False)
    assert frozen[2].numel() == 0 and frozen[3].numel() == 0 and frozen[4].numel() == 0
    assert torch.equal(full[0], frozen[0]) and torch.equal(full[1], frozen[1])
    again = layer.backward_routed(dy, None, None, x, router, w13, w2, *saved, top_k=2,
                                  routing_mode="softmax_then_topk")
    for a, b in zip(full, again):
        assert torch.equal(a, b)  # bitwise repeatable
    ops.check_status(DEV)


def test_fused_swiglu_layer_is_bit_identical():
    layer, ops = _layer()
    c1 = inputs.config1()
    w13 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w13"]))
    w2 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w2"]))
    x, router = c1["x"].to(DEV), c1["router"].to(DEV)
    plain = layer.forward_routed(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    fused = layer.forward_routed(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk",
                                 fuse_swiglu=True)
    assert torch.equal(plain[0], fused[0]) and torch.equal(plain[10], fused[10])
    ops.check_status(DEV)


def test_fused_combine_layer_matches_within_one_rounding():
    """`fuse_combine=True` changes only the order of the fp32 sum behind the output's one bf16
    rounding; everything saved for the backward pass is unchanged."""
    layer, ops = _layer()
    c1 = inputs.config1()
    w13 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w13"]))
    w2 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w2"]))
    x, router = c1["x"].to(DEV), c1["router"].to(DEV)
    residual = torch.randn(x.shape, generator=torch.Generator().manual_seed(3)).bfloat16().to(DEV)
    plain = layer.forward_routed(x, residual, router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    fused = layer.forward_routed(x, residual, router, w13, w2, top_k=2, routing_mode="softmax_then_topk",
                                 fuse_combine=True)
    ops.check_status(DEV)
    mx, mean = O.rel_errors(fused[0].cpu(), plain[0].double().cpu())
    assert mx <= 2.0 ** -6 and mean <= 1e-4, (mx, mean)
    for a, b in zip(plain[1:], fused[1:]):
        assert torch.equal(a, b)


def test_nan_tokens_and_bad_route_ids_give_nan_or_a_status_never_a_fault():
    """A diverged token (NaN activations, hence NaN logits) must come out as NaN rows, and
    caller-supplied ids outside the expert range must be reported in the status block; neither
    may index outside a buffer (every gather index is bounded on the device)."""
    layer, ops = _layer()
    from mlops_b200._lib import NativeError

    c1 = inputs.config1()
    w13 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w13"]))
    w2 = tuple(t.to(DEV) for t in O.quantize_blocks(c1["w2"]))
    x, router, dy = c1["x"].clone(), c1["router"].to(DEV), c1["dy"].to(DEV)
    x[7] = float("nan")
    x[100, 3] = float("inf")
    x = x.to(DEV)
    res = layer.forward_routed(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    ids = res[6]
    assert bool(((ids >= 0) & (ids < 8)).all())
    grads = layer.backward_routed(dy, None, None, x, router, w13, w2, *res[4:], top_k=2,
                                  routing_mode="softmax_then_topk")
    torch.cuda.synchronize()
    ops.check_status(DEV)  # NaN data is not an error: it propagates
    out = res[0]
    assert bool(torch.isnan(out[7]).all())
    clean = torch.ones(x.shape[0], dtype=torch.bool)
    clean[[7, 100]] = False
    assert bool(torch.isfinite(out.cpu()[clean]).all())
    assert bool(torch.isfinite(grads[0].cpu()[clean]).all())

    # ids outside [0, E) handed in by the caller
    x = c1["x"].to(DEV)
    bad_ids = torch.randint(0, 8, (x.shape[0], 2), generator=torch.Generator().manual_seed(2)).to(torch.int32)
    bad_ids[5, 0] = 99
    bad_ids[6, 1] = -4
    weights = torch.full((x.shape[0], 2), 0.5)
    res = layer.forward_routed(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk",
                               route=(weights.to(DEV), bad_ids.to(DEV)))
    layer.backward_routed(dy, None, None, x, router, w13, w2, *res[4:], top_k=2, routing_mode="softmax_then_topk")
    torch.cuda.synchronize()
    with pytest.raises(NativeError):
        ops.check_status(DEV)
    assert bool(torch.isfinite(res[0]).all())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_layer_on_a_device_that_is_not_current():
    """Tensors on cuda:1 while cuda:0 is the current device (a model moved with `.to`): the
    wrappers launch on the tensors' device and stream, and results equal those on cuda:0."""
    layer, ops = _layer()
    c1 = inputs.config1()
    outs = []
    for name in ("cuda:0", "cuda:1"):
        torch.cuda.set_device(0)
        w13 = tuple(t.to(name) for t in O.quantize_blocks(c1["w13"]))
        w2 = tuple(t.to(name) for t in O.quantize_blocks(c1["w2"]))
        x, router, dy = c1["x"].to(name), c1["router"].to(name), c1["dy"].to(name)
        res = layer.forward_routed(x, torch.zeros_like(x), router, w13, w2, top_k=2,
                                   routing_mode="softmax_then_topk")
        grads = layer.backward_routed(dy, None, None, x, router, w13, w2, *res[4:], top_k=2,
                                      routing_mode="softmax_then_topk")
        torch.cuda.synchronize(name)
        ops.check_status(name)
        outs.append((res[0].cpu(), grads[0].cpu(), grads[3].cpu()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
