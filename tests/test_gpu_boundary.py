"""The drop-in boundary on a B200.

(1) The opaque-operator contract the reference sets for a provider (`docs/PROVIDERS.md:86-112`,
checked by its `tests/test_custom_op_contracts.py:830-850`): `torch.library.opcheck` on the
`b200moe::` operators (schema, autograd registration, fake tensors, AOT dispatch with dynamic
shapes), functional schemas, FLOP formulas seen by `FlopCounterMode`.
(2) The reference itself calling this library: `mlops.moe(...)` with the reference's own
`BlockFP8Weight` containers on CUDA resolves to `b200.moe` (its `capture_dispatch()` says
so) and the results agree with the CPU oracle and with the reference's native-PyTorch
provider run on the CPU. The reference comes from `oracle/_ref` (see `oracle/build_ref.py`);
where it is absent these cases are skipped, the others still run."""

import pytest
import torch

import inputs
from oracle import moe_oracle as O
from oracle.build_ref import reference

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _plain_args(requires_grad=True):
    from mlops_b200 import ops

    c1 = inputs.config1()
    x = c1["x"][:128].to(DEV).requires_grad_(requires_grad)
    router = c1["router"].to(DEV).requires_grad_(requires_grad)
    w13_q, w13_s = ops.quantize_blocks(c1["w13"].to(DEV))
    w2_q, w2_s = ops.quantize_blocks(c1["w2"].to(DEV))
    bias = torch.empty(0, device=DEV)
    return (x, torch.zeros_like(x), router, w13_q, w2_q, bias, 2, "softmax_then_topk", 1, 1, 1.0, [128],
            "float32", None, None, [w13_s, w2_s])


def test_opcheck_of_the_routed_operator_pair():
    from mlops_b200 import provider

    # SchemaCheckMode's mutation check does arithmetic on every input, which E4M3 tensors have
    # no kernels for (the reference drops `test_schema` for its FP8 cases for the same reason)
    utilities = ("test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")
    results = torch.library.opcheck(provider.moe_fwd, _plain_args(), test_utils=utilities)
    assert set(results.values()) == {"SUCCESS"}, results

    args = _plain_args(requires_grad=False)
    with torch.no_grad():
        out = provider.moe_fwd(*args)
    x, _res, router, w13_q, w2_q = args[:5]
    dy = torch.randn_like(x)
    bwd_args = (dy, torch.zeros((), device=DEV), torch.zeros(8, device=DEV), x, router, w13_q, w2_q, *out[4:], 2,
                "softmax_then_topk", [128], None, None, True, True, False, args[-1])
    results = torch.library.opcheck(provider.moe_bwd, bwd_args, test_utils=("test_faketensor",))
    assert set(results.values()) == {"SUCCESS"}, results
    grads = provider.moe_bwd(*bwd_args)
    assert grads[4].numel() == 0 and grads[3].shape == w13_q.shape and grads[3].dtype == torch.bfloat16


def test_opcheck_of_the_swiglu_operator():
    from mlops_b200 import provider

    h13 = torch.randn(96, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    for limit in (None, 0.75):
        results = torch.library.opcheck(
            provider.swiglu, (h13, limit),
            test_utils=("test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic"))
        assert set(results.values()) == {"SUCCESS"}, results


def test_opcheck_of_the_lora_operator():
    from mlops_b200 import lora

    args = list(_plain_args())
    x, residual, router, w13_q, w2_q, bias = args[:6]
    g = torch.Generator().manual_seed(9)
    factors = [(torch.randn(8, 12, 256, generator=g) * 0.02), (torch.randn(8, 1024, 12, generator=g) * 0.01),
               (torch.randn(8, 12, 512, generator=g) * 0.02), (torch.randn(8, 256, 12, generator=g) * 0.01)]
    factors = [f.bfloat16().to(DEV).requires_grad_(True) for f in factors]
    op_args = (x, residual, router, w13_q, w2_q, *factors, bias, 2, "softmax_then_topk", 1.0, 1, 1, 1.0, [128],
               None, [], 1.0, args[-1])
    results = torch.library.opcheck(
        lora.moe_lora_fwd, op_args,
        test_utils=("test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic"))
    assert set(results.values()) == {"SUCCESS"}, results


def test_operator_schemas_are_functional_and_outside_the_reference_namespace():
    from mlops_b200 import lora, provider  # noqa: F401

    from mlops_b200 import composed  # noqa: F401

    for name in ("moe_fwd", "moe_bwd", "moe_lora_fwd", "moe_lora_bwd", "swiglu", "swiglu_bwd", "moe_prepare_fwd",
                 "moe_prepare_bwd", "moe_finish_fwd", "moe_finish_bwd"):
        schema = getattr(torch.ops.b200moe, name).default._schema
        assert all(argument.alias_info is None for argument in schema.arguments)
        assert all(result.alias_info is None for result in schema.returns)
        assert "!" not in str(schema)


def test_flop_counter_sees_18_d_f_per_routed_row():
    from torch.utils.flop_counter import FlopCounterMode

    from mlops_b200 import provider
    from mlops_b200.weights import BlockFP8Weight

    c1 = inputs.config1()
    x = c1["x"].to(DEV).requires_grad_(True)
    router = c1["router"].to(DEV).requires_grad_(True)
    w13 = BlockFP8Weight.quantize(c1["w13"].to(DEV)).requires_grad_(True)
    w2 = BlockFP8Weight.quantize(c1["w2"].to(DEV)).requires_grad_(True)
    with FlopCounterMode(display=False) as counter:
        out, *_ = provider.apply(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
        out.backward(c1["dy"].to(DEV))
    rows, width, inner, experts = 512 * 2, 256, 512, 8
    projections = 18 * width * inner * rows
    total = counter.get_total_flops()
    # projections + router GEMMs (2*T*D*E forward, twice that backward) + elementwise passes
    assert projections < total < projections * 1.05 + 6 * 512 * width * experts, (total, projections)


# ----------------------------------------------------------------- the reference as caller
def _reference_or_skip():
    mlops = reference()
    if mlops is None:
        pytest.skip("the reference package is not at oracle/_ref (run oracle/build_ref.py)")
    return mlops


def test_reference_dispatch_resolves_to_this_provider_on_cuda():
    mlops = _reference_or_skip()
    from mlops.block_fp8 import BlockFP8Weight as ReferenceWeight
    from mlops.dispatch import capture_dispatch, explain_implementation, use_implementation

    from mlops_b200 import ops, provider

    provider.register()
    c1 = inputs.config1()
    x = c1["x"].to(DEV).requires_grad_(True)
    router = c1["router"].to(DEV).requires_grad_(True)
    # containers of the reference's own class, quantised by its CPU path and moved over
    w13c = ReferenceWeight.quantize(c1["w13"])
    w2c = ReferenceWeight.quantize(c1["w2"])
    w13 = ReferenceWeight(w13c._data.to(DEV), w13c._scale.to(DEV), dtype=w13c.dtype).requires_grad_(True)
    w2 = ReferenceWeight(w2c._data.to(DEV), w2c._scale.to(DEV), dtype=w2c.dtype).requires_grad_(True)
    residual = torch.zeros_like(x)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    explanation = explain_implementation("moe", x, residual, router, w13, w2, **kwargs)
    assert explanation.candidates["b200.moe"].supported, explanation.candidates["b200.moe"].reason
    with capture_dispatch() as trace:
        out, aux, counts, psum = mlops.moe(x, residual, router, w13, w2, **kwargs)
    assert trace["moe"] == {"b200.moe": 1}, trace
    dy = c1["dy"].to(DEV)
    grads = torch.autograd.grad(out, [x, router, w13, w2], dy)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert counts.dtype == torch.int64 and int(counts.sum()) == 1024
    assert all(type(g) is torch.Tensor for g in grads) and grads[2].dtype == torch.bfloat16

    # against the CPU oracle on identical block-FP8 operands
    w13_q, w13_s = O.quantize_blocks(c1["w13"])
    w2_q, w2_s = O.quantize_blocks(c1["w2"])
    logits = O.router_logits(c1["x"], c1["router"])
    fwd = O.forward_block_fp8(c1["x"], torch.zeros_like(c1["x"]), logits, w13_q, w13_s, w2_q, w2_s, top_k=2,
                              routing_mode="softmax_then_topk")
    assert torch.equal(counts.cpu(), torch.bincount(fwd["ids"].reshape(-1).long(), minlength=8))
    mx, mean = O.rel_errors(out.float().cpu(), fwd["output"].float())
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)

    # against the reference's own native-PyTorch provider on the CPU (bf16 on dequantised
    # weights), at the reference's FP8-vs-bf16 bounds (tests/test_sonicmoe_block_fp8.py:350)
    xc = c1["x"].clone().requires_grad_(True)
    rc = c1["router"].clone().requires_grad_(True)
    w13c.requires_grad_(True)
    w2c.requires_grad_(True)
    with use_implementation("moe", "native_torch.moe"):
        ref_out, ref_aux, ref_counts, ref_psum = mlops.moe(xc, torch.zeros_like(xc), rc, w13c, w2c,
                                                           compute_precision="bf16", **kwargs)
    ref_grads = torch.autograd.grad(ref_out, [xc, rc, w13c, w2c], c1["dy"])

    def frob(a, e):
        return ((a.double().cpu() - e.double()).norm() / e.double().norm()).item()

    assert torch.equal(counts.cpu(), ref_counts)
    assert frob(out, ref_out) <= 4.5e-2  # measured 4.4e-2: E4M3 activation noise at this width
    assert frob(grads[0], ref_grads[0]) < 8e-2 and frob(grads[1], ref_grads[1]) < 8e-2
    assert frob(grads[2], ref_grads[2]) < 6e-2 and frob(grads[3], ref_grads[3]) < 6e-2
    torch.testing.assert_close(aux.cpu(), ref_aux, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(psum.cpu(), ref_psum, rtol=1e-3, atol=1e-3)


def test_reference_contexts_reach_the_operator():
    mlops = _reference_or_skip()
    from mlops.block_fp8 import BlockFP8Weight as ReferenceWeight
    from mlops.dispatch.context import weight_gradients_at
    from mlops.kernels.moe_router import route_weight_precision

    from mlops_b200 import provider

    provider.register()
    c1 = inputs.config1()
    x = c1["x"].to(DEV)
    router = c1["router"].to(DEV).requires_grad_(True)
    w13c, w2c = ReferenceWeight.quantize(c1["w13"]), ReferenceWeight.quantize(c1["w2"])
    w13 = ReferenceWeight(w13c._data.to(DEV), w13c._scale.to(DEV), dtype=w13c.dtype).requires_grad_(True)
    w2 = ReferenceWeight(w2c._data.to(DEV), w2c._scale.to(DEV), dtype=w2c.dtype).requires_grad_(True)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    dy = c1["dy"].to(DEV)
    out, *_ = mlops.moe(x, torch.zeros_like(x), router, w13, w2, **kwargs)
    plain = torch.autograd.grad(out, [router, w13], dy)
    # the contexts are read at apply time and travel as operator arguments; autograd hands a
    # parameter its gradient at the parameter's dtype, so a bf16-logical container still sees bf16
    with weight_gradients_at(torch.float32), route_weight_precision("input"):
        out32, *_ = mlops.moe(x, torch.zeros_like(x), router, w13, w2, **kwargs)
        same = torch.autograd.grad(out32, [router, w13], dy)
    assert torch.equal(out, out32)
    assert same[1].dtype == torch.bfloat16 and torch.equal(same[1], plain[1])
    torch.testing.assert_close(same[0], plain[0], rtol=1e-2, atol=1e-3)
    # a container whose logical dtype is fp32 receives the fp32 sums themselves
    w13_wide = ReferenceWeight(w13c._data.to(DEV), w13c._scale.to(DEV), dtype=torch.float32).requires_grad_(True)
    out_wide, *_ = mlops.moe(x, torch.zeros_like(x), router, w13_wide, w2, **kwargs)
    wide = torch.autograd.grad(out_wide, [router, w13_wide], dy)
    assert torch.equal(out, out_wide)
    assert wide[1].dtype == torch.float32 and wide[0].dtype == router.dtype
    assert torch.equal(wide[1].bfloat16(), plain[1])  # the same fp32 sums, rounded later


# ------------------------------------------------------------- the two-region composition
def _containers(requires_grad=True):
    from mlops_b200.weights import BlockFP8Weight

    c1 = inputs.config1()
    x = c1["x"].to(DEV).requires_grad_(requires_grad)
    router = c1["router"].to(DEV).requires_grad_(requires_grad)
    w13 = BlockFP8Weight.quantize(c1["w13"].to(DEV)).requires_grad_(requires_grad)
    w2 = BlockFP8Weight.quantize(c1["w2"].to(DEV)).requires_grad_(requires_grad)
    return c1, x, router, w13, w2


def test_composed_regions_agree_with_the_fused_operator():
    """`prepare` + `finish` give the fused operator's forward results bit for bit (the same
    kernels in the same order); the gradients downstream of the `h13` gradient differ by its
    bf16 rounding where it crosses the two regions."""
    from mlops_b200 import composed, ops, provider

    c1, x, router, w13, w2 = _containers()
    dy, residual = c1["dy"].to(DEV), torch.randn_like(c1["x"]).to(DEV)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    g_aux, g_psum = torch.tensor(0.3, device=DEV), torch.randn(8, device=DEV)
    fused = provider.apply(x, residual, router, w13, w2, **kwargs)
    fused_grads = torch.autograd.grad([fused[0], fused[1], fused[3]], [x, router, w13, w2], [dy, g_aux, g_psum])
    split = composed.apply(x, residual, router, w13, w2, **kwargs)
    split_grads = torch.autograd.grad([split[0], split[1], split[3]], [x, router, w13, w2], [dy, g_aux, g_psum])
    ops.check_status(DEV)
    for a, b in zip(fused, split):
        assert torch.equal(a, b)
    assert split[2].dtype == torch.int64 and not split[2].requires_grad
    assert torch.equal(fused_grads[3], split_grads[3])  # grad_w2 never sees the crossing
    # The h13 gradient is quantised to E4M3 from fp32 in the fused operator and from its bf16
    # rounding here; a few percent of its elements land on the neighbouring E4M3 value, so what is
    # computed from it agrees to E4M3 quantisation noise (about 1% in the Frobenius norm), not bits
    for name, a, b in zip(("grad_x", "grad_router", "grad_w13"), fused_grads, split_grads):
        frob = ((b.double() - a.double()).norm() / a.double().norm()).item()
        assert frob <= 2e-2, (name, frob)
    # frozen weights: no gradient, the rest unchanged
    c1, x2, router2, w13f, w2f = _containers(requires_grad=False)
    x2.requires_grad_(True)
    launches = ops.LAUNCHES
    out, *_ = composed.apply(x2, residual, router2, w13f, w2f, **kwargs)
    (gx,) = torch.autograd.grad(out, [x2], dy)
    frozen_launches = ops.LAUNCHES - launches
    launches = ops.LAUNCHES
    out, *_ = composed.apply(x, residual, router, w13, w2, **kwargs)
    trainable = torch.autograd.grad(out, [x, router, w13, w2], dy)
    assert (ops.LAUNCHES - launches) - frozen_launches == 3  # two weight gradients and the gather of x
    assert torch.equal(gx, trainable[0])  # what is still computed is bit-identical


def test_opcheck_of_the_region_operators_and_the_donating_backward():
    from mlops_b200 import composed, ops

    args = _plain_args()
    x, _res, router, w13_q, w2_q, bias = args[:6]
    w13_s, w2_s = args[-1]
    utilities = ("test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")
    prepare_args = (x, router, w13_q, bias, 2, "softmax_then_topk", 1, 1, 1.0, [128], "float32", None, [w13_s])
    results = torch.library.opcheck(composed.prepare_fwd, prepare_args, test_utils=utilities)
    assert set(results.values()) == {"SUCCESS"}, results
    with torch.no_grad():
        aux, counts, psum, logits, weights, ids, order, offsets, slots, h13 = composed.prepare_fwd(*prepare_args)
    h13 = h13.requires_grad_(True)
    weights = weights.requires_grad_(True)
    residual = torch.randn_like(x).detach().requires_grad_(True)
    finish_args = (h13, w2_q, weights, order, offsets, slots, residual, 2, None, None, [w2_s])
    results = torch.library.opcheck(composed.finish_fwd, finish_args, test_utils=utilities)
    assert set(results.values()) == {"SUCCESS"}, results

    dy = torch.randn_like(x).detach()
    plain = composed.finish_bwd(dy, h13.detach(), w2_q, weights.detach(), order, offsets, slots, 2, None, None, True,
                                [w2_s])
    donated = h13.detach().clone()
    rest = composed.finish_bwd_donate_h13(dy, donated, w2_q, weights.detach(), order, offsets, slots, 2, None, None,
                                          True, [w2_s])
    ops.check_status(DEV)
    assert torch.equal(donated, plain[0])  # the gradient now sits where h13 was
    for a, b in zip(rest, plain[1:]):
        assert torch.equal(a, b)
    schema = torch.ops.b200moe.moe_finish_bwd_donate_h13.default._schema
    assert "!" in str(schema)  # the one mutating overload says so


def test_reference_dispatch_can_select_the_composition():
    mlops = _reference_or_skip()
    from mlops.block_fp8 import BlockFP8Weight as ReferenceWeight
    from mlops.dispatch import capture_dispatch, use_implementation

    from mlops_b200 import composed, provider

    provider.register()
    composed.register()
    c1 = inputs.config1()
    x = c1["x"].to(DEV).requires_grad_(True)
    w13c, w2c = ReferenceWeight.quantize(c1["w13"]), ReferenceWeight.quantize(c1["w2"])
    w13 = ReferenceWeight(w13c._data.to(DEV), w13c._scale.to(DEV), dtype=w13c.dtype).requires_grad_(True)
    w2 = ReferenceWeight(w2c._data.to(DEV), w2c._scale.to(DEV), dtype=w2c.dtype).requires_grad_(True)
    router = c1["router"].to(DEV)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    with capture_dispatch() as trace:
        default_out, *_ = mlops.moe(x, torch.zeros_like(x), router, w13, w2, **kwargs)
        with use_implementation("moe", "b200.moe.composed"):
            out, *_ = mlops.moe(x, torch.zeros_like(x), router, w13, w2, **kwargs)
    assert trace["moe"] == {"b200.moe": 1, "b200.moe.composed": 1}, trace
    assert torch.equal(out, default_out)
    grads = torch.autograd.grad(out, [x, w13, w2], c1["dy"].to(DEV))
    assert grads[1].shape == w13.shape and grads[2].shape == w2.shape


def test_fp8_weight_gradient_recipe_through_the_operator():
    """`provider.set_weight_gradient_operands("fp8")`: the backward operator quantises both
    operands of each expert weight gradient (one scale per expert and column) and multiplies at
    the FP8 rate; activations' and the router's gradients are untouched, the expert gradients
    stay within the reference's bound for that recipe (tests/test_sonicmoe_fp8.py:114-124)."""
    from mlops_b200 import ops, provider

    c1, x, router, w13, w2 = _containers()
    dy, residual = c1["dy"].to(DEV), torch.zeros_like(c1["x"]).to(DEV)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    grads = {}
    previous = provider.set_weight_gradient_operands("bf16")
    try:
        for kind in ("bf16", "fp8"):
            provider.set_weight_gradient_operands(kind)
            out = provider.apply(x, residual, router, w13, w2, **kwargs)
            grads[kind] = torch.autograd.grad(out[0], [x, router, w13, w2], dy)
    finally:
        provider.set_weight_gradient_operands(previous)
    ops.check_status(DEV)
    assert torch.equal(grads["fp8"][0], grads["bf16"][0]) and torch.equal(grads["fp8"][1], grads["bf16"][1])
    for i in (2, 3):
        exact, fp8 = grads["bf16"][i].double(), grads["fp8"][i].double()
        assert not torch.equal(exact, fp8)
        assert ((fp8 - exact).norm() / exact.norm()).item() < 6e-2
    with pytest.raises(ValueError):
        provider.set_weight_gradient_operands("fp4")


def test_bf16_experts_run_the_bf16_path_through_the_operator(golden):
    """Plain bf16 expert tensors (the builtin's default weights) and `compute_precision="bf16"` on
    block-FP8 containers both reach the bf16 grouped GEMMs; on the same weight values the two agree
    bit for bit, and with the stored outputs of the reference's bf16 provider to rounding."""
    from mlops_b200 import ops, provider
    from mlops_b200.weights import BlockFP8Weight

    c1 = inputs.config1()
    x = c1["x"].to(DEV).requires_grad_(True)
    router = c1["router"].to(DEV).requires_grad_(True)
    dy, residual = c1["dy"].to(DEV), torch.zeros_like(c1["x"]).to(DEV)
    q13, q2 = BlockFP8Weight.quantize(c1["w13"].to(DEV)), BlockFP8Weight.quantize(c1["w2"].to(DEV))
    w13 = q13.dequantize().to(torch.bfloat16).detach().requires_grad_(True)
    w2 = q2.dequantize().to(torch.bfloat16).detach().requires_grad_(True)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    assert provider.refusal(x, residual, router, w13, w2, surface="opaque", **kwargs) is None
    assert provider.refusal(x, residual, router, w13, w2, surface="opaque", compute_precision="fp8_block",
                            **kwargs) is not None
    out = provider.apply(x, residual, router, w13, w2, **kwargs)
    grads = torch.autograd.grad(out[0], [x, router, w13, w2], dy)
    q13.requires_grad_(True), q2.requires_grad_(True)
    out_c = provider.apply(x, residual, router, q13, q2, compute_precision="bf16", **kwargs)
    grads_c = torch.autograd.grad(out_c[0], [x, router, q13, q2], dy)
    ops.check_status(DEV)
    assert torch.equal(out[0], out_c[0])
    for a, b in zip(grads, grads_c):
        assert torch.equal(a, b)
    fixture = golden("config1_native_torch.pt")
    frob = lambda a, e: ((a.double().cpu() - e.double()).norm() / e.double().norm()).item()  # noqa: E731
    assert frob(out[0], fixture["output"]) < 1e-2
    assert frob(grads[0], fixture["grad_x"]) < 1e-2
    assert frob(grads[2][:, ::16, ::8], fixture["grad_w13_sample"]) < 1e-2
