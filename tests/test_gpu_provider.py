"""The provider's `apply` / explicit `forward` / `backward` on a B200, with this package's
own weight container (the reference is not installed on the GPU machine). Contracts taken
from the reference's tests: explicit VJP == autograd bit for bit (tests/test_explicit_ops.py:
381-516), frozen inputs get no gradient and leave the others bit-identical
(tests/test_moe_frozen_gradients.py:74-116), non-reentrant activation checkpointing is
bit-identical (tests/test_moe_checkpoint.py), containers quantise as the reference's do and
re-quantise on publication (tests/test_sonicmoe_block_fp8.py:31-76)."""

import pytest
import torch

import inputs
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(requires=(True, True, True, True)):
    from mlops_b200.weights import BlockFP8Weight

    c1 = inputs.config1()
    x = c1["x"].to(DEV).requires_grad_(requires[0])
    router = c1["router"].to(DEV).requires_grad_(requires[1])
    w13 = BlockFP8Weight.quantize(c1["w13"].to(DEV)).requires_grad_(requires[2])
    w2 = BlockFP8Weight.quantize(c1["w2"].to(DEV)).requires_grad_(requires[3])
    return c1, x, router, w13, w2


def test_container_matches_oracle_and_republishes():
    from mlops_b200.weights import BlockFP8Weight

    w = inputs.block_weight().bfloat16()
    container = BlockFP8Weight.quantize(w.to(DEV))
    data, scale = O.quantize_blocks(w)
    assert torch.equal(container._data.cpu().view(torch.uint8), data.view(torch.uint8))
    assert torch.equal(container._scale.cpu(), scale)
    assert container.dtype == torch.bfloat16 and container.shape == w.shape
    torch.testing.assert_close(container.dequantize().cpu(), O.dequantize_blocks(data, scale, torch.bfloat16))
    master = (w * 2).to(DEV)
    container.copy_(master)  # publication after an optimizer step
    data2, scale2 = O.quantize_blocks(w * 2)
    assert torch.equal(container._data.cpu().view(torch.uint8), data2.view(torch.uint8))
    assert torch.equal(container._scale.cpu(), scale2)
    # straight-through gradient of quantize
    leaf = w.to(DEV).requires_grad_(True)
    BlockFP8Weight.quantize(leaf).backward(torch.ones_like(leaf))
    assert torch.equal(leaf.grad, torch.ones_like(leaf))


def test_autograd_equals_explicit_vjp_bit_for_bit():
    from mlops_b200 import provider

    c1, x, router, w13, w2 = _setup()
    dy = c1["dy"].to(DEV)
    residual = torch.zeros_like(x)
    out, aux, counts, psum = provider.apply(x, residual, router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    assert counts.dtype == torch.int64 and not counts.requires_grad
    g_aux, g_psum = torch.tensor(0.3, device=DEV), torch.randn(8, device=DEV)
    grads = torch.autograd.grad([out, aux, psum], [x, router, w13, w2], [dy, g_aux, g_psum])
    with torch.no_grad():
        res = provider.forward(x, residual, router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
        assert torch.equal(res[0], out) and torch.equal(res[1], aux) and torch.equal(res[3], psum)
        explicit = provider.backward(dy, g_aux, g_psum, x, router, w13, w2, *res[4:], top_k=2,
                                     routing_mode="softmax_then_topk", lengths=(512,))
    assert torch.equal(grads[0], explicit[0])
    assert torch.equal(grads[1], explicit[2])
    assert torch.equal(grads[2], explicit[3]) and torch.equal(grads[3], explicit[4])
    assert grads[2].dtype == torch.bfloat16 and grads[2].shape == w13.shape  # logical dtype, Linear row order
    assert type(grads[2]) is torch.Tensor


def test_frozen_inputs_get_none_and_the_rest_is_bit_identical():
    from mlops_b200 import ops, provider

    c1, x, router, w13, w2 = _setup()
    dy = c1["dy"].to(DEV)
    out, *_ = provider.apply(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    full = torch.autograd.grad(out, [x, router, w13, w2], dy)
    c1, x2, router2, w13f, w2f = _setup(requires=(True, False, False, False))
    launches = ops.LAUNCHES
    out2, *_ = provider.apply(x2, torch.zeros_like(x2), router2, w13f, w2f, top_k=2, routing_mode="softmax_then_topk")
    forward_launches = ops.LAUNCHES - launches
    (gx,) = torch.autograd.grad(out2, [x2], dy)
    frozen_backward = ops.LAUNCHES - launches - forward_launches
    assert torch.equal(gx, full[0])
    out3, *_ = provider.apply(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    launches = ops.LAUNCHES
    torch.autograd.grad(out3, [x, router, w13, w2], dy)
    # frozen: the two weight-gradient GEMMs and the gather of their x operand are not launched
    # (the dy operand is a by-product of the quantiser's pass, not a launch of its own)
    assert (ops.LAUNCHES - launches) - frozen_backward == 3


def test_activation_checkpoint_is_bit_identical():
    from torch.utils.checkpoint import checkpoint

    from mlops_b200 import provider

    c1, x, router, w13, w2 = _setup()
    dy = c1["dy"].to(DEV)

    def run(h):
        return provider.apply(h, torch.zeros_like(h), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")[0]

    plain = torch.autograd.grad(run(x), [x, w13], dy)
    again = torch.autograd.grad(checkpoint(run, x, use_reentrant=False), [x, w13], dy)
    assert torch.equal(plain[0], again[0]) and torch.equal(plain[1], again[1])


@pytest.mark.parametrize("shared_mode", ["add", "sigmoid"])
def test_shared_expert_against_torch_reference(shared_mode):
    """Shared branch vs the reference's own expression for it
    (src/mlops/kernels/moe_reference.py:93-107) evaluated by PyTorch autograd on the device."""
    from mlops_b200 import provider

    c1, x, router, w13, w2 = _setup()
    g = torch.Generator().manual_seed(3)
    sw13 = (torch.randn(768, 256, generator=g) * 0.05).bfloat16().to(DEV).requires_grad_(True)
    sw2 = (torch.randn(256, 384, generator=g) * 0.05).bfloat16().to(DEV).requires_grad_(True)
    gate_w = (torch.randn(1, 256, generator=g) * 0.05).bfloat16().to(DEV).requires_grad_(True)
    residual = torch.randn(512, 256, generator=g).bfloat16().to(DEV)
    dy = c1["dy"].to(DEV)
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk")
    out, *_ = provider.apply(x, residual, router, w13, w2, shared_w13=sw13, shared_w2=sw2,
                             shared_gate_weight=gate_w, shared_mode=shared_mode, **kwargs)
    routed_only, *_ = provider.apply(x, torch.zeros_like(residual), router, w13, w2, **kwargs)
    grads = torch.autograd.grad(out, [x, sw13, sw2], dy)
    routed_grads = torch.autograd.grad(routed_only, [x], dy)

    def reference(h):
        h13 = torch.nn.functional.linear(h, sw13)
        act = torch.nn.functional.silu(h13[:, :384].float()).to(h.dtype) * h13[:, 384:]
        shared = torch.nn.functional.linear(act, sw2)
        if shared_mode == "sigmoid":
            gate = torch.sigmoid(torch.nn.functional.linear(h, gate_w).float())
            shared = (gate * shared.float()).to(h.dtype)
        return residual + shared

    x_ref = x.detach().clone().requires_grad_(True)
    base = reference(x_ref)
    ref_grads = torch.autograd.grad(base, [x_ref, sw13, sw2], dy)
    mx, mean = O.rel_errors((out.float() - routed_only.float()).cpu(), base.detach().float().cpu())
    assert mx <= 3e-2 and mean <= 3e-3, (mx, mean)  # two bf16 roundings apart (sum, then difference)
    for actual, expected in ((grads[0].float() - routed_grads[0].float(), ref_grads[0]), (grads[1], ref_grads[1]),
                             (grads[2], ref_grads[2])):
        mx, mean = O.rel_errors(actual.float().cpu(), expected.float().cpu())
        assert mx <= 3e-2 and mean <= 3e-3, (mx, mean)
