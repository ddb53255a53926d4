"""The provider against the reference's own registry (CPU, needs the reference package, which
`oracle/build_ref.py` puts at `oracle/_ref`, or `$MLOPS_REFERENCE_SRC`; skipped where absent). Mirrors the rules the reference
tests in tests/test_implementation_registry.py: registration, duplicate ids, priority
selection, refusal reasons, forced selection of an unsupported implementation."""

import pytest
import torch

from oracle.build_ref import reference

mlops = reference()
if mlops is None:
    pytest.skip("reference package not present", allow_module_level=True)

from mlops.block_fp8 import BlockFP8Weight  # noqa: E402
from mlops.dispatch import explain_implementation, resolve_implementation, use_implementation  # noqa: E402
from mlops.dispatch.registry import implementations_for, register_implementation  # noqa: E402

from mlops_b200 import provider  # noqa: E402


def _inputs():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 256, generator=g).bfloat16()
    router = torch.randn(8, 256, generator=g)
    w13 = BlockFP8Weight.quantize((torch.randn(8, 512, 256, generator=g) * 0.02).bfloat16())
    w2 = BlockFP8Weight.quantize((torch.randn(8, 256, 256, generator=g) * 0.02).bfloat16())
    return x, router, w13, w2


def test_registers_once_with_top_priority():
    record = provider.register()
    assert provider.register() is record  # idempotent
    table = implementations_for("moe")
    assert table["b200.moe"] is record
    assert record.priority > max(i.priority for name, i in table.items() if name != "b200.moe")
    assert record.forward is not None and record.backward is not None and record.deterministic
    with pytest.raises(ValueError):
        register_implementation(record)  # duplicate id


def test_cpu_call_is_refused_with_a_reason_and_resolution_falls_to_the_reference():
    provider.register()
    x, router, w13, w2 = _inputs()
    kwargs = dict(top_k=2, routing_mode="softmax_then_topk", compute_precision="bf16")
    explanation = explain_implementation("moe", x, x, router, w13, w2, **kwargs)
    assert not explanation.candidates["b200.moe"].supported
    assert "CUDA" in explanation.candidates["b200.moe"].reason
    chosen = resolve_implementation("moe", x, x, router, w13, w2, **kwargs)
    assert chosen.implementation_id != "b200.moe"
    # the reference still serves the call end to end with the provider registered
    out, aux, counts, psum = mlops.moe(x, torch.zeros_like(x), router, w13, w2, **kwargs)
    assert out.shape == x.shape and counts.dtype == torch.int64 and int(counts.sum()) == 32


def test_forcing_the_provider_on_cpu_fails_loudly_not_silently():
    provider.register()
    x, router, w13, w2 = _inputs()
    with use_implementation("moe", "b200.moe"):
        with pytest.raises(RuntimeError, match="b200.moe"):
            mlops.moe(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")
    with pytest.raises(ValueError):
        provider.apply(x, torch.zeros_like(x), router, w13, w2, top_k=2, routing_mode="softmax_then_topk")


def test_refusal_reasons_are_specific():
    x, router, w13, w2 = _inputs()
    dense = w13.dequantize()
    narrow13 = BlockFP8Weight.quantize(torch.zeros(8, 384, 192).bfloat16())
    narrow2 = BlockFP8Weight.quantize(torch.zeros(8, 192, 192).bfloat16())
    # the device check comes first on CPU; check the remaining gates through `refusal` with
    # the device gates patched out
    real_cuda = torch.Tensor.is_cuda
    try:
        torch.Tensor.is_cuda = property(lambda self: True)
        real_cap = torch.cuda.get_device_capability
        torch.cuda.get_device_capability = lambda device=None: (10, 0)
        ok = dict(top_k=2, routing_mode="softmax_then_topk")
        assert provider.refusal(x, x, router, w13, w2, **ok) is None
        assert "BlockFP8Weight" in provider.refusal(x, x, router, dense, w2, **ok)
        assert "bf16" in provider.refusal(x.float(), x.float(), router, w13, w2, **ok)
        assert "compute_precision" in provider.refusal(x, x, router, w13, w2, compute_precision="fp4", **ok)
        assert provider.refusal(x, x, router, w13, w2, compute_precision="bf16", **ok) is None
        assert provider.refusal(x, x, router, dense, w2.dequantize(), **ok) is None          # plain bf16 experts
        assert "fp8_block" in provider.refusal(x, x, router, dense, w2.dequantize(), compute_precision="fp8_block",
                                               **ok)
        assert "top_k" in provider.refusal(x, x, router, w13, w2, top_k=9, routing_mode="softmax_then_topk")
        assert "routing mode" in provider.refusal(x, x, router, w13, w2, top_k=2, routing_mode="other")
        assert "lengths" in provider.refusal(x, x, router, w13, w2, lengths=(3,), **ok)
        assert "explicit" in provider.refusal(x, x, router, w13, w2, surface="explicit", swiglu_limit=1.0, **ok)
        assert "multiples of 128" in provider.refusal(x[:, :192], x[:, :192], router[:, :192], narrow13,
                                                      narrow2, **ok)
    finally:
        torch.Tensor.is_cuda = real_cuda
        torch.cuda.get_device_capability = real_cap
