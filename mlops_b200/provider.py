"""The `b200.moe` provider: this library behind the reference's implementation registry.

`register()` adds one `Implementation(operation="moe", implementation_id="b200.moe", ...)`
to `mlops.dispatch.registry` (als244/mlops, `src/mlops/dispatch/registry.py:31-69`), with the
`supports` / `apply` / `forward` / `backward` callables below; `apply`, `forward` and
`backward` take the arguments and return the tuples the reference documents for the `moe`
operation (`docs/OPS.md:1603-1700`, `docs/EXPLICIT_OPS.md:456-502`) and work without the
reference installed. There is no fallback: a refusal comes from `supports`, with its reason.
"""

from __future__ import annotations

import torch

from . import layer
from .weights import components, is_block_fp8

IMPLEMENTATION_ID = "b200.moe"
PRIORITY = 120  # above the reference's highest MoE implementation (110)
MAX_EXPERTS = 1024
MAX_TOP_K = 32
ROUTING_MODES = ("softmax_then_topk", "topk_then_softmax", "sigmoid_noaux_tc")


def _context_weight_gradient_dtype():
    """The reference's `weight_gradients_at(...)` context, when the reference is present."""
    try:
        from mlops.dispatch.context import weight_gradient_dtype
    except ImportError:
        return None
    return weight_gradient_dtype()


def refusal(h2, residual, router_weight, w13_experts, w2_experts, *, surface="semantic", top_k,
            routing_mode, n_group=1, topk_group=1, lengths=None, shared_w13=None, shared_w2=None,
            compute_precision=None, swiglu_limit=None, **_ignored):
    """The reason this provider cannot serve the call, or None. Metadata only."""
    tensors = (h2, residual, router_weight, w13_experts, w2_experts)
    if not all(isinstance(t, torch.Tensor) for t in tensors):
        return "MoE core arguments must be tensors"
    if not all(t.is_cuda for t in (h2, residual, router_weight)):
        return "b200.moe runs on CUDA tensors only"
    if torch.cuda.get_device_capability(h2.device) != (10, 0):
        return "b200.moe is built for compute capability 10.0 (sm_100a) only"
    if compute_precision not in (None, "fp8_block"):
        return f"b200.moe computes in block FP8; compute_precision={compute_precision!r} is not served"
    if not (is_block_fp8(w13_experts) and is_block_fp8(w2_experts)):
        return "expert weights must be BlockFP8Weight containers (E4M3, 128x128 block scales)"
    if h2.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16:
        return "h2 and residual must be bf16"
    if h2.shape != residual.shape:
        return "h2 and residual must have equal shape"
    width = h2.shape[-1]
    if router_weight.dim() != 2 or router_weight.shape[1] != width:
        return "router_weight must have shape [experts, width]"
    experts = router_weight.shape[0]
    if w13_experts.shape[0] != experts or w2_experts.shape[0] != experts:
        return "router and expert counts differ"
    inner = w2_experts.shape[2]
    if tuple(w13_experts.shape[1:]) != (2 * inner, width) or w2_experts.shape[1] != width:
        return "expert weights must be w13 [experts, 2F, D] and w2 [experts, D, F]"
    if width % 128 or inner % 128:
        return "hidden and expert widths must be multiples of 128"
    if experts > MAX_EXPERTS or not 0 < int(top_k) <= min(experts, MAX_TOP_K):
        return f"supported sizes: experts <= {MAX_EXPERTS}, 0 < top_k <= min(experts, {MAX_TOP_K})"
    if routing_mode not in ROUTING_MODES:
        return f"unsupported routing mode {routing_mode!r}"
    if routing_mode == "sigmoid_noaux_tc":
        if int(n_group) <= 0 or experts % int(n_group) or (int(n_group) > 32 and int(topk_group) < int(n_group)):
            return "sigmoid_noaux_tc needs experts divisible by n_group and n_group <= 32"
    rows = h2.numel() // width
    normalized = (rows,) if lengths is None else tuple(int(v) for v in lengths)
    if sum(normalized) != rows:
        return "lengths must cover all hidden rows"
    if surface == "explicit" and (swiglu_limit is not None or shared_w13 is not None):
        return "the explicit surface is the routed part only (no shared expert, no swiglu_limit)"
    if (shared_w13 is None) != (shared_w2 is None):
        return "shared_w13 and shared_w2 come together"
    return None


class _Routed(torch.autograd.Function):
    """Autograd node of the routed part. Inputs 0-4 are differentiable; the containers receive
    plain tensors at their logical dtype (or at the context's weight-gradient dtype)."""

    @staticmethod
    def forward(ctx, h2, residual, router_weight, w13_experts, w2_experts, router_bias, options):
        w13, w2 = components(w13_experts), components(w2_experts)
        result = layer.forward_routed(h2, residual, router_weight, w13, w2, router_bias=router_bias, **options)
        output, aux, counts, probability_sum = result[:4]
        ctx.save_for_backward(h2, router_weight, *w13, *w2, *result[4:])
        ctx.options = options
        ctx.weight_grad_dtype = _context_weight_gradient_dtype()
        ctx.logical = (w13_experts.dtype, w2_experts.dtype)
        ctx.mark_non_differentiable(counts)
        return output, aux, counts, probability_sum

    @staticmethod
    def backward(ctx, grad_output, grad_aux, _grad_counts, grad_probability_sum):
        h2, router_weight, w13_d, w13_s, w2_d, w2_s, *saved = ctx.saved_tensors
        need = ctx.needs_input_grad
        options = ctx.options
        if grad_output is None:
            grad_output = torch.zeros_like(h2)
        wdtype = ctx.weight_grad_dtype
        grads = layer.backward_routed(
            grad_output, grad_aux, grad_probability_sum, h2, router_weight, (w13_d, w13_s), (w2_d, w2_s),
            *saved, top_k=options["top_k"], routing_mode=options["routing_mode"], lengths=options["lengths"],
            swiglu_limit=options["swiglu_limit"], weight_grad_dtype=ctx.logical[0] if wdtype is None else wdtype,
            router_grad_dtype=wdtype, need_router=need[2], need_w13=need[3], need_w2=need[4],
        )
        grad_h2, grad_residual, grad_router, grad_w13, grad_w2 = grads
        return (
            grad_h2 if need[0] else None, grad_residual if need[1] else None,
            grad_router if need[2] else None, grad_w13 if need[3] else None,
            grad_w2 if need[4] else None, None, None,
        )


class _Shared(torch.autograd.Function):
    """The always-on shared expert (bf16 library GEMMs, this library's SwiGLU kernels)."""

    @staticmethod
    def forward(ctx, h2, shared_w13, shared_w2, swiglu_limit):
        flat = h2.reshape(-1, h2.shape[-1])
        y, h13 = layer.shared_expert_forward(flat, shared_w13, shared_w2, swiglu_limit=swiglu_limit)
        ctx.save_for_backward(flat, shared_w13, shared_w2, h13)
        ctx.limit = swiglu_limit
        ctx.shape = h2.shape
        return y.reshape(h2.shape)

    @staticmethod
    def backward(ctx, grad_y):
        flat, shared_w13, shared_w2, h13 = ctx.saved_tensors
        need_weights = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        gx, gw13, gw2 = layer.shared_expert_backward(
            grad_y.reshape(flat.shape).contiguous(), flat, shared_w13, shared_w2, h13,
            swiglu_limit=ctx.limit, need_weights=need_weights,
        )
        return gx.reshape(ctx.shape), gw13, gw2, None


def supports(h2, residual, router_weight, w13_experts, w2_experts, **kwargs):
    from mlops.dispatch.registry import SupportResult

    reason = refusal(h2, residual, router_weight, w13_experts, w2_experts, **kwargs)
    return SupportResult.yes() if reason is None else SupportResult.no(reason)


def apply(h2, residual, router_weight, w13_experts, w2_experts, *, top_k, routing_mode, router_bias=None,
          n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, shared_w13=None, shared_w2=None,
          shared_gate_weight=None, shared_mode="add", compute_precision=None, swiglu_limit=None):
    """`(output, aux, counts int64 [E], probability_sum fp32 [E])`; differentiable in `h2`,
    `residual`, `router_weight`, both expert containers and the shared weights."""
    reason = refusal(h2, residual, router_weight, w13_experts, w2_experts, top_k=top_k, routing_mode=routing_mode,
                     n_group=n_group, topk_group=topk_group, lengths=lengths, shared_w13=shared_w13,
                     shared_w2=shared_w2, compute_precision=compute_precision)
    if reason is not None:
        raise ValueError(reason)
    base = residual
    if shared_w13 is not None:
        shared = _Shared.apply(h2, shared_w13, shared_w2, None if swiglu_limit is None else float(swiglu_limit))
        if shared_mode == "sigmoid":
            gate = torch.sigmoid(torch.nn.functional.linear(h2, shared_gate_weight).float())
            shared = (gate * shared.float()).to(residual.dtype)
        elif shared_mode != "add":
            raise ValueError(f"unsupported shared_mode {shared_mode!r}")
        base = residual + shared
    rows = h2.numel() // h2.shape[-1]
    options = dict(
        top_k=int(top_k), routing_mode=str(routing_mode), n_group=int(n_group), topk_group=int(topk_group),
        routed_scaling=float(routed_scaling),
        lengths=(rows,) if lengths is None else tuple(int(v) for v in lengths),
        swiglu_limit=None if swiglu_limit is None else float(swiglu_limit),
    )
    bias = None if router_bias is None or router_bias.numel() == 0 else router_bias
    return _Routed.apply(h2, base, router_weight, w13_experts, w2_experts, bias, options)


def forward(h2, residual, router_weight, w13_experts, w2_experts, *, top_k, routing_mode, router_bias=None,
            n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, weight_precision="float32",
            swiglu_implementation=None, swiglu_limit=None):
    """Explicit surface: output, statistics and the VJP residuals, in the reference's order
    `(output, aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets,
    slots, h13)`."""
    del swiglu_implementation
    if weight_precision != "float32":
        raise ValueError("b200.moe keeps route weights in fp32")
    return layer.forward_routed(
        h2, residual, router_weight, components(w13_experts), components(w2_experts), top_k=int(top_k),
        routing_mode=str(routing_mode), router_bias=router_bias, n_group=int(n_group), topk_group=int(topk_group),
        routed_scaling=float(routed_scaling), lengths=lengths, swiglu_limit=swiglu_limit,
    )


def backward(grad_output, grad_aux, grad_probability_sum, h2, router_weight, w13_experts, w2_experts, logits,
             route_weights, route_ids, order, offsets, slots, h13, *, top_k, routing_mode, lengths,
             swiglu_implementation=None, **kwargs):
    """Explicit VJP: `(grad_h2, grad_residual, grad_router, grad_w13, grad_w2)`."""
    del swiglu_implementation
    wdtype = kwargs.pop("weight_grad_dtype", None)
    if wdtype is None:
        wdtype = _context_weight_gradient_dtype() or w13_experts.dtype
    return layer.backward_routed(
        grad_output, grad_aux, grad_probability_sum, h2, router_weight, components(w13_experts),
        components(w2_experts), logits, route_weights, route_ids, order, offsets, slots, h13, top_k=int(top_k),
        routing_mode=str(routing_mode), lengths=lengths, weight_grad_dtype=wdtype, **kwargs,
    )


_REGISTERED = None


def register(priority: int = PRIORITY):
    """Register `b200.moe` with the reference's registry (idempotent). Needs `mlops`
    importable; everything else in this module works without it."""
    global _REGISTERED
    if _REGISTERED is not None:
        return _REGISTERED
    from mlops.dispatch.registry import Implementation, register_implementation

    _REGISTERED = register_implementation(
        Implementation(
            operation="moe", implementation_id=IMPLEMENTATION_ID, provider="b200", priority=int(priority),
            deterministic=True, supports=supports, apply=apply, forward=forward, backward=backward,
        )
    )
    return _REGISTERED
