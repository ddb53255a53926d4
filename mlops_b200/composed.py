"""The routed layer as two opaque regions, `b200.moe.composed`.

`prepare` = router logits + top-k + sort + up projection -> the pre-activation `h13` and the
routing tensors; `finish` = SwiGLU + down projection + combine. Keeping the region that
produces the saved residual apart from the one that consumes it lets AOTAutograd
rematerialise `h13` (replay `prepare`) without replaying the down projection: the shape of the
reference's default implementation (`src/mlops/providers/builtin/moe_composed.py:1-7`,
operators `:267-343`, `:580-614`, the `donate_h13` overload `:671-710`).

Each region is a functional custom-operator pair with fake implementations, autograd
registered with `register_autograd`, FLOP formulas (the reference's `moe_prepare` /
`moe_finish` split, `src/mlops/dispatch/logical_costs.py:401-439`) and the container dispatch
of `provider.py`. The `h13` gradient crosses the boundary between the regions in bf16, so
`prepare`'s backward quantises it once more for its E4M3 input-gradient product; the fused
operator of `provider.py` skips that pass, which is why it stays the default.
"""

from __future__ import annotations

import torch
from torch.utils.flop_counter import register_flop_formula

from . import layer, ops, provider

IMPLEMENTATION_ID = "b200.moe.composed"
PRIORITY = 115  # above the reference's implementations (110), below the fused `b200.moe` (120)

_TEN = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
             torch.Tensor, torch.Tensor, torch.Tensor]


def _scale_of(weight_components):
    if len(weight_components) != 1:
        raise ValueError("a region operator takes the block scales of its one weight as weight_components; pass "
                         "the weight container and leave the list empty")
    return weight_components[0]


# ----------------------------------------------------------------------------- prepare
@torch.library.custom_op("b200moe::moe_prepare_fwd", mutates_args=())
def prepare_fwd(h2: torch.Tensor, router_weight: torch.Tensor, w13_experts: torch.Tensor, router_bias: torch.Tensor,
                top_k: int, routing_mode: str, n_group: int, topk_group: int, routed_scaling: float,
                lengths: list[int], weight_precision: str, weight_grad_dtype: torch.dtype | None,
                weight_components: list[torch.Tensor]) -> _TEN:
    """`(aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets, slots,
    h13)`: everything up to the pre-activation (gate columns then up columns)."""
    del weight_grad_dtype
    if weight_precision not in provider.ROUTE_WEIGHT_PRECISIONS:
        raise ValueError(f"unsupported route-weight precision {weight_precision!r}")
    w13_scale = _scale_of(weight_components)
    experts = router_weight.shape[0]
    with torch.no_grad(), torch.cuda.device(h2.device):
        flat = h2.reshape(-1, h2.shape[-1]).contiguous()
        normalized = layer._normalized_lengths(lengths, flat.shape[0])
        logits = layer.router_logits(flat, router_weight)
        route_weights, route_ids = ops.route_topk(
            logits, int(top_k), str(routing_mode), bias=None if router_bias.numel() == 0 else router_bias,
            n_group=int(n_group), topk_group=int(topk_group), routed_scaling=float(routed_scaling))
        order, offsets, slots, counts = ops.sort_assignments(route_ids, experts)
        x_q, x_s = ops.quantize_rows_scatter(flat, slots)
        h13 = ops.grouped_gemm_fp8(x_q, x_s, w13_experts, w13_scale, offsets)
        aux, counts, probability_sum = layer.routing_statistics(
            logits, route_ids, counts, routing_mode=str(routing_mode), lengths=normalized, experts=experts)
    return aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets, slots, h13


@prepare_fwd.register_fake
def _prepare_fwd_fake(h2, router_weight, w13_experts, router_bias, top_k, routing_mode, n_group, topk_group,
                      routed_scaling, lengths, weight_precision, weight_grad_dtype, weight_components):
    rows = h2.numel() // h2.shape[-1]
    experts, assignments = router_weight.shape[0], rows * int(top_k)
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=h2.device)  # noqa: E731
    return (new((), torch.float32), new((experts,), torch.int64), new((experts,), torch.float32),
            new((rows, experts), torch.float32), new((rows, int(top_k)), torch.float32),
            new((rows, int(top_k)), torch.int32), new((assignments,), torch.int32),
            new((experts + 1,), torch.int32), new((rows, int(top_k)), torch.int32),
            new((assignments, w13_experts.shape[1]), h2.dtype))


@torch.library.custom_op("b200moe::moe_prepare_bwd", mutates_args=())
def prepare_bwd(grad_aux: torch.Tensor, grad_probability_sum: torch.Tensor, grad_route_weights: torch.Tensor,
                grad_h13: torch.Tensor, h2: torch.Tensor, router_weight: torch.Tensor, w13_experts: torch.Tensor,
                logits: torch.Tensor, route_weights: torch.Tensor, route_ids: torch.Tensor, order: torch.Tensor,
                offsets: torch.Tensor, slots: torch.Tensor, top_k: int, routing_mode: str, lengths: list[int],
                weight_grad_dtype: torch.dtype | None, need_router: bool, need_w13: bool,
                weight_components: list[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """`(grad_h2, grad_router, grad_w13)`; a weight nobody asked a gradient for gets an empty
    placeholder and its GEMM is not launched."""
    w13_scale = _scale_of(weight_components)
    experts = w13_experts.shape[0]
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    with torch.no_grad(), torch.cuda.device(h2.device):
        flat = h2.reshape(-1, h2.shape[-1]).contiguous()
        normalized = layer._normalized_lengths(lengths, flat.shape[0])
        counts = (offsets[1:] - offsets[:-1]).long()
        gh = grad_h13.contiguous()
        gh_q, gh_s = ops.quantize_rows(gh)  # the bf16 gradient that crossed the regions, as E4M3
        if need_w13:
            x_rows = ops.dispatch(flat, order, int(top_k))
            grad_w13 = ops.grouped_wgrad(gh, x_rows, offsets, experts, wdtype)
            del x_rows
        else:
            grad_w13 = torch.empty(0, dtype=wdtype, device=h2.device)
        grad_rows = ops.grouped_gemm_fp8(gh_q, gh_s, w13_experts, w13_scale, offsets, b_mn_major=True)
        grad_h2 = ops.dispatch_backward(grad_rows, slots)
        grad_logits = layer.routing_gradient(grad_aux, grad_probability_sum, grad_route_weights, route_weights,
                                             route_ids, logits, counts, routing_mode=str(routing_mode),
                                             lengths=normalized)
        if need_router:
            rdtype = router_weight.dtype if weight_grad_dtype is None else weight_grad_dtype
            grad_router = layer._router_weight_gradient(grad_logits, flat, rdtype)
        else:
            grad_router = torch.empty(0, dtype=router_weight.dtype, device=h2.device)
        grad_h2.addmm_(grad_logits.to(flat.dtype), getattr(router_weight, "_data", router_weight).to(flat.dtype))
    return grad_h2.reshape(h2.shape), grad_router, grad_w13


@prepare_bwd.register_fake
def _prepare_bwd_fake(grad_aux, grad_probability_sum, grad_route_weights, grad_h13, h2, router_weight, w13_experts,
                      logits, route_weights, route_ids, order, offsets, slots, top_k, routing_mode, lengths,
                      weight_grad_dtype, need_router, need_w13, weight_components):
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    rdtype = router_weight.dtype if weight_grad_dtype is None else weight_grad_dtype
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=h2.device)  # noqa: E731
    return (torch.empty_like(h2, memory_format=torch.contiguous_format),
            new(tuple(router_weight.shape), rdtype) if need_router else new((0,), router_weight.dtype),
            new(tuple(w13_experts.shape), wdtype) if need_w13 else new((0,), wdtype))


def _prepare_context(ctx, inputs, output):
    (h2, router_weight, w13_experts, _bias, top_k, routing_mode, _n_group, _topk_group, _scaling, lengths,
     _precision, weight_grad_dtype, weight_components) = inputs
    (_aux, counts, _psum, logits, route_weights, route_ids, order, offsets, slots, _h13) = output
    ctx.save_for_backward(h2, router_weight, w13_experts, logits, route_weights, route_ids, order, offsets, slots,
                          *weight_components)
    ctx.top_k, ctx.routing_mode, ctx.lengths = int(top_k), routing_mode, list(lengths)
    ctx.weight_grad_dtype, ctx.components = weight_grad_dtype, len(weight_components)
    ctx.logical = w13_experts.dtype if w13_experts.dtype != torch.float8_e4m3fn else torch.bfloat16
    ctx.mark_non_differentiable(counts, logits, route_ids, order, offsets, slots)


def _prepare_autograd_backward(ctx, grad_aux, _g_counts, grad_probability_sum, _g_logits, grad_route_weights,
                               _g_ids, _g_order, _g_offsets, _g_slots, grad_h13):
    saved = ctx.saved_tensors
    tensors, components = saved[:9], list(saved[9:])
    h2, router_weight, w13_experts, _logits, route_weights = tensors[:5]
    device = h2.device
    if grad_aux is None:
        grad_aux = torch.zeros((), dtype=torch.float32, device=device)
    if grad_probability_sum is None:
        grad_probability_sum = torch.zeros(router_weight.shape[0], dtype=torch.float32, device=device)
    if grad_route_weights is None:
        grad_route_weights = torch.zeros_like(route_weights)
    if grad_h13 is None:
        rows = h2.numel() // h2.shape[-1] * ctx.top_k
        grad_h13 = torch.zeros((rows, w13_experts.shape[1]), dtype=h2.dtype, device=device)
    need = ctx.needs_input_grad
    wdtype = ctx.weight_grad_dtype
    if wdtype is None and ctx.logical != torch.bfloat16:
        wdtype = ctx.logical
    grad_h2, grad_router, grad_w13 = prepare_bwd(
        grad_aux, grad_probability_sum, grad_route_weights, grad_h13, *tensors, ctx.top_k, ctx.routing_mode,
        ctx.lengths, wdtype, bool(need[1]), bool(need[2]), components)
    if ctx.weight_grad_dtype is None and need[1] and grad_router.dtype != router_weight.dtype:
        grad_router = grad_router.to(router_weight.dtype)
    return (grad_h2 if need[0] else None, grad_router if need[1] else None, grad_w13 if need[2] else None,
            *([None] * 9), [None] * ctx.components)


prepare_fwd.register_autograd(_prepare_autograd_backward, setup_context=_prepare_context)


# ------------------------------------------------------------------------------ finish
@torch.library.custom_op("b200moe::moe_finish_fwd", mutates_args=())
def finish_fwd(h13: torch.Tensor, w2_experts: torch.Tensor, route_weights: torch.Tensor, order: torch.Tensor,
               offsets: torch.Tensor, slots: torch.Tensor, residual: torch.Tensor, top_k: int,
               weight_grad_dtype: torch.dtype | None, swiglu_limit: float | None,
               weight_components: list[torch.Tensor]) -> torch.Tensor:
    """`residual + sum_k w_k . W2[e_k] swiglu(h13[row_k])`, shaped like `residual`."""
    del order, top_k, weight_grad_dtype
    w2_scale = _scale_of(weight_components)
    with torch.no_grad(), torch.cuda.device(h13.device):
        a_q, a_s, _ = ops.swiglu_quantize(h13.contiguous(), limit=swiglu_limit)
        expert_output = ops.grouped_gemm_fp8(a_q, a_s, w2_experts, w2_scale, offsets)
        flat = residual.reshape(-1, residual.shape[-1]).contiguous()
        return ops.combine(expert_output, slots, route_weights.float().contiguous(), flat).reshape(residual.shape)


@finish_fwd.register_fake
def _finish_fwd_fake(h13, w2_experts, route_weights, order, offsets, slots, residual, top_k, weight_grad_dtype,
                     swiglu_limit, weight_components):
    return torch.empty_like(residual, memory_format=torch.contiguous_format)


def _finish_backward(grad_output, h13, w2_experts, w2_scale, route_weights, order, offsets, slots, *, need_w2,
                     weight_grad_dtype, swiglu_limit, destination=None):
    experts = w2_experts.shape[0]
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    with torch.no_grad(), torch.cuda.device(h13.device):
        grad_flat = grad_output.reshape(-1, grad_output.shape[-1]).contiguous()
        if need_w2:
            dy_q, dy_s, dy_rows = ops.quantize_rows_scatter(grad_flat, slots, with_copy=True)
        else:
            dy_q, dy_s = ops.quantize_rows_scatter(grad_flat, slots)
        r = ops.grouped_gemm_fp8(dy_q, dy_s, w2_experts, w2_scale, offsets, b_mn_major=True)
        dscore, _, _, grad_h13, act_scaled = ops.dswiglu_routed(
            h13, r, route_weights.float().contiguous(), order, limit=swiglu_limit, quantized=False, rounded=True,
            scaled_activation=need_w2, rounded_out=destination)
        grad_route_weights = ops.gather_scalar(dscore, slots)
        if need_w2:
            grad_w2 = ops.grouped_wgrad(dy_rows, act_scaled, offsets, experts, wdtype)
        else:
            grad_w2 = torch.empty(0, dtype=wdtype, device=h13.device)
    return grad_h13, grad_w2, grad_route_weights, grad_output.clone()


_FOUR = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


@torch.library.custom_op("b200moe::moe_finish_bwd", mutates_args=())
def finish_bwd(grad_output: torch.Tensor, h13: torch.Tensor, w2_experts: torch.Tensor, route_weights: torch.Tensor,
               order: torch.Tensor, offsets: torch.Tensor, slots: torch.Tensor, top_k: int,
               weight_grad_dtype: torch.dtype | None, swiglu_limit: float | None, need_w2: bool,
               weight_components: list[torch.Tensor]) -> _FOUR:
    """`(grad_h13 bf16, grad_w2, grad_route_weights, grad_residual)`."""
    del top_k
    return _finish_backward(grad_output, h13, w2_experts, _scale_of(weight_components), route_weights, order,
                            offsets, slots, need_w2=need_w2, weight_grad_dtype=weight_grad_dtype,
                            swiglu_limit=swiglu_limit)


@finish_bwd.register_fake
def _finish_bwd_fake(grad_output, h13, w2_experts, route_weights, order, offsets, slots, top_k, weight_grad_dtype,
                     swiglu_limit, need_w2, weight_components):
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    return (torch.empty_like(h13, memory_format=torch.contiguous_format),
            torch.empty(tuple(w2_experts.shape) if need_w2 else (0,), dtype=wdtype, device=h13.device),
            torch.empty_like(route_weights, dtype=torch.float32, memory_format=torch.contiguous_format),
            torch.empty_like(grad_output, memory_format=torch.contiguous_format))


@torch.library.custom_op("b200moe::moe_finish_bwd_donate_h13", mutates_args=("h13",))
def finish_bwd_donate_h13(grad_output: torch.Tensor, h13: torch.Tensor, w2_experts: torch.Tensor,
                          route_weights: torch.Tensor, order: torch.Tensor, offsets: torch.Tensor,
                          slots: torch.Tensor, top_k: int, weight_grad_dtype: torch.dtype | None,
                          swiglu_limit: float | None, need_w2: bool,
                          weight_components: list[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The same backward for a caller that no longer needs `h13`: the gradient of `h13` is
    written over `h13` itself (2 x rows x 2F bytes of HBM not allocated); returns `(grad_w2,
    grad_route_weights, grad_residual)`. Every element of `h13` is read by the thread that
    overwrites it, before it does (the reference's overload:
    src/mlops/providers/builtin/moe_composed.py:671-710)."""
    del top_k
    if not h13.is_contiguous():
        raise ValueError("donate_h13 writes the gradient over h13: it must be contiguous")
    _gh, grad_w2, grad_route_weights, grad_residual = _finish_backward(
        grad_output, h13, w2_experts, _scale_of(weight_components), route_weights, order, offsets, slots,
        need_w2=need_w2, weight_grad_dtype=weight_grad_dtype, swiglu_limit=swiglu_limit, destination=h13)
    return grad_w2, grad_route_weights, grad_residual


@finish_bwd_donate_h13.register_fake
def _finish_bwd_donate_fake(grad_output, h13, w2_experts, route_weights, order, offsets, slots, top_k,
                            weight_grad_dtype, swiglu_limit, need_w2, weight_components):
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    return (torch.empty(tuple(w2_experts.shape) if need_w2 else (0,), dtype=wdtype, device=h13.device),
            torch.empty_like(route_weights, dtype=torch.float32, memory_format=torch.contiguous_format),
            torch.empty_like(grad_output, memory_format=torch.contiguous_format))


def _finish_context(ctx, inputs, output):
    (h13, w2_experts, route_weights, order, offsets, slots, _residual, top_k, weight_grad_dtype, swiglu_limit,
     weight_components) = inputs
    ctx.save_for_backward(h13, w2_experts, route_weights, order, offsets, slots, *weight_components)
    ctx.top_k, ctx.weight_grad_dtype, ctx.swiglu_limit = int(top_k), weight_grad_dtype, swiglu_limit
    ctx.components = len(weight_components)
    ctx.logical = w2_experts.dtype if w2_experts.dtype != torch.float8_e4m3fn else torch.bfloat16


def _finish_autograd_backward(ctx, grad_output):
    saved = ctx.saved_tensors
    tensors, components = saved[:6], list(saved[6:])
    need = ctx.needs_input_grad
    wdtype = ctx.weight_grad_dtype
    if wdtype is None and ctx.logical != torch.bfloat16:
        wdtype = ctx.logical
    grad_h13, grad_w2, grad_route_weights, grad_residual = finish_bwd(
        grad_output.contiguous(), *tensors, ctx.top_k, wdtype, ctx.swiglu_limit, bool(need[1]), components)
    return (grad_h13 if need[0] else None, grad_w2 if need[1] else None,
            grad_route_weights if need[2] else None, None, None, None, grad_residual if need[6] else None,
            None, None, None, [None] * ctx.components)


finish_fwd.register_autograd(_finish_autograd_backward, setup_context=_finish_context)


def _region_flops(h2_rows, width, experts, assignments, packed, inner, *, prepare, forward):
    try:
        from mlops.dispatch import logical_costs
    except ImportError:
        logical_costs = None
    if logical_costs is not None:
        if prepare:
            return logical_costs._moe_prepare_flops(h2_rows, width, experts, assignments, packed, forward=forward)
        return logical_costs._moe_finish_flops(assignments, inner, width, forward=forward)
    if prepare:
        router = 2 * h2_rows * width * experts + 3 * h2_rows * experts
        up = 2 * assignments * width * packed
        return router + up if forward else 2 * router - 3 * h2_rows * experts + 2 * up
    activation, down, combine = 5 * assignments * inner, 2 * assignments * inner * width, 2 * assignments * width
    return activation + down + combine if forward else 2 * activation + 2 * down + combine


@register_flop_formula(torch.ops.b200moe.moe_prepare_fwd, get_raw=True)
def _prepare_fwd_flops(h2, router_weight, w13_experts, router_bias, top_k, *_rest, out_val=None, **_kwargs):
    rows = h2.numel() // h2.shape[-1]
    return _region_flops(rows, h2.shape[-1], router_weight.shape[0], rows * int(top_k), w13_experts.shape[1], 0,
                         prepare=True, forward=True)


@register_flop_formula(torch.ops.b200moe.moe_prepare_bwd, get_raw=True)
def _prepare_bwd_flops(grad_aux, grad_probability_sum, grad_route_weights, grad_h13, h2, router_weight,
                       w13_experts, *_rest, out_val=None, **_kwargs):
    rows = h2.numel() // h2.shape[-1]
    return _region_flops(rows, h2.shape[-1], router_weight.shape[0], grad_h13.shape[0], w13_experts.shape[1], 0,
                         prepare=True, forward=False)


@register_flop_formula(torch.ops.b200moe.moe_finish_fwd, get_raw=True)
def _finish_fwd_flops(h13, w2_experts, *_rest, out_val=None, **_kwargs):
    return _region_flops(0, w2_experts.shape[1], 0, h13.shape[0], 0, w2_experts.shape[2], prepare=False,
                         forward=True)


@register_flop_formula([torch.ops.b200moe.moe_finish_bwd, torch.ops.b200moe.moe_finish_bwd_donate_h13],
                       get_raw=True)
def _finish_bwd_flops(grad_output, h13, w2_experts, *_rest, out_val=None, **_kwargs):
    return _region_flops(0, w2_experts.shape[1], 0, h13.shape[0], 0, w2_experts.shape[2], prepare=False,
                         forward=False)


_OPERATORS = [prepare_fwd, prepare_bwd, finish_fwd, finish_bwd, finish_bwd_donate_h13]
provider._CONTAINER_OPERATORS.extend(_OPERATORS)
for _cls in list(provider._DISPATCH_REGISTERED):  # containers registered before this module loaded
    for _op in _OPERATORS:
        _op.register_torch_dispatch(_cls, provider._unwrap_containers)


# ------------------------------------------------------------------------------- provider
def supports(h2, residual, router_weight, w13_experts, w2_experts, *, surface, **kwargs):
    from mlops.dispatch.registry import SupportResult

    if surface == "explicit":
        return SupportResult.no("the two-region composition is a semantic-only implementation")
    reason = provider.refusal(h2, residual, router_weight, w13_experts, w2_experts, surface=surface, **kwargs)
    return SupportResult.yes() if reason is None else SupportResult.no(reason)


def apply(h2, residual, router_weight, w13_experts, w2_experts, *, top_k, routing_mode, router_bias=None,
          n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, shared_w13=None, shared_w2=None,
          shared_gate_weight=None, shared_mode="add", compute_precision=None, swiglu_limit=None):
    """`(output, aux, counts, probability_sum)` through the two regions; same contract as
    `provider.apply`."""
    reason = provider.refusal(h2, residual, router_weight, w13_experts, w2_experts, top_k=top_k,
                              routing_mode=routing_mode, n_group=n_group, topk_group=topk_group, lengths=lengths,
                              shared_w13=shared_w13, shared_w2=shared_w2, compute_precision=compute_precision)
    if reason is not None:
        raise ValueError(reason)
    for weight in (w13_experts, w2_experts):
        if type(weight) not in provider._DISPATCH_REGISTERED:
            provider.register_container(type(weight))
    limit = None if swiglu_limit is None else float(swiglu_limit)
    base = residual
    if shared_w13 is not None:
        base = residual + provider.shared_expert(h2, shared_w13, shared_w2, shared_gate_weight, shared_mode, limit)
    rows = h2.numel() // h2.shape[-1]
    normalized = [rows] if lengths is None else [int(v) for v in lengths]
    bias = router_bias if router_bias is not None else torch.empty(0, dtype=torch.float32, device=h2.device)
    wgd = provider._context_weight_gradient_dtype()
    aux, counts, probability_sum, _logits, route_weights, _ids, order, offsets, slots, h13 = prepare_fwd(
        h2, router_weight, w13_experts, bias, int(top_k), str(routing_mode), int(n_group), int(topk_group),
        float(routed_scaling), normalized, provider._context_route_weight_precision(), wgd, [])
    output = finish_fwd(h13, w2_experts, route_weights, order, offsets, slots, base, int(top_k), wgd, limit, [])
    return output, aux, counts, probability_sum


_REGISTERED = None


def register(priority: int = PRIORITY):
    """Register `b200.moe.composed` with the reference's registry (idempotent)."""
    global _REGISTERED
    if _REGISTERED is not None:
        return _REGISTERED
    from mlops.dispatch.registry import Implementation, register_implementation

    provider._register_reference_containers()
    _REGISTERED = register_implementation(
        Implementation(operation="moe", implementation_id=IMPLEMENTATION_ID, provider="b200",
                       priority=int(priority), deterministic=True, supports=supports, apply=apply))
    return _REGISTERED


__all__ = ["apply", "finish_bwd", "finish_bwd_donate_h13", "finish_fwd", "prepare_bwd", "prepare_fwd", "register",
           "supports"]
