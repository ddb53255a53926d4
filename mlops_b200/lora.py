"""Expert LoRA on the block-FP8 path: `expert_lora(...)` with the reference's signature and
results (`src/mlops/lora/experts.py:53-167` of als244/mlops).

    h13 = x W13^T + s (x A13^T) B13^T  ->  SwiGLU  ->  y = a W2^T + s (a A2^T) B2^T

Factors: `a13 [E, r, D]`, `b13 [E, 2F, r]`, `a2 [E, r, F]`, `b2 [E, D, r]` (bf16). The base
products are the E4M3 tcgen05 GEMMs; each LoRA term is formed by the rank-r kernels
(`lora_project`, `lora_expand`) and enters its base GEMM as an addend before the one rounding
(and before SwiGLU for the up projection), the form of the reference's fused provider
(`src/mlops/providers/sonicmoe/lora.py:1062-1130`). A frozen base launches no base weight
gradient; the factors' gradients are grouped weight gradients with one narrow side on the
tcgen05 weight-gradient kernel. The reference validates `implementation=` against a literal
tuple, so this function is reached by importing it, not through that argument.

Like the plain layer, the computation is a functional custom-operator pair
(`b200moe::moe_lora_fwd` / `b200moe::moe_lora_bwd`) with fake implementations and autograd
registered on the forward operator, so it can be traced and counted like the reference's
operators (`docs/PROVIDERS.md:86-112`).
"""

from __future__ import annotations

import math

import torch
from torch.utils.flop_counter import register_flop_formula

from . import layer, ops, provider
from .weights import holds_blocks


def _pad_rank(factor, axis):
    """Ranks are padded with zeros to a multiple of 8 (16-byte rows for the kernels), as the
    reference pads them (`providers/sonicmoe/lora.py:965-975`)."""
    rank = factor.shape[axis]
    padded = -(-rank // 8) * 8
    if padded == rank:
        return factor.contiguous(), rank
    shape = list(factor.shape)
    shape[axis] = padded
    out = factor.new_zeros(shape)
    out.narrow(axis, 0, rank).copy_(factor)
    return out, rank


def _kernel_factors(a13, b13, a2, b2):
    """The factors as the rank-r kernels read them: ranks padded, the B factors rank-major
    (`[E, r, wide]`) so every kernel stages its factor with 16-byte loads (a few MB per call)."""
    a13p, rank = _pad_rank(a13.detach(), 1)
    b13p, _ = _pad_rank(b13.detach(), 2)
    a2p, _ = _pad_rank(a2.detach(), 1)
    b2p, _ = _pad_rank(b2.detach(), 2)
    return a13p, b13p.transpose(1, 2).contiguous(), a2p, b2p.transpose(1, 2).contiguous(), rank


_THIRTEEN = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                  torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                  torch.Tensor]
_NINE = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
              torch.Tensor, torch.Tensor, torch.Tensor]


@torch.library.custom_op("b200moe::moe_lora_fwd", mutates_args=())
def moe_lora_fwd(hidden: torch.Tensor, residual: torch.Tensor, router_weight: torch.Tensor, gate_up: torch.Tensor,
                 down: torch.Tensor, a13: torch.Tensor, b13: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor,
                 router_bias: torch.Tensor, top_k: int, routing_mode: str, scale: float, n_group: int,
                 topk_group: int, routed_scaling: float, lengths: list[int], swiglu_limit: float | None,
                 gradient_destinations: list[torch.Tensor], gradient_scale: float,
                 weight_components: list[torch.Tensor]) -> _THIRTEEN:
    """`(output, aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets,
    slots, h13, t1, t2)`: the plain layer's results and residuals plus the two rank-r
    intermediates `t1 = x A13^T`, `t2 = act A2^T` the factor gradients need.
    `gradient_destinations` (none, or four buffers for a13, b13, a2, b2) and `gradient_scale`
    are not read here: they name where the backward pass accumulates the factor gradients."""
    del gradient_destinations, gradient_scale
    w13, w2 = provider._with_scales(gate_up, down, weight_components)
    experts = gate_up.shape[0]
    with torch.no_grad(), torch.cuda.device(hidden.device):
        flat = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        residual_flat = residual.reshape_as(flat).contiguous()
        a13p, b13t, a2p, b2t, _rank = _kernel_factors(a13, b13, a2, b2)
        logits = layer.router_logits(flat, router_weight)
        weights, ids = ops.route_topk(
            logits, top_k, routing_mode, bias=None if router_bias.numel() == 0 else router_bias, n_group=n_group,
            topk_group=topk_group, routed_scaling=routed_scaling)
        order, offsets, slots, counts = ops.sort_assignments(ids, experts)
        # one pass over the tokens: E4M3 rows for the base product, bf16 rows for the rank-r one
        x_q, x_s, x_rows = ops.quantize_rows_scatter(flat, slots, with_copy=True)
        t1 = ops.lora_project(x_rows, a13p, offsets, rank_major=True)
        c1 = ops.lora_expand(t1, b13t, offsets, wide_major=False, scale=scale)
        h13 = ops.grouped_gemm_fp8(x_q, x_s, *w13, offsets, addend=c1)
        a_q, a_s, act = ops.swiglu_quantize(h13, limit=swiglu_limit, quantized=True, rounded=True)
        t2 = ops.lora_project(act, a2p, offsets, rank_major=True)
        c2 = ops.lora_expand(t2, b2t, offsets, wide_major=False, scale=scale)
        y = ops.grouped_gemm_fp8(a_q, a_s, *w2, offsets, addend=c2)
        output = ops.combine(y, slots, weights, residual_flat).reshape(hidden.shape)
        aux, counts, probability_sum = layer.routing_statistics(
            logits, ids, counts, routing_mode=routing_mode, lengths=tuple(lengths), experts=experts)
    return output, aux, counts, probability_sum, logits, weights, ids, order, offsets, slots, h13, t1, t2


@moe_lora_fwd.register_fake
def _moe_lora_fwd_fake(hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, router_bias, top_k,
                       routing_mode, scale, n_group, topk_group, routed_scaling, lengths, swiglu_limit,
                       gradient_destinations, gradient_scale, weight_components):
    rows = hidden.numel() // hidden.shape[-1]
    experts, assignments = router_weight.shape[0], rows * int(top_k)
    padded = -(-a13.shape[1] // 8) * 8
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=hidden.device)  # noqa: E731
    return (
        torch.empty_like(hidden, memory_format=torch.contiguous_format),
        new((), torch.float32), new((experts,), torch.int64), new((experts,), torch.float32),
        new((rows, experts), torch.float32), new((rows, int(top_k)), torch.float32),
        new((rows, int(top_k)), torch.int32), new((assignments,), torch.int32),
        new((experts + 1,), torch.int32), new((rows, int(top_k)), torch.int32),
        new((assignments, gate_up.shape[1]), hidden.dtype), new((assignments, padded), hidden.dtype),
        new((assignments, padded), hidden.dtype),
    )


def _lora_backward(grad_output, grad_aux, grad_probability_sum, hidden, router_weight, gate_up, down, a13, b13, a2,
                   b2, logits, route_weights, route_ids, order, offsets, slots, h13, t1, t2, top_k, routing_mode,
                   scale, lengths, weight_grad_dtype, swiglu_limit, need_router, need_w13, need_w2, need_factors,
                   weight_components, destinations=None, gradient_scale=1.0):
    """The backward pass of both operators below. With `destinations` (buffers for a13, b13, a2,
    b2) the factor gradients are added, times `gradient_scale`, into those buffers by the
    weight-gradient GEMMs' own stores and empty placeholders are returned in their place."""
    (w13_d, w13_s), (w2_d, w2_s) = provider._with_scales(gate_up, down, weight_components)
    experts = w13_d.shape[0]
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    weights, ids = route_weights, route_ids
    with torch.no_grad(), torch.cuda.device(hidden.device):
        flat = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        dy = grad_output.reshape_as(flat).contiguous()
        a13p, b13t, a2p, b2t, rank = _kernel_factors(a13, b13, a2, b2)
        counts = (offsets[1:] - offsets[:-1]).long()
        empty = lambda dtype: torch.empty(0, dtype=dtype, device=flat.device)  # noqa: E731

        dy_q, dy_s, dy_rows = ops.quantize_rows_scatter(dy, slots, with_copy=True)
        t2g = ops.lora_project(dy_rows, b2t, offsets, rank_major=True)              # dy B2      [R, r]
        r_add = ops.lora_expand(t2g, a2p, offsets, wide_major=False, scale=scale)   # s dy B2 A2 [R, F]
        r = ops.grouped_gemm_fp8(dy_q, dy_s, w2_d, w2_s, offsets, b_mn_major=True, addend=r_add)
        dscore, gh_q, gh_s, gh_b, act_scaled = ops.dswiglu_routed(
            h13, r, weights, order, limit=swiglu_limit, quantized=True, rounded=True, scaled_activation=True)
        grad_route_weights = ops.gather_scalar(dscore, slots)

        x_rows = ops.dispatch(flat, order, top_k)
        dt1 = ops.lora_project(gh_b, b13t, offsets, rank_major=True)                # gh B13     [R, r]
        fdtype = a13.dtype
        grad_a13 = grad_b13 = grad_a2 = grad_b2 = empty(fdtype)
        if need_factors:
            row_weight = weights.reshape(-1)[order.long()].float()[:, None]
            into = dict(zip(("a13", "b13", "a2", "b2"), destinations)) if destinations else {}
            product = lambda name, left, right: ops.grouped_wgrad(  # noqa: E731
                left, right, offsets, experts, fdtype, accumulate_into=into.get(name),
                scale=gradient_scale if into else 1.0)
            grad_b2 = product("b2", dy_rows, (t2.float() * (row_weight * scale)).to(t2.dtype))
            grad_a2 = product("a2", (t2g.float() * scale).to(t2g.dtype), act_scaled)
            grad_b13 = product("b13", gh_b, (t1.float() * scale).to(t1.dtype))
            grad_a13 = product("a13", (dt1.float() * scale).to(dt1.dtype), x_rows)
            if into:  # the buffers hold the gradients; nothing is handed back
                grad_a13 = grad_b13 = grad_a2 = grad_b2 = empty(fdtype)
            else:
                grad_b2, grad_b13 = grad_b2[:, :, :rank].contiguous(), grad_b13[:, :, :rank].contiguous()
                grad_a2, grad_a13 = grad_a2[:, :rank].contiguous(), grad_a13[:, :rank].contiguous()
        dx_add = ops.lora_expand(dt1, a13p, offsets, wide_major=False, scale=scale)
        grad_rows = ops.grouped_gemm_fp8(gh_q, gh_s, w13_d, w13_s, offsets, b_mn_major=True, addend=dx_add)
        grad_h2 = ops.dispatch_backward(grad_rows, slots)

        # a trainable base gets its gradient as in the plain layer
        grad_w13 = ops.grouped_wgrad(gh_b, x_rows, offsets, experts, wdtype) if need_w13 else empty(wdtype)
        grad_w2 = ops.grouped_wgrad(dy_rows, act_scaled, offsets, experts, wdtype) if need_w2 else empty(wdtype)

        grad_logits = layer.routing_gradient(
            grad_aux, grad_probability_sum, grad_route_weights, weights, ids, logits, counts,
            routing_mode=routing_mode, lengths=tuple(lengths))
        rdtype = router_weight.dtype if weight_grad_dtype is None else weight_grad_dtype
        grad_router = (layer._router_weight_gradient(grad_logits, flat, rdtype) if need_router
                       else empty(router_weight.dtype))
        grad_h2.addmm_(grad_logits.to(flat.dtype), getattr(router_weight, "_data", router_weight).to(flat.dtype))
    return (grad_h2.reshape(hidden.shape), grad_output.clone(), grad_router, grad_w13, grad_w2, grad_a13, grad_b13,
            grad_a2, grad_b2)




@torch.library.custom_op("b200moe::moe_lora_bwd", mutates_args=())
def moe_lora_bwd(grad_output: torch.Tensor, grad_aux: torch.Tensor, grad_probability_sum: torch.Tensor,
                 hidden: torch.Tensor, router_weight: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor,
                 a13: torch.Tensor, b13: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor, logits: torch.Tensor,
                 route_weights: torch.Tensor, route_ids: torch.Tensor, order: torch.Tensor, offsets: torch.Tensor,
                 slots: torch.Tensor, h13: torch.Tensor, t1: torch.Tensor, t2: torch.Tensor, top_k: int,
                 routing_mode: str, scale: float, lengths: list[int], weight_grad_dtype: torch.dtype | None,
                 swiglu_limit: float | None, need_router: bool, need_w13: bool, need_w2: bool,
                 need_factors: bool, weight_components: list[torch.Tensor]) -> _NINE:
    """`(grad_hidden, grad_residual, grad_router, grad_w13, grad_w2, grad_a13, grad_b13, grad_a2,
    grad_b2)`; gradients whose flag is false are empty placeholders and are not computed (a
    frozen base launches no base-weight gradient: `tests/test_sonicmoe_lora.py:209-233`)."""
    return _lora_backward(grad_output, grad_aux, grad_probability_sum, hidden, router_weight, gate_up, down, a13, b13,
                          a2, b2, logits, route_weights, route_ids, order, offsets, slots, h13, t1, t2, top_k,
                          routing_mode, scale, lengths, weight_grad_dtype, swiglu_limit, need_router, need_w13,
                          need_w2, need_factors, weight_components)


_FIVE = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


@torch.library.custom_op("b200moe::moe_lora_bwd_into",
                         mutates_args=("dest_a13", "dest_b13", "dest_a2", "dest_b2"))
def moe_lora_bwd_into(grad_output: torch.Tensor, grad_aux: torch.Tensor, grad_probability_sum: torch.Tensor,
                      hidden: torch.Tensor, router_weight: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor,
                      a13: torch.Tensor, b13: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor,
                      logits: torch.Tensor, route_weights: torch.Tensor, route_ids: torch.Tensor,
                      order: torch.Tensor, offsets: torch.Tensor, slots: torch.Tensor, h13: torch.Tensor,
                      t1: torch.Tensor, t2: torch.Tensor, dest_a13: torch.Tensor, dest_b13: torch.Tensor,
                      dest_a2: torch.Tensor, dest_b2: torch.Tensor, gradient_scale: float, top_k: int,
                      routing_mode: str, scale: float, lengths: list[int], weight_grad_dtype: torch.dtype | None,
                      swiglu_limit: float | None, need_router: bool, need_w13: bool, need_w2: bool,
                      weight_components: list[torch.Tensor]) -> _FIVE:
    """The backward pass with explicit destinations for the factor gradients:
    `dest += gradient_scale * gradient`, formed in the store of each weight-gradient GEMM, so the
    micro-batches of an accumulation window add up in the caller's buffers with no pass of their
    own. Returns `(grad_hidden, grad_residual, grad_router, grad_w13, grad_w2)`. The form of the
    reference's accumulating operators (src/mlops/providers/sonicmoe/lora_destinations.py:1-16)."""
    result = _lora_backward(grad_output, grad_aux, grad_probability_sum, hidden, router_weight, gate_up, down, a13,
                            b13, a2, b2, logits, route_weights, route_ids, order, offsets, slots, h13, t1, t2, top_k,
                            routing_mode, scale, lengths, weight_grad_dtype, swiglu_limit, need_router, need_w13,
                            need_w2, True, weight_components, destinations=(dest_a13, dest_b13, dest_a2, dest_b2),
                            gradient_scale=gradient_scale)
    return result[:5]


@moe_lora_bwd_into.register_fake
def _moe_lora_bwd_into_fake(grad_output, grad_aux, grad_probability_sum, hidden, router_weight, gate_up, down, a13,
                            b13, a2, b2, logits, route_weights, route_ids, order, offsets, slots, h13, t1, t2,
                            dest_a13, dest_b13, dest_a2, dest_b2, gradient_scale, top_k, routing_mode, scale,
                            lengths, weight_grad_dtype, swiglu_limit, need_router, need_w13, need_w2,
                            weight_components):
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    rdtype = router_weight.dtype if weight_grad_dtype is None else weight_grad_dtype
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=hidden.device)  # noqa: E731
    return (torch.empty_like(hidden, memory_format=torch.contiguous_format),
            torch.empty_like(grad_output, memory_format=torch.contiguous_format),
            new(tuple(router_weight.shape), rdtype) if need_router else new((0,), router_weight.dtype),
            new(tuple(gate_up.shape), wdtype) if need_w13 else new((0,), wdtype),
            new(tuple(down.shape), wdtype) if need_w2 else new((0,), wdtype))


@moe_lora_bwd.register_fake
def _moe_lora_bwd_fake(grad_output, grad_aux, grad_probability_sum, hidden, router_weight, gate_up, down, a13, b13,
                       a2, b2, logits, route_weights, route_ids, order, offsets, slots, h13, t1, t2, top_k,
                       routing_mode, scale, lengths, weight_grad_dtype, swiglu_limit, need_router, need_w13,
                       need_w2, need_factors, weight_components):
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    rdtype = router_weight.dtype if weight_grad_dtype is None else weight_grad_dtype
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=hidden.device)  # noqa: E731
    factor = lambda f: new(tuple(f.shape), f.dtype) if need_factors else new((0,), f.dtype)  # noqa: E731
    return (
        torch.empty_like(hidden, memory_format=torch.contiguous_format),
        torch.empty_like(grad_output, memory_format=torch.contiguous_format),
        new(tuple(router_weight.shape), rdtype) if need_router else new((0,), router_weight.dtype),
        new(tuple(gate_up.shape), wdtype) if need_w13 else new((0,), wdtype),
        new(tuple(down.shape), wdtype) if need_w2 else new((0,), wdtype),
        factor(a13), factor(b13), factor(a2), factor(b2),
    )


def _lora_flops(hidden, router_weight, gate_up, down, a13, top_k, forward, frozen_base):
    base = provider._logical_flops(hidden, router_weight, gate_up, down, top_k, forward)
    rows = (hidden.numel() // hidden.shape[-1]) * int(top_k)
    width, packed, inner, rank = hidden.shape[-1], gate_up.shape[1], down.shape[2], a13.shape[1]
    branch = 2 * rows * rank * (width + packed + inner + width)  # project + expand, both projections
    if forward:
        return base + branch
    if frozen_base:  # no base weight gradient: the input-gradient half of the backward products
        base -= 2 * rows * width * packed + 2 * rows * inner * width
    return base + 2 * branch


@register_flop_formula(torch.ops.b200moe.moe_lora_fwd, get_raw=True)
def _moe_lora_fwd_flops(hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, router_bias, top_k,
                        *_rest, out_val=None, **_kwargs):
    return _lora_flops(hidden, router_weight, gate_up, down, a13, top_k, True, False)


@register_flop_formula(torch.ops.b200moe.moe_lora_bwd, get_raw=True)
def _moe_lora_bwd_flops(grad_output, grad_aux, grad_probability_sum, hidden, router_weight, gate_up, down, a13,
                        b13, a2, b2, logits, route_weights, route_ids, order, offsets, slots, h13, t1, t2, top_k,
                        routing_mode, scale, lengths, weight_grad_dtype, swiglu_limit, need_router, need_w13,
                        need_w2, *_rest, out_val=None, **_kwargs):
    return _lora_flops(hidden, router_weight, gate_up, down, a13, top_k, False, not (need_w13 or need_w2))


def _setup_context(ctx, inputs, output):
    (hidden, _residual, router_weight, gate_up, down, a13, b13, a2, b2, _bias, top_k, routing_mode, scale,
     _n_group, _topk_group, _scaling, lengths, swiglu_limit, gradient_destinations, gradient_scale,
     weight_components) = inputs
    (_out, _aux, counts, _psum, logits, weights, ids, order, offsets, slots, h13, t1, t2) = output
    ctx.save_for_backward(hidden, router_weight, gate_up, down, a13, b13, a2, b2, logits, weights, ids, order,
                          offsets, slots, h13, t1, t2, *weight_components)
    ctx.destinations, ctx.gradient_scale = list(gradient_destinations), float(gradient_scale)
    ctx.top_k, ctx.routing_mode, ctx.scale = int(top_k), routing_mode, float(scale)
    ctx.lengths, ctx.swiglu_limit, ctx.components = list(lengths), swiglu_limit, len(weight_components)
    ctx.weight_grad_dtype = provider._context_weight_gradient_dtype()
    ctx.logical = gate_up.dtype if gate_up.dtype != torch.float8_e4m3fn else torch.bfloat16
    ctx.mark_non_differentiable(counts, logits, weights, ids, order, offsets, slots, h13, t1, t2)


def _autograd_backward(ctx, grad_output, grad_aux, _g_counts, grad_probability_sum, *_metadata_grads):
    saved = ctx.saved_tensors
    tensors, components = saved[:17], list(saved[17:])
    hidden, router_weight = tensors[0], tensors[1]
    if grad_output is None:
        grad_output = torch.zeros_like(hidden)
    if grad_aux is None:
        grad_aux = torch.zeros((), dtype=torch.float32, device=hidden.device)
    if grad_probability_sum is None:
        grad_probability_sum = torch.zeros(router_weight.shape[0], dtype=torch.float32, device=hidden.device)
    need = ctx.needs_input_grad
    wdtype = ctx.weight_grad_dtype
    if wdtype is None and ctx.logical != torch.bfloat16:
        wdtype = ctx.logical
    if ctx.destinations:
        grads = (*moe_lora_bwd_into(
            grad_output, grad_aux, grad_probability_sum, *tensors, *ctx.destinations, ctx.gradient_scale, ctx.top_k,
            ctx.routing_mode, ctx.scale, ctx.lengths, wdtype, ctx.swiglu_limit, bool(need[2]), bool(need[3]),
            bool(need[4]), components), None, None, None, None)  # the factors' gradients sit in the buffers
    else:
        grads = moe_lora_bwd(
            grad_output, grad_aux, grad_probability_sum, *tensors, ctx.top_k, ctx.routing_mode, ctx.scale,
            ctx.lengths, wdtype, ctx.swiglu_limit, bool(need[2]), bool(need[3]), bool(need[4]),
            bool(any(need[5:9])), components)
    grad_router = grads[2]
    if ctx.weight_grad_dtype is None and need[2] and grad_router.dtype != router_weight.dtype:
        grad_router = grad_router.to(router_weight.dtype)
    picked = [grads[0], grads[1], grad_router, *grads[3:]]
    return (*[g if (n and g is not None) else None for g, n in zip(picked, need[:9])], *([None] * 9),
            [None] * len(ctx.destinations), None, [None] * ctx.components)


moe_lora_fwd.register_autograd(_autograd_backward, setup_context=_setup_context)
provider._CONTAINER_OPERATORS.extend([moe_lora_fwd, moe_lora_bwd, moe_lora_bwd_into])
for _cls in list(provider._DISPATCH_REGISTERED):  # containers registered before this module loaded
    for _op in (moe_lora_fwd, moe_lora_bwd, moe_lora_bwd_into):
        _op.register_torch_dispatch(_cls, provider._unwrap_containers)


def expert_lora(hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, *, top_k, routing_mode, scale,
                router_bias=None, n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, swiglu_limit=None,
                implementation="b200", compute_precision=None, gradient_destinations=None, gradient_scale=1.0):
    """Returns `(output, aux, counts, probability_sum)`, differentiable in `hidden`, `residual`,
    `router_weight`, the four factors and (when they ask for it) the base containers.

    `gradient_destinations` (a dict with buffers for all of `a13`, `b13`, `a2`, `b2`: each the
    factor's shape, contiguous, bf16 or fp32, not overlapping) makes the backward pass ADD
    `gradient_scale` times each factor's gradient into its buffer, inside the weight-gradient
    GEMM's store, instead of returning it: the gradients of an accumulation window's
    micro-batches sum in place (the factors' own `.grad` stays untouched). Ranks must be
    multiples of 8 for this form (no padded rank to crop). Reference:
    src/mlops/providers/sonicmoe/lora_destinations.py:28-432."""
    if implementation not in ("auto", "b200"):
        raise ValueError(f"mlops_b200.expert_lora serves implementation 'b200' (or 'auto'), not {implementation!r}")
    if compute_precision not in (None, "fp8_block"):
        raise ValueError("mlops_b200.expert_lora computes the base in block FP8 only")
    if not (holds_blocks(gate_up) and holds_blocks(down)):
        raise ValueError("gate_up and down must be block-FP8 containers (E4M3, 128x128 block scales)")
    if swiglu_limit is not None:
        swiglu_limit = float(swiglu_limit)
        if not swiglu_limit > 0:
            raise ValueError("swiglu_limit must be positive")
    experts, two_f, width = gate_up.shape
    rank = a13.shape[1]
    expected = {"a13": (experts, rank, width), "b13": (experts, two_f, rank), "a2": (experts, rank, two_f // 2),
                "b2": (experts, width, rank)}
    for name, factor in (("a13", a13), ("b13", b13), ("a2", a2), ("b2", b2)):
        if tuple(factor.shape) != expected[name] or factor.dtype != torch.bfloat16:
            raise ValueError(f"{name} must be bf16 with shape {expected[name]}")
    if rank > 64:
        raise ValueError("ranks up to 64 are supported")
    destinations = []
    if gradient_destinations is not None:
        if sorted(gradient_destinations) != ["a13", "a2", "b13", "b2"]:
            raise ValueError("gradient_destinations names a buffer for each of a13, b13, a2, b2")
        if rank % 8:
            raise ValueError("gradient destinations need a rank that is a multiple of 8")
        destinations = [gradient_destinations[name] for name in ("a13", "b13", "a2", "b2")]
        spans = []
        for name, buffer in zip(("a13", "b13", "a2", "b2"), destinations):
            if tuple(buffer.shape) != expected[name] or not buffer.is_contiguous() or \
                    buffer.dtype not in (torch.bfloat16, torch.float32) or buffer.device != hidden.device:
                raise ValueError(f"destination {name}: a contiguous bf16 or fp32 {expected[name]} tensor on the "
                                 "layer's device is needed")
            first = buffer.data_ptr()
            last = first + buffer.numel() * buffer.element_size()
            if any(first < stop and start < last for start, stop in spans):
                raise ValueError("gradient destinations must not overlap")
            spans.append((first, last))
        if not math.isfinite(float(gradient_scale)):
            raise ValueError("gradient_scale must be finite")
    for weight in (gate_up, down):
        if type(weight) not in provider._DISPATCH_REGISTERED:
            provider.register_container(type(weight))
    rows = hidden.numel() // hidden.shape[-1]
    normalized = [rows] if lengths is None else [int(v) for v in lengths]
    bias = router_bias if router_bias is not None else torch.empty(0, dtype=torch.float32, device=hidden.device)
    outputs = moe_lora_fwd(hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, bias, int(top_k),
                           str(routing_mode), float(scale), int(n_group), int(topk_group), float(routed_scaling),
                           normalized, swiglu_limit, destinations, float(gradient_scale), [])
    return outputs[:4]
