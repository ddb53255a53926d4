"""The routed MoE layer on block-FP8 experts: stateless forward and VJP.

`forward_routed` / `backward_routed` mirror the reference's shared mechanics
(`src/mlops/providers/moe_common.py:174-378`): same argument meaning, same ordered
results and the same residual tuple `(logits, route_weights, route_ids, order, offsets,
slots, h13)` with `h13` holding gate columns then up columns, so the explicit VJP surface
(`src/mlops/explicit/moe.py:12-119`) can be served from here. What differs is below that
boundary: the expert products are E4M3 x E4M3 on tcgen05 with 128x128 weight-block and
1x128 activation-block scales, the gather is fused into the quantiser, SwiGLU into the
activation quantiser, and the route-weight gradient, the SwiGLU backward and the
quantisation of the pre-activation gradient are one pass.

Every step is an asynchronous launch on the current CUDA stream; nothing here reads
device memory on the host.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch

from . import ops

BLOCK_N_DEFAULT = 256


# ------------------------------------------------------------------------- router GEMM
def router_logits(hidden, router_weight):
    """fp32 logits `[rows, E]`: operands at the activation's dtype, fp32 sums and output
    (reference: src/mlops/kernels/router.py:53-64). A plain library GEMM."""
    weight = getattr(router_weight, "_data", router_weight)
    return torch.mm(hidden, weight.to(hidden.dtype).t(), out_dtype=torch.float32)


def _router_weight_gradient(grad_logits, hidden, dtype):
    """`grad_logits.T @ hidden` with the cotangent carried as two bf16 pieces so an fp32
    master keeps an fp32-quality gradient (reference: src/mlops/kernels/router.py:92-110)."""
    high = grad_logits.to(hidden.dtype)
    gradient = torch.mm(high.t(), hidden, out_dtype=torch.float32)
    residue = (grad_logits.float() - high.float()).to(hidden.dtype)
    gradient.add_(torch.mm(residue.t(), hidden, out_dtype=torch.float32))
    return gradient.to(dtype)


# ---------------------------------------------------------------- routing statistics
def routing_statistics(logits, route_ids, counts, *, routing_mode, lengths, experts):
    """`(aux, counts, probability_sum)` of one routing decision (reference:
    src/mlops/providers/moe_common.py:32-71). `counts` is the int64 histogram the sort kernel
    already produced. The pass over the `[T, E]` logits is one kernel (column sums of the
    probabilities, formed in a fixed order); what is left is `[E]`-sized arithmetic."""
    rows = logits.shape[0]
    if routing_mode == "sigmoid_noaux_tc":
        aux = torch.zeros((), dtype=torch.float32, device=logits.device)
        probability_sum = None
        start = 0
        for length in lengths:  # the auxiliary loss of this mode is per sequence
            stop = start + int(length)
            segment_sum = ops.routing_probability_sum(logits[start:stop], routing_mode)
            if len(lengths) == 1:
                segment_counts = counts
            else:
                segment_counts = torch.bincount(route_ids[start:stop].reshape(-1).long(), minlength=experts)
            frequency = segment_counts.float() * experts / (route_ids.shape[1] * int(length))
            aux = aux + (frequency * (segment_sum / int(length))).sum()
            probability_sum = segment_sum if probability_sum is None else probability_sum + segment_sum
            start = stop
    else:
        probability_sum = ops.routing_probability_sum(logits, routing_mode)
        frequency = counts.float() / route_ids.numel()
        aux = experts * (frequency * (probability_sum / rows)).sum()
    return aux, counts, probability_sum


def routing_gradient(grad_aux, grad_probability_sum, grad_route_weights, route_weights, route_ids,
                     logits, counts, *, routing_mode, lengths):
    """fp32 gradient of the logits from the cotangents of the route weights, the auxiliary
    loss and the probability sum (reference: src/mlops/providers/moe_common.py:74-124,
    src/mlops/kernels/moe_router.py:403-502): one kernel per sequence for the sigmoid mode's
    per-sequence auxiliary loss, one kernel otherwise."""
    tokens, experts = logits.shape
    if routing_mode != "sigmoid_noaux_tc" or grad_aux is None or len(lengths) == 1:
        frequency, aux_scale = None, 0.0
        if grad_aux is not None:
            if routing_mode == "sigmoid_noaux_tc":
                frequency = counts.float() * experts / (route_ids.shape[1] * tokens)
                aux_scale = 1.0 / tokens
            else:
                frequency = counts.float() / route_ids.numel()
                aux_scale = experts / tokens
        return ops.routing_gradient(logits, route_ids, route_weights, grad_route_weights, routing_mode,
                                    grad_aux=grad_aux, frequency=frequency, aux_scale=aux_scale,
                                    grad_probability_sum=grad_probability_sum)
    grad_logits = torch.empty((tokens, experts), dtype=torch.float32, device=logits.device)
    start = 0
    for length in lengths:
        stop = start + int(length)
        segment = torch.bincount(route_ids[start:stop].reshape(-1).long(), minlength=experts).float()
        frequency = segment * experts / (route_ids.shape[1] * int(length))
        ops.routing_gradient(logits[start:stop], route_ids[start:stop], route_weights[start:stop],
                             grad_route_weights[start:stop], routing_mode, grad_aux=grad_aux, frequency=frequency,
                             aux_scale=1.0 / int(length), grad_probability_sum=grad_probability_sum,
                             out=grad_logits[start:stop])
        start = stop
    return grad_logits


# ------------------------------------------------------------------------------ forward
def _normalized_lengths(lengths, rows):
    normalized = (rows,) if lengths is None else tuple(int(v) for v in lengths)
    if not normalized or any(v <= 0 for v in normalized) or sum(normalized) != rows:
        raise ValueError("MoE lengths must be positive and cover every hidden row")
    return normalized


def forward_routed(
    h2: torch.Tensor,
    residual: torch.Tensor,
    router_weight: torch.Tensor,
    w13: tuple[torch.Tensor, torch.Tensor],
    w2: tuple[torch.Tensor, torch.Tensor],
    *,
    top_k: int,
    routing_mode: str,
    router_bias: torch.Tensor | None = None,
    n_group: int = 1,
    topk_group: int = 1,
    routed_scaling: float = 1.0,
    lengths: Sequence[int] | None = None,
    swiglu_limit: float | None = None,
    block_n: int = BLOCK_N_DEFAULT,
    route: tuple[torch.Tensor, torch.Tensor] | None = None,
    fuse_swiglu: bool = False,
    fuse_combine: bool = False,
) -> tuple[torch.Tensor, ...]:
    """Returns `(output, aux, counts, probability_sum, logits, route_weights, route_ids,
    order, offsets, slots, h13)`.

    `w13 = (data E4M3 [E, 2F, D], scale fp32 [E, 2F/128, D/128])` with gate rows then up
    rows, `w2 = (data [E, D, F], scale)`: the components of a block-FP8 weight container. Plain
    bf16 tensors `w13 [E, 2F, D]`, `w2 [E, D, F]` select the bf16 compute path instead (bf16
    grouped GEMMs with fp32 sums, no quantisation anywhere).
    `route = (route_weights, route_ids)` bypasses the selection (the logits and the
    statistics are still computed). `fuse_swiglu` runs SwiGLU and the activation quantiser in
    the up GEMM's epilogue (bit-identical results; measured 7% slower than the two-kernel form
    at DeepSeek-V3 shapes because the longer tile epilogue stalls the MMA pipeline, hence off
    by default). `fuse_combine` forms the route-weighted sum in the down GEMM's store with fp32
    atomics instead of writing expert-order rows for `combine`: not bitwise repeatable, and
    slower for top-8 routing (a token row is read-modify-written eight times in HBM), so it is
    off by default as well."""
    bf16_weights = isinstance(w13, torch.Tensor)
    if bf16_weights:
        _check_bf16_weights(w13, w2)
        w13_data, w2_data = w13, w2
        w13_scale = w2_scale = None
    else:
        w13_data, w13_scale = w13
        w2_data, w2_scale = w2
    experts = w13_data.shape[0]
    with torch.no_grad():
        original_shape = h2.shape
        h2_flat = h2.reshape(-1, h2.shape[-1]).contiguous()
        residual_flat = residual.reshape_as(h2_flat).contiguous()
        normalized = _normalized_lengths(lengths, h2_flat.shape[0])
        logits = router_logits(h2_flat, router_weight)
        if route is None:
            bias = None if router_bias is None or router_bias.numel() == 0 else router_bias
            route_weights, route_ids = ops.route_topk(
                logits, int(top_k), str(routing_mode), bias=bias, n_group=int(n_group),
                topk_group=int(topk_group), routed_scaling=float(routed_scaling),
            )
        else:
            route_weights, route_ids = route
            route_weights = route_weights.float().contiguous()
            route_ids = route_ids.to(torch.int32).contiguous()
        order, offsets, slots, counts = ops.sort_assignments(route_ids, experts)
        if route is not None:
            # the sort reported ids outside [0, experts) and placed them on the nearest expert;
            # the residual handed to the statistics and to the backward pass says the same
            route_ids = route_ids.clamp(0, experts - 1)
        if bf16_weights:
            # the bf16 compute path (reference: src/mlops/kernels/moe_grouped_gemm.py:201-299 around
            # the builtin's dispatch / SwiGLU / combine): nothing is quantised
            x_rows = ops.dispatch(h2_flat, order, int(top_k))
            h13 = ops.grouped_gemm_bf16(x_rows, w13_data, offsets)
            del x_rows
            _q, _s, act = ops.swiglu_quantize(h13, limit=swiglu_limit, quantized=False, rounded=True)
            expert_output = ops.grouped_gemm_bf16(act, w2_data, offsets)
            output = ops.combine(expert_output, slots, route_weights, residual_flat).reshape(original_shape)
            aux, counts, probability_sum = routing_statistics(
                logits, route_ids, counts, routing_mode=str(routing_mode), lengths=normalized, experts=experts
            )
            return (output, aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets, slots,
                    h13)
        # every token quantised once, its E4M3 row written to each of its K expert-ordered rows
        x_q, x_s = ops.quantize_rows_scatter(h2_flat, slots)
        if fuse_swiglu and w2_data.shape[2] % 128 == 0:
            h13, a_q, a_s = ops.grouped_gemm_fp8_swiglu(x_q, x_s, w13_data, w13_scale, offsets, limit=swiglu_limit)
        else:
            h13 = ops.grouped_gemm_fp8(x_q, x_s, w13_data, w13_scale, offsets, block_n=block_n)
            a_q, a_s, _ = ops.swiglu_quantize(h13, limit=swiglu_limit)
        if fuse_combine:
            output = ops.grouped_gemm_fp8_combine(
                a_q, a_s, w2_data, w2_scale, offsets, order, route_weights, h2_flat.shape[0],
                residual=residual_flat).reshape(original_shape)
        else:
            expert_output = ops.grouped_gemm_fp8(a_q, a_s, w2_data, w2_scale, offsets, block_n=block_n)
            output = ops.combine(expert_output, slots, route_weights, residual_flat).reshape(original_shape)
        aux, counts, probability_sum = routing_statistics(
            logits, route_ids, counts, routing_mode=str(routing_mode), lengths=normalized, experts=experts
        )
    return (output, aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets, slots, h13)


def _check_bf16_weights(w13, w2):
    if not isinstance(w2, torch.Tensor) or w13.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
        raise ValueError("the bf16 compute path takes both expert weights as plain bf16 tensors")
    if w13.dim() != 3 or w2.dim() != 3 or w13.shape[0] != w2.shape[0] or w13.shape[1] != 2 * w2.shape[2] \
            or w13.shape[2] != w2.shape[1]:
        raise ValueError("expected w13 [E, 2F, D] and w2 [E, D, F]")
    if w13.shape[2] % 8 or w2.shape[2] % 8:
        raise ValueError("the bf16 grouped GEMM needs D and F to be multiples of 8")


# ----------------------------------------------------------------------------- backward
def _weight_gradient(g_rows, x_rows, offsets, experts, dtype, operands):
    """`out[e] = g_rows[rows_e].T @ x_rows[rows_e]` from bf16 operands, or from their column-scaled
    E4M3 forms."""
    if operands == "bf16":
        return ops.grouped_wgrad(g_rows, x_rows, offsets, experts, dtype)
    g_q, g_s = ops.quantize_columns(g_rows, offsets, experts)
    x_q, x_s = ops.quantize_columns(x_rows, offsets, experts)
    return ops.grouped_wgrad_fp8(g_q, g_s, x_q, x_s, offsets, experts, dtype)


def backward_routed(
    grad_output: torch.Tensor,
    grad_aux: torch.Tensor | None,
    grad_probability_sum: torch.Tensor | None,
    h2: torch.Tensor,
    router_weight: torch.Tensor,
    w13: tuple[torch.Tensor, torch.Tensor],
    w2: tuple[torch.Tensor, torch.Tensor],
    logits: torch.Tensor,
    route_weights: torch.Tensor,
    route_ids: torch.Tensor,
    order: torch.Tensor,
    offsets: torch.Tensor,
    slots: torch.Tensor,
    h13: torch.Tensor,
    *,
    top_k: int,
    routing_mode: str,
    lengths: Sequence[int] | None = None,
    weight_grad_dtype: torch.dtype | None = None,
    swiglu_limit: float | None = None,
    need_router: bool = True,
    need_w13: bool = True,
    need_w2: bool = True,
    router_grad_dtype: torch.dtype | None = None,
    block_n: int = BLOCK_N_DEFAULT,
    weight_grad_operands: str = "bf16",
) -> tuple[torch.Tensor, ...]:
    """VJPs for `h2, residual, router_weight, w13, w2` in order. A gradient nobody asked
    for (`need_* = False`) is an empty placeholder and its GEMM is not launched
    (reference: src/mlops/providers/moe_common.py:127-139, 269-378). Input gradients are
    E4M3 products against the stored weights read along their rows; weight gradients are
    bf16-operand products with fp32 sums, written at `weight_grad_dtype` (bf16 when None).
    `weight_grad_operands="fp8"` selects the reference's optional FP8 weight-gradient recipe
    instead (src/mlops/kernels/quack_moe/wgrad.py:30-69): both operands of each product are
    quantised to E4M3 with one scale per expert and column and multiplied at the FP8 rate."""
    if weight_grad_operands not in ("bf16", "fp8"):
        raise ValueError("weight_grad_operands is 'bf16' or 'fp8'")
    bf16_weights = isinstance(w13, torch.Tensor)
    if bf16_weights:
        _check_bf16_weights(w13, w2)
        w13_data, w2_data = w13.contiguous(), w2.contiguous()
        w13_scale = w2_scale = None
    else:
        w13_data, w13_scale = w13
        w2_data, w2_scale = w2
    experts = w13_data.shape[0]
    wdtype = torch.bfloat16 if weight_grad_dtype is None else weight_grad_dtype
    with torch.no_grad():
        original_shape = h2.shape
        h2_flat = h2.reshape(-1, h2.shape[-1]).contiguous()
        grad_flat = grad_output.reshape_as(h2_flat).contiguous()
        normalized = _normalized_lengths(lengths, h2_flat.shape[0])
        counts = (offsets[1:] - offsets[:-1]).long()

        if bf16_weights:
            dy_rows = ops.dispatch(grad_flat, order, int(top_k))
            r = ops.grouped_gemm_bf16(dy_rows, w2_data, offsets, b_mn_major=True)
            dscore, _gq, _gs, gh_b, act_scaled = ops.dswiglu_routed(
                h13, r, route_weights, order, limit=swiglu_limit, quantized=False, rounded=True,
                scaled_activation=need_w2,
            )
            del r
            grad_route_weights = ops.gather_scalar(dscore, slots)
            if need_w2:
                grad_w2 = _weight_gradient(dy_rows, act_scaled, offsets, experts, wdtype, weight_grad_operands)
                del act_scaled
            else:
                grad_w2 = torch.empty(0, dtype=wdtype, device=h2.device)
            del dy_rows
            if need_w13:
                x_rows = ops.dispatch(h2_flat, order, int(top_k))
                grad_w13 = _weight_gradient(gh_b, x_rows, offsets, experts, wdtype, weight_grad_operands)
                del x_rows
            else:
                grad_w13 = torch.empty(0, dtype=wdtype, device=h2.device)
            grad_rows = ops.grouped_gemm_bf16(gh_b, w13_data, offsets, b_mn_major=True)
            del gh_b
            grad_h2 = ops.dispatch_backward(grad_rows, slots)
            return _finish_backward(grad_h2, grad_output, grad_aux, grad_probability_sum, grad_route_weights,
                                    route_weights, route_ids, logits, counts, routing_mode, normalized,
                                    router_weight, h2_flat, need_router, router_grad_dtype, original_shape,
                                    grad_w13, grad_w2)
        # one pass over dy: E4M3 rows for the input gradient and, when the down weight's gradient
        # is wanted, the same rows in bf16 as its operand
        if need_w2:
            dy_q, dy_s, dy_rows = ops.quantize_rows_scatter(grad_flat, slots, with_copy=True)
        else:
            dy_q, dy_s = ops.quantize_rows_scatter(grad_flat, slots)
        r = ops.grouped_gemm_fp8(dy_q, dy_s, w2_data, w2_scale, offsets, b_mn_major=True, block_n=block_n)
        dscore, gh_q, gh_s, gh_b, act_scaled = ops.dswiglu_routed(
            h13, r, route_weights, order, limit=swiglu_limit, quantized=True, rounded=need_w13,
            scaled_activation=need_w2,
        )
        grad_route_weights = ops.gather_scalar(dscore, slots)
        if need_w2:
            grad_w2 = _weight_gradient(dy_rows, act_scaled, offsets, experts, wdtype, weight_grad_operands)
            del dy_rows, act_scaled
        else:
            grad_w2 = torch.empty(0, dtype=wdtype, device=h2.device)
        if need_w13:
            x_rows = ops.dispatch(h2_flat, order, int(top_k))
            grad_w13 = _weight_gradient(gh_b, x_rows, offsets, experts, wdtype, weight_grad_operands)
            del x_rows, gh_b
        else:
            grad_w13 = torch.empty(0, dtype=wdtype, device=h2.device)
        grad_rows = ops.grouped_gemm_fp8(gh_q, gh_s, w13_data, w13_scale, offsets, b_mn_major=True,
                                         block_n=block_n)
        grad_h2 = ops.dispatch_backward(grad_rows, slots)
        return _finish_backward(grad_h2, grad_output, grad_aux, grad_probability_sum, grad_route_weights,
                                route_weights, route_ids, logits, counts, routing_mode, normalized, router_weight,
                                h2_flat, need_router, router_grad_dtype, original_shape, grad_w13, grad_w2)


def _finish_backward(grad_h2, grad_output, grad_aux, grad_probability_sum, grad_route_weights, route_weights,
                     route_ids, logits, counts, routing_mode, normalized, router_weight, h2_flat, need_router,
                     router_grad_dtype, original_shape, grad_w13, grad_w2):
    """The router's share of the backward pass: the routing VJP, the router weight's gradient and
    the router's contribution to the input gradient."""
    with torch.no_grad():
        grad_logits = routing_gradient(
            grad_aux, grad_probability_sum, grad_route_weights, route_weights, route_ids, logits, counts,
            routing_mode=str(routing_mode), lengths=normalized,
        )
        router_operand = getattr(router_weight, "_data", router_weight)
        if need_router:
            rdtype = router_weight.dtype if router_grad_dtype is None else router_grad_dtype
            grad_router = _router_weight_gradient(grad_logits, h2_flat, rdtype)
        else:
            grad_router = torch.empty(0, dtype=router_weight.dtype, device=h2_flat.device)
        grad_h2.addmm_(grad_logits.to(h2_flat.dtype), router_operand.to(h2_flat.dtype))
    return (grad_h2.reshape(original_shape), grad_output.clone(), grad_router, grad_w13, grad_w2)


# ------------------------------------------------------------------------ shared expert
def shared_expert_forward(h2_flat, shared_w13, shared_w2, *, swiglu_limit=None):
    """The always-on shared expert: `W2s . swiglu(W13s . x)` with bf16 dense library GEMMs
    (the reference never quantises it: src/mlops/moe.py:12-37, docs/EXPERT_PARALLEL.md) and
    this library's SwiGLU kernel in between. Returns `(y [T, D], h13 [T, 2Fs])`; h13 is the
    residual its backward needs."""
    with torch.no_grad():
        h13 = h2_flat @ shared_w13.t()
        _, _, act = ops.swiglu_quantize(h13, limit=swiglu_limit, quantized=False, rounded=True)
        return act @ shared_w2.t(), h13


def shared_expert_backward(grad_y, h2_flat, shared_w13, shared_w2, h13, *, swiglu_limit=None,
                           need_weights=True):
    """VJP of `shared_expert_forward`: `(grad_h2, grad_w13, grad_w2)` (weights' entries are
    None when not needed)."""
    with torch.no_grad():
        rows = h2_flat.shape[0]
        r = grad_y @ shared_w2
        ones = torch.ones(rows, dtype=torch.float32, device=h2_flat.device)
        identity = torch.arange(rows, dtype=torch.int32, device=h2_flat.device)
        _, _, _, grad_h13, act = ops.dswiglu_routed(
            h13, r, ones, identity, limit=swiglu_limit, quantized=False, rounded=True,
            scaled_activation=need_weights,
        )
        grad_h2 = grad_h13 @ shared_w13
        if not need_weights:
            return grad_h2, None, None
        return grad_h2, grad_h13.t() @ h2_flat, grad_y.t() @ act
