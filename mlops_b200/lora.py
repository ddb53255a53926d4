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
"""

from __future__ import annotations

import torch

from . import layer, ops
from .weights import components


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


class _ExpertLoRA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, router_bias, options):
        w13, w2 = components(gate_up), components(down)
        experts = w13[0].shape[0]
        top_k, scale, limit = options["top_k"], options["scale"], options["swiglu_limit"]
        flat = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        residual_flat = residual.reshape_as(flat).contiguous()
        a13p, rank = _pad_rank(a13.detach(), 1)
        b13p, _ = _pad_rank(b13.detach(), 2)
        a2p, _ = _pad_rank(a2.detach(), 1)
        b2p, _ = _pad_rank(b2.detach(), 2)
        # the B factors are also kept rank-major ([E, r, wide]): every rank-r kernel then stages
        # its factor with 16-byte loads (a few MB, transposed once per call)
        b13t = b13p.transpose(1, 2).contiguous()
        b2t = b2p.transpose(1, 2).contiguous()
        logits = layer.router_logits(flat, router_weight)
        weights, ids = ops.route_topk(
            logits, top_k, options["routing_mode"], bias=router_bias, n_group=options["n_group"],
            topk_group=options["topk_group"], routed_scaling=options["routed_scaling"],
        )
        order, offsets, slots, counts = ops.sort_assignments(ids, experts)
        x_rows = ops.dispatch(flat, order, top_k)
        x_q, x_s = ops.quantize_rows(x_rows)
        t1 = ops.lora_project(x_rows, a13p, offsets, rank_major=True)
        c1 = ops.lora_expand(t1, b13t, offsets, wide_major=False, scale=scale)
        h13 = ops.grouped_gemm_fp8(x_q, x_s, *w13, offsets, addend=c1)
        a_q, a_s, act = ops.swiglu_quantize(h13, limit=limit, quantized=True, rounded=True)
        t2 = ops.lora_project(act, a2p, offsets, rank_major=True)
        c2 = ops.lora_expand(t2, b2t, offsets, wide_major=False, scale=scale)
        y = ops.grouped_gemm_fp8(a_q, a_s, *w2, offsets, addend=c2)
        output = ops.combine(y, slots, weights, residual_flat).reshape(hidden.shape)
        aux, counts, probability_sum = layer.routing_statistics(
            logits, ids, counts, routing_mode=options["routing_mode"], lengths=options["lengths"], experts=experts)
        ctx.save_for_backward(flat, router_weight, *w13, *w2, a13p, b13t, a2p, b2t, logits, weights, ids, order,
                              offsets, slots, h13, t1, t2)
        ctx.options, ctx.rank, ctx.shape = options, rank, hidden.shape
        ctx.logical = (gate_up.dtype, down.dtype)
        ctx.mark_non_differentiable(counts)
        return output, aux, counts, probability_sum

    @staticmethod
    def backward(ctx, grad_output, grad_aux, _grad_counts, grad_probability_sum):
        (flat, router_weight, w13_d, w13_s, w2_d, w2_s, a13, b13, a2, b2, logits, weights, ids, order, offsets,
         slots, h13, t1, t2) = ctx.saved_tensors
        options, rank = ctx.options, ctx.rank
        need = ctx.needs_input_grad
        top_k, scale, limit = options["top_k"], options["scale"], options["swiglu_limit"]
        experts = w13_d.shape[0]
        if grad_output is None:
            grad_output = torch.zeros(ctx.shape, dtype=flat.dtype, device=flat.device)
        dy = grad_output.reshape_as(flat).contiguous()
        counts = (offsets[1:] - offsets[:-1]).long()
        need_factors = any(need[5:9])

        dy_rows = ops.dispatch(dy, order, top_k)
        dy_q, dy_s = ops.quantize_rows(dy_rows)
        t2g = ops.lora_project(dy_rows, b2, offsets, rank_major=True)           # dy B2      [R, r]
        r_add = ops.lora_expand(t2g, a2, offsets, wide_major=False, scale=scale)  # s dy B2 A2 [R, F]
        r = ops.grouped_gemm_fp8(dy_q, dy_s, w2_d, w2_s, offsets, b_mn_major=True, addend=r_add)
        dscore, gh_q, gh_s, gh_b, act_scaled = ops.dswiglu_routed(
            h13, r, weights, order, limit=limit, quantized=True, rounded=True, scaled_activation=True)
        grad_route_weights = ops.gather_scalar(dscore, slots)

        x_rows = ops.dispatch(flat, order, top_k)
        dt1 = ops.lora_project(gh_b, b13, offsets, rank_major=True)             # gh B13     [R, r]
        grad_a13 = grad_b13 = grad_a2 = grad_b2 = None
        if need_factors:
            row_weight = weights.reshape(-1)[order.long()].float()[:, None]
            fdtype = a13.dtype
            grad_b2 = ops.grouped_wgrad(dy_rows, (t2.float() * (row_weight * scale)).to(t2.dtype), offsets,
                                        experts, fdtype)[:, :, :rank]
            grad_a2 = ops.grouped_wgrad((t2g.float() * scale).to(t2g.dtype), act_scaled, offsets, experts,
                                        fdtype)[:, :rank]
            grad_b13 = ops.grouped_wgrad(gh_b, (t1.float() * scale).to(t1.dtype), offsets, experts,
                                         fdtype)[:, :, :rank]
            grad_a13 = ops.grouped_wgrad((dt1.float() * scale).to(dt1.dtype), x_rows, offsets, experts,
                                         fdtype)[:, :rank]
        dx_add = ops.lora_expand(dt1, a13, offsets, wide_major=False, scale=scale)
        grad_rows = ops.grouped_gemm_fp8(gh_q, gh_s, w13_d, w13_s, offsets, b_mn_major=True, addend=dx_add)
        grad_h2 = ops.dispatch_backward(grad_rows, slots)

        grad_w13 = grad_w2 = None
        if need[3]:  # a trainable base gets its gradient as in the plain layer
            grad_w13 = ops.grouped_wgrad(gh_b, x_rows, offsets, experts, ctx.logical[0])
        if need[4]:
            grad_w2 = ops.grouped_wgrad(dy_rows, act_scaled, offsets, experts, ctx.logical[1])

        grad_logits = layer.routing_gradient(
            grad_aux, grad_probability_sum, grad_route_weights, weights, ids, logits, counts,
            routing_mode=options["routing_mode"], lengths=options["lengths"])
        grad_router = None
        if need[2]:
            grad_router = layer._router_weight_gradient(grad_logits, flat, router_weight.dtype)
        grad_h2.addmm_(grad_logits.to(flat.dtype), getattr(router_weight, "_data", router_weight).to(flat.dtype))
        contig = lambda t: None if t is None else t.contiguous()  # noqa: E731
        return (grad_h2.reshape(ctx.shape) if need[0] else None, grad_output.clone() if need[1] else None,
                grad_router, grad_w13, grad_w2, contig(grad_a13) if need[5] else None,
                contig(grad_b13) if need[6] else None, contig(grad_a2) if need[7] else None,
                contig(grad_b2) if need[8] else None, None, None)


def expert_lora(hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, *, top_k, routing_mode, scale,
                router_bias=None, n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, swiglu_limit=None,
                implementation="b200", compute_precision=None):
    """Returns `(output, aux, counts, probability_sum)`, differentiable in `hidden`, `residual`,
    `router_weight`, the four factors and (when they ask for it) the base containers."""
    if implementation not in ("auto", "b200"):
        raise ValueError(f"mlops_b200.expert_lora serves implementation 'b200' (or 'auto'), not {implementation!r}")
    if compute_precision not in (None, "fp8_block"):
        raise ValueError("mlops_b200.expert_lora computes the base in block FP8 only")
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
    rows = hidden.numel() // hidden.shape[-1]
    options = dict(
        top_k=int(top_k), routing_mode=str(routing_mode), scale=float(scale), n_group=int(n_group),
        topk_group=int(topk_group), routed_scaling=float(routed_scaling), swiglu_limit=swiglu_limit,
        lengths=(rows,) if lengths is None else tuple(int(v) for v in lengths),
    )
    bias = None if router_bias is None or router_bias.numel() == 0 else router_bias
    return _ExpertLoRA.apply(hidden, residual, router_weight, gate_up, down, a13, b13, a2, b2, bias, options)
