"""CPU restatement of the reference's routed-MoE expert path (als244/mlops).

TEST INFRASTRUCTURE ONLY. Nothing in the `mlops_b200` package imports this module; it
is called by `tests/`, by `__graft_entry__.smoke()` as the checker and by `bench.py`'s
CPU-baseline leg. It is plain PyTorch on CPU tensors and follows the reference function
by function (citations are paths inside the reference project).

Pinned against the reference itself: `tests/golden/make_golden.py` imports the reference
(`src/mlops`) in the build container, runs its `route`, `sort_assignments`,
`quantize_blocks`, `quantize_rows_fp8_reference`, `native_torch.moe` and the
expert-parallel reference on seeded inputs and stores the results as fixtures;
`tests/test_oracle_golden.py` checks every function below against those fixtures.
The 1x128 activation-scale quantiser has no counterpart in the reference's
registry-dispatched path (its in-tree recipe is one scale per row): for that mode the
*quantiser* parity is unpinned; the GEMM on given operands is pinned by the
float64-of-dequantised-operands method the reference's own tests use
(tests/test_block_fp8_transpose_gemm.py:447-459).
"""

from __future__ import annotations

import torch

BLOCK = 128
E4M3_MAX = 448.0
FP8 = torch.float8_e4m3fn


# --------------------------------------------------------------------------- routing
def route(logits, top_k, mode, *, bias=None, n_group=1, topk_group=1, routed_scaling=1.0):
    """(weights fp32 [T,K], ids int32 [T,K]).

    Follows src/mlops/kernels/moe_router.py:290-344 (`route`, CPU branch) and its twin
    `route_torch` :347-400: stable descending sorts, so ties go to the lowest index."""
    logits = logits.float()
    tokens, experts = logits.shape
    if mode == "sigmoid_noaux_tc":
        scores = torch.sigmoid(logits)
        selection = scores + (0.0 if bias is None else bias.float())
        if int(topk_group) >= int(n_group):
            masked = selection
        else:
            grouped = selection.view(tokens, int(n_group), experts // int(n_group))
            grouped, _ = torch.sort(grouped, dim=-1, descending=True, stable=True)
            group_scores = grouped[..., : min(2, grouped.shape[-1])].sum(-1)
            _, group_ids = torch.sort(group_scores, dim=-1, descending=True, stable=True)
            group_mask = torch.zeros(tokens, int(n_group), dtype=torch.bool)
            group_mask.scatter_(1, group_ids[:, : int(topk_group)], True)
            expert_mask = group_mask.repeat_interleave(experts // int(n_group), dim=1)
            masked = selection.masked_fill(~expert_mask, float("-inf"))
        _, selected = torch.sort(masked, dim=-1, descending=True, stable=True)
        selected = selected[:, : int(top_k)]
        picked = scores.gather(1, selected)
        weights = picked / picked.sum(-1, keepdim=True) * float(routed_scaling)
        return weights, selected.to(torch.int32)
    if mode not in ("softmax_then_topk", "topk_then_softmax"):
        raise ValueError(f"unsupported routing mode {mode!r}")
    values = torch.softmax(logits, -1) if mode == "softmax_then_topk" else logits
    values, indices = torch.sort(values, dim=-1, descending=True, stable=True)
    selected = values[:, :top_k]
    if mode == "topk_then_softmax":
        selected = torch.softmax(selected, -1)
    return selected.contiguous(), indices[:, :top_k].to(torch.int32)


def sort_assignments(route_ids, experts):
    """(order int32 [R], offsets int32 [E+1], slots int32 like route_ids).
    Follows src/mlops/kernels/moe_dispatch.py:106-119."""
    flat = route_ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True).to(torch.int32)
    counts = torch.bincount(flat, minlength=experts)
    offsets = torch.zeros(experts + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0).to(torch.int32)
    slots = torch.empty_like(flat, dtype=torch.int32)
    slots[order.long()] = torch.arange(flat.numel(), dtype=torch.int32)
    return order, offsets, slots.view_as(route_ids)


def routing_statistics(logits, route_ids, *, routing_mode, lengths, experts):
    """(aux, counts int64 [E], probability_sum fp32 [E]).
    Follows src/mlops/providers/moe_common.py:32-71."""
    rows = logits.shape[0]
    if routing_mode == "sigmoid_noaux_tc":
        scores = torch.sigmoid(logits.float())
        probabilities = scores / scores.sum(-1, keepdim=True)
    else:
        probabilities = torch.softmax(logits.float(), dim=-1)
    probability_sum = probabilities.sum(0)
    counts = torch.bincount(route_ids.reshape(-1).long(), minlength=experts)
    if routing_mode == "sigmoid_noaux_tc":
        aux = torch.zeros((), dtype=torch.float32)
        start = 0
        for length in lengths:
            stop = start + int(length)
            seg = torch.bincount(route_ids[start:stop].reshape(-1).long(), minlength=experts)
            frequency = seg.float() * experts / (route_ids.shape[1] * int(length))
            aux = aux + (frequency * probabilities[start:stop].mean(0)).sum()
            start = stop
    else:
        frequency = counts.float() / route_ids.numel()
        aux = experts * (frequency * (probability_sum / rows)).sum()
    return aux, counts, probability_sum


def _probabilities(logits, routing_mode):
    if routing_mode == "sigmoid_noaux_tc":
        scores = torch.sigmoid(logits.float())
        return scores, scores / scores.sum(-1, keepdim=True)
    return None, torch.softmax(logits.float(), dim=-1)


def routing_gradient(grad_aux, grad_probability_sum, grad_route_weights, route_weights, route_ids,
                     logits, counts, *, routing_mode, lengths):
    """fp32 gradient of the logits from the cotangents of the route weights, the auxiliary
    loss and the probability sum. Follows src/mlops/providers/moe_common.py:74-124 and
    src/mlops/kernels/moe_router.py:403-502 (`route_backward`, `add_aux_gradient_`,
    `add_sequence_aux_gradient_`); pinned against the reference's `routing_gradient` fixture.
    `counts` is the int64 histogram of `route_ids` over the experts."""
    tokens, experts = logits.shape
    selected = route_ids.long()
    grad_w = grad_route_weights.float()
    scores, probabilities = _probabilities(logits, routing_mode)
    grad_logits = torch.zeros_like(logits, dtype=torch.float32)
    if routing_mode == "sigmoid_noaux_tc":
        weights = route_weights.float()
        picked = scores.gather(1, selected)
        picked_sum = picked.sum(-1, keepdim=True)
        scaling = weights.sum(-1, keepdim=True)
        dot = (grad_w * weights).sum(-1, keepdim=True)
        grad_logits.scatter_(1, selected, ((scaling * grad_w - dot) / picked_sum) * picked * (1.0 - picked))
    elif routing_mode == "topk_then_softmax":
        weights = route_weights.float()
        grad_logits.scatter_(1, selected, weights * (grad_w - (grad_w * weights).sum(-1, keepdim=True)))
    else:
        top = probabilities.gather(1, selected)
        dot = (grad_w * top).sum(-1, keepdim=True)
        grad_logits.copy_(-probabilities * dot)
        grad_logits.scatter_add_(1, selected, grad_w * top)

    if grad_aux is not None:
        if routing_mode == "sigmoid_noaux_tc":
            row_sum = scores.sum(-1, keepdim=True)
            start = 0
            for length in lengths:
                stop = start + int(length)
                if len(lengths) == 1:
                    segment = counts.float()
                else:
                    segment = torch.bincount(
                        route_ids[start:stop].reshape(-1).long(), minlength=experts
                    ).float()
                frequency = segment * experts / (route_ids.shape[1] * int(length))
                coefficient = grad_aux.float() / (int(length) * row_sum[start:stop])
                part = probabilities[start:stop]
                score_gradient = coefficient * (frequency.unsqueeze(0) - (part @ frequency).unsqueeze(1))
                grad_logits[start:stop].add_(score_gradient * scores[start:stop] * (1.0 - scores[start:stop]))
                start = stop
        else:
            frequency = counts.float() / route_ids.numel()
            coefficient = grad_aux.float() * experts / tokens
            grad_logits.add_(
                coefficient * probabilities * (frequency.unsqueeze(0) - (probabilities @ frequency).unsqueeze(1))
            )

    if grad_probability_sum is not None:
        jacobian_scale = probabilities if scores is None else (1.0 - scores) * probabilities
        grad_sum = grad_probability_sum.float()
        grad_logits.add_(jacobian_scale * (grad_sum.unsqueeze(0) - (probabilities @ grad_sum).unsqueeze(1)))
    return grad_logits


# ---------------------------------------------------------------------- quantisation
def _blocks(width):
    return -(-width // BLOCK)


def _expanded(scale, out, inner):
    return scale.repeat_interleave(BLOCK, 1).repeat_interleave(BLOCK, 2)[:, :out, :inner]


def quantize_blocks(weight):
    """(data E4M3, scale fp32 [E, ceil(out/128), ceil(in/128)]): scale = max(amax/448,
    1e-12). Follows src/mlops/kernels/block_fp8.py:88-93 (the non-Triton branch)."""
    value = weight.float()
    experts, out, inner = value.shape
    rows, cols = _blocks(out) * BLOCK, _blocks(inner) * BLOCK
    padded = value
    if (rows, cols) != (out, inner):
        padded = value.new_zeros(experts, rows, cols)
        padded[:, :out, :inner] = value
    blocks = padded.view(experts, rows // BLOCK, BLOCK, cols // BLOCK, BLOCK)
    scale = (blocks.abs().amax(dim=(2, 4)) / E4M3_MAX).clamp_min(1e-12)
    data = (value / _expanded(scale, out, inner)).clamp(-E4M3_MAX, E4M3_MAX)
    return data.to(FP8), scale


def dequantize_blocks(data, scale, dtype=torch.float32):
    """Follows src/mlops/kernels/block_fp8.py:96-99."""
    _e, out, inner = data.shape
    return (data.float() * _expanded(scale.float(), out, inner)).to(dtype)


def quantize_rows(value, *, gather=None, mode="1x128"):
    """(data E4M3 [rows, N], scales fp32 [rows, blocks]).

    mode "row": src/mlops/kernels/quack_moe/quantize_rows.py:210-226
    (`quantize_rows_fp8_reference`): scale = max(amax * (1/448), 1e-12).
    mode "1x128": the same equations applied to every 128-column block of the row."""
    rows = value if gather is None else value[gather.long()]
    rows = rows.float()
    n = rows.shape[1]
    if mode == "row":
        amax = rows.abs().amax(dim=1)
        scales = torch.clamp_min(amax * (1.0 / 448.0), 1e-12)
        quantized = torch.clamp(rows / scales[:, None], -448.0, 448.0)
        return quantized.to(FP8), scales[:, None].contiguous()
    nb = _blocks(n)
    padded = rows
    if nb * BLOCK != n:
        padded = rows.new_zeros(rows.shape[0], nb * BLOCK)
        padded[:, :n] = rows
    blocks = padded.view(rows.shape[0], nb, BLOCK)
    amax = blocks.abs().amax(dim=2)
    scales = torch.clamp_min(amax * (1.0 / 448.0), 1e-12)
    quantized = torch.clamp(blocks / scales[:, :, None], -448.0, 448.0)
    return quantized.view(rows.shape[0], nb * BLOCK)[:, :n].to(FP8).contiguous(), scales


def dequantize_rows(data, scales, dtype=torch.float64):
    """`data * scale` per row or per 1x128 block, at `dtype`."""
    rows, n = data.shape
    value = data.to(dtype)
    if scales.dim() == 1 or scales.shape[1] == 1:
        return value * scales.reshape(rows, 1).to(dtype)
    expanded = scales.to(dtype).repeat_interleave(BLOCK, 1)[:, :n]
    return value * expanded


# ------------------------------------------------------------------------------ GEMMs
def grouped_block_gemm(a_q, a_scale, b_q, b_scale, offsets, *, b_mn_major=False,
                       dtype=torch.float64):
    """Product of the dequantised operands per group, at `dtype` (float64 by default:
    the comparison the reference's GEMM tests make,
    tests/test_block_fp8_transpose_gemm.py:447-459,486-498).
    `b_q [G,N,K]` with scales `[G,N/128,K/128]`; with `b_mn_major` the stored weight is
    `[G,K,N]` (scales `[G,K/128,N/128]`) and is read along its rows (an input gradient)."""
    a = dequantize_rows(a_q, a_scale, dtype)
    groups = b_q.shape[0]
    n = b_q.shape[2] if b_mn_major else b_q.shape[1]
    out = torch.zeros((a_q.shape[0], n), dtype=dtype)
    offs = offsets.tolist()
    for g in range(groups):
        lo, hi = offs[g], offs[g + 1]
        if hi > lo:  # weights are dequantised one expert at a time (memory)
            b = dequantize_blocks(b_q[g:g + 1], b_scale[g:g + 1], dtype)[0]
            out[lo:hi] = a[lo:hi] @ (b if b_mn_major else b.t())
    return out


def grouped_mm(a, b, offsets, *, b_mn_major=False, dtype=torch.float64):
    """`out[rows_e] = a[rows_e] @ b[e].T` (`b [E, N, K]`) or `a[rows_e] @ b[e]` (`b [E, K, N]`,
    `b_mn_major`): the dense per-expert products of the bf16 path
    (src/mlops/kernels/moe_grouped_gemm.py:185-198), at `dtype`."""
    n = b.shape[2] if b_mn_major else b.shape[1]
    out = torch.zeros((a.shape[0], n), dtype=dtype)
    offs = offsets.tolist()
    for e in range(len(offs) - 1):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            w = b[e % b.shape[0]].to(dtype)
            out[lo:hi] = a[lo:hi].to(dtype) @ (w if b_mn_major else w.t())
    return out


def grouped_wgrad(g, x, offsets, groups, dtype=torch.float64):
    """`out[e] = g[rows_e].T @ x[rows_e]`; zeros for an expert without rows.
    Follows src/mlops/kernels/moe_grouped_gemm.py:185-198,300-342."""
    out = torch.zeros((groups, g.shape[1], x.shape[1]), dtype=dtype)
    offs = offsets.tolist()
    for e in range(groups):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            out[e] = g[lo:hi].to(dtype).t() @ x[lo:hi].to(dtype)
    return out


# ------------------------------------------------------------------ SwiGLU and combine
def quantize_columns(value, offsets, groups):
    """(data E4M3 [rows, N] token-major, scales fp32 [groups, N]): one scale per column over the
    rows of each group, `scale = max(amax * (1/448), 1e-12)`, `q = clamp(x / scale)` -- the row
    quantiser's equations applied to the columns of an expert's token block, as the reference's
    FP8 weight gradient quantises both of its operands
    (src/mlops/kernels/quack_moe/quantize_transpose.py:126-133; the reference's implementation is a
    CUDA-only Triton kernel, so this restatement follows its stated equations: parity unpinned).
    `offsets` holds segments * groups + 1 boundaries; range i belongs to group i % groups."""
    rows = value.float()
    n = rows.shape[1]
    bounds = [int(v) for v in offsets.tolist()]
    ranges = len(bounds) - 1
    amax = rows.new_zeros(groups, n)
    for i in range(ranges):
        lo, hi = bounds[i], bounds[i + 1]
        if hi > lo:
            block = rows[lo:hi].abs()
            block = torch.where(torch.isnan(block), torch.zeros_like(block), block)  # a NaN never sets a scale
            amax[i % groups] = torch.maximum(amax[i % groups], block.amax(dim=0))
    scales = torch.clamp_min(amax * (1.0 / 448.0), 1e-12)
    data = torch.zeros(rows.shape, dtype=FP8)
    for i in range(ranges):
        lo, hi = bounds[i], bounds[i + 1]
        if hi > lo:
            data[lo:hi] = torch.clamp(rows[lo:hi] / scales[i % groups][None, :], -448.0, 448.0).to(FP8)
    return data, scales


def grouped_wgrad_fp8(g_q, g_scale, x_q, x_scale, offsets, groups, dtype=torch.float64):
    """`out[e] = (g_scale[e][:, None] * x_scale[e][None, :]) * (g_q[rows_e].T @ x_q[rows_e])`: the
    reference's FP8 weight gradient on given operands (src/mlops/kernels/quack_moe/wgrad.py:30-69:
    one product over all of the expert's tokens, `acc * xs * ws` at the end)."""
    bounds = [int(v) for v in offsets.tolist()]
    ranges = len(bounds) - 1
    out = torch.zeros(groups, g_q.shape[1], x_q.shape[1], dtype=dtype)
    for i in range(ranges):
        lo, hi = bounds[i], bounds[i + 1]
        if hi > lo:
            out[i % groups] += g_q[lo:hi].to(dtype).t() @ x_q[lo:hi].to(dtype)
    return out * g_scale.to(dtype)[:, :, None] * x_scale.to(dtype)[:, None, :]


def swiglu(h13, limit=None):
    """fp32 `silu(gate) * up` of h13 = [gate | up], GLM clamp when `limit` is given.
    Follows src/mlops/kernels/quack_moe/swiglu_rows.py:49-80 (fp32, rounded by the
    caller once) and src/mlops/kernels/moe_reference.py:12-17 (clamp)."""
    width = h13.shape[1] // 2
    gate, up = h13[:, :width].float(), h13[:, width:].float()
    if limit is not None:
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
    return gate * torch.sigmoid(gate) * up


def dswiglu_routed(h13, r, score, limit=None):
    """(dscore [rows], grad_h13 fp32 [rows, 2F], act_scaled fp32 [rows, F]).
    Follows src/mlops/kernels/quack_moe/swiglu_rows.py:100-199."""
    width = h13.shape[1] // 2
    raw_gate, raw_up = h13[:, :width].float(), h13[:, width:].float()
    gate, up = raw_gate, raw_up
    if limit is not None:
        gate, up = raw_gate.clamp(max=limit), raw_up.clamp(-limit, limit)
    sig = torch.sigmoid(gate)
    silu = gate * sig
    act = silu * up
    rf = r.float()
    dscore = (rf * act).sum(-1)
    g = score[:, None].float() * rf
    dgate = g * up * (sig + silu * (1.0 - sig))
    dup = g * silu
    if limit is not None:
        dgate = torch.where(raw_gate <= limit, dgate, torch.zeros_like(dgate))
        dup = torch.where((raw_up >= -limit) & (raw_up <= limit), dup, torch.zeros_like(dup))
    return dscore, torch.cat([dgate, dup], dim=1), score[:, None].float() * act


def combine(source, slots, weights, residual):
    """`residual + sum_k w[:,k] * source[slots[:,k]]`, fp32 sums in slot order, one
    rounding to bf16. Follows the kernel order of
    src/mlops/kernels/moe_dispatch.py:21-72 (residual first, then k = 0..K-1)."""
    tokens, top_k = slots.shape
    acc = (torch.zeros((tokens, source.shape[1]), dtype=torch.float32) if residual is None
           else residual.float().clone())
    for k in range(top_k):
        rows = source[slots[:, k].long()].float()
        if weights is not None:
            acc = torch.addcmul(acc, rows, weights[:, k].float()[:, None])
        else:
            acc = acc + rows
    return acc.to(torch.bfloat16)


# -------------------------------------------------------------------- the whole layer
def router_logits(h2, router_weight, operand_dtype=torch.bfloat16):
    """fp32 logits from operands at the activation's dtype with fp32 sums: what the
    reference computes on CUDA (src/mlops/kernels/router.py:53-64)."""
    return h2.to(operand_dtype).float() @ router_weight.to(operand_dtype).float().t()


def forward_block_fp8(h2, residual, logits, w13_q, w13_s, w2_q, w2_s, *, top_k, routing_mode,
                      router_bias=None, n_group=1, topk_group=1, routed_scaling=1.0,
                      swiglu_limit=None, act_scale="1x128", gemm_dtype=torch.float64):
    """The routed layer with quantised activations ("identical block-FP8 operands"):
    route -> sort -> gather+quantise -> up GEMM (bf16 h13, gate rows then up rows) ->
    SwiGLU (fp32) -> quantise -> down GEMM (bf16 rows) -> combine.
    Orchestration follows src/mlops/providers/moe_common.py:174-266 with the FP8 steps
    of src/mlops/providers/sonicmoe/block_fp8.py:114-166 in place of the bf16 GEMMs.
    Returns a dict of every intermediate."""
    experts = w13_q.shape[0]
    weights, ids = route(logits, top_k, routing_mode, bias=router_bias, n_group=n_group,
                         topk_group=topk_group, routed_scaling=routed_scaling)
    order, offsets, slots = sort_assignments(ids, experts)
    token_of_row = torch.div(order.long(), int(top_k), rounding_mode="floor")
    x_q, x_s = quantize_rows(h2, gather=token_of_row, mode=act_scale)
    h13 = grouped_block_gemm(x_q, x_s, w13_q, w13_s, offsets, dtype=gemm_dtype).to(torch.bfloat16)
    act = swiglu(h13, swiglu_limit)
    a_q, a_s = quantize_rows(act, mode=act_scale)
    y = grouped_block_gemm(a_q, a_s, w2_q, w2_s, offsets, dtype=gemm_dtype).to(torch.bfloat16)
    output = combine(y, slots, weights, residual)
    return dict(weights=weights, ids=ids, order=order, offsets=offsets, slots=slots, x_q=x_q,
                x_s=x_s, h13=h13, a_q=a_q, a_s=a_s, y=y, output=output)


def backward_block_fp8(grad_output, h2, fwd, w13_q, w13_s, w2_q, w2_s, *, top_k, swiglu_limit=None,
                       act_scale="1x128", gemm_dtype=torch.float64):
    """VJP of `forward_block_fp8` for (h2 routed part, route weights, w13, w2), FP8 input
    gradients and bf16-operand weight gradients (as the reference's fp8_block form:
    src/mlops/providers/sonicmoe/moe.py:517-619, providers/sonicmoe/fp8.py:15-17).
    Orchestration follows src/mlops/providers/moe_common.py:269-378."""
    experts = w13_q.shape[0]
    order, offsets, slots, weights = fwd["order"], fwd["offsets"], fwd["slots"], fwd["weights"]
    token_of_row = torch.div(order.long(), int(top_k), rounding_mode="floor")
    dy_q, dy_s = quantize_rows(grad_output, gather=token_of_row, mode=act_scale)
    r = grouped_block_gemm(dy_q, dy_s, w2_q, w2_s, offsets, b_mn_major=True, dtype=gemm_dtype).to(torch.bfloat16)
    score = weights.reshape(-1)[order.long()].float()
    dscore, grad_h13, act_scaled = dswiglu_routed(fwd["h13"], r, score, swiglu_limit)
    grad_route_weights = dscore[slots.reshape(-1).long()].view_as(weights)
    gh_q, gh_s = quantize_rows(grad_h13, mode=act_scale)
    grad_rows = grouped_block_gemm(gh_q, gh_s, w13_q, w13_s, offsets, b_mn_major=True,
                                   dtype=gemm_dtype).to(torch.bfloat16)
    grad_h2 = combine(grad_rows, slots, None, None)
    dy_rows = grad_output[token_of_row].to(torch.bfloat16)
    x_rows = h2[token_of_row].to(torch.bfloat16)
    grad_w2 = grouped_wgrad(dy_rows, act_scaled.to(torch.bfloat16), offsets, experts, gemm_dtype)
    grad_w13 = grouped_wgrad(grad_h13.to(torch.bfloat16), x_rows, offsets, experts, gemm_dtype)
    return dict(r=r, dscore=dscore, grad_route_weights=grad_route_weights, grad_h13=grad_h13,
                grad_rows=grad_rows, grad_h2=grad_h2, grad_w2=grad_w2, grad_w13=grad_w13)


def forward_bf16(h2, residual, logits, w13, w2, *, top_k, routing_mode, router_bias=None, n_group=1,
                 topk_group=1, routed_scaling=1.0, swiglu_limit=None, gemm_dtype=torch.float64):
    """The routed layer on plain bf16 expert weights: route -> sort -> gather -> up product (bf16
    h13, gate rows then up rows) -> SwiGLU (fp32, one rounding) -> down product (bf16 rows) ->
    combine. Orchestration: src/mlops/providers/moe_common.py:174-266 around the bf16 grouped
    products of src/mlops/kernels/moe_grouped_gemm.py:185-198."""
    experts = w13.shape[0]
    weights, ids = route(logits, top_k, routing_mode, bias=router_bias, n_group=n_group,
                         topk_group=topk_group, routed_scaling=routed_scaling)
    order, offsets, slots = sort_assignments(ids, experts)
    token_of_row = torch.div(order.long(), int(top_k), rounding_mode="floor")
    x_rows = h2[token_of_row].to(torch.bfloat16)
    h13 = grouped_mm(x_rows, w13, offsets, dtype=gemm_dtype).to(torch.bfloat16)
    act = swiglu(h13, swiglu_limit).to(torch.bfloat16)
    y = grouped_mm(act, w2, offsets, dtype=gemm_dtype).to(torch.bfloat16)
    output = combine(y, slots, weights, residual)
    return dict(weights=weights, ids=ids, order=order, offsets=offsets, slots=slots, h13=h13, act=act, y=y,
                output=output)


def backward_bf16(grad_output, h2, fwd, w13, w2, *, top_k, swiglu_limit=None, gemm_dtype=torch.float64):
    """VJP of `forward_bf16` (src/mlops/providers/moe_common.py:269-378): every product on bf16
    operands with wide sums, each intermediate rounded to bf16 where the device stores it."""
    experts = w13.shape[0]
    order, offsets, slots, weights = fwd["order"], fwd["offsets"], fwd["slots"], fwd["weights"]
    token_of_row = torch.div(order.long(), int(top_k), rounding_mode="floor")
    dy_rows = grad_output[token_of_row].to(torch.bfloat16)
    r = grouped_mm(dy_rows, w2, offsets, b_mn_major=True, dtype=gemm_dtype).to(torch.bfloat16)
    score = weights.reshape(-1)[order.long()].float()
    dscore, grad_h13, act_scaled = dswiglu_routed(fwd["h13"], r, score, swiglu_limit)
    grad_route_weights = dscore[slots.reshape(-1).long()].view_as(weights)
    gh = grad_h13.to(torch.bfloat16)
    grad_rows = grouped_mm(gh, w13, offsets, b_mn_major=True, dtype=gemm_dtype).to(torch.bfloat16)
    grad_h2 = combine(grad_rows, slots, None, None)
    x_rows = h2[token_of_row].to(torch.bfloat16)
    grad_w2 = grouped_wgrad(dy_rows, act_scaled.to(torch.bfloat16), offsets, experts, gemm_dtype)
    grad_w13 = grouped_wgrad(gh, x_rows, offsets, experts, gemm_dtype)
    return dict(r=r, dscore=dscore, grad_route_weights=grad_route_weights, grad_h13=grad_h13,
                grad_rows=grad_rows, grad_h2=grad_h2, grad_w2=grad_w2, grad_w13=grad_w13)


def rel_errors(actual, expected):
    """(max, mean) relative error of `actual` against `expected`: |a - e| / max(|e|, rms(e)).
    Large elements are judged by their true relative error, small ones against the tensor's
    RMS, so a bf16 rounding (2^-9 relative) reads as about 2e-3 wherever it falls. The
    parity tests require max <= 2e-2 and mean <= 2e-3."""
    a, e = actual.double(), expected.double()
    rms = e.pow(2).mean().sqrt().clamp_min(1e-30)
    diff = (a - e).abs() / torch.maximum(e.abs(), rms)
    return diff.max().item(), diff.mean().item()


# ------------------------------------------------------------------------ expert LoRA
def _factor_rows(rows, factor, offsets, transpose):
    """Per expert `rows_e @ factor[e]` (or `@ factor[e].T`), float64, zeros for empty experts."""
    out = torch.zeros((rows.shape[0], factor.shape[1] if transpose else factor.shape[2]), dtype=torch.float64)
    offs = offsets.tolist()
    for e in range(factor.shape[0]):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            f = factor[e].double()
            out[lo:hi] = rows[lo:hi].double() @ (f.t() if transpose else f)
    return out


def forward_lora_block_fp8(h2, residual, logits, w13_q, w13_s, w2_q, w2_s, a13, b13, a2, b2, *, top_k,
                           routing_mode, scale, router_bias=None, n_group=1, topk_group=1,
                           routed_scaling=1.0, swiglu_limit=None):
    """`h13 = x W13^T + s (x A13^T) B13^T -> SwiGLU -> y = a W2^T + s (a A2^T) B2^T` with the
    base products on block-FP8 operands and the LoRA branch in bf16 (semantics:
    src/mlops/lora/experts.py:140-167, src/mlops/lora/grouped.py:19-110). Rounding points:
    the rank-r intermediate and the LoRA term are bf16, the sum is rounded once."""
    bf = torch.bfloat16
    experts = w13_q.shape[0]
    weights, ids = route(logits, top_k, routing_mode, bias=router_bias, n_group=n_group,
                         topk_group=topk_group, routed_scaling=routed_scaling)
    order, offsets, slots = sort_assignments(ids, experts)
    token = torch.div(order.long(), int(top_k), rounding_mode="floor")
    x_rows = h2[token].to(bf)
    x_q, x_s = quantize_rows(x_rows)
    t1 = _factor_rows(x_rows, a13, offsets, True).to(bf)
    c1 = (scale * _factor_rows(t1, b13, offsets, True)).to(bf)
    h13 = (grouped_block_gemm(x_q, x_s, w13_q, w13_s, offsets) + c1.double()).to(bf)
    act = swiglu(h13, swiglu_limit)
    a_q, a_s = quantize_rows(act)
    act_b = act.to(bf)
    t2 = _factor_rows(act_b, a2, offsets, True).to(bf)
    c2 = (scale * _factor_rows(t2, b2, offsets, True)).to(bf)
    y = (grouped_block_gemm(a_q, a_s, w2_q, w2_s, offsets) + c2.double()).to(bf)
    output = combine(y, slots, weights, residual)
    return dict(weights=weights, ids=ids, order=order, offsets=offsets, slots=slots, x_rows=x_rows, h13=h13,
                act=act_b, t1=t1, t2=t2, y=y, output=output)


def backward_lora_block_fp8(grad_output, fwd, w13_q, w13_s, w2_q, w2_s, a13, b13, a2, b2, *, top_k, scale,
                            swiglu_limit=None, r_for_backward=None):
    """VJP of `forward_lora_block_fp8` for the hidden rows (expert part), the route weights and
    the four factors (frozen base). `r_for_backward`: the device's `dy W2 + s dy B2 A2` rows, so
    that (with the device's h13 / t1 / t2 in `fwd`) every later product has bit-identical
    operands on both sides; `r` is still computed here and returned."""
    bf = torch.bfloat16
    experts = w13_q.shape[0]
    order, offsets, slots, weights = fwd["order"], fwd["offsets"], fwd["slots"], fwd["weights"]
    token = torch.div(order.long(), int(top_k), rounding_mode="floor")
    dy_rows = grad_output[token].to(bf)
    dy_q, dy_s = quantize_rows(dy_rows)
    t2g = _factor_rows(dy_rows, b2, offsets, False).to(bf)                      # dy B2
    r_add = (scale * _factor_rows(t2g, a2, offsets, False)).to(bf)              # s dy B2 A2
    r = (grouped_block_gemm(dy_q, dy_s, w2_q, w2_s, offsets, b_mn_major=True) + r_add.double()).to(bf)
    score = weights.reshape(-1)[order.long()].float()
    dscore, grad_h13, act_scaled = dswiglu_routed(fwd["h13"], r if r_for_backward is None else r_for_backward,
                                                  score, swiglu_limit)
    gh_b = grad_h13.to(bf)
    gh_q, gh_s = quantize_rows(grad_h13)
    dt1 = _factor_rows(gh_b, b13, offsets, False).to(bf)                        # gh B13
    dx_add = (scale * _factor_rows(dt1, a13, offsets, False)).to(bf)
    grad_rows = (grouped_block_gemm(gh_q, gh_s, w13_q, w13_s, offsets, b_mn_major=True) + dx_add.double()).to(bf)
    grad_h2 = combine(grad_rows, slots, None, None)
    w_col = score[:, None]
    grad_b2 = grouped_wgrad(dy_rows, (fwd["t2"].float() * (w_col * scale)).to(bf), offsets, experts)
    grad_a2 = grouped_wgrad((t2g.float() * scale).to(bf), act_scaled.to(bf), offsets, experts)
    grad_b13 = grouped_wgrad(gh_b, (fwd["t1"].float() * scale).to(bf), offsets, experts)
    grad_a13 = grouped_wgrad((dt1.float() * scale).to(bf), fwd["x_rows"], offsets, experts)
    return dict(r=r, grad_h2=grad_h2, grad_route_weights=dscore[slots.reshape(-1).long()].view_as(weights),
                grad_a13=grad_a13, grad_b13=grad_b13, grad_a2=grad_a2, grad_b2=grad_b2)


# ------------------------------------------- the whole layer, one expert at a time
def layer_expert_major(h2, residual, grad_output, logits, w13_q, w13_s, w2_q, w2_s, *, top_k, routing_mode,
                       router_bias=None, n_group=1, topk_group=1, routed_scaling=1.0, swiglu_limit=None,
                       h13_for_backward=None, r_for_backward=None, keep_weight_grads=(),
                       gemm_dtype=torch.float32):
    """`forward_block_fp8` followed by `backward_block_fp8`, reorganised so that each expert's
    two weights are dequantised ONCE and used for its four products (forward up / down, the two
    input gradients) and its two weight gradients. Same equations, same rounding points; it
    exists so that layers with hundreds of large experts (256 x [4096, 7168]) can be checked in
    seconds and in bounded memory. Weight gradients are kept only for the experts listed in
    `keep_weight_grads` (dicts expert -> fp32 tensor); `h13_for_backward`, when given, is the
    saved pre-activation the backward half differentiates at (the device's own, so both sides
    take the derivative at the same point), and `r_for_backward` the device's `dy W2` rows: with
    both, every product of the backward half has bit-identical operands on the two sides (a
    one-ulp bf16 difference in `r` otherwise moves single weight-gradient elements by more than
    the rounding of the product itself). `r` is still computed here and returned."""
    experts = w13_q.shape[0]
    weights, ids = route(logits, top_k, routing_mode, bias=router_bias, n_group=n_group,
                         topk_group=topk_group, routed_scaling=routed_scaling)
    order, offsets, slots = sort_assignments(ids, experts)
    token_of_row = torch.div(order.long(), int(top_k), rounding_mode="floor")
    rows = order.numel()
    inner = w2_q.shape[2]
    x_q, x_s = quantize_rows(h2, gather=token_of_row)
    dy_q, dy_s = quantize_rows(grad_output, gather=token_of_row)
    x_f, dy_f = dequantize_rows(x_q, x_s, gemm_dtype), dequantize_rows(dy_q, dy_s, gemm_dtype)
    score = weights.reshape(-1)[order.long()].float()
    h13 = torch.zeros((rows, 2 * inner), dtype=torch.bfloat16)
    y = torch.zeros((rows, h2.shape[1]), dtype=torch.bfloat16)
    r = torch.zeros((rows, inner), dtype=torch.bfloat16)
    grad_rows = torch.zeros((rows, h2.shape[1]), dtype=torch.bfloat16)
    dscore = torch.zeros(rows, dtype=torch.float32)
    grad_w13, grad_w2 = {}, {}
    offs = offsets.tolist()
    for e in range(experts):
        lo, hi = offs[e], offs[e + 1]
        if hi == lo:
            if e in keep_weight_grads:
                grad_w13[e] = torch.zeros(tuple(w13_q.shape[1:]), dtype=torch.float32)
                grad_w2[e] = torch.zeros(tuple(w2_q.shape[1:]), dtype=torch.float32)
            continue
        w13 = dequantize_blocks(w13_q[e:e + 1], w13_s[e:e + 1], gemm_dtype)[0]
        w2 = dequantize_blocks(w2_q[e:e + 1], w2_s[e:e + 1], gemm_dtype)[0]
        h13[lo:hi] = (x_f[lo:hi] @ w13.t()).to(torch.bfloat16)
        a_q, a_s = quantize_rows(swiglu(h13[lo:hi], swiglu_limit))
        y[lo:hi] = (dequantize_rows(a_q, a_s, gemm_dtype) @ w2.t()).to(torch.bfloat16)
        r[lo:hi] = (dy_f[lo:hi] @ w2).to(torch.bfloat16)
        saved = h13[lo:hi] if h13_for_backward is None else h13_for_backward[lo:hi]
        r_used = r[lo:hi] if r_for_backward is None else r_for_backward[lo:hi]
        ds, grad_h13, act_scaled = dswiglu_routed(saved, r_used, score[lo:hi], swiglu_limit)
        dscore[lo:hi] = ds
        gh_q, gh_s = quantize_rows(grad_h13)
        grad_rows[lo:hi] = (dequantize_rows(gh_q, gh_s, gemm_dtype) @ w13).to(torch.bfloat16)
        if e in keep_weight_grads:
            tokens_e = token_of_row[lo:hi]
            dy_rows = grad_output[tokens_e].to(torch.bfloat16).to(gemm_dtype)
            x_rows = h2[tokens_e].to(torch.bfloat16).to(gemm_dtype)
            grad_w2[e] = (dy_rows.t() @ act_scaled.to(torch.bfloat16).to(gemm_dtype)).float()
            grad_w13[e] = (grad_h13.to(torch.bfloat16).to(gemm_dtype).t() @ x_rows).float()
    output = combine(y, slots, weights, residual)
    grad_h2 = combine(grad_rows, slots, None, None)
    grad_route_weights = dscore[slots.reshape(-1).long()].view_as(weights)
    return dict(weights=weights, ids=ids, order=order, offsets=offsets, slots=slots, h13=h13, y=y,
                output=output, r=r, grad_rows=grad_rows, grad_h2=grad_h2,
                grad_route_weights=grad_route_weights, grad_w13=grad_w13, grad_w2=grad_w2)


def plain_max_rel(actual, expected, floor=1e-2):
    """The plain maximum relative error `|a - e| / |e|` over the elements whose magnitude is at
    least `floor` x rms(e) (elements nearer zero have no meaningful relative error), with the
    share of elements that takes part. Reported beside `rel_errors`, whose denominator is
    floored at the tensor's RMS."""
    a, e = actual.double(), expected.double()
    rms = e.pow(2).mean().sqrt().clamp_min(1e-30)
    mask = e.abs() >= floor * rms
    if not bool(mask.any()):
        return 0.0, 0.0
    return ((a - e).abs()[mask] / e.abs()[mask]).max().item(), mask.double().mean().item()
