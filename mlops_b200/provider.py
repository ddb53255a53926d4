"""The `b200.moe` provider: this library behind the reference's implementation registry.

`register()` adds one `Implementation(operation="moe", implementation_id="b200.moe", ...)`
to `mlops.dispatch.registry` (als244/mlops, `src/mlops/dispatch/registry.py:31-69`), with the
`supports` / `apply` / `forward` / `backward` callables below; they take the arguments and
return the tuples the reference documents for the `moe` operation (`docs/OPS.md:1603-1700`,
`docs/EXPLICIT_OPS.md:456-502`) and work without the reference installed. There is no
fallback: a refusal comes from `supports`, with its reason.

Opaque-operator contract (`docs/PROVIDERS.md:86-112`, the shape of
`src/mlops/providers/builtin/moe.py:122-472`): the routed layer is the functional custom
operator pair `b200moe::moe_fwd` / `b200moe::moe_bwd` (`mutates_args=()`), each with a fake
implementation that states its outputs' shapes, dtypes and device, autograd registered with
`register_autograd` (`needs_input_grad` becomes the backward operator's `need_*` flags, a
gradient nobody asked for is an empty placeholder turned into `None`), a FLOP formula for
`FlopCounterMode`, and `register_torch_dispatch` handlers that take a weight container apart
(its E4M3 data in place, its block scales appended to the trailing `weight_components`
list) before the operator runs on plain tensors. The operators live in their own namespace:
the reference asserts that `torch.ops.mlops` holds exactly its own manifest
(`tests/test_custom_op_contracts.py:787-791`).
"""

from __future__ import annotations

import os

import torch
from torch.utils.flop_counter import register_flop_formula

from . import layer
from . import ops as kernels
from .weights import BlockFP8Weight, holds_blocks, split

IMPLEMENTATION_ID = "b200.moe"
PRIORITY = 120  # above the reference's highest MoE implementation (110)
MAX_EXPERTS = 1024
MAX_TOP_K = 32
ROUTING_MODES = ("softmax_then_topk", "topk_then_softmax", "sigmoid_noaux_tc")
ROUTE_WEIGHT_PRECISIONS = ("float32", "input")


# The optional FP8 weight-gradient recipe (both operands of dW13 and dW2 quantised to E4M3 with
# one scale per expert and column; the reference's `fp8_current` weight gradient,
# src/mlops/kernels/quack_moe/wgrad.py:30-69). A process-wide recipe choice like the reference's
# container type, read when a backward runs; bf16 operands are the default.
WEIGHT_GRADIENT_OPERANDS = os.environ.get("B200MOE_WGRAD_OPERANDS", "bf16")


def set_weight_gradient_operands(kind: str) -> str:
    """`"bf16"` (default) or `"fp8"`; returns the previous setting."""
    global WEIGHT_GRADIENT_OPERANDS
    if kind not in ("bf16", "fp8"):
        raise ValueError("weight-gradient operands are 'bf16' or 'fp8'")
    previous, WEIGHT_GRADIENT_OPERANDS = WEIGHT_GRADIENT_OPERANDS, kind
    return previous


# ----------------------------------------------------------------- the reference's contexts
def _context_weight_gradient_dtype():
    """The reference's `weight_gradients_at(...)` context, when the reference is present."""
    try:
        from mlops.dispatch.context import weight_gradient_dtype
    except ImportError:
        return None
    return weight_gradient_dtype()


def _context_route_weight_precision() -> str:
    """The reference's `route_weight_precision(...)` context ("float32" without it). Both of
    its values give fp32 route weights here, as they do in the reference: "input" means the
    dtype of the logits, and the logits of this path are fp32
    (`src/mlops/kernels/moe_router.py:254-270`, `kernels/router.py:53-64`)."""
    try:
        from mlops.kernels.moe_router import current_route_weight_precision
    except ImportError:
        return "float32"
    return current_route_weight_precision()


# ------------------------------------------------------------------------------ refusals
def refusal(h2, residual, router_weight, w13_experts, w2_experts, *, surface="semantic", top_k,
            routing_mode, n_group=1, topk_group=1, lengths=None, shared_w13=None, shared_w2=None,
            compute_precision=None, swiglu_limit=None, **_ignored):
    """The reason this provider cannot serve the call, or None. Metadata only."""
    tensors = (h2, residual, router_weight, w13_experts, w2_experts)
    if not all(isinstance(t, torch.Tensor) for t in tensors):
        return "MoE core arguments must be tensors"
    if not all(t.is_cuda for t in tensors):
        return "b200.moe runs on CUDA tensors only"
    if len({t.device for t in tensors}) != 1:
        return "b200.moe needs every argument on one device"
    if torch.cuda.get_device_capability(h2.device) != (10, 0):
        return "b200.moe is built for compute capability 10.0 (sm_100a) only"
    if compute_precision not in (None, "fp8_block", "bf16"):
        return f"b200.moe computes in block FP8 or bf16; compute_precision={compute_precision!r} is not served"
    containers = holds_blocks(w13_experts) and holds_blocks(w2_experts)
    plain = _plain_bf16(w13_experts) and _plain_bf16(w2_experts)
    if not (containers or plain):
        return ("expert weights must be BlockFP8Weight containers (E4M3, 128x128 block scales) or plain bf16 "
                "tensors")
    if plain and compute_precision == "fp8_block":
        return "plain bf16 expert weights are multiplied in bf16; quantise them (BlockFP8Weight.quantize) for fp8_block"
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
    if containers and (width % 128 or inner % 128):
        return "hidden and expert widths must be multiples of 128"
    if plain and (width % 8 or inner % 8):
        return "hidden and expert widths must be multiples of 8"
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


def _plain_bf16(weight) -> bool:
    return type(weight) in (torch.Tensor, torch.nn.Parameter) and weight.dtype == torch.bfloat16 and weight.dim() == 3


def _operands(weight):
    """What the layer takes for one expert weight: the bf16 tensor, or (E4M3 data, block scales)."""
    return weight if _plain_bf16(weight) else split(weight)


class _DequantizedCopy(torch.autograd.Function):
    """bf16 values of a block-FP8 container for the bf16 compute path; the gradient of the copy is
    the container's gradient (the reference multiplies the dequantised weights the same way,
    src/mlops/providers/expert_weights.py:46-52)."""

    @staticmethod
    def forward(ctx, container):
        data, scale = split(container)
        rows, cols = data.shape[1], data.shape[2]
        wide = scale.repeat_interleave(128, 1)[:, :rows].repeat_interleave(128, 2)[:, :, :cols]
        return (data.float() * wide).to(torch.bfloat16)

    @staticmethod
    def backward(ctx, grad):
        return grad


# ------------------------------------------------------------------ the operator pair
_ELEVEN = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]
_FIVE = tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


def _with_scales(w13_data, w2_data, weight_components):
    if w13_data.dtype == torch.bfloat16 and w2_data.dtype == torch.bfloat16 and len(weight_components) == 0:
        return w13_data, w2_data  # plain bf16 weights: the bf16 compute path
    if len(weight_components) != 2:
        raise ValueError("b200moe operators take the two block-scale tensors (w13's, then w2's) as "
                         "weight_components; pass the weight containers and leave the list empty")
    return (w13_data, weight_components[0]), (w2_data, weight_components[1])


@torch.library.custom_op("b200moe::moe_fwd", mutates_args=())
def moe_fwd(h2: torch.Tensor, residual: torch.Tensor, router_weight: torch.Tensor, w13_experts: torch.Tensor,
            w2_experts: torch.Tensor, router_bias: torch.Tensor, top_k: int, routing_mode: str, n_group: int,
            topk_group: int, routed_scaling: float, lengths: list[int], weight_precision: str,
            weight_grad_dtype: torch.dtype | None, swiglu_limit: float | None,
            weight_components: list[torch.Tensor]) -> _ELEVEN:
    """`(output, aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets,
    slots, h13)`; `w13_experts` / `w2_experts` are the E4M3 data, `weight_components` their
    scales. `router_bias` with no elements means none."""
    del weight_grad_dtype
    if weight_precision not in ROUTE_WEIGHT_PRECISIONS:
        raise ValueError(f"unsupported route-weight precision {weight_precision!r}")
    w13, w2 = _with_scales(w13_experts, w2_experts, weight_components)
    with torch.cuda.device(h2.device):
        return layer.forward_routed(
            h2, residual, router_weight, w13, w2, top_k=top_k, routing_mode=routing_mode,
            router_bias=None if router_bias.numel() == 0 else router_bias, n_group=n_group,
            topk_group=topk_group, routed_scaling=routed_scaling, lengths=lengths, swiglu_limit=swiglu_limit)


@moe_fwd.register_fake
def _moe_fwd_fake(h2, residual, router_weight, w13_experts, w2_experts, router_bias, top_k, routing_mode,
                  n_group, topk_group, routed_scaling, lengths, weight_precision, weight_grad_dtype,
                  swiglu_limit, weight_components):
    rows = h2.numel() // h2.shape[-1]
    experts = router_weight.shape[0]
    assignments = rows * int(top_k)
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=h2.device)  # noqa: E731
    return (
        torch.empty_like(h2, memory_format=torch.contiguous_format),
        new((), torch.float32), new((experts,), torch.int64), new((experts,), torch.float32),
        new((rows, experts), torch.float32), new((rows, int(top_k)), torch.float32),
        new((rows, int(top_k)), torch.int32), new((assignments,), torch.int32),
        new((experts + 1,), torch.int32), new((rows, int(top_k)), torch.int32),
        new((assignments, w13_experts.shape[1]), h2.dtype),
    )


def _logical_dtype(weight_grad_dtype, fallback):
    return fallback if weight_grad_dtype is None else weight_grad_dtype


@torch.library.custom_op("b200moe::moe_bwd", mutates_args=())
def moe_bwd(grad_output: torch.Tensor, grad_aux: torch.Tensor, grad_probability_sum: torch.Tensor,
            h2: torch.Tensor, router_weight: torch.Tensor, w13_experts: torch.Tensor, w2_experts: torch.Tensor,
            logits: torch.Tensor, route_weights: torch.Tensor, route_ids: torch.Tensor, order: torch.Tensor,
            offsets: torch.Tensor, slots: torch.Tensor, h13: torch.Tensor, top_k: int, routing_mode: str,
            lengths: list[int], weight_grad_dtype: torch.dtype | None, swiglu_limit: float | None,
            need_router: bool, need_w13: bool, need_w2: bool,
            weight_components: list[torch.Tensor]) -> _FIVE:
    """`(grad_h2, grad_residual, grad_router, grad_w13, grad_w2)`; a gradient whose `need_*`
    flag is false is an empty placeholder and its GEMM is not launched."""
    w13, w2 = _with_scales(w13_experts, w2_experts, weight_components)
    wdtype = _logical_dtype(weight_grad_dtype, torch.bfloat16)
    with torch.cuda.device(h2.device):
        return layer.backward_routed(
            grad_output, grad_aux, grad_probability_sum, h2, router_weight, w13, w2, logits, route_weights,
            route_ids, order, offsets, slots, h13, top_k=top_k, routing_mode=routing_mode, lengths=lengths,
            weight_grad_dtype=wdtype, router_grad_dtype=weight_grad_dtype, swiglu_limit=swiglu_limit,
            need_router=need_router, need_w13=need_w13, need_w2=need_w2,
            weight_grad_operands=WEIGHT_GRADIENT_OPERANDS)


@moe_bwd.register_fake
def _moe_bwd_fake(grad_output, grad_aux, grad_probability_sum, h2, router_weight, w13_experts, w2_experts,
                  logits, route_weights, route_ids, order, offsets, slots, h13, top_k, routing_mode, lengths,
                  weight_grad_dtype, swiglu_limit, need_router, need_w13, need_w2, weight_components):
    wdtype = _logical_dtype(weight_grad_dtype, torch.bfloat16)
    rdtype = _logical_dtype(weight_grad_dtype, router_weight.dtype)
    new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=h2.device)  # noqa: E731
    return (
        torch.empty_like(h2, memory_format=torch.contiguous_format),
        torch.empty_like(grad_output, memory_format=torch.contiguous_format),
        new(tuple(router_weight.shape), rdtype) if need_router else new((0,), router_weight.dtype),
        new(tuple(w13_experts.shape), wdtype) if need_w13 else new((0,), wdtype),
        new(tuple(w2_experts.shape), wdtype) if need_w2 else new((0,), wdtype),
    )


def _logical_flops(h2, router_weight, w13_experts, w2_experts, top_k, forward):
    """The reference's own count (`src/mlops/dispatch/logical_costs.py:390-470`): router GEMM,
    `2*D*2F + 2*F*D = 6*D*F` per routed row for the two projections (twice that backward,
    `18*D*F` in all), plus the elementwise passes."""
    try:
        from mlops.dispatch import logical_costs
    except ImportError:
        logical_costs = None
    if logical_costs is not None:
        return logical_costs.moe(h2, h2, router_weight, w13_experts, w2_experts, top_k=top_k,
                                 entrypoint="forward" if forward else "backward").logical_flops
    rows = h2.numel() // h2.shape[-1]
    width, experts = h2.shape[-1], router_weight.shape[0]
    assignments, packed, inner = rows * int(top_k), w13_experts.shape[1], w2_experts.shape[2]
    router = 2 * rows * width * experts + 3 * rows * experts
    up = 2 * assignments * width * packed
    activation, down, combine = 5 * assignments * inner, 2 * assignments * inner * width, 2 * assignments * width
    if forward:
        return router + up + activation + down + combine
    return 2 * router - 3 * rows * experts + 2 * up + 2 * activation + 2 * down + combine


@register_flop_formula(torch.ops.b200moe.moe_fwd, get_raw=True)
def _moe_fwd_flops(h2, residual, router_weight, w13_experts, w2_experts, router_bias, top_k, *_rest,
                   out_val=None, **_kwargs):
    return _logical_flops(h2, router_weight, w13_experts, w2_experts, top_k, True)


@register_flop_formula(torch.ops.b200moe.moe_bwd, get_raw=True)
def _moe_bwd_flops(grad_output, grad_aux, grad_probability_sum, h2, router_weight, w13_experts, w2_experts,
                   logits, route_weights, route_ids, order, offsets, slots, h13, top_k, *_rest, out_val=None,
                   **_kwargs):
    return _logical_flops(h2, router_weight, w13_experts, w2_experts, top_k, False)


def _setup_context(ctx, inputs, output):
    (h2, _residual, router_weight, w13_experts, w2_experts, _bias, top_k, routing_mode, _n_group, _topk_group,
     _scaling, lengths, _precision, weight_grad_dtype, swiglu_limit, weight_components) = inputs
    (_out, _aux, counts, _psum, logits, route_weights, route_ids, order, offsets, slots, h13) = output
    ctx.save_for_backward(h2, router_weight, w13_experts, w2_experts, logits, route_weights, route_ids, order,
                          offsets, slots, h13, *weight_components)
    ctx.top_k, ctx.routing_mode, ctx.lengths = int(top_k), routing_mode, list(lengths)
    ctx.weight_grad_dtype, ctx.swiglu_limit = weight_grad_dtype, swiglu_limit
    # the gradient of a container goes out at its logical dtype unless the context names one
    ctx.logical = (w13_experts.dtype if w13_experts.dtype != torch.float8_e4m3fn else torch.bfloat16)
    ctx.mark_non_differentiable(counts, logits, route_weights, route_ids, order, offsets, slots, h13)
    ctx.components = len(weight_components)


def _requested(gradient, needed):
    return gradient if needed else None


def _autograd_backward(ctx, grad_output, grad_aux, _g_counts, grad_probability_sum, *_metadata_grads):
    saved = ctx.saved_tensors
    tensors, components = saved[:11], list(saved[11:])
    h2, router_weight = tensors[0], tensors[1]
    if grad_output is None:
        grad_output = torch.zeros_like(h2)
    if grad_aux is None:
        grad_aux = torch.zeros((), dtype=torch.float32, device=h2.device)
    if grad_probability_sum is None:
        grad_probability_sum = torch.zeros(router_weight.shape[0], dtype=torch.float32, device=h2.device)
    need = ctx.needs_input_grad
    # None keeps "own dtypes" (the router's; bf16 for E4M3 data); a container whose logical dtype
    # is not bf16 names that dtype, and the router's gradient is brought back to the router's
    wdtype = ctx.weight_grad_dtype
    if wdtype is None and ctx.logical != torch.bfloat16:
        wdtype = ctx.logical
    grad_h2, grad_residual, grad_router, grad_w13, grad_w2 = moe_bwd(
        grad_output, grad_aux, grad_probability_sum, *tensors, ctx.top_k, ctx.routing_mode, ctx.lengths,
        wdtype, ctx.swiglu_limit, bool(need[2]), bool(need[3]), bool(need[4]), components)
    if ctx.weight_grad_dtype is None and need[2] and grad_router.dtype != router_weight.dtype:
        grad_router = grad_router.to(router_weight.dtype)
    return (_requested(grad_h2, need[0]), _requested(grad_residual, need[1]), _requested(grad_router, need[2]),
            _requested(grad_w13, need[3]), _requested(grad_w2, need[4]), *([None] * 10),
            [None] * ctx.components)  # a list input answers with a list of the same length


moe_fwd.register_autograd(_autograd_backward, setup_context=_setup_context)


# --------------------------------------------------------------- SwiGLU of the shared expert
@torch.library.custom_op("b200moe::swiglu", mutates_args=())
def swiglu(h13: torch.Tensor, limit: float | None) -> torch.Tensor:
    """`silu(gate) * up` of `h13 = [gate | up]` (fp32 math, one rounding), clamped when `limit`
    is given (`src/mlops/kernels/moe_reference.py:12-17`)."""
    flat = h13.reshape(-1, h13.shape[-1])
    if flat.stride(-1) != 1:
        flat = flat.contiguous()
    _, _, act = kernels.swiglu_quantize(flat, limit=limit, quantized=False, rounded=True)
    return act.reshape(*h13.shape[:-1], h13.shape[-1] // 2)


@swiglu.register_fake
def _swiglu_fake(h13, limit):
    return h13.new_empty((*h13.shape[:-1], h13.shape[-1] // 2))


@torch.library.custom_op("b200moe::swiglu_bwd", mutates_args=())
def swiglu_bwd(h13: torch.Tensor, grad_act: torch.Tensor, limit: float | None) -> torch.Tensor:
    """Gradient of `swiglu` for `h13` (no gradient through a clamped value)."""
    flat = h13.reshape(-1, h13.shape[-1])
    grad = grad_act.reshape(-1, grad_act.shape[-1])
    if flat.stride(-1) != 1:
        flat = flat.contiguous()
    if grad.stride(-1) != 1:
        grad = grad.contiguous()
    rows = flat.shape[0]
    ones = torch.ones(rows, dtype=torch.float32, device=flat.device)
    identity = torch.arange(rows, dtype=torch.int32, device=flat.device)
    _, _, _, grad_h13, _ = kernels.dswiglu_routed(flat, grad, ones, identity, limit=limit, quantized=False,
                                                  rounded=True)
    return grad_h13.reshape(h13.shape)


@swiglu_bwd.register_fake
def _swiglu_bwd_fake(h13, grad_act, limit):
    return torch.empty_like(h13, memory_format=torch.contiguous_format)


def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])
    ctx.limit = inputs[1]


def _swiglu_backward(ctx, grad_act):
    (h13,) = ctx.saved_tensors
    return swiglu_bwd(h13, grad_act.contiguous(), ctx.limit), None


swiglu.register_autograd(_swiglu_backward, setup_context=_swiglu_setup)


@register_flop_formula(torch.ops.b200moe.swiglu, get_raw=True)
def _swiglu_flops(h13, limit, *_rest, out_val=None, **_kwargs):
    return 5 * (h13.numel() // 2)


@register_flop_formula(torch.ops.b200moe.swiglu_bwd, get_raw=True)
def _swiglu_bwd_flops(h13, grad_act, limit, *_rest, out_val=None, **_kwargs):
    return 10 * (h13.numel() // 2)


# ------------------------------------------------------------- containers at the boundary
_CONTAINER_OPERATORS: list = [moe_fwd, moe_bwd]
_DISPATCH_REGISTERED: set = set()


def _unwrap_containers(_mode_or_cls, func, _types, args, kwargs):
    """A call that carries weight containers: each container becomes its data in place and its
    block scales join the operator's trailing `weight_components` list, in weight order (the
    convention of `src/mlops/providers/sonicmoe/fp8.py:196-225`)."""
    if kwargs:
        raise ValueError("b200moe operators take positional arguments")
    args = list(args)
    slot = max(index for index, value in enumerate(args) if isinstance(value, list))
    components = list(args[slot])
    for index, value in enumerate(args):
        if not isinstance(value, torch.Tensor) or isinstance(value, torch._subclasses.FakeTensor):
            continue
        if holds_blocks(value) and type(value) is not torch.Tensor:
            components.append(value._scale)
            args[index] = value._data
        elif type(value) in _DISPATCH_REGISTERED and isinstance(getattr(value, "_data", None), torch.Tensor):
            args[index] = value._data  # a compute-dtype wrapper (the router's BF16ComputeWeight)
    args[slot] = components
    return func(*args)


def register_container(cls) -> None:
    """Teach the operators to accept instances of the tensor subclass `cls` (a block-FP8
    container with `_data` / `_scale`, or a wrapper whose payload is `_data`)."""
    if cls in _DISPATCH_REGISTERED:
        return
    for operator in _CONTAINER_OPERATORS:
        operator.register_torch_dispatch(cls, _unwrap_containers)
    _DISPATCH_REGISTERED.add(cls)


def _register_reference_containers() -> None:
    try:
        from mlops.block_fp8 import BlockFP8Weight as ReferenceBlockWeight
    except ImportError:
        return
    register_container(ReferenceBlockWeight)
    try:
        from mlops.bf16_compute import BF16ComputeWeight
    except ImportError:
        return
    register_container(BF16ComputeWeight)


register_container(BlockFP8Weight)


# --------------------------------------------------------------------------- the provider
def supports(h2, residual, router_weight, w13_experts, w2_experts, **kwargs):
    from mlops.dispatch.registry import SupportResult

    reason = refusal(h2, residual, router_weight, w13_experts, w2_experts, **kwargs)
    return SupportResult.yes() if reason is None else SupportResult.no(reason)


def shared_expert(h2, shared_w13, shared_w2, shared_gate_weight=None, shared_mode="add", swiglu_limit=None):
    """The always-on shared expert, `W2s . swiglu(W13s . x)` (optionally sigmoid-gated), as an
    ordinary differentiable graph: bf16 library GEMMs, as the reference computes it
    (`src/mlops/moe.py:12-37`; it never quantises the shared expert), around this library's
    SwiGLU operator."""
    act = swiglu(torch.nn.functional.linear(h2, shared_w13), swiglu_limit)
    shared = torch.nn.functional.linear(act, shared_w2)
    if shared_mode == "sigmoid":
        gate = torch.sigmoid(torch.nn.functional.linear(h2, shared_gate_weight).float())
        shared = (gate * shared.float()).to(h2.dtype)
    elif shared_mode != "add":
        raise ValueError(f"unsupported shared_mode {shared_mode!r}")
    return shared


def apply(h2, residual, router_weight, w13_experts, w2_experts, *, top_k, routing_mode, router_bias=None,
          n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, shared_w13=None, shared_w2=None,
          shared_gate_weight=None, shared_mode="add", compute_precision=None, swiglu_limit=None):
    """`(output, aux, counts int64 [E], probability_sum fp32 [E])`; differentiable in `h2`,
    `residual`, `router_weight`, both expert containers and the shared weights. Reads the
    reference's weight-gradient dtype and route-weight precision contexts here, at apply
    time, and hands them to the operator as arguments (`docs/PROVIDERS.md:40-45`)."""
    reason = refusal(h2, residual, router_weight, w13_experts, w2_experts, top_k=top_k, routing_mode=routing_mode,
                     n_group=n_group, topk_group=topk_group, lengths=lengths, shared_w13=shared_w13,
                     shared_w2=shared_w2, compute_precision=compute_precision)
    if reason is not None:
        raise ValueError(reason)
    if compute_precision == "bf16" and holds_blocks(w13_experts):
        w13_experts, w2_experts = _DequantizedCopy.apply(w13_experts), _DequantizedCopy.apply(w2_experts)
    for weight in (w13_experts, w2_experts):
        if not _plain_bf16(weight) and type(weight) not in _DISPATCH_REGISTERED:
            register_container(type(weight))
    limit = None if swiglu_limit is None else float(swiglu_limit)
    base = residual
    if shared_w13 is not None:
        base = residual + shared_expert(h2, shared_w13, shared_w2, shared_gate_weight, shared_mode, limit)
    rows = h2.numel() // h2.shape[-1]
    normalized = [rows] if lengths is None else [int(v) for v in lengths]
    bias = router_bias if router_bias is not None else torch.empty(0, dtype=torch.float32, device=h2.device)
    outputs = moe_fwd(h2, base, router_weight, w13_experts, w2_experts, bias, int(top_k), str(routing_mode),
                      int(n_group), int(topk_group), float(routed_scaling), normalized,
                      _context_route_weight_precision(), _context_weight_gradient_dtype(), limit, [])
    return outputs[:4]


def forward(h2, residual, router_weight, w13_experts, w2_experts, *, top_k, routing_mode, router_bias=None,
            n_group=1, topk_group=1, routed_scaling=1.0, lengths=None, weight_precision="float32",
            swiglu_implementation=None, swiglu_limit=None):
    """Explicit surface: output, statistics and the VJP residuals, in the reference's order
    `(output, aux, counts, probability_sum, logits, route_weights, route_ids, order, offsets,
    slots, h13)`."""
    del swiglu_implementation
    if weight_precision not in ROUTE_WEIGHT_PRECISIONS:
        raise ValueError(f"unsupported route-weight precision {weight_precision!r}")
    return layer.forward_routed(
        h2, residual, router_weight, _operands(w13_experts), _operands(w2_experts), top_k=int(top_k),
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
    kwargs.setdefault("weight_grad_operands", WEIGHT_GRADIENT_OPERANDS)
    return layer.backward_routed(
        grad_output, grad_aux, grad_probability_sum, h2, router_weight, _operands(w13_experts),
        _operands(w2_experts), logits, route_weights, route_ids, order, offsets, slots, h13, top_k=int(top_k),
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

    _register_reference_containers()
    _REGISTERED = register_implementation(
        Implementation(
            operation="moe", implementation_id=IMPLEMENTATION_ID, provider="b200", priority=int(priority),
            deterministic=True, supports=supports, apply=apply, forward=forward, backward=backward,
        )
    )
    return _REGISTERED
