"""Tensor-level wrappers over the C ABI: each function unpacks torch CUDA tensors into
pointers / pitches, allocates the outputs with torch's caching allocator and enqueues the
kernel on the current CUDA stream. No function synchronises, reads device memory on the
host, or has a non-CUDA path: a CPU tensor is an error.

Names follow the reference's raw kernel functions (`route`, `sort_assignments`,
`quantize_rows_fp8`, `grouped_block_gemm`, `combine`, ...) so call sites read like
`src/mlops/providers/moe_common.py` of the reference.
"""

from __future__ import annotations

import functools
import os

import torch

from ._lib import NativeError, check, lib

ROUTING_MODES = {"topk_then_softmax": 0, "softmax_then_topk": 1, "sigmoid_noaux_tc": 2}
FP8 = torch.float8_e4m3fn

_STATUS: dict[int, torch.Tensor] = {}

# Instrumentation read by the bench: kernels launched through this module, and (when a list
# is installed) one (start_event, end_event, kind, flops) record per tensor-core launch.
LAUNCHES = 0
GEMM_TIMINGS: list | None = None


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


class _Timed:
    """Brackets a launch with CUDA events on the launching stream when timings are wanted."""

    def __init__(self, kind: str, flops: float):
        self.kind, self.flops = kind, flops

    def __enter__(self):
        if GEMM_TIMINGS is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.stop = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if GEMM_TIMINGS is not None:
            self.stop.record()
            GEMM_TIMINGS.append((self.start, self.stop, self.kind, self.flops))
        return False


# B200MOE_NVTX=1 brackets every wrapper call with an NVTX range named after it, so a timeline
# shows the phases of a step as the reference's expert-parallel runtime marks its own
# (src/mlops/expert_parallel/quack/streams.py:36-71). Off by default: a range costs a few
# hundred nanoseconds on the host per launch.
NVTX = os.environ.get("B200MOE_NVTX", "0") == "1"


def _on_tensor_device(fn):
    """Runs `fn` with the device of its first CUDA tensor argument current, so the kernels are
    launched on that device and on ITS current stream whatever device the caller had selected
    (a model moved with `.to("cuda:1")` while cuda:0 is current). The library launches on the
    current device; the wrappers therefore never rely on the caller having set it."""

    @functools.wraps(fn)
    def on_device(*args, **kwargs):
        for value in (*args, *kwargs.values()):
            if isinstance(value, torch.Tensor) and value.is_cuda:
                if value.device.index == torch.cuda.current_device():
                    break
                with torch.cuda.device(value.device):
                    return fn(*args, **kwargs)
        return fn(*args, **kwargs)

    if not NVTX:
        return on_device

    @functools.wraps(fn)
    def ranged(*args, **kwargs):
        torch.cuda.nvtx.range_push("b200moe." + fn.__name__)
        try:
            return on_device(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()

    return ranged


def set_cta_limit(ctas: int) -> None:
    """Cap the CTAs of the persistent GEMM kernels (0 = every SM), so that communication
    kernels running beside them find free SMs."""
    check(lib.b200moe_set_cta_limit(int(ctas)), "set_cta_limit")


def set_gemm_pair(mode: int) -> None:
    """1: the CTA-pair form of the wide FP8 GEMM (cta_group::2, 256 x 256 tiles); -1 (default)
    and 0: the single-CTA form. Bit-identical results either way."""
    check(lib.b200moe_set_gemm_pair(int(mode)), "set_gemm_pair")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors) -> torch.device:
    device = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise NativeError("mlops_b200 kernels take CUDA tensors only (no CPU path)")
        if device is None:
            device = t.device
        elif t.device != device:
            raise NativeError("tensors live on different devices")
    return device


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def status_block(device) -> torch.Tensor:
    """The per-device int32[4] block the kernels report bounded-wait and validation
    failures into. Created (zeroed) on first use."""
    index = torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    block = _STATUS.get(index)
    if block is None:
        block = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", index))
        _STATUS[index] = block
    return block


def check_status(device=None) -> None:
    """Synchronising check of the status block; raises when a kernel reported a failure.
    Not called on the forward/backward path (it reads device memory)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    block = _STATUS.get(index)
    if block is None:
        return
    code, where_block, where, detail = block.tolist()
    if code != 0:
        block.zero_()
        names = {1: "bounded wait ran out", 2: "malformed offsets or ids"}
        raise NativeError(
            f"device status: {names.get(code, code)} (block {where_block}, where {where}, detail {detail})"
        )


# ----------------------------------------------------------------------------- routing
@_on_tensor_device
def route_topk(logits, top_k, mode, *, bias=None, n_group=1, topk_group=1, routed_scaling=1.0):
    """(weights fp32 [T,K], ids int32 [T,K]) of fp32 logits [T,E]."""
    _need_cuda(logits, bias)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise NativeError("logits must be fp32 [tokens, experts] with unit inner stride")
    tokens, experts = logits.shape
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device=logits.device)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    check(
        lib.b200moe_route_topk(
            logits.data_ptr(), logits.stride(0), tokens, experts, int(top_k), ROUTING_MODES[mode],
            _ptr(bias), int(n_group), int(topk_group), float(routed_scaling),
            weights.data_ptr(), ids.data_ptr(), _stream(),
        ),
        "route_topk",
    )
    _count()
    return weights, ids


@_on_tensor_device
def routing_probability_sum(logits, mode):
    """fp32 `[E]`: column sums of softmax(logits) (or of the per-token normalised sigmoid scores
    for mode "sigmoid_noaux_tc") over the rows of fp32 `logits [T, E]`; bitwise repeatable."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise NativeError("logits must be fp32 [tokens, experts] with unit inner stride")
    tokens, experts = logits.shape
    out = torch.empty(experts, dtype=torch.float32, device=logits.device)
    nbytes = lib.b200moe_routing_probability_sum_workspace_bytes(tokens, experts)
    workspace = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=logits.device)
    check(
        lib.b200moe_routing_probability_sum(logits.data_ptr(), logits.stride(0), tokens, experts,
                                            ROUTING_MODES[mode], workspace.data_ptr(), out.data_ptr(), _stream()),
        "routing_probability_sum",
    )
    _count(2)
    return out


@_on_tensor_device
def routing_gradient(logits, route_ids, route_weights, grad_route_weights, mode, *, grad_aux=None, frequency=None,
                     aux_scale=0.0, grad_probability_sum=None, out=None):
    """fp32 gradient of `logits [T, E]` (see `b200moe_routing_gradient`); `out` receives it when
    given (a row slice of a larger gradient, for per-sequence calls)."""
    device = _need_cuda(logits, route_ids, route_weights, grad_route_weights, grad_aux, frequency,
                        grad_probability_sum, out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise NativeError("logits must be fp32 [tokens, experts] with unit inner stride")
    tokens, experts = logits.shape
    top_k = route_ids.shape[1]
    if out is None:
        out = torch.empty((tokens, experts), dtype=torch.float32, device=device)
    as_f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()  # noqa: E731
    ids = route_ids if route_ids.dtype == torch.int32 and route_ids.is_contiguous() else \
        route_ids.to(torch.int32).contiguous()
    weights, grads = as_f32(route_weights), as_f32(grad_route_weights)
    grad_aux, frequency, grad_probability_sum = as_f32(grad_aux), as_f32(frequency), as_f32(grad_probability_sum)
    if tokens:
        check(
            lib.b200moe_routing_gradient(
                logits.data_ptr(), logits.stride(0), tokens, experts, top_k, ROUTING_MODES[mode], ids.data_ptr(),
                _ptr(weights), grads.data_ptr(), _ptr(grad_aux), _ptr(frequency), float(aux_scale),
                _ptr(grad_probability_sum), out.data_ptr(), out.stride(0), _stream(),
            ),
            "routing_gradient",
        )
        _count()
    return out


@_on_tensor_device
def sort_assignments(route_ids, experts):
    """(order int32 [R], offsets int32 [E+1], slots int32 [T,K], counts int64 [E])."""
    _need_cuda(route_ids)
    flat = route_ids.reshape(-1)
    if flat.dtype != torch.int32 or not flat.is_contiguous():
        flat = flat.to(torch.int32).contiguous()
    n = flat.numel()
    device = flat.device
    order = torch.empty(n, dtype=torch.int32, device=device)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=device)
    slots = torch.empty(n, dtype=torch.int32, device=device)
    counts = torch.empty(experts, dtype=torch.int64, device=device)
    nbytes = lib.b200moe_sort_assignments_workspace_bytes(n, experts)
    workspace = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=device)
    check(
        lib.b200moe_sort_assignments(
            flat.data_ptr(), n, experts, order.data_ptr(), offsets.data_ptr(), slots.data_ptr(),
            counts.data_ptr(), workspace.data_ptr(), status_block(device).data_ptr(), _stream(),
        ),
        "sort_assignments",
    )
    _count(3 if n > 0 else 1)
    return order, offsets, slots.view(route_ids.shape), counts


@_on_tensor_device
def sort_assignments_static(route_ids, experts, order, offsets, slots, counts):
    """`sort_assignments` into caller-provided outputs, using the library's built-in scratch
    instead of a workspace: for callers that cannot allocate (all device memory owned by their
    own arena, or a call site where the CUDA allocator must not run). Nothing is allocated
    here. Limit: ceil(assignments / 4096) * experts <= 262144. Calls share the scratch, so
    keep them ordered on one stream; the first call on a device should happen outside stream
    capture. `route_ids` must be contiguous int32."""
    _need_cuda(route_ids, order, offsets, slots, counts)
    if route_ids.dtype != torch.int32 or not route_ids.is_contiguous():
        raise NativeError("route_ids must be contiguous int32 (no copy is made here)")
    check(
        lib.b200moe_sort_assignments_static(
            route_ids.data_ptr(), route_ids.numel(), experts, order.data_ptr(), offsets.data_ptr(),
            slots.data_ptr(), _ptr(counts), status_block(route_ids.device).data_ptr(), _stream(),
        ),
        "sort_assignments_static",
    )
    _count(3 if route_ids.numel() > 0 else 1)


# ------------------------------------------------------------------------ quantisation
def _scale_buffer(rows, blocks, device):
    """Scales are stored block-major ([blocks, rows]) so that the GEMM epilogue's 32
    lanes read 32 consecutive floats; the returned view is [rows, blocks]."""
    return torch.empty((blocks, max(rows, 1)), dtype=torch.float32, device=device)[:, :rows].t()


@_on_tensor_device
def quantize_rows(x, *, gather=None, gather_div=1, mode="1x128", with_copy=False, copy_out=None):
    """E4M3 rows and fp32 scales of bf16 `x [T, D]`; output row r reads input row
    `gather[r] // gather_div`. Returns (q [R, D] float8_e4m3fn, scales [R, blocks]); with
    `with_copy` also the gathered bf16 rows themselves, written by the same pass (into
    `copy_out [R, D]` when given)."""
    _need_cuda(x, gather)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise NativeError("x must be bf16 [rows, width] with unit inner stride")
    rows = x.shape[0] if gather is None else gather.numel()
    width = x.shape[1]
    q = torch.empty((rows, width), dtype=FP8, device=x.device)
    blocks = (width + 127) // 128 if mode == "1x128" else 1
    scales = _scale_buffer(rows, blocks, x.device)
    copy = None
    if copy_out is not None:
        if copy_out.shape != (rows, width) or copy_out.dtype != torch.bfloat16 or copy_out.stride(1) != 1:
            raise NativeError("copy_out must be bf16 [rows, width] with unit inner stride")
        copy, with_copy = copy_out, True
    elif with_copy:
        copy = torch.empty((rows, width), dtype=torch.bfloat16, device=x.device)
    if rows == 0:
        return (q, scales, copy) if with_copy else (q, scales)
    check(
        lib.b200moe_quantize_rows(
            x.data_ptr(), x.stride(0), x.shape[0], _ptr(gather), int(gather_div), rows, width, q.data_ptr(),
            q.stride(0), scales.data_ptr(), scales.stride(0), scales.stride(1),
            0 if mode == "1x128" else 1, _ptr(copy), width if copy is None else copy.stride(0),
            status_block(x.device).data_ptr(), _stream(),
        ),
        "quantize_rows",
    )
    _count()
    return (q, scales, copy) if with_copy else (q, scales)


@_on_tensor_device
def quantize_rows_scatter(x, slots, *, with_copy=False):
    """`quantize_rows(x, gather=order, gather_div=K)` computed from the token's side: every row
    of bf16 `x [T, D]` is quantised once (1x128 scales) and written to the K rows `slots[t, :]`
    (the sort's inverse permutation, int32 `[T, K]`). Returns `(q [T*K, D], scales [T*K, blocks])`
    and, with `with_copy`, the bf16 rows in the same order."""
    _need_cuda(x, slots)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise NativeError("x must be bf16 [rows, width] with unit inner stride")
    if slots.dtype != torch.int32 or slots.dim() != 2 or slots.shape[0] != x.shape[0] or not slots.is_contiguous():
        raise NativeError("slots must be contiguous int32 [rows of x, fan-out]")
    tokens, width = x.shape
    fanout = slots.shape[1]
    rows = tokens * fanout
    q = torch.empty((rows, width), dtype=FP8, device=x.device)
    scales = _scale_buffer(rows, (width + 127) // 128, x.device)
    copy = torch.empty((rows, width), dtype=torch.bfloat16, device=x.device) if with_copy else None
    if rows:
        check(
            lib.b200moe_quantize_rows_scatter(
                x.data_ptr(), x.stride(0), tokens, slots.data_ptr(), fanout, rows, width, q.data_ptr(), q.stride(0),
                scales.data_ptr(), scales.stride(0), scales.stride(1), _ptr(copy),
                width if copy is None else copy.stride(0), status_block(x.device).data_ptr(), _stream(),
            ),
            "quantize_rows_scatter",
        )
        _count()
    return (q, scales, copy) if with_copy else (q, scales)


@_on_tensor_device
def swiglu_quantize(h13, *, limit=None, quantized=True, rounded=False):
    """SwiGLU of h13 = [gate | up]. Returns (act_q, scales, act_bf16); entries not asked
    for are None."""
    _need_cuda(h13)
    rows, two_f = h13.shape
    width = two_f // 2
    device = h13.device
    act_q = scales = act = None
    if quantized:
        act_q = torch.empty((rows, width), dtype=FP8, device=device)
        scales = _scale_buffer(rows, (width + 127) // 128, device)
    if rounded:
        act = torch.empty((rows, width), dtype=torch.bfloat16, device=device)
    if rows == 0:
        return act_q, scales, act
    check(
        lib.b200moe_swiglu_quantize(
            h13.data_ptr(), h13.stride(0), rows, width, _ptr(act_q), width, _ptr(scales),
            0 if scales is None else scales.stride(0), 0 if scales is None else scales.stride(1),
            _ptr(act), width, 0.0 if limit is None else float(limit), 0 if limit is None else 1,
            _stream(),
        ),
        "swiglu_quantize",
    )
    _count()
    return act_q, scales, act


@_on_tensor_device
def dswiglu_routed(h13, r, route_weights, order, *, limit=None, quantized=True, rounded=False,
                   scaled_activation=False, rounded_out=None, scaled_out=None):
    """One pass over h13 and r: returns (dscore [rows] fp32, grad_h13_q, grad_h13_scales,
    grad_h13_bf16, act_scaled)."""
    _need_cuda(h13, r, route_weights, order)
    rows, two_f = h13.shape
    width = two_f // 2
    device = h13.device
    dscore = torch.empty(rows, dtype=torch.float32, device=device)
    gq = gs = gb = a_s = None
    if quantized:
        gq = torch.empty((rows, two_f), dtype=FP8, device=device)
        gs = _scale_buffer(rows, (two_f + 127) // 128, device)
    if rounded:
        gb = torch.empty((rows, two_f), dtype=torch.bfloat16, device=device) if rounded_out is None else rounded_out
    if scaled_activation:
        a_s = torch.empty((rows, width), dtype=torch.bfloat16, device=device) if scaled_out is None else scaled_out
    weights_flat = route_weights.reshape(-1)
    if rows == 0:
        return dscore, gq, gs, gb, a_s
    check(
        lib.b200moe_dswiglu_routed(
            h13.data_ptr(), h13.stride(0), r.data_ptr(), r.stride(0), weights_flat.data_ptr(),
            weights_flat.numel(), order.data_ptr(), rows, width, dscore.data_ptr(), _ptr(gq), two_f, _ptr(gs),
            0 if gs is None else gs.stride(0), 0 if gs is None else gs.stride(1), _ptr(gb),
            two_f if gb is None else gb.stride(0), _ptr(a_s), width if a_s is None else a_s.stride(0),
            0.0 if limit is None else float(limit), 0 if limit is None else 1,
            status_block(device).data_ptr(), _stream(),
        ),
        "dswiglu_routed",
    )
    _count()
    return dscore, gq, gs, gb, a_s


@_on_tensor_device
def quantize_blocks(weight):
    """(data E4M3 [E,out,in], scale fp32 [E, ceil(out/128), ceil(in/128)]) of a bf16 or
    fp32 weight."""
    _need_cuda(weight)
    if weight.dim() != 3:
        raise NativeError("Expected an [experts, out, in] weight")
    weight = weight.contiguous()
    if weight.dtype not in (torch.bfloat16, torch.float32):
        weight = weight.float()
    experts, out, inner = weight.shape
    data = torch.empty(weight.shape, dtype=FP8, device=weight.device)
    scale = torch.empty(
        (experts, (out + 127) // 128, (inner + 127) // 128), dtype=torch.float32, device=weight.device
    )
    check(
        lib.b200moe_quantize_blocks(
            weight.data_ptr(), 1 if weight.dtype == torch.float32 else 0, experts, out, inner,
            data.data_ptr(), scale.data_ptr(), _stream(),
        ),
        "quantize_blocks",
    )
    _count()
    return data, scale


# ------------------------------------------------------------------------------- GEMMs
@_on_tensor_device
def grouped_gemm_fp8(a_q, a_scale, b_q, b_scale, offsets, *, b_mn_major=False, block_n=256, out=None,
                     addend=None, row_map=None):
    """bf16 `[rows, N]` of the grouped block-FP8 product. `b_q` is `[G, N, K]`
    (`b_mn_major=False`) or `[G, K, N]` read along its rows (`b_mn_major=True`);
    `a_scale` is `[rows, K/128]` (any strides) or `[rows]`/`[rows, 1]` for one scale per row.
    `row_map` (int32 `[rows]`, a permutation) stores product row r at `out[row_map[r]]`."""
    device = _need_cuda(a_q, a_scale, b_q, b_scale, offsets, addend, row_map)
    rows, k = a_q.shape
    weights = b_q.shape[0]
    groups = offsets.numel() - 1  # a multiple of `weights`: group g multiplies weight g % weights
    n = b_q.shape[2] if b_mn_major else b_q.shape[1]
    kb = b_q.shape[1] if b_mn_major else b_q.shape[2]
    if kb != k:
        raise NativeError(f"contraction sizes differ: A has {k}, B has {kb}")
    if not b_q.is_contiguous() or not b_scale.is_contiguous():
        raise NativeError("weights and their scales must be contiguous")
    if a_scale.dim() == 1:
        a_scale = a_scale.unsqueeze(1)
    kblocks = (k + 127) // 128
    if a_scale.shape[1] == 1:
        as_kb = 0  # one scale per row, applied to every K block
    elif a_scale.shape[1] == kblocks:
        as_kb = a_scale.stride(1)
    else:
        raise NativeError("a_scale must have 1 or ceil(K/128) columns")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
    if rows == 0:
        return out
    with _Timed("fp8", 2.0 * rows * n * k):
        if row_map is None:
            check(
                lib.b200moe_grouped_gemm_fp8(
                    a_q.data_ptr(), a_q.stride(0), a_scale.data_ptr(), a_scale.stride(0), as_kb,
                    b_q.data_ptr(), b_scale.data_ptr(), out.data_ptr(), out.stride(0), _ptr(addend),
                    0 if addend is None else addend.stride(0), offsets.data_ptr(),
                    groups, weights, rows, n, k, 1 if b_mn_major else 0, int(block_n),
                    status_block(device).data_ptr(), _stream(),
                ),
                "grouped_gemm_fp8",
            )
        else:
            if row_map.dtype != torch.int32 or row_map.numel() != rows or not row_map.is_contiguous():
                raise NativeError("row_map must be a contiguous int32 vector with one entry per row")
            check(
                lib.b200moe_grouped_gemm_fp8_scatter(
                    a_q.data_ptr(), a_q.stride(0), a_scale.data_ptr(), a_scale.stride(0), as_kb,
                    b_q.data_ptr(), b_scale.data_ptr(), out.data_ptr(), out.stride(0), row_map.data_ptr(),
                    _ptr(addend), 0 if addend is None else addend.stride(0), offsets.data_ptr(),
                    groups, weights, rows, n, k, 1 if b_mn_major else 0, int(block_n),
                    status_block(device).data_ptr(), _stream(),
                ),
                "grouped_gemm_fp8_scatter",
            )
    _count()
    return out


@_on_tensor_device
def grouped_gemm_fp8_combine(a_q, a_scale, b_q, b_scale, offsets, order, route_weights, tokens, *,
                             residual=None, addend=None):
    """Down projection with the combine fused into its store: returns bf16 `[tokens, N]` =
    `residual + sum over the token's assignments of weight * bf16(product row)`. The sum is
    formed with fp32 atomics in arrival order, so it is not bitwise repeatable (the unfused
    `grouped_gemm_fp8` + `combine` is). `order [rows]` is the sort's permutation (assignment
    index of every expert-order row), `route_weights [tokens, K]` fp32."""
    device = _need_cuda(a_q, a_scale, b_q, b_scale, offsets, order, route_weights, residual, addend)
    rows, k = a_q.shape
    weights = b_q.shape[0]
    groups = offsets.numel() - 1
    n = b_q.shape[1]
    if b_q.shape[2] != k:
        raise NativeError(f"contraction sizes differ: A has {k}, B has {b_q.shape[2]}")
    if not b_q.is_contiguous() or not b_scale.is_contiguous():
        raise NativeError("weights and their scales must be contiguous")
    if a_scale.dim() == 1:
        a_scale = a_scale.unsqueeze(1)
    kblocks = (k + 127) // 128
    as_kb = 0 if a_scale.shape[1] == 1 else a_scale.stride(1)
    if a_scale.shape[1] not in (1, kblocks):
        raise NativeError("a_scale must have 1 or ceil(K/128) columns")
    top_k = route_weights.shape[1]
    row_token = torch.div(order, top_k, rounding_mode="floor").to(torch.int32)
    row_weight = route_weights.reshape(-1).float()[order.long()].contiguous()
    sums = torch.zeros((tokens, n), dtype=torch.float32, device=device)
    out = torch.empty((tokens, n), dtype=torch.bfloat16, device=device)
    if rows:
        with _Timed("fp8", 2.0 * rows * n * k):
            check(
                lib.b200moe_grouped_gemm_fp8_combine(
                    a_q.data_ptr(), a_q.stride(0), a_scale.data_ptr(), a_scale.stride(0), as_kb,
                    b_q.data_ptr(), b_scale.data_ptr(), sums.data_ptr(), sums.stride(0), tokens,
                    row_token.data_ptr(), row_weight.data_ptr(), _ptr(addend),
                    0 if addend is None else addend.stride(0), offsets.data_ptr(), groups, weights, rows, n, k,
                    0, status_block(device).data_ptr(), _stream(),
                ),
                "grouped_gemm_fp8_combine",
            )
        _count()
    if tokens:
        check(
            lib.b200moe_finish_combine(
                sums.data_ptr(), sums.stride(0), _ptr(residual), 0 if residual is None else residual.stride(0),
                out.data_ptr(), out.stride(0), tokens, n, _stream(),
            ),
            "finish_combine",
        )
        _count()
    return out


@_on_tensor_device
def grouped_gemm_fp8_swiglu(a_q, a_scale, w13_q, w13_scale, offsets, *, limit=None, out=None):
    """Up projection with the SwiGLU epilogue fused. Returns `(h13 bf16 [rows, 2F], act_q E4M3
    [rows, F], act_scale [rows, F/128])`: the same three tensors as `grouped_gemm_fp8` followed
    by `swiglu_quantize`, from one kernel."""
    device = _need_cuda(a_q, a_scale, w13_q, w13_scale, offsets)
    rows, k = a_q.shape
    weights, two_f, kb = w13_q.shape
    if kb != k or two_f % 256:
        raise NativeError("w13 must be [E, 2F, K] with F a multiple of 128")
    width = two_f // 2
    groups = offsets.numel() - 1
    if a_scale.dim() == 1:
        a_scale = a_scale.unsqueeze(1)
    as_kb = 0 if a_scale.shape[1] == 1 else a_scale.stride(1)
    h13 = torch.empty((rows, two_f), dtype=torch.bfloat16, device=device) if out is None else out
    act_q = torch.empty((rows, width), dtype=FP8, device=device)
    scales = _scale_buffer(rows, width // 128, device)
    if rows == 0:
        return h13, act_q, scales
    with _Timed("fp8", 2.0 * rows * two_f * k):
        check(
            lib.b200moe_grouped_gemm_fp8_swiglu(
                a_q.data_ptr(), a_q.stride(0), a_scale.data_ptr(), a_scale.stride(0), as_kb, w13_q.data_ptr(),
                w13_scale.data_ptr(), h13.data_ptr(), h13.stride(0), act_q.data_ptr(), act_q.stride(0),
                scales.data_ptr(), scales.stride(0), scales.stride(1), offsets.data_ptr(), groups, weights, rows,
                width, k, 0.0 if limit is None else float(limit), 0 if limit is None else 1,
                status_block(device).data_ptr(), _stream(),
            ),
            "grouped_gemm_fp8_swiglu",
        )
    _count()
    return h13, act_q, scales


@_on_tensor_device
def grouped_wgrad(g, x, offsets, groups, out_dtype=torch.bfloat16, *, accumulate_into=None, scale=1.0):
    """`[G, M, N]` with `out[e] = g[rows_e].T @ x[rows_e]` (bf16 operands, fp32 sums).
    `offsets` has `segments * groups + 1` entries; expert e sums over the ranges
    `offsets[s*groups+e] .. offsets[s*groups+e+1]`. With `accumulate_into` (a contiguous bf16 or
    fp32 `[G, M, N]` buffer, e.g. a parameter's `.grad`) the product, times `scale`, is added to
    the buffer in the GEMM's store and the buffer is returned."""
    device = _need_cuda(g, x, offsets, accumulate_into)
    rows, m = g.shape
    n = x.shape[1]
    segments = (offsets.numel() - 1) // groups
    if accumulate_into is not None:
        out = accumulate_into
        if tuple(out.shape) != (groups, m, n) or not out.is_contiguous() or \
                out.dtype not in (torch.bfloat16, torch.float32):
            raise NativeError(f"accumulate_into must be a contiguous bf16 or fp32 [{groups}, {m}, {n}] tensor")
        if rows:
            with _Timed("wgrad_bf16", 2.0 * rows * m * n):
                check(
                    lib.b200moe_grouped_wgrad_bf16_accumulate(
                        g.data_ptr(), g.stride(0), x.data_ptr(), x.stride(0), offsets.data_ptr(), groups, segments,
                        rows, m, n, out.data_ptr(), 1 if out.dtype == torch.float32 else 0, float(scale),
                        status_block(device).data_ptr(), _stream(),
                    ),
                    "grouped_wgrad_accumulate",
                )
            _count()
        return out
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise NativeError("weight gradients are written as bf16 or fp32")
    if rows == 0:
        return torch.zeros((groups, m, n), dtype=out_dtype, device=device)
    out = torch.empty((groups, m, n), dtype=out_dtype, device=device)
    with _Timed("wgrad_bf16", 2.0 * rows * m * n):
        check(
            lib.b200moe_grouped_wgrad_bf16(
                g.data_ptr(), g.stride(0), x.data_ptr(), x.stride(0), offsets.data_ptr(), groups, segments, rows,
                m, n, out.data_ptr(), 1 if out_dtype == torch.float32 else 0,
                status_block(device).data_ptr(), _stream(),
            ),
            "grouped_wgrad",
        )
    _count()
    if scale != 1.0:
        out.mul_(scale)
    return out


@_on_tensor_device
def grouped_gemm_bf16(a, b, offsets, *, b_mn_major=False, addend=None, alpha=1.0):
    """`out[rows_e] = a[rows_e] @ op(b[e])` in bf16 with fp32 sums. `b` is `[E, N, K]` (K-major: the
    stored `nn.Linear` weight, `y = x W^T`) or, with `b_mn_major`, `[E, K, N]` read along its rows
    (`dx = dy W` on the same stored weight). More groups than weights: group g uses `b[g % E]`."""
    device = _need_cuda(a, b, offsets, addend)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.stride(1) != 1 or not b.is_contiguous():
        raise NativeError("a must be bf16 rows with unit inner stride and b a contiguous bf16 [experts, ., .] tensor")
    rows, k = a.shape
    weights = b.shape[0]
    n = b.shape[2] if b_mn_major else b.shape[1]
    if (b.shape[1] if b_mn_major else b.shape[2]) != k:
        raise NativeError("inner dimensions of a and b differ")
    groups = offsets.numel() - 1
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
    if rows:
        with _Timed("gemm_bf16", 2.0 * rows * n * k):
            check(
                lib.b200moe_grouped_gemm_bf16(
                    a.data_ptr(), a.stride(0), b.data_ptr(), out.data_ptr(), out.stride(0), _ptr(addend),
                    0 if addend is None else addend.stride(0), offsets.data_ptr(), groups, weights, rows, n, k,
                    1 if b_mn_major else 0, float(alpha), status_block(device).data_ptr(), _stream(),
                ),
                "grouped_gemm_bf16",
            )
        _count()
    return out


@_on_tensor_device
def build_copies(keys, weights, world, local, send_copies):
    """The sender's plan of a de-duplicated dispatch in one launch: `(token [copies] int32, meta
    [copies, 2K] int32 = [local expert ids or -1 | route-weight bits], token_copies [tokens, world]
    int32)`. `keys [tokens, K]` int32 placement keys (rank = key // local), `weights [tokens, K]`
    fp32, `send_copies`: copies per destination rank (host integers, from the plan)."""
    import ctypes

    device = _need_cuda(keys, weights)
    if keys.dtype != torch.int32 or weights.dtype != torch.float32 or not keys.is_contiguous() \
            or not weights.is_contiguous():
        raise NativeError("keys must be contiguous int32 [tokens, K] and weights contiguous fp32 [tokens, K]")
    tokens, top_k = keys.shape
    starts = [0]
    for v in send_copies:
        starts.append(starts[-1] + int(v))
    copies = starts[-1]
    token = torch.empty(copies, dtype=torch.int32, device=device)
    meta = torch.empty((copies, 2 * top_k), dtype=torch.int32, device=device)
    token_copies = torch.empty((tokens, world), dtype=torch.int32, device=device)
    check(
        lib.b200moe_build_copies(keys.data_ptr(), weights.data_ptr(), tokens, top_k, world, local,
                                 (ctypes.c_int32 * (world + 1))(*starts), token.data_ptr(), meta.data_ptr(),
                                 token_copies.data_ptr(), status_block(device).data_ptr(), _stream()),
        "build_copies",
    )
    _count()
    return token, meta, token_copies


def peer_dispatch_rows(src, gather, dest_ptrs, dest_pitch, dest_rows, send_start, dest_row0, *, stream=None):
    """Gather + transfer of an expert-parallel dispatch in one kernel: send row i is
    `src[gather[i]]` (bf16); rows `[send_start[r], send_start[r+1])` go, in order, to rows
    `dest_row0[r]...` of the arena at `dest_ptrs[r]` (device addresses valid in this process: the
    peers' symmetric-memory buffers). Plain stores over NVLink; the caller orders the ranks
    afterwards. `stream`: the torch stream to launch on (default: the current one)."""
    import ctypes

    device = _need_cuda(src, gather)
    if src.dtype != torch.bfloat16 or src.stride(1) != 1 or gather.dtype != torch.int32:
        raise NativeError("src must be bf16 rows with unit inner stride, gather int32")
    world = len(dest_ptrs)
    rows = gather.numel()
    if len(send_start) != world + 1 or len(dest_row0) != world:
        raise NativeError("send_start needs world + 1 entries and dest_row0 world entries")
    ptrs = (ctypes.c_void_p * world)(*[int(p) for p in dest_ptrs])
    starts = (ctypes.c_int32 * (world + 1))(*[int(v) for v in send_start])
    row0 = (ctypes.c_longlong * world)(*[int(v) for v in dest_row0])
    with torch.cuda.device(device):
        launch_stream = (torch.cuda.current_stream() if stream is None else stream).cuda_stream
        check(
            lib.b200moe_peer_dispatch_rows(src.data_ptr(), src.stride(0), src.shape[0], gather.data_ptr(), rows,
                                           src.shape[1], ptrs, int(dest_pitch), int(dest_rows), starts, row0, world,
                                           status_block(device).data_ptr(), launch_stream),
            "peer_dispatch_rows",
        )
    _count()


@_on_tensor_device
def quantize_columns(x, offsets, groups):
    """Column-scaled E4M3 of bf16 rows `x [rows, width]`: one scale per (group, column) over the
    group's rows, `scale = max(amax * fp32(1/448), 1e-12)`. Returns `(q [rows, width] E4M3,
    scales [groups, width] fp32)`; `offsets` as for `grouped_wgrad` (segments * groups + 1)."""
    device = _need_cuda(x, offsets)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise NativeError("x must be bf16 [rows, width] with unit inner stride")
    rows, width = x.shape
    segments = (offsets.numel() - 1) // groups
    q = torch.empty((rows, width), dtype=FP8, device=device)
    scales = torch.empty((groups, width), dtype=torch.float32, device=device)
    check(
        lib.b200moe_quantize_columns(x.data_ptr(), x.stride(0), rows, width, offsets.data_ptr(), groups, segments,
                                     q.data_ptr(), q.stride(0), scales.data_ptr(), _stream()),
        "quantize_columns",
    )
    _count(3)
    return q, scales


@_on_tensor_device
def grouped_wgrad_fp8(g_q, g_scale, x_q, x_scale, offsets, groups, out_dtype=torch.bfloat16, *,
                      accumulate_into=None, scale=1.0):
    """`[G, M, N]` with `out[e] = (g_scale[e][:, None] * x_scale[e][None, :]) * (g_q[rows_e].T @ x_q[rows_e])`
    from column-scaled E4M3 operands (`quantize_columns`), fp32 sums over all of an expert's rows."""
    device = _need_cuda(g_q, g_scale, x_q, x_scale, offsets, accumulate_into)
    rows, m = g_q.shape
    n = x_q.shape[1]
    segments = (offsets.numel() - 1) // groups
    if accumulate_into is not None:
        out = accumulate_into
        if tuple(out.shape) != (groups, m, n) or not out.is_contiguous() or \
                out.dtype not in (torch.bfloat16, torch.float32):
            raise NativeError(f"accumulate_into must be a contiguous bf16 or fp32 [{groups}, {m}, {n}] tensor")
    else:
        if out_dtype not in (torch.bfloat16, torch.float32):
            raise NativeError("weight gradients are written as bf16 or fp32")
        out = torch.empty((groups, m, n), dtype=out_dtype, device=device)
    with _Timed("wgrad_fp8", 2.0 * rows * m * n):
        check(
            lib.b200moe_grouped_wgrad_fp8(
                g_q.data_ptr(), g_q.stride(0), g_scale.data_ptr(), x_q.data_ptr(), x_q.stride(0), x_scale.data_ptr(),
                offsets.data_ptr(), groups, segments, rows, m, n, out.data_ptr(),
                1 if out.dtype == torch.float32 else 0, float(scale), 1 if accumulate_into is not None else 0,
                status_block(device).data_ptr(), _stream(),
            ),
            "grouped_wgrad_fp8",
        )
    _count()
    return out


# B200MOE_LORA_SIMT=1: the rank-r products of expert LoRA on the SIMT kernels (csrc/lora.cu) instead
# of the tensor-core grouped GEMM
_LORA_TENSOR_CORES = os.environ.get("B200MOE_LORA_SIMT", "0") != "1"


@_on_tensor_device
def lora_project(x, factor, offsets, *, rank_major):
    """`t [rows, r] = x[row] . factor[expert(row)]`; factor `[E, r, K]` (`rank_major`) or `[E, K, r]`."""
    device = _need_cuda(x, factor, offsets)
    rows, k = x.shape
    experts = factor.shape[0]
    rank = factor.shape[1] if rank_major else factor.shape[2]
    factor = factor.contiguous()
    if _LORA_TENSOR_CORES and rank % 8 == 0 and k % 8 == 0 and x.dtype == torch.bfloat16 and \
            factor.dtype == torch.bfloat16 and x.stride(1) == 1:
        # a GEMM with one narrow side: the bf16 grouped GEMM on the tensor cores (the TMA unit
        # zero-fills the unused part of the tile), memory-bound as it should be
        return grouped_gemm_bf16(x, factor, offsets, b_mn_major=not rank_major)
    out = torch.empty((rows, rank), dtype=torch.bfloat16, device=device)
    if rows == 0:
        return out
    check(
        lib.b200moe_lora_project(x.data_ptr(), x.stride(0), factor.data_ptr(), 1 if rank_major else 0,
                                 offsets.data_ptr(), experts, rows, k, rank, out.data_ptr(), out.stride(0),
                                 _stream()),
        "lora_project",
    )
    _count()
    return out


@_on_tensor_device
def lora_expand(t, factor, offsets, *, wide_major, scale=1.0):
    """`c [rows, N] = scale * t[row] . factor[expert(row)]`; factor `[E, N, r]` (`wide_major`) or
    `[E, r, N]`."""
    device = _need_cuda(t, factor, offsets)
    rows, rank = t.shape
    experts = factor.shape[0]
    n = factor.shape[1] if wide_major else factor.shape[2]
    factor = factor.contiguous()
    if _LORA_TENSOR_CORES and rank % 8 == 0 and n % 8 == 0 and t.dtype == torch.bfloat16 and \
            factor.dtype == torch.bfloat16 and t.stride(1) == 1:
        return grouped_gemm_bf16(t, factor, offsets, b_mn_major=not wide_major, alpha=scale)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
    if rows == 0:
        return out
    check(
        lib.b200moe_lora_expand(t.data_ptr(), t.stride(0), factor.data_ptr(), 1 if wide_major else 0,
                                offsets.data_ptr(), experts, rows, n, rank, float(scale), out.data_ptr(),
                                out.stride(0), _stream()),
        "lora_expand",
    )
    _count()
    return out


# ---------------------------------------------------------------------- permutation I/O
@_on_tensor_device
def combine(source, slots, weights, residual):
    """`residual + sum_k weights[:, k] * source[slots[:, k]]` as bf16 `[T, D]`."""
    device = _need_cuda(source, slots, weights, residual)
    tokens, top_k = slots.shape
    width = source.shape[1]
    out = torch.empty((tokens, width), dtype=torch.bfloat16, device=device)
    if tokens == 0:
        return out
    check(
        lib.b200moe_combine(
            source.data_ptr(), source.stride(0), source.shape[0], slots.data_ptr(), _ptr(weights),
            _ptr(residual), 0 if residual is None else residual.stride(0), out.data_ptr(),
            out.stride(0), tokens, width, top_k, _stream(),
        ),
        "combine",
    )
    _count()
    return out


def dispatch_backward(source, slots):
    """Scatter-sum of expert-ordered rows back to their tokens."""
    return combine(source, slots, None, None)


@_on_tensor_device
def dispatch(x, order, top_k):
    """bf16 rows of `x` in expert order: row j is `x[order[j] // top_k]`."""
    device = _need_cuda(x, order)
    rows = order.numel()
    out = torch.empty((rows, x.shape[1]), dtype=torch.bfloat16, device=device)
    if rows == 0:
        return out
    check(
        lib.b200moe_gather_rows(
            x.data_ptr(), x.stride(0), x.shape[0], order.data_ptr(), int(top_k), rows, x.shape[1],
            out.data_ptr(), out.stride(0), status_block(device).data_ptr(), _stream(),
        ),
        "dispatch",
    )
    _count()
    return out


@_on_tensor_device
def gather_scalar(values, slots):
    """`values[slots]` (fp32), shaped like `slots`."""
    _need_cuda(values, slots)
    out = torch.empty(slots.shape, dtype=torch.float32, device=values.device)
    check(
        lib.b200moe_gather_scalar(
            values.data_ptr(), values.numel(), slots.data_ptr(), slots.numel(), out.data_ptr(),
            status_block(values.device).data_ptr(), _stream()
        ),
        "gather_scalar",
    )
    _count()
    return out
