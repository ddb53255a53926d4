"""Expert parallelism for the routed layer: experts sharded over the ranks of one process
group, token rows exchanged with NCCL all-to-all over NVLink.

Behavioural model: the reference's expert-parallel layer
(`src/mlops/expert_parallel/quack/layer.py:28-281`, runtime `quack/runtime.py:198-441`):
rank g owns `E/G` experts and its own `T` tokens; a forward pass dispatches every routed row
to the rank that owns its expert, runs the expert math there and combines the rows back at
the token's owner; the backward pass sends `dy` rows along the saved plan and returns `dx`
rows and the route-weight gradients. Expert weight gradients stay local; replicated
parameters (router, shared expert) are reduced by the caller
(`synchronize_replicated_gradients`). The transport differs on purpose: the reference drives
MoonEP's peer-memory kernels, here rows land in local HBM through `all_to_all_single`
before any kernel of this library reads them, and the rows of a rank arrive as
`[source rank][local expert]` segments that the GEMMs consume directly (weight index =
segment % local experts; weight gradients sum over the segments of an expert).

The exchange plan needs the per-rank row counts on the host (split sizes of the collective):
one small device-to-host copy per forward pass; the backward pass reuses the plan.

Everything that only plans or moves rows (`ExchangePlan`, `make_plan`, `exchange`) works on
CPU tensors with a gloo group as well, which is how its tests run without a GPU.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ExpertParallelConfig:
    hidden: int
    experts: int
    intermediate: int
    top_k: int
    routing_mode: str = "softmax_then_topk"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling: float = 1.0
    swiglu_limit: float | None = None
    expert_map: str = "contiguous"  # "contiguous": expert e on rank e // (E/G); "strided": rank e % G

    def validate(self, world: int) -> None:
        if self.experts % world:
            raise ValueError(f"experts ({self.experts}) must divide evenly over {world} ranks")
        if world > 128 or self.top_k > 32:
            raise ValueError("supported: at most 128 ranks and top_k <= 32")
        if self.hidden % 128 or self.intermediate % 128:
            raise ValueError("hidden and intermediate must be multiples of 128")
        if self.expert_map not in ("contiguous", "strided"):
            raise ValueError(f"unknown expert_map {self.expert_map!r}")
        if not 0 < self.top_k <= self.experts:
            raise ValueError("top_k must be within the expert count")


def handshake(config: ExpertParallelConfig, group) -> None:
    """Every rank must hold the same configuration; a mismatch raises on every rank before
    any kernel is launched (reference: quack/runtime_resources.py:36-40)."""
    world = dist.get_world_size(group)
    config.validate(world)
    gathered = [None] * world
    dist.all_gather_object(gathered, asdict(config), group=group)
    if any(other != gathered[0] for other in gathered):
        raise RuntimeError(f"expert-parallel configurations differ across ranks: {gathered}")


def placement(config: ExpertParallelConfig, world: int, device=None) -> torch.Tensor:
    """`key[e]` = rank(e) * (E/G) + local index(e): sorting assignments by key groups them by
    destination rank, then by local expert."""
    experts, local = config.experts, config.experts // world
    e = torch.arange(experts, device=device)
    if config.expert_map == "contiguous":
        return e.to(torch.int32)
    return ((e % world) * local + e // world).to(torch.int32)


@dataclass
class ExchangePlan:
    send_splits: list[int]        # rows this rank sends to each rank
    recv_splits: list[int]        # rows this rank receives from each rank
    segment_offsets: torch.Tensor  # int32 [G * E/G + 1]: received rows as [source][local expert]
    recv_rows: int
    send_rows: int


def make_plan(send_counts: torch.Tensor, group) -> ExchangePlan:
    """`send_counts [E]`: rows per placement key held by this rank (any integer dtype, on the
    group's device). One all-to-all of the counts, one host read of the split sizes."""
    world = dist.get_world_size(group)
    local = send_counts.numel() // world
    mine = send_counts.to(torch.int64).view(world, local).contiguous()
    theirs = torch.empty_like(mine)
    dist.all_to_all_single(theirs, mine, group=group)
    sizes = torch.stack([mine.sum(1), theirs.sum(1)]).cpu()  # the one device-to-host copy
    send_splits, recv_splits = sizes[0].tolist(), sizes[1].tolist()
    offsets = torch.zeros(world * local + 1, dtype=torch.int32, device=send_counts.device)
    offsets[1:] = theirs.reshape(-1).cumsum(0).to(torch.int32)
    return ExchangePlan(send_splits, recv_splits, offsets, int(sum(recv_splits)), int(sum(send_splits)))


def exchange(rows: torch.Tensor, plan: ExchangePlan, group, *, back: bool = False, async_op: bool = False):
    """Dispatch (`back=False`: send my sorted rows, receive the rows of my experts) or return
    (`back=True`: the inverse). Returns `(received, work)`; `work` is None unless `async_op`."""
    send, recv = (plan.recv_splits, plan.send_splits) if back else (plan.send_splits, plan.recv_splits)
    total = plan.send_rows if back else plan.recv_rows
    received = torch.empty((total, *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    payload, target = rows, received
    if rows.dtype == torch.float8_e4m3fn:  # collectives move bytes
        payload, target = rows.view(torch.uint8), received.view(torch.uint8)
    work = dist.all_to_all_single(target, payload.contiguous(), output_split_sizes=recv, input_split_sizes=send,
                                  group=group, async_op=async_op)
    return received, (work if async_op else None)


class ExpertParallelMoE:
    """One expert-parallel MoE layer. `w13 = (data [E/G, 2F, D], scale)`, `w2 = (data
    [E/G, D, F], scale)` are this rank's shard; `router_weight [E, D]`, `router_bias` and the
    optional `shared = (w13 [2Fs, D], w2 [D, Fs])` bf16 pair are replicated.

    `forward` returns `(output, aux, counts, probability_sum, saved)`; `backward(saved, dy)`
    returns `dict(grad_x, grad_router, grad_w13, grad_w2, grad_shared_w13, grad_shared_w2)`
    with local expert gradients and UN-reduced replicated gradients."""

    def __init__(self, config: ExpertParallelConfig, ep_group, *, router_weight, w13, w2, router_bias=None,
                 shared=None, device=None, weight_grad_dtype=torch.bfloat16):
        self.config = config
        self.group = ep_group
        self.world = dist.get_world_size(ep_group)
        self.rank = dist.get_rank(ep_group)
        handshake(config, ep_group)
        self.local_experts = config.experts // self.world
        if w13[0].shape[0] != self.local_experts or w2[0].shape[0] != self.local_experts:
            raise ValueError("w13 / w2 must hold this rank's E/G experts")
        self.device = torch.device(device) if device is not None else w13[0].device
        self.router_weight, self.router_bias = router_weight, router_bias
        self.w13, self.w2, self.shared = w13, w2, shared
        self.weight_grad_dtype = weight_grad_dtype
        self.keys = placement(config, self.world, self.device)
        self.side_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.bytes_moved = 0
        self.last_recv_rows = 0
        self.profile = False  # when set, phase boundaries are marked with CUDA events
        self._marks = []

    # ------------------------------------------------------------------ reference API
    def expert_parameters(self):
        return [*self.w13, *self.w2]

    def replicated_parameters(self):
        extra = [] if self.shared is None else list(self.shared)
        bias = [] if self.router_bias is None else [self.router_bias]
        return [self.router_weight, *bias, *extra]

    def synchronize_replicated_parameters(self):
        for tensor in self.replicated_parameters():
            dist.broadcast(tensor, src=dist.get_global_rank(self.group, 0), group=self.group)

    @staticmethod
    def synchronize_replicated_gradients(gradients, group):
        """SUM all-reduce of the replicated parameters' gradients, called by the owner of the
        accumulation window; expert shards are never reduced over the EP group."""
        for tensor in gradients:
            if tensor is not None and tensor.numel():
                dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)

    def report(self):
        return dict(world=self.world, rank=self.rank, local_experts=self.local_experts,
                    expert_map=self.config.expert_map, transport="nccl all_to_all_single, bf16 rows",
                    bytes_moved=self.bytes_moved)

    def _mark(self, name):
        if self.profile:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            self._marks.append((name, event))

    def phase_times(self):
        """`[(phase, milliseconds)]` between consecutive marks of the profiled calls so far
        (synchronises); clears the marks."""
        torch.cuda.synchronize()
        marks, self._marks = self._marks, []
        return [(b[0], a[1].elapsed_time(b[1])) for a, b in zip(marks, marks[1:])]

    # ----------------------------------------------------------------------- forward
    def forward(self, x, residual=None, expert_ids=None, routing_weights=None):
        from . import layer, ops

        cfg = self.config
        with torch.no_grad():
            self._mark("start")
            flat = x.reshape(-1, x.shape[-1]).contiguous()
            tokens = flat.shape[0]
            base = torch.zeros_like(flat) if residual is None else residual.reshape_as(flat).contiguous()
            logits = layer.router_logits(flat, self.router_weight)
            if expert_ids is None:
                weights, ids = ops.route_topk(logits, cfg.top_k, cfg.routing_mode, bias=self.router_bias,
                                              n_group=cfg.n_group, topk_group=cfg.topk_group,
                                              routed_scaling=cfg.routed_scaling)
            else:
                ids = expert_ids.to(torch.int32).contiguous()
                weights = routing_weights.float().contiguous()
            keys = ids if cfg.expert_map == "contiguous" else self.keys[ids.long()]
            order, _offsets, slots, key_counts = ops.sort_assignments(keys, cfg.experts)
            self._mark("route+sort")
            plan = make_plan(key_counts, self.group)
            self.last_recv_rows = plan.recv_rows
            self._mark("plan")

            rows = ops.dispatch(flat, order, cfg.top_k)
            row_weights = weights.reshape(-1)[order.long()].contiguous()
            self._mark("gather rows")
            recv_x, work_x = exchange(rows, plan, self.group, async_op=True)
            recv_w, work_w = exchange(row_weights, plan, self.group, async_op=True)
            self.bytes_moved += rows.numel() * 2

            shared_h13 = None
            if self.shared is not None:  # overlaps the dispatch
                side = self.side_stream
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    y_shared, shared_h13 = layer.shared_expert_forward(flat, *self.shared,
                                                                       swiglu_limit=cfg.swiglu_limit)
                    base = base + y_shared
                for tensor in (base, shared_h13):  # produced on the side stream, consumed on this one
                    tensor.record_stream(torch.cuda.current_stream())
            work_x.wait()
            work_w.wait()
            self._mark("dispatch a2a (+shared fwd)")

            x_q, x_s = ops.quantize_rows(recv_x)
            h13 = ops.grouped_gemm_fp8(x_q, x_s, *self.w13, plan.segment_offsets)
            a_q, a_s, _ = ops.swiglu_quantize(h13, limit=cfg.swiglu_limit)
            y = ops.grouped_gemm_fp8(a_q, a_s, *self.w2, plan.segment_offsets)
            self._mark("expert fwd")
            y_back, _ = exchange(y, plan, self.group, back=True)
            self._mark("combine a2a")
            self.bytes_moved += y.numel() * 2
            if self.shared is not None:
                torch.cuda.current_stream().wait_stream(self.side_stream)
            output = ops.combine(y_back, slots, weights, base).reshape(x.shape)

            # the sort counted by placement key; statistics want expert order
            counts = key_counts if cfg.expert_map == "contiguous" else key_counts[self.keys.long()]
            aux, counts, psum = layer.routing_statistics(
                logits, ids, counts, routing_mode=cfg.routing_mode, lengths=(tokens,), experts=cfg.experts)
        self._mark("combine+stats")
        saved = dict(flat=flat, logits=logits, weights=weights, ids=ids, order=order, slots=slots, plan=plan,
                     recv_x=recv_x, recv_w=recv_w, h13=h13, shared_h13=shared_h13, counts=counts,
                     shape=x.shape)
        return output, aux, counts, psum, saved

    # ---------------------------------------------------------------------- backward
    def backward(self, saved, grad_output, grad_aux=None, grad_probability_sum=None, *, need_router=True,
                 need_experts=True):
        from . import layer, ops

        cfg = self.config
        plan = saved["plan"]
        with torch.no_grad():
            flat = saved["flat"]
            self._mark("bwd start")
            dy = grad_output.reshape_as(flat).contiguous()
            dy_rows = ops.dispatch(dy, saved["order"], cfg.top_k)
            self._mark("gather dy rows")
            recv_dy, work = exchange(dy_rows, plan, self.group, async_op=True)
            self.bytes_moved += dy_rows.numel() * 2
            shared_grads = (None, None, None)
            if self.shared is not None:  # overlaps the dispatch of dy
                side = self.side_stream
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    shared_grads = layer.shared_expert_backward(dy, flat, *self.shared, saved["shared_h13"],
                                                                swiglu_limit=cfg.swiglu_limit,
                                                                need_weights=need_experts)
                for tensor in shared_grads:
                    if tensor is not None:
                        tensor.record_stream(torch.cuda.current_stream())
            work.wait()
            self._mark("dy dispatch a2a (+shared bwd)")

            identity = torch.arange(plan.recv_rows, dtype=torch.int32, device=flat.device)
            dy_q, dy_s = ops.quantize_rows(recv_dy)
            r = ops.grouped_gemm_fp8(dy_q, dy_s, *self.w2, plan.segment_offsets, b_mn_major=True)
            dscore, gh_q, gh_s, gh_b, act_scaled = ops.dswiglu_routed(
                saved["h13"], r, saved["recv_w"], identity, limit=cfg.swiglu_limit, quantized=True,
                rounded=need_experts, scaled_activation=need_experts)
            grad_rows = ops.grouped_gemm_fp8(gh_q, gh_s, *self.w13, plan.segment_offsets, b_mn_major=True)
            self._mark("expert dgrad")
            back_rows, work_rows = exchange(grad_rows, plan, self.group, back=True, async_op=True)
            back_score, work_score = exchange(dscore, plan, self.group, back=True, async_op=True)
            self.bytes_moved += grad_rows.numel() * 2
            grad_w13 = grad_w2 = None
            if need_experts:  # local weight gradients overlap the return of dx rows
                grad_w2 = ops.grouped_wgrad(recv_dy, act_scaled, plan.segment_offsets, self.local_experts,
                                            self.weight_grad_dtype)
                grad_w13 = ops.grouped_wgrad(gh_b, saved["recv_x"], plan.segment_offsets, self.local_experts,
                                             self.weight_grad_dtype)
            self._mark("expert wgrad (issued)")
            work_rows.wait()
            work_score.wait()
            self._mark("dx return a2a (+wgrad)")
            grad_x = ops.dispatch_backward(back_rows, saved["slots"])
            grad_route_weights = ops.gather_scalar(back_score, saved["slots"])
            grad_logits = layer.routing_gradient(
                grad_aux, grad_probability_sum, grad_route_weights, saved["weights"], saved["ids"],
                saved["logits"], saved["counts"], routing_mode=cfg.routing_mode, lengths=(flat.shape[0],))
            grad_router = None
            if need_router:
                grad_router = layer._router_weight_gradient(grad_logits, flat, self.router_weight.dtype)
            grad_x.addmm_(grad_logits.to(flat.dtype), self.router_weight.to(flat.dtype))
            if self.shared is not None:
                torch.cuda.current_stream().wait_stream(self.side_stream)
                grad_x.add_(shared_grads[0])
        self._mark("scatter+router grads")
        return dict(grad_x=grad_x.reshape(saved["shape"]), grad_router=grad_router, grad_w13=grad_w13,
                    grad_w2=grad_w2, grad_shared_w13=shared_grads[1], grad_shared_w2=shared_grads[2])

    def forward_backward(self, x, residual, grad_output):
        output, aux, counts, _psum, saved = self.forward(x, residual)
        grads = self.backward(saved, grad_output)
        return output, grads["grad_x"], aux, counts

    def close(self):
        self.side_stream = None
