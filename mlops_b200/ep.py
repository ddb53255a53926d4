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
    # send a token once to every rank that holds any of its experts (with the list of those
    # experts) instead of once per expert; the receiver replicates.  Pays off when the experts of
    # a token cluster on few ranks: group-limited routing with a contiguous map (reference:
    # expert_parallel/quack/runtime.py:106, "dedup")
    dedup: bool = False
    # with `dedup`: the expert side forms, per received token copy, the route-weighted sum of the
    # copy's expert outputs (in slot order, fp32, one rounding) and returns ONE row per copy
    # instead of one per assignment; the owner adds the partial sums of a token in rank order.
    # The input gradient comes back the same way. The reference's layers return pre-weighted
    # rows likewise (kernels/quack_moe/fp8.py:41-45, 81-95). Halves the return exchanges when a
    # token's experts sit on half as many ranks as it has experts; the output then carries one
    # more bf16 rounding than the single-GPU layer (which sums all K rows before rounding).
    presum: bool = False
    # with `dedup`: how the token rows travel. "nccl": gathered into a send buffer, then an
    # all-to-all. "peer": ONE kernel per rank gathers the rows and writes them straight into the
    # destinations' receive arenas in NVLink peer memory (mlops_b200/peer.py); the small per-copy
    # metadata and the returns stay on the library all-to-all.
    transport: str = "nccl"

    def validate(self, world: int) -> None:
        if self.transport not in ("nccl", "peer"):
            raise ValueError(f"unknown transport {self.transport!r}")
        if self.transport == "peer" and not self.dedup:
            raise ValueError("the peer transport carries the de-duplicated dispatch: it needs dedup")
        if self.transport == "peer" and world > 16:
            raise ValueError("the peer transport serves at most 16 ranks")
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
        if self.presum and not self.dedup:
            raise ValueError("presum returns one row per token copy: it needs dedup")


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
    # de-duplicated dispatch: token copies instead of rows (None when not used)
    send_copies: list[int] | None = None
    recv_copies: list[int] | None = None
    recv_copies_device: torch.Tensor | None = None  # the same counts as an int64 device tensor


def copy_mask(keys: torch.Tensor, world: int, local: int) -> torch.Tensor:
    """`[tokens, world]` bool: the ranks that hold at least one of a token's experts
    (`keys [tokens, K]` are placement keys, rank = key // local)."""
    mask = torch.zeros((keys.shape[0], world), dtype=torch.bool, device=keys.device)
    mask.scatter_(1, torch.div(keys.long(), local, rounding_mode="floor"), True)
    return mask


def build_copies(mask: torch.Tensor, keys: torch.Tensor, weights: torch.Tensor, local: int, copies: int):
    """The sender's side of a de-duplicated dispatch. One copy per (rank, token) pair of `mask`,
    ordered by rank, then token. Returns `(token [copies] int32, ids [copies, K] int32,
    route_weight [copies, K] fp32, token_copies [tokens, world] int32)`: which token a copy is,
    for each of the token's K assignments the local expert on the copy's rank (-1: that
    assignment lives elsewhere) with its route weight, and for every token the position of its
    copy for each rank (-1: none). No host synchronisation: `copies` comes from the plan."""
    tokens, world = mask.shape
    device = mask.device
    flat = mask.t().reshape(-1)  # rank-major
    slot = torch.where(flat, flat.long().cumsum(0) - 1, copies)  # unused pairs go to a dump slot
    token_of = torch.empty(copies + 1, dtype=torch.int64, device=device)
    rank_of = torch.empty(copies + 1, dtype=torch.int64, device=device)
    token_of.scatter_(0, slot, torch.arange(tokens, device=device).repeat(world))
    rank_of.scatter_(0, slot, torch.arange(world, device=device).repeat_interleave(tokens))
    token_of, rank_of = token_of[:copies], rank_of[:copies]
    key = keys.long()[token_of]  # [copies, K]
    here = torch.div(key, local, rounding_mode="floor") == rank_of[:, None]
    ids = torch.where(here, key - rank_of[:, None] * local, -1).to(torch.int32)
    route_weight = torch.where(here, weights.float()[token_of], 0.0)
    token_copies = torch.where(flat, slot, -1).view(world, tokens).t().to(torch.int32).contiguous()
    return token_of.to(torch.int32), ids.contiguous(), route_weight.contiguous(), token_copies


def expand_copies(ids: torch.Tensor, recv_copies, local: int, rows: int, sort=None, counts_device=None):
    """The receiver's side: `ids [copies, K]` (local expert or -1) of the copies received from
    each rank (`recv_copies[s]` of them from rank s, in token order). Returns `(assignment
    [rows] int32, segment_offsets int32 [world * local + 1])`: the received assignments as
    `[source rank][local expert][token]` rows -- exactly the layout and order a row-per-assignment
    dispatch delivers -- each named by `copy * K + slot`."""
    if sort is None:
        from . import ops

        sort = ops.sort_assignments
    world = len(recv_copies)
    device = ids.device
    # (the counts as a device tensor, when the plan kept them: a host list would have to be copied
    # to the device, and a pageable copy waits for the stream)
    counts = counts_device if counts_device is not None else torch.tensor(recv_copies, device=device)
    source = torch.repeat_interleave(torch.arange(world, device=device), counts, output_size=ids.shape[0])
    # assignments that live on another rank sort behind every real (source, expert) group
    key = torch.where(ids >= 0, source[:, None] * local + ids.long(), world * local).to(torch.int32)
    order, offsets, _slots, _counts = sort(key.contiguous(), world * local + 1)
    return order[:rows].contiguous(), offsets[: world * local + 1].contiguous()



def make_plans(send_counts: torch.Tensor, group, copy_counts: torch.Tensor | None = None) -> list[ExchangePlan]:
    """`send_counts [C, E]`: rows per placement key of each of C token chunks held by this rank
    (any integer dtype, on the group's device); `copy_counts [C, G]` (optional): token copies per
    destination rank for a de-duplicated dispatch. One all-to-all of all the counts and one host
    read of the split sizes give one plan per chunk."""
    world = dist.get_world_size(group)
    chunks, experts = send_counts.shape
    local = experts // world
    mine = send_counts.to(torch.int64).view(chunks, world, local).permute(1, 0, 2).contiguous()  # [G, C, El]
    if copy_counts is not None:  # one more column per (rank, chunk)
        mine = torch.cat([mine, copy_counts.to(torch.int64).t().reshape(world, chunks, 1)], dim=2).contiguous()
    theirs = torch.empty_like(mine)
    dist.all_to_all_single(theirs, mine, group=group)
    sizes = [mine[:, :, :local].sum(2), theirs[:, :, :local].sum(2)]
    if copy_counts is not None:
        sizes += [mine[:, :, local], theirs[:, :, local]]
    sizes = torch.stack(sizes).cpu()  # the one device-to-host copy: [2 or 4, G, C]
    plans = []
    for c in range(chunks):
        send_splits, recv_splits = sizes[0, :, c].tolist(), sizes[1, :, c].tolist()
        offsets = torch.zeros(world * local + 1, dtype=torch.int32, device=send_counts.device)
        offsets[1:] = theirs[:, c, :local].reshape(-1).cumsum(0).to(torch.int32)
        plan = ExchangePlan(send_splits, recv_splits, offsets, int(sum(recv_splits)), int(sum(send_splits)))
        if copy_counts is not None:
            plan.send_copies, plan.recv_copies = sizes[2, :, c].tolist(), sizes[3, :, c].tolist()
            plan.recv_copies_device = theirs[:, c, local].contiguous()
        plans.append(plan)
    return plans


def regroup_index(segment_offsets: torch.Tensor, world: int, local: int, rows: int):
    """Received rows sit as `[source rank][local expert]` segments (`segment_offsets`, int32
    `[world * local + 1]`). Returns `(offsets, source)`: int32 `offsets [local + 1]` of the same
    rows grouped by expert, the sources in rank order inside an expert, and int32 `source
    [rows]`, the received position of every row of that order. Multiplying in expert order keeps
    the GEMM groups `world` times larger, so far fewer partly filled 128-row tiles; the
    gather is free in the quantiser and the way back is the GEMM's scattered store. No host
    synchronisation (`rows` is already known from the plan)."""
    device = segment_offsets.device
    seg = segment_offsets.long()
    cnt = (seg[1:] - seg[:-1]).view(world, local)
    offsets = torch.zeros(local + 1, dtype=torch.int64, device=device)
    offsets[1:] = cnt.sum(0).cumsum(0)
    first = offsets[:-1].unsqueeze(0) + (cnt.cumsum(0) - cnt)  # [world, local]: where a segment starts
    segment = torch.repeat_interleave(torch.arange(world * local, device=device), cnt.reshape(-1),
                                      output_size=rows)
    arrival = torch.arange(rows, device=device)
    destination = first.reshape(-1)[segment] + (arrival - seg[:-1][segment])
    source = torch.empty(rows, dtype=torch.int32, device=device)
    source[destination] = arrival.to(torch.int32)
    return offsets.to(torch.int32), source


def make_plan(send_counts: torch.Tensor, group) -> ExchangePlan:
    """The single-chunk form of `make_plans`: `send_counts [E]`."""
    return make_plans(send_counts.reshape(1, -1), group)[0]


def exchange(rows: torch.Tensor, plan: ExchangePlan, group, *, back: bool = False, async_op: bool = False,
             out: torch.Tensor | None = None, copies: bool = False):
    """Dispatch (`back=False`: send my sorted rows, receive the rows of my experts) or return
    (`back=True`: the inverse). Returns `(received, work)`; `work` is None unless `async_op`.
    `out` (optional) receives the rows instead of a fresh tensor. `copies`: the rows are the
    token copies of a de-duplicated dispatch (or, with `back`, one row per copy going home)."""
    if copies and back:
        send, recv, total = plan.recv_copies, plan.send_copies, int(sum(plan.send_copies))
    elif copies:
        send, recv, total = plan.send_copies, plan.recv_copies, int(sum(plan.recv_copies))
    else:
        send, recv = (plan.recv_splits, plan.send_splits) if back else (plan.send_splits, plan.recv_splits)
        total = plan.send_rows if back else plan.recv_rows
    received = out if out is not None else torch.empty((total, *rows.shape[1:]), dtype=rows.dtype,
                                                       device=rows.device)
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
                 shared=None, device=None, weight_grad_dtype=torch.bfloat16, chunks=None, comm_sms=0,
                 lora=None, frozen_base=False):
        self.config = config
        self.frozen_base = bool(frozen_base)  # `forward_backward` then skips the base weight gradients
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
        # token chunks per step; None: chosen per call so that an expert still gets about 2048
        # rows per chunk (between 2 and 4 chunks)
        self.chunks = None if chunks is None else int(chunks)
        self.comm_sms = int(comm_sms) if self.world > 1 else 0
        if self.comm_sms and self.device.type == "cuda":
            # optional: the statically scheduled kernels (weight gradients) leave these SMs to the
            # all-to-all kernels.  Off by default: the FP8 GEMMs draw their tiles dynamically and
            # adapt to whatever SMs the collectives hold, and the weight gradients overlap only
            # the last return, where starting some CTAs late costs less than a narrower grid.
            from . import ops

            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            ops.set_cta_limit(max(sms - self.comm_sms, 2) // 2 * 2)
        # expert LoRA on this rank's shard: dict(a13 [E/G, r, D], b13 [E/G, 2F, r], a2 [E/G, r, F],
        # b2 [E/G, D, r] bf16, scale).  The factors are kept as the rank kernels want them: rank
        # padded to a multiple of 8, B factors rank-major.
        self.lora = None
        if lora is not None:
            from .lora import _pad_rank

            a13, rank = _pad_rank(lora["a13"].detach(), 1)
            b13, _ = _pad_rank(lora["b13"].detach(), 2)
            a2, _ = _pad_rank(lora["a2"].detach(), 1)
            b2, _ = _pad_rank(lora["b2"].detach(), 2)
            if a13.shape[0] != self.local_experts or rank > 64:
                raise ValueError("LoRA factors must hold this rank's experts, with rank <= 64")
            self.lora = dict(a13=a13, b13t=b13.transpose(1, 2).contiguous(), a2=a2,
                             b2t=b2.transpose(1, 2).contiguous(), scale=float(lora["scale"]), rank=rank)
        self.keys = placement(config, self.world, self.device)
        self.side_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.arena = None  # receive arenas in peer memory, created at the first step that needs them
        # the receiver's per-chunk planning (small tensor ops) runs here, beside the GEMMs
        # (high priority: its kernels are tiny and on the critical path of the next chunk, while the
        # GEMMs they run beside fill every SM)
        self.plan_stream = torch.cuda.Stream(device=self.device, priority=-1) if self.device.type == "cuda" else None
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
                    expert_map=self.config.expert_map, dedup=self.config.dedup,
                    transport="nccl all_to_all_single, bf16 rows",
                    chunks=self.chunks,
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
    def _peer_arena(self, rows_per_peer: int, width: int):
        """The arena of the peer transport (collective when it has to be created or grown: every
        rank calls this at the same step with its own chunk size, and the largest one decides)."""
        from .peer import PeerArena

        if self.arena is not None and self.arena.fits(rows_per_peer, width):
            return self.arena
        need = torch.tensor([rows_per_peer], dtype=torch.int64, device=self.device)
        dist.all_reduce(need, op=dist.ReduceOp.MAX, group=self.group)
        if self.arena is not None:
            self.arena.close()
        self.arena = PeerArena(self.group, self.device, int(need.item()), width)
        return self.arena

    def forward(self, x, residual=None, expert_ids=None, routing_weights=None):
        """Tokens are processed in `self.chunks` contiguous chunks: the dispatch of chunk c+1
        and the return of chunk c are in flight while chunk c's expert GEMMs run."""
        from . import layer, ops

        cfg = self.config
        with torch.no_grad():
            self._mark("start")
            flat = x.reshape(-1, x.shape[-1]).contiguous()
            tokens, width = flat.shape
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
            wanted = self.chunks
            if wanted is None:
                # more chunks hide more of the first dispatch and the last return, fewer keep
                # the GEMM groups large: measured best at 8 GPUs with 4 (2048 rows per expert
                # and chunk), at 2 GPUs with 2
                rows_per_expert = tokens * cfg.top_k // max(self.local_experts, 1)
                wanted = max(2, min(4, rows_per_expert // 2048))
            chunks = max(1, min(wanted, tokens))
            bounds = [tokens * c // chunks for c in range(chunks + 1)]
            dedup = cfg.dedup and self.world > 1
            parts = []
            for c in range(chunks):
                lo, hi = bounds[c], bounds[c + 1]
                order, _offsets, slots, key_counts = ops.sort_assignments(keys[lo:hi], cfg.experts)
                parts.append(dict(lo=lo, hi=hi, order=order, slots=slots, key_counts=key_counts))
                if dedup:
                    parts[-1]["mask"] = copy_mask(keys[lo:hi], self.world, self.local_experts)
            self._mark("route+sort")
            plans = make_plans(torch.stack([part["key_counts"] for part in parts]), self.group,
                               copy_counts=torch.stack([part["mask"].sum(0) for part in parts]) if dedup else None)
            self._mark("plan")
            total = sum(plan.recv_rows for plan in plans)
            self.last_recv_rows = total
            starts = [0]
            for plan in plans:
                starts.append(starts[-1] + plan.recv_rows)
            recv_x = recv_w = None
            if not dedup:
                recv_x = torch.empty((total, width), dtype=flat.dtype, device=flat.device)
                recv_w = torch.empty(total, dtype=torch.float32, device=flat.device)
            # what the backward pass reads, all in expert order (within a chunk)
            x_rows = torch.empty((total, width), dtype=flat.dtype, device=flat.device)
            row_w = torch.empty(total, dtype=torch.float32, device=flat.device)
            h13 = torch.empty((total, 2 * cfg.intermediate), dtype=torch.bfloat16, device=flat.device)
            lora = self.lora
            t1 = t2 = None
            if lora is not None:  # x A13^T and act A2^T of every row: the factor gradients need them
                t1 = torch.empty((total, lora["a13"].shape[1]), dtype=torch.bfloat16, device=flat.device)
                t2 = torch.empty_like(t1)
            regroup = [None] * chunks  # filled per chunk while its rows are in flight

            arena = None
            if dedup and cfg.transport == "peer":
                arena = self._peer_arena(max(b - a for a, b in zip(bounds[:-1], bounds[1:])), width)

            def send(c):
                part = parts[c]
                lo, hi = part["lo"], part["hi"]
                if dedup:
                    # one copy of a token per destination rank, and what to do with it there:
                    # K (local expert or -1, route weight) pairs, the weights as raw bits
                    if flat.is_cuda:  # one launch
                        token, meta, token_copies = ops.build_copies(
                            keys[lo:hi].to(torch.int32).contiguous(), weights[lo:hi].contiguous(), self.world,
                            self.local_experts, plans[c].send_copies)
                    else:
                        token, copy_ids, copy_w, token_copies = build_copies(
                            part["mask"], keys[lo:hi], weights[lo:hi], self.local_experts,
                            int(sum(plans[c].send_copies)))
                        meta = torch.cat([copy_ids, copy_w.view(torch.int32)], dim=1)
                    part["copy_token"], part["token_copies"] = token, token_copies
                    if c == 0:
                        self._mark("first copies built")
                    if arena is not None:
                        # gather + transfer in one kernel, straight into the peers' arenas
                        wx = arena.dispatch(flat[lo:hi], token, plans[c].send_copies)
                        rows, got_rows = None, wx.rows
                        part["arena_rows"] = arena.received_index(plans[c].recv_copies_device,
                                                                  int(sum(plans[c].recv_copies)))
                        self.bytes_moved += token.numel() * width * 2
                    else:
                        rows = ops.dispatch(flat[lo:hi], token, 1)
                        got_rows, wx = exchange(rows, plans[c], self.group, async_op=True, copies=True)
                        self.bytes_moved += rows.numel() * 2
                    got_meta, ww = exchange(meta, plans[c], self.group, async_op=True, copies=True)
                    part["recv_copies"], part["recv_meta"] = got_rows, got_meta
                    return rows, meta, wx, ww
                rows = ops.dispatch(flat[lo:hi], part["order"], cfg.top_k)
                row_weights = weights[lo:hi].reshape(-1)[part["order"].long()].contiguous()
                _, wx = exchange(rows, plans[c], self.group, async_op=True, out=recv_x[starts[c]:starts[c + 1]])
                _, ww = exchange(row_weights, plans[c], self.group, async_op=True,
                                 out=recv_w[starts[c]:starts[c + 1]])
                self.bytes_moved += rows.numel() * 2
                return rows, row_weights, wx, ww

            in_flight = send(0)
            self._mark("first dispatch issued")
            shared_h13 = None
            if self.shared is not None:  # overlaps the first dispatch
                side = self.side_stream
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    y_shared, shared_h13 = layer.shared_expert_forward(flat, *self.shared,
                                                                       swiglu_limit=cfg.swiglu_limit)
                    base = base + y_shared
                for tensor in (base, shared_h13):  # produced on the side stream, consumed on this one
                    tensor.record_stream(torch.cuda.current_stream())

            def prepare(c, meta_work, after):
                """The receiver's plan of chunk c (which received copy feeds which expert-order row, the
                regroup index, the per-row route weights), computed on the planning stream as soon as
                the chunk's metadata has arrived: beside the previous chunk's GEMMs, not between them.
                `after`: an event on the calling stream behind everything the plan reads (the host may
                queue this plan later than that point, after the launches that are more urgent)."""
                part = parts[c]
                current = torch.cuda.current_stream()
                side = self.plan_stream
                side.wait_event(after)
                with torch.cuda.stream(side):
                    meta_work.wait()
                    meta = part["recv_meta"]
                    meta.record_stream(side)
                    offsets, source = regroup_index(plans[c].segment_offsets, self.world, self.local_experts,
                                                    plans[c].recv_rows)
                    # the copies become this rank's assignments: [source][expert][token] rows as a
                    # row-per-assignment dispatch delivers them, then expert order
                    assignment, _segments = expand_copies(meta[:, :cfg.top_k].contiguous(), plans[c].recv_copies,
                                                          self.local_experts, plans[c].recv_rows,
                                                          counts_device=plans[c].recv_copies_device)
                    pick = assignment[source.long()].contiguous()  # expert-order row -> copy * K + slot
                    out = dict(offsets=offsets, source=source, pick=pick)
                    copy_weights = meta[:, cfg.top_k:].contiguous().view(torch.float32)
                    if cfg.presum:
                        # copy_rows[c, k]: the expert-order row of assignment k of copy c (-1: not here)
                        copies_here = meta.shape[0]
                        copy_rows = torch.full((copies_here * cfg.top_k,), -1, dtype=torch.int32, device=flat.device)
                        copy_rows[pick.long()] = torch.arange(pick.numel(), dtype=torch.int32, device=flat.device)
                        out["copy_rows"] = copy_rows.view(copies_here, cfg.top_k)
                        out["copy_weights"] = copy_weights
                    out["gather"] = pick
                    if arena is not None:
                        # the copies sit in one fixed segment per source rank: name them by arena row
                        copy, slot = torch.div(pick, cfg.top_k, rounding_mode="floor"), pick % cfg.top_k
                        arena_rows = part.pop("arena_rows")
                        arena_rows.record_stream(side)
                        out["gather"] = (arena_rows[copy.long()] * cfg.top_k + slot).to(torch.int32)
                    out["row_weights"] = copy_weights.reshape(-1)[pick.long()]
                    done = torch.cuda.Event()
                    done.record()
                for tensor in out.values():
                    tensor.record_stream(current)
                return out, done

            def issued():
                event = torch.cuda.Event()
                event.record()
                return event

            prepared = [None] * chunks
            if dedup:
                prepared[0] = prepare(0, in_flight[3], issued())
            returns = []
            for c in range(chunks):
                nxt = send(c + 1) if c + 1 < chunks else None
                sent = issued() if nxt is not None else None
                if not dedup:
                    regroup[c] = regroup_index(plans[c].segment_offsets, self.world, self.local_experts,
                                               plans[c].recv_rows)
                in_flight[2].wait()
                in_flight[3].wait()
                in_flight = nxt
                rows = slice(starts[c], starts[c + 1])
                # expert order from here on: gathered by the quantiser, given back in arrival
                # order by the down projection's store
                if dedup:
                    part = parts[c]
                    plan_c, plan_done = prepared[c]
                    torch.cuda.current_stream().wait_event(plan_done)
                    self._mark("dispatch wait")
                    part.pop("recv_meta")
                    regroup[c] = (plan_c["offsets"], plan_c["source"])
                    offsets, source = regroup[c]
                    part["pick"] = plan_c["pick"]
                    if cfg.presum:
                        part["copy_rows"], part["copy_weights"] = plan_c["copy_rows"], plan_c["copy_weights"]
                    if arena is not None:
                        part["arena_pick"] = plan_c["gather"]
                    x_q, x_s, _ = ops.quantize_rows(part.pop("recv_copies"), gather=plan_c["gather"],
                                                    gather_div=cfg.top_k, copy_out=x_rows[rows])
                    row_w[rows] = plan_c["row_weights"]
                else:
                    self._mark("dispatch wait")
                    offsets, source = regroup[c]
                    x_q, x_s, _ = ops.quantize_rows(recv_x[rows], gather=source, copy_out=x_rows[rows])
                    row_w[rows] = recv_w[rows][source.long()]
                presum = dedup and cfg.presum  # rows stay in expert order; one weighted row per copy goes back
                if lora is None:
                    ops.grouped_gemm_fp8(x_q, x_s, *self.w13, offsets, out=h13[rows])
                    a_q, a_s, _ = ops.swiglu_quantize(h13[rows], limit=cfg.swiglu_limit)
                    y = ops.grouped_gemm_fp8(a_q, a_s, *self.w2, offsets, row_map=None if presum else source)
                else:
                    # each LoRA term enters its base product as an addend before the one rounding
                    # (the single-GPU form: mlops_b200/lora.py)
                    t1[rows] = ops.lora_project(x_rows[rows], lora["a13"], offsets, rank_major=True)
                    c1 = ops.lora_expand(t1[rows], lora["b13t"], offsets, wide_major=False, scale=lora["scale"])
                    ops.grouped_gemm_fp8(x_q, x_s, *self.w13, offsets, out=h13[rows], addend=c1)
                    a_q, a_s, act = ops.swiglu_quantize(h13[rows], limit=cfg.swiglu_limit, quantized=True,
                                                        rounded=True)
                    t2[rows] = ops.lora_project(act, lora["a2"], offsets, rank_major=True)
                    c2 = ops.lora_expand(t2[rows], lora["b2t"], offsets, wide_major=False, scale=lora["scale"])
                    y = ops.grouped_gemm_fp8(a_q, a_s, *self.w2, offsets, row_map=None if presum else source,
                                             addend=c2)
                if presum:
                    y = ops.combine(y, parts[c]["copy_rows"], parts[c]["copy_weights"], None)
                self._mark("expert fwd")
                y_back, work = exchange(y, plans[c], self.group, back=True, async_op=True, copies=presum)
                if dedup and nxt is not None:
                    # queued only now, behind this chunk's launches: the host reaches the GEMMs sooner; on
                    # the device the plan still starts as soon as chunk c + 1's metadata is there
                    prepared[c + 1] = prepare(c + 1, nxt[3], sent)
                self.bytes_moved += y.numel() * 2
                returns.append((y, y_back, work))
            if self.shared is not None:
                torch.cuda.current_stream().wait_stream(self.side_stream)
            output = torch.empty_like(flat)
            for c, (y, y_back, work) in enumerate(returns):
                work.wait()
                part = parts[c]
                if dedup and cfg.presum:  # the partial sums of a token, in rank order, onto its base row
                    output[part["lo"]:part["hi"]] = ops.combine(y_back, part["token_copies"], None,
                                                                base[part["lo"]:part["hi"]])
                else:
                    output[part["lo"]:part["hi"]] = ops.combine(
                        y_back, part["slots"], weights[part["lo"]:part["hi"]], base[part["lo"]:part["hi"]])
            self._mark("combine a2a wait + combine")
            key_counts = torch.stack([part["key_counts"] for part in parts]).sum(0)
            # the sort counted by placement key; statistics want expert order
            counts = key_counts if cfg.expert_map == "contiguous" else key_counts[self.keys.long()]
            aux, counts, psum = layer.routing_statistics(
                logits, ids, counts, routing_mode=cfg.routing_mode, lengths=(tokens,), experts=cfg.experts)
        self._mark("stats")
        saved = dict(flat=flat, logits=logits, weights=weights, ids=ids, parts=parts, plans=plans, starts=starts,
                     x_rows=x_rows, row_w=row_w, regroup=regroup, h13=h13, shared_h13=shared_h13, counts=counts,
                     shape=x.shape, t1=t1, t2=t2)
        return output.reshape(x.shape), aux, counts, psum, saved

    # ---------------------------------------------------------------------- backward
    def backward(self, saved, grad_output, grad_aux=None, grad_probability_sum=None, *, need_router=True,
                 need_experts=True, need_lora=True):
        from . import layer, ops

        cfg = self.config
        plans, parts, starts = saved["plans"], saved["parts"], saved["starts"]
        chunks = len(plans)
        with torch.no_grad():
            self._mark("bwd start")
            flat = saved["flat"]
            tokens, width = flat.shape
            total = starts[-1]
            dy = grad_output.reshape_as(flat).contiguous()
            dedup = "pick" in parts[0]
            recv_dy = None if dedup else torch.empty((total, width), dtype=flat.dtype, device=flat.device)
            regroup = saved["regroup"]
            lora = self.lora  # its terms are part of the input gradient whether or not the factors train
            factor_grads = lora is not None and need_lora
            keep_rows = need_experts or lora is not None
            dy_rows = torch.empty((total, width), dtype=flat.dtype, device=flat.device) if keep_rows else None
            t2g = dt1 = None
            if factor_grads:
                t2g, dt1 = torch.empty_like(saved["t1"]), torch.empty_like(saved["t1"])

            def send(c):
                part = parts[c]
                if dedup and "arena_pick" in part:  # the same copies, the same way as in the forward pass
                    work = self.arena.dispatch(dy[part["lo"]:part["hi"]], part["copy_token"], plans[c].send_copies)
                    part["recv_dy_copies"] = work.rows
                    self.bytes_moved += part["copy_token"].numel() * width * 2
                    return None, work
                if dedup:  # the same copies as in the forward pass
                    rows = ops.dispatch(dy[part["lo"]:part["hi"]], part["copy_token"], 1)
                    part["recv_dy_copies"], work = exchange(rows, plans[c], self.group, async_op=True, copies=True)
                else:
                    rows = ops.dispatch(dy[part["lo"]:part["hi"]], part["order"], cfg.top_k)
                    _, work = exchange(rows, plans[c], self.group, async_op=True,
                                       out=recv_dy[starts[c]:starts[c + 1]])
                self.bytes_moved += rows.numel() * 2
                return rows, work

            in_flight = send(0)
            shared_grads = (None, None, None)
            if self.shared is not None:  # overlaps the first dispatch of dy
                side = self.side_stream
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    shared_grads = layer.shared_expert_backward(dy, flat, *self.shared, saved["shared_h13"],
                                                                swiglu_limit=cfg.swiglu_limit,
                                                                need_weights=need_experts)
                for tensor in shared_grads:
                    if tensor is not None:
                        tensor.record_stream(torch.cuda.current_stream())
            gh_b = act_scaled = None
            if keep_rows:
                gh_b = torch.empty((total, 2 * cfg.intermediate), dtype=torch.bfloat16, device=flat.device)
                act_scaled = torch.empty((total, cfg.intermediate), dtype=torch.bfloat16, device=flat.device)
            returns = []
            for c in range(chunks):
                nxt = send(c + 1) if c + 1 < chunks else None
                in_flight[1].wait()
                in_flight = nxt
                self._mark("dy dispatch wait")
                rows = slice(starts[c], starts[c + 1])
                count = starts[c + 1] - starts[c]
                identity = torch.arange(count, dtype=torch.int32, device=flat.device)
                offsets, source = regroup[c]
                if dedup:
                    arrived, div = parts[c].pop("recv_dy_copies"), cfg.top_k
                    gather = parts[c].get("arena_pick", parts[c]["pick"])
                else:
                    arrived, gather, div = recv_dy[rows], source, 1
                if keep_rows:
                    dy_q, dy_s, _ = ops.quantize_rows(arrived, gather=gather, gather_div=div, copy_out=dy_rows[rows])
                else:
                    dy_q, dy_s = ops.quantize_rows(arrived, gather=gather, gather_div=div)
                r_add = dx_add = None
                if lora is not None:
                    dy_b2 = ops.lora_project(dy_rows[rows], lora["b2t"], offsets, rank_major=True)
                    r_add = ops.lora_expand(dy_b2, lora["a2"], offsets, wide_major=False, scale=lora["scale"])
                    if factor_grads:
                        t2g[rows] = dy_b2
                r = ops.grouped_gemm_fp8(dy_q, dy_s, *self.w2, offsets, b_mn_major=True, addend=r_add)
                dscore, gh_q, gh_s, _, _ = ops.dswiglu_routed(
                    saved["h13"][rows], r, saved["row_w"][rows], identity, limit=cfg.swiglu_limit, quantized=True,
                    rounded=keep_rows, scaled_activation=keep_rows,
                    rounded_out=None if gh_b is None else gh_b[rows],
                    scaled_out=None if act_scaled is None else act_scaled[rows])
                if lora is not None:
                    gh_b13 = ops.lora_project(gh_b[rows], lora["b13t"], offsets, rank_major=True)
                    dx_add = ops.lora_expand(gh_b13, lora["a13"], offsets, wide_major=False, scale=lora["scale"])
                    if factor_grads:
                        dt1[rows] = gh_b13
                presum = dedup and cfg.presum
                grad_rows = ops.grouped_gemm_fp8(gh_q, gh_s, *self.w13, offsets, b_mn_major=True,
                                                 row_map=None if presum else source, addend=dx_add)
                if presum:  # one row per copy: the sum of the copy's assignments, in slot order
                    grad_rows = ops.combine(grad_rows, parts[c]["copy_rows"], None, None)
                dscore_arrival = torch.empty_like(dscore)
                dscore_arrival[source.long()] = dscore
                dscore = dscore_arrival
                self._mark("expert dgrad")
                back_rows, work_rows = exchange(grad_rows, plans[c], self.group, back=True, async_op=True,
                                                copies=presum)
                back_score, work_score = exchange(dscore, plans[c], self.group, back=True, async_op=True)
                self.bytes_moved += grad_rows.numel() * 2
                returns.append((grad_rows, dscore, back_rows, back_score, work_rows, work_score))
            grad_w13 = grad_w2 = None
            lora_grads = {}
            # every chunk is one segment of expert-ordered rows
            all_offsets = torch.cat(
                [regroup[c][0][: -1 if c + 1 < chunks else None] + starts[c] for c in range(chunks)])
            if factor_grads:  # grouped weight gradients with one narrow side (lora.py, single GPU)
                scale, rank = lora["scale"], lora["rank"]
                narrow = lambda t, factor: (t.float() * factor).to(t.dtype)  # noqa: E731
                experts_here, fdtype = self.local_experts, torch.bfloat16
                lora_grads["grad_b2"] = ops.grouped_wgrad(
                    dy_rows, narrow(saved["t2"], saved["row_w"][:, None] * scale), all_offsets, experts_here,
                    fdtype)[:, :, :rank].contiguous()
                lora_grads["grad_a2"] = ops.grouped_wgrad(narrow(t2g, scale), act_scaled, all_offsets,
                                                          experts_here, fdtype)[:, :rank].contiguous()
                lora_grads["grad_b13"] = ops.grouped_wgrad(gh_b, narrow(saved["t1"], scale), all_offsets,
                                                           experts_here, fdtype)[:, :, :rank].contiguous()
                lora_grads["grad_a13"] = ops.grouped_wgrad(narrow(dt1, scale), saved["x_rows"], all_offsets,
                                                           experts_here, fdtype)[:, :rank].contiguous()
            if need_experts:  # local weight gradients over every chunk; overlaps the last return
                grad_w2 = ops.grouped_wgrad(dy_rows, act_scaled, all_offsets, self.local_experts,
                                            self.weight_grad_dtype)
                grad_w13 = ops.grouped_wgrad(gh_b, saved["x_rows"], all_offsets, self.local_experts,
                                             self.weight_grad_dtype)
            self._mark("expert wgrad (issued)")
            grad_x = torch.empty_like(flat)
            grad_route_weights = torch.empty_like(saved["weights"])
            for c, (_rows, _score, back_rows, back_score, work_rows, work_score) in enumerate(returns):
                work_rows.wait()
                work_score.wait()
                part = parts[c]
                if dedup and cfg.presum:
                    grad_x[part["lo"]:part["hi"]] = ops.dispatch_backward(back_rows, part["token_copies"])
                else:
                    grad_x[part["lo"]:part["hi"]] = ops.dispatch_backward(back_rows, part["slots"])
                grad_route_weights[part["lo"]:part["hi"]] = ops.gather_scalar(back_score, part["slots"])
            self._mark("dx return wait + scatter")
            grad_logits = layer.routing_gradient(
                grad_aux, grad_probability_sum, grad_route_weights, saved["weights"], saved["ids"],
                saved["logits"], saved["counts"], routing_mode=cfg.routing_mode, lengths=(tokens,))
            grad_router = None
            if need_router:
                grad_router = layer._router_weight_gradient(grad_logits, flat, self.router_weight.dtype)
            grad_x.addmm_(grad_logits.to(flat.dtype), self.router_weight.to(flat.dtype))
            if self.shared is not None:
                torch.cuda.current_stream().wait_stream(self.side_stream)
                grad_x.add_(shared_grads[0])
        self._mark("router grads")
        return dict(grad_x=grad_x.reshape(saved["shape"]), grad_router=grad_router, grad_w13=grad_w13,
                    grad_w2=grad_w2, grad_shared_w13=shared_grads[1], grad_shared_w2=shared_grads[2], **lora_grads)

    def forward_backward(self, x, residual, grad_output):
        output, aux, counts, _psum, saved = self.forward(x, residual)
        grads = self.backward(saved, grad_output, need_experts=not self.frozen_base)
        return output, grads["grad_x"], aux, counts

    def close(self):
        if self.comm_sms and self.device.type == "cuda":
            from . import ops

            ops.set_cta_limit(0)
        if self.arena is not None:
            self.arena.close()
            self.arena = None
        self.side_stream = self.plan_stream = None


def parity_check(group, device, *, routing_mode="softmax_then_topk", n_group=1, topk_group=1,
                 routed_scaling=1.0, shared=False, presum=False, transport="nccl", tokens=384, width=512,
                 inner=256, experts_per_rank=4, seed=5) -> dict:
    """The expert-parallel layer against the single-GPU layer on the gathered weights, on a
    small case with this group's world size: every rank builds the same global experts, keeps
    its shard, runs `ExpertParallelMoE` on its own tokens and `layer.forward_routed /
    backward_routed` on the full weights, and compares. The outputs must be bit-equal (the
    expert math is row-wise identical whichever rank runs it; with `presum`, which rounds the
    per-rank partial sums, equal within the bf16 tolerance instead) and the gradients agree to
    rounding (input gradient: maximum 2e-2, or 4e-2 with `presum`, mean 2e-3); expert weight gradients are compared with the all-reduced single-GPU ones (every
    rank's tokens contribute to an expert). Raises AssertionError on a mismatch; returns the
    measured figures. This is the expectation the reference's multi-rank tests form
    (`tests/expert_parallel/gpu/reference_quack.py:14-69`: run the oracle on global weights,
    all-reduce the expected expert gradients, slice the own shard)."""
    from . import layer, ops

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    experts = experts_per_rank * world
    if n_group > 1:  # group-limited routing: one group per rank, half of the groups eligible
        n_group, topk_group = world, max(1, world // 2)
        top_k = min(4, experts_per_rank * topk_group)
    else:
        n_group = topk_group = 1
        top_k = min(4, experts)
    g = torch.Generator().manual_seed(seed)  # global parameters: identical on every rank
    router = (torch.randn(experts, width, generator=g) * 0.05).to(device)
    bias = (torch.randn(experts, generator=g) * 0.1).to(device) if routing_mode == "sigmoid_noaux_tc" else None
    w13 = ops.quantize_blocks((torch.randn(experts, 2 * inner, width, generator=g) * 0.05).bfloat16().to(device))
    w2 = ops.quantize_blocks((torch.randn(experts, width, inner, generator=g) * 0.05).bfloat16().to(device))
    shared_w = None
    if shared:
        shared_w = ((torch.randn(2 * inner, width, generator=g) * 0.05).bfloat16().to(device),
                    (torch.randn(width, inner, generator=g) * 0.05).bfloat16().to(device))
    gl = torch.Generator().manual_seed(100 + rank)  # this rank's tokens
    x = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    residual = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    dy = torch.randn(tokens, width, generator=gl).bfloat16().to(device)
    dedup = n_group > 1
    config = ExpertParallelConfig(hidden=width, experts=experts, intermediate=inner, top_k=top_k,
                                  routing_mode=routing_mode, n_group=n_group, topk_group=topk_group,
                                  routed_scaling=routed_scaling, expert_map="contiguous" if dedup else "strided",
                                  dedup=dedup, presum=bool(presum and dedup),
                                  transport=transport if dedup else "nccl")
    keys = placement(config, world)
    mine = sorted((e for e in range(experts) if int(keys[e]) // experts_per_rank == rank), key=lambda e: int(keys[e]))
    pick = torch.tensor(mine, device=device)
    module = ExpertParallelMoE(config, group, router_weight=router, router_bias=bias,
                               w13=(w13[0][pick].contiguous(), w13[1][pick].contiguous()),
                               w2=(w2[0][pick].contiguous(), w2[1][pick].contiguous()), shared=shared_w,
                               device=device, weight_grad_dtype=torch.float32, chunks=2)
    output, aux, counts, _psum, saved = module.forward(x, residual)
    grads = module.backward(saved, dy)
    torch.cuda.synchronize(device)
    ops.check_status(device)

    base, shared_h13 = residual, None
    if shared:
        y_shared, shared_h13 = layer.shared_expert_forward(x, *shared_w)
        base = residual + y_shared
    kwargs = dict(top_k=top_k, routing_mode=routing_mode, router_bias=bias, n_group=n_group,
                  topk_group=topk_group, routed_scaling=routed_scaling)
    ref = layer.forward_routed(x, base, router, w13, w2, **kwargs)
    ref_grads = layer.backward_routed(dy, None, None, x, router, w13, w2, *ref[4:], top_k=top_k,
                                      routing_mode=routing_mode, weight_grad_dtype=torch.float32)
    expected_x = ref_grads[0]
    if shared:
        expected_x = expected_x + layer.shared_expert_backward(dy, x, *shared_w, shared_h13)[0]

    def rel(actual, expected):
        a, e = actual.double(), expected.double()
        rms = e.pow(2).mean().sqrt().clamp_min(1e-30)
        return (a - e).abs() / torch.maximum(e.abs(), rms)

    def max_rel(actual, expected):
        return rel(actual, expected).max().item()

    result = {"world": world, "experts": experts, "top_k": top_k, "tokens_per_rank": tokens,
              "routing": routing_mode, "dedup_dispatch": dedup, "presum_return": config.presum,
              "transport": config.transport,
              "counts_equal": bool(torch.equal(counts, ref[2])),
              "output_bit_equal": bool(torch.equal(output, ref[0])),
              "output_max_rel": max_rel(output, ref[0]),
              "grad_x_max_rel": max_rel(grads["grad_x"], expected_x),
              "grad_x_mean_rel": rel(grads["grad_x"], expected_x).mean().item(),
              "grad_router_max_rel": max_rel(grads["grad_router"], ref_grads[2])}
    for name, full in (("grad_w13", ref_grads[3]), ("grad_w2", ref_grads[4])):
        total = full.clone()
        dist.all_reduce(total, group=group)
        result[name + "_max_rel"] = max_rel(grads[name], total[pick])
    flags = torch.tensor([float(result["counts_equal"]), float(result["output_bit_equal"]),
                          -result["output_max_rel"], -result["grad_x_max_rel"], -result["grad_router_max_rel"],
                          -result["grad_w13_max_rel"], -result["grad_w2_max_rel"], -result["grad_x_mean_rel"]],
                         device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN, group=group)  # the worst rank decides
    worst = flags.tolist()
    result.update(counts_equal=bool(worst[0] == 1.0), output_bit_equal=bool(worst[1] == 1.0),
                  output_max_rel=-worst[2], grad_x_max_rel=-worst[3], grad_router_max_rel=-worst[4],
                  grad_w13_max_rel=-worst[5], grad_w2_max_rel=-worst[6], grad_x_mean_rel=-worst[7])
    module.close()
    assert result["counts_equal"], f"expert counts differ from the single-GPU layer: {result}"
    if config.presum:
        assert result["output_max_rel"] <= 2e-2, f"expert-parallel output outside the bf16 tolerance: {result}"
    else:
        assert result["output_bit_equal"], f"expert-parallel output differs from the single-GPU layer: {result}"
    # With pre-summed returns every rank's partial sum of a token's input-gradient rows is rounded
    # to bf16 before the owner adds them; where partials cancel, an element can be off by a few
    # bf16 ulps of a PARTIAL (2.1e-2 of the tensor's rms seen at 4 ranks), so the maximum gets a
    # wider bound there while the mean stays at the parity tolerance.
    assert result["grad_x_max_rel"] <= (4e-2 if config.presum else 2e-2), result
    assert result["grad_x_mean_rel"] <= 2e-3 and result["grad_router_max_rel"] <= 2e-3, result
    assert result["grad_w13_max_rel"] <= 1e-3 and result["grad_w2_max_rel"] <= 1e-3, result
    return result


# ---------------------------------------------------------------- the module contract
class _ExpertParallelFunction(torch.autograd.Function):
    """Autograd node of one expert-parallel layer call: forward and backward are the runtime's
    own (collectives included); the saved plan travels in the context."""

    @staticmethod
    def forward(ctx, runtime, x, residual, expert_ids, routing_weights, router_weight, w13, w2, *shared):
        output, aux, counts, psum, saved = runtime.forward(x, residual, expert_ids, routing_weights)
        ctx.runtime, ctx.saved, ctx.shared = runtime, saved, len(shared)
        ctx.mark_non_differentiable(counts)
        return output, aux, counts, psum

    @staticmethod
    def backward(ctx, grad_output, grad_aux, _grad_counts, grad_psum):
        need = ctx.needs_input_grad  # runtime, x, residual, ids, weights, router, w13, w2, shared...
        if grad_output is None:
            grad_output = torch.zeros(ctx.saved["shape"], dtype=ctx.saved["flat"].dtype,
                                      device=ctx.saved["flat"].device)
        grads = ctx.runtime.backward(ctx.saved, grad_output, grad_aux, grad_psum, need_router=bool(need[5]),
                                     need_experts=bool(need[6] or need[7] or any(need[8:])))
        ctx.saved = None  # the plan and the saved rows are released with the first backward
        shared = [grads["grad_shared_w13"], grads["grad_shared_w2"]][:ctx.shared]
        return (None, grads["grad_x"] if need[1] else None, grad_output if need[2] else None, None, None,
                grads["grad_router"] if need[5] else None, grads["grad_w13"] if need[6] else None,
                grads["grad_w2"] if need[7] else None, *[g if n else None for g, n in zip(shared, need[8:])])


class ExpertParallelLayer(torch.nn.Module):
    """`ExpertParallelMoE` as a module with ordinary autograd, the contract of the reference's
    layer (`src/mlops/expert_parallel/quack/layer.py:28-59, 107-155, 219-246, 267-281`):

    * `forward(x[, expert_ids, routing_weights])` with `x` bf16 `[tokens_per_rank, D]` (or any
      leading shape) on the module's device returns the layer output; supplying both routing
      tensors bypasses the layer's router (how externally routed models compose with it);
      `last_statistics` holds `(aux, counts, probability_sum)` of the last call, `aux` and
      `probability_sum` differentiable.
    * `expert_parameters()` yields this rank's shard (`gate_up_weight [E/G, 2F, D]`,
      `down_weight [E/G, D, F]` block-FP8 containers), `replicated_parameters()` the router and
      the shared expert; `synchronize_replicated_parameters()` broadcasts the latter from rank 0
      and `synchronize_replicated_gradients()` SUM-all-reduces their gradients (called by the
      owner of the accumulation window; expert shards are never reduced over the group).
    * `close()` releases the runtime; a closed layer refuses calls.
    """

    def __init__(self, config: ExpertParallelConfig, ep_group, *, gate_up_weight, down_weight, router_weight,
                 router_bias=None, shared=None, device=None, weight_grad_dtype=None, chunks=None):
        super().__init__()
        from .weights import holds_blocks, split

        if not (holds_blocks(gate_up_weight) and holds_blocks(down_weight)):
            raise ValueError("gate_up_weight and down_weight must be block-FP8 containers of this rank's experts")
        self.config, self.ep_group = config, ep_group
        self.gate_up_weight = torch.nn.Parameter(gate_up_weight, requires_grad=gate_up_weight.requires_grad)
        self.down_weight = torch.nn.Parameter(down_weight, requires_grad=down_weight.requires_grad)
        self.router_weight = torch.nn.Parameter(router_weight, requires_grad=router_weight.requires_grad)
        self.router_bias = router_bias
        self.shared_w13 = self.shared_w2 = None
        if shared is not None:
            self.shared_w13 = torch.nn.Parameter(shared[0], requires_grad=shared[0].requires_grad)
            self.shared_w2 = torch.nn.Parameter(shared[1], requires_grad=shared[1].requires_grad)
        grad_dtype = weight_grad_dtype or gate_up_weight.dtype
        self._runtime = ExpertParallelMoE(
            config, ep_group, router_weight=self.router_weight.detach(), router_bias=router_bias,
            w13=split(gate_up_weight), w2=split(down_weight),
            shared=None if shared is None else (self.shared_w13.detach(), self.shared_w2.detach()),
            device=device, weight_grad_dtype=grad_dtype, chunks=chunks)
        self._closed = False
        self.last_statistics = None
        self.synchronize_replicated_parameters()

    def expert_parameters(self):
        yield self.gate_up_weight
        yield self.down_weight

    def replicated_parameters(self):
        yield self.router_weight
        if self.shared_w13 is not None:
            yield self.shared_w13
            yield self.shared_w2

    def synchronize_replicated_parameters(self):
        with torch.no_grad():
            for parameter in self.replicated_parameters():
                dist.broadcast(parameter.data, src=dist.get_global_rank(self.ep_group, 0), group=self.ep_group)
            if self.router_bias is not None:
                dist.broadcast(self.router_bias, src=dist.get_global_rank(self.ep_group, 0), group=self.ep_group)

    def synchronize_replicated_gradients(self):
        ExpertParallelMoE.synchronize_replicated_gradients(
            [p.grad for p in self.replicated_parameters()], self.ep_group)

    def forward(self, x, expert_ids=None, routing_weights=None):
        if self._closed:
            raise RuntimeError("Layer is closed")
        if x.dtype != torch.bfloat16 or x.device != self._runtime.device or x.shape[-1] != self.config.hidden:
            raise ValueError("Expected BF16 input on the configured CUDA device")
        if (expert_ids is None) != (routing_weights is None):
            raise ValueError("Supply both routing tensors or neither")
        shared = () if self.shared_w13 is None else (self.shared_w13, self.shared_w2)
        output, aux, counts, psum = _ExpertParallelFunction.apply(
            self._runtime, x, torch.zeros_like(x), expert_ids, routing_weights, self.router_weight,
            self.gate_up_weight, self.down_weight, *shared)
        self.last_statistics = (aux, counts, psum)
        return output

    def close(self):
        if not self._closed:
            self._runtime.close()
            self._closed = True
