"""Benchmark of the routed-MoE expert path: one step = forward + backward of one MoE layer
over one batch of synthetic tokens.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c3|c1] [--impl reference]

Prints ONE JSON line (rank 0). `value` is tokens/s of the whole job with the inputs resident
in HBM; `e2e` is the same step fed from pinned host buffers (host->device copies of the
step's inputs and a device->host read of its result inside the timed region; the upload of
the next step's inputs runs on a copy stream beside the current step); `roofline`
describes the dominant kernel (the block-FP8 grouped GEMM), timed live with CUDA events on
the launching stream; `cpu_baseline` is the CPU oracle timed on a bounded sample of the same
workload on this machine's host cores. `--impl reference` times that CPU path alone.

Workloads (shapes only; weights are random, data synthetic, seeded):
  c4  DeepSeek-V3-shaped: D=7168, 256 experts, F=2048, sigmoid/group top-8, one shared expert,
      T=32768 tokens per GPU (the configuration the headline metric is quoted on)
  c4p the same layer at profiling size (32 experts, T=4096: the same 1024 rows per expert,
      a few GB on the device) for ncu captures
  c5  Qwen3-30B-A3B-shaped with rank-16 LoRA on a frozen base and Zipf(1.2) expert popularity:
      D=2048, 128 experts, F=768, softmax top-8, T=65536 per GPU (expert-parallel at N > 1)
  c3  Mixtral-8x7B-shaped: D=4096, 8 experts, F=14336, softmax top-2, T=16384
  c1  the small CPU-runnable case: D=256, 8 experts, F=512, softmax top-2, T=512
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    "c4": dict(name="deepseek_v3_shaped_moe_layer", T=32768, D=7168, E=256, F=2048, K=8,
               mode="sigmoid_noaux_tc", n_group=8, topk_group=4, scaling=2.5, shared=True),
    "c4p": dict(name="deepseek_v3_shaped_moe_layer_profile_size", T=4096, D=7168, E=32, F=2048, K=8,
                mode="sigmoid_noaux_tc", n_group=8, topk_group=4, scaling=2.5, shared=True),
    "c3": dict(name="mixtral_8x7b_shaped_moe_layer", T=16384, D=4096, E=8, F=14336, K=2,
               mode="softmax_then_topk", n_group=1, topk_group=1, scaling=1.0, shared=False),
    "c5": dict(name="qwen3_30b_a3b_shaped_moe_layer_lora_zipf", T=65536, D=2048, E=128, F=768, K=8,
               mode="softmax_then_topk", n_group=1, topk_group=1, scaling=1.0, shared=False, lora_rank=16,
               zipf=1.2),
    "c1": dict(name="small_moe_layer", T=512, D=256, E=8, F=512, K=2,
               mode="softmax_then_topk", n_group=1, topk_group=1, scaling=1.0, shared=False),
}
NOMINAL_FP8_TFLOPS = 4500.0
FALLBACK_BF16_SUSTAINED = 1400.0


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": FALLBACK_BF16_SUSTAINED}, "fallback"


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample(cfg, tokens, seed=0):
    """Forward + backward of the CPU oracle on `tokens` tokens of the workload's shapes with
    `experts_sampled` experts (weights of every sampled expert are dequantised per product, as
    the reference's CPU provider does). Returns seconds per step."""
    from oracle import moe_oracle as O

    g = torch.Generator().manual_seed(seed)
    D, F, K = cfg["D"], cfg["F"], cfg["K"]
    E = cfg["E_cpu"]
    x = torch.randn(tokens, D, generator=g).bfloat16()
    dy = torch.randn(tokens, D, generator=g).bfloat16()
    router = torch.randn(E, D, generator=g) * 0.02
    w13 = O.quantize_blocks((torch.randn(E, 2 * F, D, generator=g) * 0.02).bfloat16())
    w2 = O.quantize_blocks((torch.randn(E, D, F, generator=g) * 0.02).bfloat16())
    bias = torch.randn(E, generator=g) * 0.1 if cfg["mode"] == "sigmoid_noaux_tc" else None
    n_group = cfg["n_group"] if E % cfg["n_group"] == 0 else 1

    def step():
        logits = O.router_logits(x, router)
        fwd = O.forward_block_fp8(x, torch.zeros_like(x), logits, *w13, *w2, top_k=K, routing_mode=cfg["mode"],
                                  router_bias=bias, n_group=n_group, topk_group=min(cfg["topk_group"], n_group),
                                  routed_scaling=cfg["scaling"], gemm_dtype=torch.float32)
        O.backward_block_fp8(dy, x, fwd, *w13, *w2, top_k=K, gemm_dtype=torch.float32)

    step()  # warm-up (allocator, thread pool)
    start = time.perf_counter()
    step()
    return time.perf_counter() - start


def cpu_baseline(cfg, budget_tokens):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    seconds = cpu_sample(cfg, budget_tokens)
    return {
        "value": budget_tokens / seconds, "unit": "tokens/s", "cores": threads, "kind": "port",
        "sample": f"{budget_tokens} tokens, {cfg['E_cpu']} of {cfg['E']} experts, D={cfg['D']} F={cfg['F']} "
                  f"top-{cfg['K']} forward+backward, CPU oracle (fp32 products of dequantised E4M3 operands), "
                  f"{seconds:.1f} s per step",
    }


def reference_arm(args, cfg):
    """The reference's CPU path: its native-PyTorch provider cannot travel to this machine
    (Python sources, not installed here), so the timed code is the CPU oracle port."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    tokens = cfg["cpu_tokens"]
    times = []
    for _ in range(max(args.warmup, 0)):
        cpu_sample(cfg, tokens)
    for _ in range(max(args.steps, 1)):
        times.append(cpu_sample(cfg, tokens))
    mean = sum(times) / len(times)
    value = tokens / mean
    sample = (f"{tokens} tokens, {cfg['E_cpu']} of {cfg['E']} experts, same D/F/top-k, forward+backward, "
              f"CPU oracle port, {threads} threads")
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic", "config": {"workload": cfg["name"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------- GPU arm
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.file.seek(0)
        clocks, max_clock, reasons = [], None, set()
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                  parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        loaded = [c for c in clocks if c > 0.5 * (max(clocks) if clocks else 1)]
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def make_weights(cfg, experts_local, device, seed):
    """Random block-FP8 experts, quantised by this library's kernel a few experts at a time."""
    from mlops_b200 import ops

    D, F = cfg["D"], cfg["F"]
    g = torch.Generator(device=device).manual_seed(seed)
    w13_q = torch.empty((experts_local, 2 * F, D), dtype=torch.float8_e4m3fn, device=device)
    w13_s = torch.empty((experts_local, 2 * F // 128, D // 128), dtype=torch.float32, device=device)
    w2_q = torch.empty((experts_local, D, F), dtype=torch.float8_e4m3fn, device=device)
    w2_s = torch.empty((experts_local, D // 128, F // 128), dtype=torch.float32, device=device)
    chunk = max(1, min(experts_local, (1 << 28) // (2 * F * D)))
    for lo in range(0, experts_local, chunk):
        hi = min(lo + chunk, experts_local)
        w = (torch.randn(hi - lo, 2 * F, D, device=device, generator=g) * 0.02).bfloat16()
        w13_q[lo:hi], w13_s[lo:hi] = ops.quantize_blocks(w)
        w = (torch.randn(hi - lo, D, F, device=device, generator=g) * 0.02).bfloat16()
        w2_q[lo:hi], w2_s[lo:hi] = ops.quantize_blocks(w)
    return (w13_q, w13_s), (w2_q, w2_s)


def gpu_arm(args, cfg):
    from mlops_b200 import layer, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        # the all-to-all kernels run beside the GEMMs on at most this many SMs; the FP8 GEMMs draw
        # their tiles dynamically and take whatever SMs are left
        comm_sms = int(os.environ.get("B200MOE_EP_COMM_SMS", "32"))
        os.environ.setdefault("NCCL_MAX_CTAS", str(comm_sms))
        dist.init_process_group("nccl", device_id=device)
    T, D, E, F, K = cfg["T"], cfg["D"], cfg["E"], cfg["F"], cfg["K"]
    experts_local = E // world

    g = torch.Generator(device=device).manual_seed(1234 + rank)
    gw = torch.Generator(device=device).manual_seed(99)  # replicated parameters: same on every rank
    x_host = torch.randn(T, D, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
    dy_host = torch.randn(T, D, generator=torch.Generator().manual_seed(1000 + rank)).bfloat16().pin_memory()
    x = x_host.to(device)
    dy = dy_host.to(device)
    residual = torch.zeros_like(x)
    router = torch.randn(E, D, device=device, generator=gw) * 0.02
    # The selection bias of a trained DeepSeek-style router is the correction that BALANCES expert
    # load; a random bias of the survey's scale (0.1) does the opposite at the sigmoid's tail
    # (experts between 0 and 8555 rows for a mean of 1024). 0.001 keeps the bias path exercised
    # and the load near uniform (config 5 is the skewed-load workload).
    bias = torch.randn(E, device=device, generator=gw) * 0.001 if cfg["mode"] == "sigmoid_noaux_tc" else None
    w13, w2 = make_weights(cfg, experts_local, device, seed=7 + rank)
    shared = None
    if cfg["shared"]:
        shared = ((torch.randn(2 * F, D, device=device, generator=gw) * 0.02).bfloat16(),
                  (torch.randn(D, F, device=device, generator=gw) * 0.02).bfloat16())
    del g

    lora = None
    if cfg.get("lora_rank"):
        from mlops_b200.lora import expert_lora
        from mlops_b200.weights import BlockFP8Weight

        r = cfg["lora_rank"]
        # skew lives in the data: x[:, 0] = 1 and Wr[:, 0] = log p_e shift the logits by log p_e
        popularity = torch.arange(1, E + 1, device=device).float().pow(-cfg["zipf"])
        router[:, 0] = torch.log(popularity / popularity.sum())
        x[:, 0] = 1.0
        x_host[:, 0] = 1.0
        gf = torch.Generator(device=device).manual_seed(31 + rank)  # this rank's experts' factors
        El = experts_local
        factors = [(torch.randn(El, r, D, device=device, generator=gf) * 0.02).bfloat16(),
                   (torch.randn(El, 2 * F, r, device=device, generator=gf) * 0.01).bfloat16(),
                   (torch.randn(El, r, F, device=device, generator=gf) * 0.02).bfloat16(),
                   (torch.randn(El, D, r, device=device, generator=gf) * 0.01).bfloat16()]
        for f in factors:
            f.requires_grad_(True)
        lora = dict(factors=factors, w13=BlockFP8Weight(*w13), w2=BlockFP8Weight(*w2))

    route_kwargs = dict(top_k=K, routing_mode=cfg["mode"], router_bias=bias, n_group=cfg["n_group"],
                        topk_group=cfg["topk_group"], routed_scaling=cfg["scaling"])
    ep = None
    if distributed:
        from mlops_b200 import ep as ep_module

        # Group-limited routing with balanced load: experts in contiguous blocks, so a token's
        # experts sit on few ranks and it is sent once per rank (de-duplicated dispatch).
        # Skewed popularity (the LoRA workload): experts strided over the ranks, one row per
        # assignment.
        dedup = os.environ.get("B200MOE_EP_DEDUP", "1" if cfg["n_group"] > 1 else "0") == "1"
        expert_map = os.environ.get("B200MOE_EP_MAP", "contiguous" if dedup else "strided")

        ep = ep_module.ExpertParallelMoE(
            ep_module.ExpertParallelConfig(hidden=D, experts=E, intermediate=F, top_k=K, routing_mode=cfg["mode"],
                                           n_group=cfg["n_group"], topk_group=cfg["topk_group"],
                                           routed_scaling=cfg["scaling"], expert_map=expert_map, dedup=dedup),
            dist.group.WORLD, router_weight=router, router_bias=bias, w13=w13, w2=w2, shared=shared,
            device=device, chunks=int(os.environ["B200MOE_EP_CHUNKS"]) if "B200MOE_EP_CHUNKS" in os.environ else None,
            comm_sms=int(os.environ.get("B200MOE_EP_LIMIT_SMS", "0")),
            lora=None if lora is None else dict(zip(("a13", "b13", "a2", "b2"), lora["factors"]), scale=1.0),
            frozen_base=lora is not None)

    rows_received = []

    def step(x_in, dy_in):
        if ep is not None:
            result = ep.forward_backward(x_in, residual, dy_in)
            rows_received.append(ep.last_recv_rows)
            return result
        if lora is not None:
            x_leaf = x_in.detach().requires_grad_(True)
            out, aux, counts, _ = expert_lora(x_leaf, residual, router, lora["w13"], lora["w2"], *lora["factors"],
                                              top_k=K, routing_mode=cfg["mode"], scale=1.0)
            grads = torch.autograd.grad(out, [x_leaf, *lora["factors"]], dy_in)
            return out.detach(), grads[0], aux.detach(), counts
        base, shared_h13 = residual, None
        if shared is not None:
            y_shared, shared_h13 = layer.shared_expert_forward(x_in, *shared)
            base = residual + y_shared
        result = layer.forward_routed(x_in, base, router, w13, w2, **route_kwargs)
        grads = layer.backward_routed(dy_in, None, None, x_in, router, w13, w2, *result[4:], top_k=K,
                                      routing_mode=cfg["mode"])
        grad_x = grads[0]
        if shared is not None:
            gx_s, _gw13_s, _gw2_s = layer.shared_expert_backward(dy_in, x_in, *shared, shared_h13)
            grad_x = grad_x + gx_s
        return result[0], grad_x, result[1], result[2]

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop)], device=device)
        if distributed:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return elapsed.item() / steps

    # ---- device-resident timing (the `value`)
    for _ in range(args.warmup):
        step(x, dy)
    ops.check_status(device)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ops.GEMM_TIMINGS = []
    launches_before = ops.LAUNCHES
    ms_per_step = timed(lambda: step(x, dy), args.steps)
    launches = ops.LAUNCHES - launches_before
    timings, ops.GEMM_TIMINGS = ops.GEMM_TIMINGS, None
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status(device)

    # ---- end to end from pinned host buffers
    host_result = torch.empty(4, dtype=torch.float32).pin_memory()

    # The step's inputs come from pinned host memory every step and a summary of its results
    # goes back.  The upload of step i+1 runs on a copy stream while step i computes (what an
    # input pipeline does: two device buffers); the first timed step uploads its own inputs
    # inside the timed region and the last one prefetches nothing, so the region holds exactly
    # `steps` uploads and `steps` read-backs.
    copy_stream = torch.cuda.Stream(device=device)
    buffers = [(x, dy), (torch.empty_like(x), torch.empty_like(dy))]
    uploaded = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    state = dict(i=0, steps=0)

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])  # the step that read this buffer has finished
            buffers[slot][0].copy_(x_host, non_blocking=True)
            buffers[slot][1].copy_(dy_host, non_blocking=True)
            uploaded[slot].record(copy_stream)

    def e2e_begin(steps):
        state["i"], state["steps"] = 0, steps
        for event in consumed:
            event.record(torch.cuda.current_stream())

    def e2e_step():
        i, slot = state["i"], state["i"] % 2
        if i == 0:
            upload(slot)
        if i + 1 < state["steps"]:
            upload((i + 1) % 2)
        torch.cuda.current_stream().wait_event(uploaded[slot])
        out, grad_x, aux, counts = step(*buffers[slot])
        consumed[slot].record(torch.cuda.current_stream())
        summary = torch.stack([out.sum(dtype=torch.float32), grad_x.sum(dtype=torch.float32), aux.float(),
                               counts.float().max()])
        host_result.copy_(summary, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        state["i"] = i + 1

    e2e_begin(1)
    e2e_step()
    e2e_begin(args.steps)
    e2e_ms = timed(e2e_step, args.steps)
    h2d = x_host.numel() * 2 + dy_host.numel() * 2
    d2h = host_result.numel() * 4

    per_rank_rows = None
    if distributed:
        mine = torch.tensor([rows_received[-1]], device=device, dtype=torch.int64)
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        per_rank_rows = [int(t.item()) for t in gathered]
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    fp8 = [(s.elapsed_time(e), fl) for s, e, kind, fl in timings if kind == "fp8"]
    wg = [(s.elapsed_time(e), fl) for s, e, kind, fl in timings if kind == "wgrad_bf16"]
    fp8_ms = sum(t for t, _ in fp8)
    fp8_flops = sum(f for _, f in fp8)
    achieved = fp8_flops / (fp8_ms * 1e-3) / 1e12 if fp8_ms > 0 else 0.0
    peak_fp8 = 2.0 * peaks["bf16_tflops_sustained"]
    rows = T * K
    routed_flops = (12.0 if lora is not None else 18.0) * D * F * rows  # a frozen base has no base wgrad
    shared_flops = 18.0 * D * F * T if cfg["shared"] else 0.0
    tokens_total = T * world
    line = {
        "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": tokens_total / (ms_per_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["name"], "tokens_per_gpu": T, "hidden": D, "experts": E, "intermediate": F,
                   "top_k": K, "routing": cfg["mode"],
                   "router_bias": "N(0, 0.001), balanced load" if bias is not None else None, "shared_expert": bool(cfg["shared"]),
                   "expert_parallel": world, "expert_map": ep.config.expert_map if distributed else "local",
                   "dedup_dispatch": bool(distributed and ep.config.dedup),
                   "rows_per_rank": per_rank_rows, "weights": "block-FP8 e4m3 128x128, random N(0,0.02)",
                   "activations": "e4m3 1x128 blocks", "weight_grads": "bf16 operands, fp32 sums, bf16 out",
                   "l2": "inputs exceed L2 (no flush needed)" if T * D * 2 > (126 << 20) else "inputs fit L2"},
        "tflops_per_gpu": (routed_flops + shared_flops) / (ms_per_step * 1e-3) / 1e12,
        "gpu_launches": launches,
        "e2e": {"value": tokens_total / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "roofline": {"kernel": "grouped_gemm_fp8_kernel", "bound": "tensor", "achieved": achieved,
                     "peak": peak_fp8, "unit": "TFLOP/s", "frac": achieved / peak_fp8 if peak_fp8 else None,
                     "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_kind}); "
                                    "FP8 issues at twice the bf16 rate",
                     "frac_of_nominal_fp8": achieved / NOMINAL_FP8_TFLOPS,
                     "launches_timed": len(fp8), "ms_in_kernel_per_step": fp8_ms / max(args.steps, 1),
                     "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(args.workload)},
        "wgrad": {"kernel": "grouped_wgrad_kernel", "achieved_tflops":
                  (sum(f for _, f in wg) / (sum(t for t, _ in wg) * 1e-3) / 1e12) if wg else None,
                  "peak_bf16_sustained": peaks["bf16_tflops_sustained"]},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(cfg, cfg["cpu_tokens"])
    print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


# DRAM bytes (read + write) per launch of the dominant kernel, averaged over its four launches
# of a step, from the ncu capture summarised in profiles/grouped_gemm_fp8_c4p.md (6.19 GB over
# four launches at 32768 rows x 32 experts). Traffic is operands once + output once, so the
# full-size figure scales with rows and experts (x8).
TRAFFIC_BYTES_PER_LAUNCH: dict[str, float] = {"c4p": 6.19e9 / 4, "c4": 8 * 6.19e9 / 4}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = parser.parse_args()
    cfg = dict(WORKLOADS[args.workload])
    # bounded CPU sample: a few experts of the same shape, a few hundred tokens
    cfg["E_cpu"] = min(cfg["E"], 8)
    cfg["cpu_tokens"] = 256 if args.workload != "c1" else 512
    if args.impl == "reference":
        reference_arm(args, cfg)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the CUDA path has no CPU fallback)")
    gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
