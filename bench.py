"""Benchmark of the routed-MoE expert path: one step = forward + backward of one MoE layer
over one batch of synthetic tokens, through the provider's public call (`provider.apply`, the
function the reference's registry dispatches to) and PyTorch autograd.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c3|c5|c2|c1|c4p]
                    [--impl reference] [--no-cpu] [--no-extras]

Prints ONE JSON line (rank 0).
  value         tokens/s of the whole job with the step's inputs resident in HBM
  e2e           the same step fed from pinned host buffers: host->device copies of the step's
                inputs and a device->host read of its summary (loss-like scalars; a training
                step hands no tensor back to the host) inside the timed region
  roofline      the dominant kernel (block-FP8 grouped GEMM) timed live with CUDA events on the
                launching stream: algorithmic FLOP / time against measured and nominal peaks
  cpu_baseline  the reference's own CPU code (from `oracle/_ref`, else the oracle port) on a
                bounded sample, timed on this machine's host cores
  workloads     (N = 1) the other configurations, three timed steps each: the standalone
                grouped GEMM (c2, beside the reference's Triton kernel when it runs), the
                Mixtral-shaped layer (c3), the Qwen3-shaped layer with LoRA and skew (c5), and the
                headline layer with a skewed selection bias, N(0, 0.1) (c4_skewed)
  hbm_kernels   (N = 1) GB/s of the routing / sort / quantise / SwiGLU / combine kernels
  ep_check      (N > 1) the expert-parallel layer against the single-GPU layer on the gathered
                weights, on a small case, before the timed region
`--impl reference` times the reference's CPU path alone (rank 0).

Workloads (shapes only; weights are random, data synthetic, seeded):
  c4  DeepSeek-V3-shaped: D=7168, 256 experts, F=2048, sigmoid/group top-8, one shared expert,
      T=32768 tokens per GPU (the configuration the headline metric is quoted on)
  c4p the same layer at profiling size (32 experts, T=4096: the same 1024 rows per expert,
      a few GB on the device) for ncu captures
  c5  Qwen3-30B-A3B-shaped with rank-16 LoRA on a frozen base and Zipf(1.2) expert popularity:
      D=2048, 128 experts, F=768, softmax top-8, T=65536 per GPU (expert-parallel at N > 1)
  c3  Mixtral-8x7B-shaped: D=4096, 8 experts, F=14336, softmax top-2, T=16384
  c2  standalone block-FP8 grouped GEMM: 32 groups, 65536 rows split Zipf(1.1), K=4096, N=2048
  c1  the small CPU-runnable case: D=256, 8 experts, F=512, softmax top-2, T=512
"""

from __future__ import annotations

import argparse
import gc
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
    "c2": dict(name="standalone_block_fp8_grouped_gemm", groups=32, rows=65536, K=4096, N=2048, zipf=1.1),
}
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_BF16_SUSTAINED = 1400.0
BALANCED_BIAS_STD = 0.001
SKEWED_BIAS_STD = 0.1

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the four FP8 GEMM launches of
# one step, from the ncu capture of `python bench.py --workload c4p --steps 1 --warmup 1
# --no-cpu --no-extras` (forward up, forward down, input gradient of down, input gradient of
# up). Traffic is operands once + output once, so the full-size layer (8x the rows and
# experts) scales by 8.
GEMM_DRAM_BYTES_C4P = (1.271e9 + 0.278e9, 0.540e9 + 0.439e9, 0.742e9 + 0.130e9, 1.097e9 + 0.460e9)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": FALLBACK_BF16_SUSTAINED}, "fallback"


# ------------------------------------------------------------------------------ CPU arms
def reference_package():
    """The reference itself (`oracle/_ref`, put there by `oracle/build_ref.py`), or None."""
    from oracle.build_ref import reference

    try:
        return reference()
    except Exception as error:  # an import failure is reported, not hidden
        print(f"reference import failed: {error!r}", file=sys.stderr)
        return None


def _threads():
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    return threads


def reference_c1(mlops):
    """The reference's native-PyTorch provider on the small configuration exactly as specified
    (T=512, D=256, 8 experts, top-2 softmax, F=512, seed 0): forward + backward wall time,
    2 warm-ups, best of 5 and median."""
    from mlops.block_fp8 import BlockFP8Weight
    from mlops.dispatch import use_implementation

    torch.manual_seed(0)
    x = torch.randn(512, 256).bfloat16().requires_grad_(True)
    router = (torch.randn(8, 256) * 0.02).requires_grad_(True)
    w13 = BlockFP8Weight.quantize((torch.randn(8, 1024, 256) * 0.02).bfloat16()).requires_grad_(True)
    w2 = BlockFP8Weight.quantize((torch.randn(8, 256, 512) * 0.02).bfloat16()).requires_grad_(True)
    dy = torch.randn(512, 256).bfloat16()

    def step():
        with use_implementation("moe", "native_torch.moe"):
            out, _aux, _counts, _psum = mlops.moe(x, torch.zeros_like(x), router, w13, w2, top_k=2,
                                                  routing_mode="softmax_then_topk", compute_precision="bf16")
        torch.autograd.grad(out, [x, router, w13, w2], dy)

    for _ in range(2):
        step()
    times = []
    for _ in range(5):
        start = time.perf_counter()
        step()
        times.append(time.perf_counter() - start)
    best, median = min(times), statistics.median(times)
    return {"implementation": "native_torch.moe via mlops.moe", "tokens": 512, "ms_best": best * 1e3,
            "ms_median": median * 1e3, "tokens_per_s_best": 512 / best, "tokens_per_s_median": 512 / median}


def reference_sample_step(mlops, cfg, tokens, experts, seed=0):
    """One forward + backward of `tokens` tokens of the workload's shapes over `experts` experts
    through the reference's gather-based CPU expert computation
    (`mlops.expert_parallel.reference.expert_computation`: bf16 weights dequantised from the
    block-FP8 containers, fp32 accumulation) with the reference's own router. Returns a closure
    that runs one step."""
    from mlops.block_fp8 import BlockFP8Weight
    from mlops.expert_parallel.reference import expert_computation, router_logits
    from mlops.kernels.moe_router import route

    g = torch.Generator().manual_seed(seed)
    D, F, K = cfg["D"], cfg["F"], cfg["K"]
    x = torch.randn(tokens, D, generator=g).bfloat16().requires_grad_(True)
    dy = torch.randn(tokens, D, generator=g).bfloat16()
    router = torch.randn(experts, D, generator=g) * 0.02
    w13 = BlockFP8Weight.quantize((torch.randn(experts, 2 * F, D, generator=g) * 0.02).bfloat16())
    w2 = BlockFP8Weight.quantize((torch.randn(experts, D, F, generator=g) * 0.02).bfloat16())
    bias = torch.randn(experts, generator=g) * SKEWED_BIAS_STD if cfg["mode"] == "sigmoid_noaux_tc" else None
    n_group = cfg["n_group"] if experts % cfg["n_group"] == 0 and experts // cfg["n_group"] >= 2 else 1
    topk_group = cfg["topk_group"] if n_group > 1 else 1
    shared = ()
    if cfg.get("shared"):
        shared = tuple((torch.randn(*shape, generator=g) * 0.02).bfloat16().requires_grad_(True)
                       for shape in ((F, D), (F, D), (D, F)))

    def step():
        with torch.no_grad():
            logits = router_logits(x.detach(), router)
            weights, ids = route(logits, K, cfg["mode"], bias=bias, n_group=n_group, topk_group=topk_group,
                                 routed_scaling=cfg["scaling"])
        dense13 = w13.dequantize(dtype=torch.bfloat16).requires_grad_(True)  # per call, as the provider does
        dense2 = w2.dequantize(dtype=torch.bfloat16).requires_grad_(True)
        out = expert_computation(x, ids, weights, dense13[:, :F], dense13[:, F:], dense2, shared_weights=shared)
        torch.autograd.grad(out, [x, dense13, dense2, *shared], dy)

    return step


def port_sample_step(cfg, tokens, experts, seed=0):
    """The same sample through this repository's CPU oracle (used only where the reference
    package is not at hand)."""
    from oracle import moe_oracle as O

    g = torch.Generator().manual_seed(seed)
    D, F, K = cfg["D"], cfg["F"], cfg["K"]
    x = torch.randn(tokens, D, generator=g).bfloat16()
    dy = torch.randn(tokens, D, generator=g).bfloat16()
    router = torch.randn(experts, D, generator=g) * 0.02
    w13 = O.quantize_blocks((torch.randn(experts, 2 * F, D, generator=g) * 0.02).bfloat16())
    w2 = O.quantize_blocks((torch.randn(experts, D, F, generator=g) * 0.02).bfloat16())
    bias = torch.randn(experts, generator=g) * SKEWED_BIAS_STD if cfg["mode"] == "sigmoid_noaux_tc" else None
    n_group = cfg["n_group"] if experts % cfg["n_group"] == 0 and experts // cfg["n_group"] >= 2 else 1

    def step():
        logits = O.router_logits(x, router)
        fwd = O.forward_block_fp8(x, torch.zeros_like(x), logits, *w13, *w2, top_k=K, routing_mode=cfg["mode"],
                                  router_bias=bias, n_group=n_group,
                                  topk_group=cfg["topk_group"] if n_group > 1 else 1,
                                  routed_scaling=cfg["scaling"], gemm_dtype=torch.float32)
        O.backward_block_fp8(dy, x, fwd, *w13, *w2, top_k=K, gemm_dtype=torch.float32)

    return step


SAMPLE_LADDER = ((16, 8), (32, 8), (64, 8), (128, 16), (256, 32))  # (tokens, experts), ascending cost


def cpu_sample(cfg, tokens, experts):
    """`(step, kind, description)` of a bounded CPU sample of a layer workload."""
    experts = min(experts, cfg["E"])
    mlops = reference_package()
    shape = f"{tokens} tokens, {experts} of {cfg['E']} experts, D={cfg['D']} F={cfg['F']} top-{min(cfg['K'], experts)}"
    sample_cfg = dict(cfg, K=min(cfg["K"], experts))
    if mlops is not None:
        return (reference_sample_step(mlops, sample_cfg, tokens, experts), "reference",
                f"{shape}, forward+backward, the reference's expert_parallel.reference.expert_computation "
                "with its own router (bf16 on block-FP8 weights dequantised per call, CPU)")
    return (port_sample_step(sample_cfg, tokens, experts), "port",
            f"{shape}, forward+backward, CPU oracle port (fp32 products of dequantised E4M3 operands); "
            "the reference package was not found at oracle/_ref")


def choose_sample(cfg, calls, budget_seconds):
    """The largest sample of the ladder whose `calls` steps fit `budget_seconds` on this machine:
    each rung is timed once, from the smallest up, until the next one would not fit. Returns
    `(step, kind, description, tokens, seconds of the last timed step)`."""
    chosen = None
    for tokens, experts in SAMPLE_LADDER:
        step, kind, description = cpu_sample(cfg, tokens, experts)
        start = time.perf_counter()
        step()
        seconds = time.perf_counter() - start
        if chosen is not None and seconds * calls > budget_seconds:
            break
        chosen = (step, kind, description, tokens, seconds)
        if seconds * calls * 2.5 > budget_seconds:  # the next rung costs at least twice as much
            break
    return chosen


def cpu_baseline(cfg):
    threads = _threads()
    step, kind, description, tokens, _ = choose_sample(cfg, calls=1, budget_seconds=20.0)
    start = time.perf_counter()
    step()
    seconds = time.perf_counter() - start
    result = {"value": tokens / seconds, "unit": "tokens/s", "cores": threads, "kind": kind,
              "sample": f"{description}; {seconds:.1f} s per step", "torch_threads": torch.get_num_threads()}
    mlops = reference_package()
    if mlops is not None:
        result["c1_native_torch"] = reference_c1(mlops)
    return result


def reference_arm(args, cfg):
    """The reference's own CPU implementation of the path on this machine's host cores, on a
    bounded sample of the GPU arm's workload sized so that the whole run ends within a few
    minutes (rank 0 only; other ranks exit without work)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = _threads()
    calls = max(args.steps, 1) + max(args.warmup, 0)
    step, kind, description, tokens, _ = choose_sample(cfg, calls=calls, budget_seconds=150.0)
    for _ in range(max(args.warmup, 0)):
        step()
    times = []
    for _ in range(max(args.steps, 1)):
        start = time.perf_counter()
        step()
        times.append(time.perf_counter() - start)
    mean = sum(times) / len(times)
    value = tokens / mean
    line = {
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if kind == "reference"
        else "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["name"], "sample": description, "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": description},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    mlops = reference_package()
    if mlops is not None:
        line["c1_native_torch"] = reference_c1(mlops)
    print(json.dumps(line))


# ------------------------------------------------------------------------------ GPU arm
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


def timed_steps(fn, steps, device, distributed=False):
    """Milliseconds per call: CUDA events on the current stream around `steps` calls, barrier +
    synchronize on both sides, max over ranks."""
    import torch.distributed as dist

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

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


class Layer:
    """One workload on one device (or one rank): parameters, inputs and `step(x, dy)`, which runs
    forward + backward through the public call and returns `(output, grad_x, aux, counts)`."""

    def __init__(self, cfg, device, *, world=1, rank=0, group=None, bias_std=BALANCED_BIAS_STD, bf16_weights=False):
        from mlops_b200 import provider
        from mlops_b200.weights import BlockFP8Weight

        self.cfg, self.device, self.world = cfg, device, world
        T, D, E, F, K = cfg["T"], cfg["D"], cfg["E"], cfg["F"], cfg["K"]
        experts_local = E // world
        gw = torch.Generator(device=device).manual_seed(99)  # replicated parameters: same on every rank
        self.x_host = torch.randn(T, D, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
        self.dy_host = torch.randn(T, D, generator=torch.Generator().manual_seed(1000 + rank)).bfloat16().pin_memory()
        self.router = torch.randn(E, D, device=device, generator=gw) * 0.02
        # The selection bias of a trained DeepSeek-style router is the correction that BALANCES
        # expert load; a random bias of scale 0.1 does the opposite at the sigmoid's
        # tail (experts between 0 and ~8500 rows for a mean of 1024). The headline uses 0.001
        # (bias path exercised, load near uniform); `c4_skewed` reports 0.1 beside it.
        self.bias_std = bias_std
        self.bias = (torch.randn(E, device=device, generator=gw) * bias_std
                     if cfg["mode"] == "sigmoid_noaux_tc" else None)
        self.shared = None
        if cfg["shared"]:
            self.shared = ((torch.randn(2 * F, D, device=device, generator=gw) * 0.02).bfloat16(),
                           (torch.randn(D, F, device=device, generator=gw) * 0.02).bfloat16())
        self.factors = None
        if cfg.get("lora_rank"):
            # skew lives in the data: x[:, 0] = 1 and Wr[:, 0] = log p_e shift the logits by log p_e
            popularity = torch.arange(1, E + 1, device=device).float().pow(-cfg["zipf"])
            self.router[:, 0] = torch.log(popularity / popularity.sum())
            self.x_host[:, 0] = 1.0
            r = cfg["lora_rank"]
            gf = torch.Generator(device=device).manual_seed(31 + rank)  # this rank's experts' factors
            El = experts_local
            self.factors = [(torch.randn(El, r, D, device=device, generator=gf) * 0.02).bfloat16(),
                            (torch.randn(El, 2 * F, r, device=device, generator=gf) * 0.01).bfloat16(),
                            (torch.randn(El, r, F, device=device, generator=gf) * 0.02).bfloat16(),
                            (torch.randn(El, D, r, device=device, generator=gf) * 0.01).bfloat16()]
        self.x = self.x_host.to(device)
        self.dy = self.dy_host.to(device)
        self.residual = torch.zeros_like(self.x)
        self.w13, self.w2 = make_weights(cfg, experts_local, device, seed=7 + rank)
        self.route_kwargs = dict(top_k=K, routing_mode=cfg["mode"], router_bias=self.bias, n_group=cfg["n_group"],
                                 topk_group=cfg["topk_group"], routed_scaling=cfg["scaling"])
        self.rows_received = []
        self.ep = None
        self.provider = provider
        if world > 1:
            self._make_expert_parallel(group)
        else:
            # what a trainer holds: parameters that ask for gradients (a frozen base under LoRA)
            frozen = self.factors is not None
            if bf16_weights:
                # plain bf16 experts with the same values: the bf16 compute path
                self.w13_param = BlockFP8Weight(*self.w13).dequantize().to(torch.bfloat16).requires_grad_(not frozen)
                self.w2_param = BlockFP8Weight(*self.w2).dequantize().to(torch.bfloat16).requires_grad_(not frozen)
                self.w13 = self.w2 = None
            else:
                self.w13_param = BlockFP8Weight(*self.w13).requires_grad_(not frozen)
                self.w2_param = BlockFP8Weight(*self.w2).requires_grad_(not frozen)
            self.router_param = self.router.requires_grad_(not frozen)
            if self.shared is not None:
                self.shared = tuple(w.requires_grad_(True) for w in self.shared)
            if self.factors is not None:
                self.factors = [f.requires_grad_(True) for f in self.factors]

    def _make_expert_parallel(self, group):
        from mlops_b200 import ep as ep_module

        cfg = self.cfg
        # Group-limited routing with balanced load: experts in contiguous blocks, so a token's
        # experts sit on few ranks and it is sent once per rank (de-duplicated dispatch).
        # Skewed popularity (the LoRA workload): experts strided over the ranks, one row per
        # assignment.
        dedup = os.environ.get("B200MOE_EP_DEDUP", "1" if cfg["n_group"] > 1 else "0") == "1"
        expert_map = os.environ.get("B200MOE_EP_MAP", "contiguous" if dedup else "strided")
        # one pre-weighted row per token copy on the way back (the reference's layers return
        # pre-weighted rows too); B200MOE_EP_PRESUM=0 returns one row per assignment
        presum = dedup and os.environ.get("B200MOE_EP_PRESUM", "1") == "1"
        # the token rows of a de-duplicated dispatch travel by this library's own kernel over NVLink
        # peer memory (B200MOE_EP_TRANSPORT=nccl: through a send buffer and the library all-to-all)
        # (default: on the world sizes it was verified on; B200MOE_EP_TRANSPORT=peer selects it up to 16 ranks)
        default_transport = "peer" if self.world <= 4 else "nccl"
        transport = os.environ.get("B200MOE_EP_TRANSPORT", default_transport) if dedup and self.world <= 16 else "nccl"
        self.transport = transport
        lora = None
        if self.factors is not None:
            lora = dict(zip(("a13", "b13", "a2", "b2"), self.factors), scale=1.0)
        self.ep = ep_module.ExpertParallelMoE(
            ep_module.ExpertParallelConfig(hidden=cfg["D"], experts=cfg["E"], intermediate=cfg["F"], top_k=cfg["K"],
                                           routing_mode=cfg["mode"], n_group=cfg["n_group"],
                                           topk_group=cfg["topk_group"], routed_scaling=cfg["scaling"],
                                           expert_map=expert_map, dedup=dedup, presum=presum, transport=transport),
            group, router_weight=self.router, router_bias=self.bias, w13=self.w13, w2=self.w2, shared=self.shared,
            device=self.device,
            chunks=int(os.environ["B200MOE_EP_CHUNKS"]) if "B200MOE_EP_CHUNKS" in os.environ else None,
            comm_sms=int(os.environ.get("B200MOE_EP_LIMIT_SMS", "0")), lora=lora, frozen_base=lora is not None)

    def step(self, x_in, dy_in):
        if self.ep is not None:
            result = self.ep.forward_backward(x_in, self.residual, dy_in)
            self.rows_received.append(self.ep.last_recv_rows)
            return result
        x_leaf = x_in.detach().requires_grad_(True)
        if self.factors is not None:
            from mlops_b200.lora import expert_lora

            out, aux, counts, _ = expert_lora(x_leaf, self.residual, self.router_param, self.w13_param,
                                              self.w2_param, *self.factors, top_k=self.cfg["K"],
                                              routing_mode=self.cfg["mode"], scale=1.0)
            grads = torch.autograd.grad(out, [x_leaf, *self.factors], dy_in)
            return out.detach(), grads[0], aux.detach(), counts
        shared = {} if self.shared is None else dict(shared_w13=self.shared[0], shared_w2=self.shared[1])
        out, aux, counts, _ = self.provider.apply(x_leaf, self.residual, self.router_param, self.w13_param,
                                                  self.w2_param, **self.route_kwargs, **shared)
        leaves = [x_leaf, self.router_param, self.w13_param, self.w2_param, *(self.shared or ())]
        grads = torch.autograd.grad(out, leaves, dy_in)
        return out.detach(), grads[0], aux.detach(), counts

    def flops(self):
        cfg = self.cfg
        rows = cfg["T"] * cfg["K"]
        routed = (12.0 if self.factors is not None else 18.0) * cfg["D"] * cfg["F"] * rows  # frozen base: no wgrad
        shared = 18.0 * cfg["D"] * cfg["F"] * cfg["T"] if cfg["shared"] else 0.0
        return routed, shared


def gemm_summary(timings, steps):
    fp8 = [(s.elapsed_time(e), fl) for s, e, kind, fl in timings if kind == "fp8"]
    bf16 = [(s.elapsed_time(e), fl) for s, e, kind, fl in timings if kind == "gemm_bf16"]
    wg = [(s.elapsed_time(e), fl) for s, e, kind, fl in timings if kind in ("wgrad_bf16", "wgrad_fp8")]
    fp8_ms, fp8_flops = sum(t for t, _ in fp8), sum(f for _, f in fp8)
    return {
        "fp8_tflops": fp8_flops / (fp8_ms * 1e-3) / 1e12 if fp8_ms > 0 else None,
        "fp8_ms_per_step": fp8_ms / max(steps, 1), "fp8_launches": len(fp8),
        "wgrad_tflops": (sum(f for _, f in wg) / (sum(t for t, _ in wg) * 1e-3) / 1e12) if wg else None,
        "wgrad_ms_per_step": sum(t for t, _ in wg) / max(steps, 1),
        # the bf16 forward / input-gradient GEMMs (plain bf16 experts) and the rank-r LoRA products
        "bf16_tflops": (sum(f for _, f in bf16) / (sum(t for t, _ in bf16) * 1e-3) / 1e12) if bf16 else None,
        "bf16_ms_per_step": sum(t for t, _ in bf16) / max(steps, 1),
    }


def run_layer(layer, steps, warmup, device, distributed=False):
    """`(ms per step, launches, gemm summary)` of a layer with resident inputs."""
    from mlops_b200 import ops

    for _ in range(warmup):
        layer.step(layer.x, layer.dy)
    ops.check_status(device)
    ops.GEMM_TIMINGS = []
    before = ops.LAUNCHES
    ms = timed_steps(lambda: layer.step(layer.x, layer.dy), steps, device, distributed)
    launches = ops.LAUNCHES - before
    timings, ops.GEMM_TIMINGS = ops.GEMM_TIMINGS, None
    ops.check_status(device)
    return ms, launches, gemm_summary(timings, steps)


def measure_fp8_peak(device, seconds=1.5):
    """cuBLAS FP8 (E4M3 x E4M3 -> bf16, fp32 accumulate) on 8192^3 through `torch._scaled_mm`:
    best of 10 single calls (burst) and back to back for `seconds` (sustained): the measured
    dense FP8 tensor peak of this GPU, in TFLOP/s."""
    n = 8192
    a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()  # column-major operand
    one = torch.ones((), device=device)
    run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
    try:
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run()
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        flops = 2.0 * n ** 3
        calls = max(10, int(seconds * 1e3 / best))
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(calls):
            run()
        e.record()
        torch.cuda.synchronize()
        sustained = flops * calls / (s.elapsed_time(e) * 1e-3) / 1e12
        return {"burst": flops / (best * 1e-3) / 1e12, "sustained": sustained, "seconds": s.elapsed_time(e) * 1e-3,
                "how": "torch._scaled_mm e4m3 x e4m3 -> bf16, 8192^3"}
    except Exception as error:
        return {"burst": None, "sustained": None, "how": f"torch._scaled_mm failed: {error!r}"}


def time_kernel(fn, reps=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def hbm_kernels(cfg, device, peaks):
    """The HBM-bound kernels of the path on the workload's shapes, each timed alone with CUDA
    events: algorithmic bytes / time, against the measured copy bandwidth and the nominal 8 TB/s.
    (The logits and the sort's ids fit in L2; the row kernels' operands are far larger.)"""
    from mlops_b200 import ops

    T, D, E, F, K = cfg["T"], cfg["D"], cfg["E"], cfg["F"], cfg["K"]
    R = T * K
    g = torch.Generator(device=device).manual_seed(5)
    x = torch.randn(T, D, device=device, generator=g).bfloat16()
    logits = torch.randn(T, E, device=device, generator=g)
    bias = torch.randn(E, device=device, generator=g) * BALANCED_BIAS_STD
    route = lambda: ops.route_topk(logits, K, cfg["mode"], bias=bias if cfg["mode"] == "sigmoid_noaux_tc" else None,  # noqa: E731
                                   n_group=cfg["n_group"], topk_group=cfg["topk_group"],
                                   routed_scaling=cfg["scaling"])
    weights, ids = route()
    order, offsets, slots, _counts = ops.sort_assignments(ids, E)
    h13 = torch.randn(R, 2 * F, device=device, generator=g).bfloat16()
    r = torch.randn(R, F, device=device, generator=g).bfloat16()
    y = torch.randn(R, D, device=device, generator=g).bfloat16()
    cases = {
        "route_topk": (route, 4.0 * T * E + 8.0 * T * K),
        "sort_assignments": (lambda: ops.sort_assignments(ids, E), 4.0 * R * 2 + 8.0 * R),
        # forward: every token quantised once and written to its K rows (what the layer runs)
        "quantize_rows_scatter": (lambda: ops.quantize_rows_scatter(x, slots),
                                  2.0 * T * D + R * D + 4.0 * R * D / 128),
        # backward: the same pass also writes the bf16 rows in expert order for the weight gradient
        "quantize_rows_scatter_with_copy": (lambda: ops.quantize_rows_scatter(x, slots, with_copy=True),
                                            2.0 * T * D + R * D + 4.0 * R * D / 128 + 2.0 * R * D),
        # row-major form (one warp per output row), used where rows arrive in another order
        "quantize_rows_gather": (lambda: ops.quantize_rows(x, gather=order, gather_div=K),
                                 2.0 * T * D + R * D + 4.0 * R * D / 128),
        "swiglu_quantize": (lambda: ops.swiglu_quantize(h13), 4.0 * R * F + R * F + 4.0 * R * F / 128),
        "dswiglu_routed": (lambda: ops.dswiglu_routed(h13, r, weights, order, quantized=True, rounded=True,
                                                      scaled_activation=True),
                           (4.0 + 2.0) * R * F + 2.0 * R * F + 4.0 * R * F + 2.0 * R * F + 4.0 * R * (2 * F) / 128),
        "combine": (lambda: ops.combine(y, slots, weights, x), 2.0 * R * D + 2.0 * T * D + 2.0 * T * D),
    }
    out = {}
    for name, (fn, nbytes) in cases.items():
        ms = time_kernel(fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "algorithmic_bytes": nbytes, "gb_per_s": gbs,
                     "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS}
    ops.check_status(device)
    return out


def run_c2(device, peaks, fp8_peak, steps=3, warmup=2):
    """The standalone grouped GEMM: 32 groups, 65536 rows split by a multinomial draw with
    Zipf(1.1) popularity, K=4096, N=2048; A in E4M3 with 1x128 scales (and, for the reference's
    kernel, with one scale per row: its only mode), B in E4M3 with 128x128 scales, bf16 out."""
    from mlops_b200 import ops

    cfg = WORKLOADS["c2"]
    G, R, K, N = cfg["groups"], cfg["rows"], cfg["K"], cfg["N"]
    g = torch.Generator().manual_seed(0)
    p = torch.arange(1, G + 1).float().pow(-cfg["zipf"])
    counts = torch.bincount(torch.multinomial(p / p.sum(), R, replacement=True, generator=g), minlength=G)
    offsets = torch.zeros(G + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0).to(torch.int32)
    offsets = offsets.to(device)
    gd = torch.Generator(device=device).manual_seed(1)
    a = torch.randn(R, K, device=device, generator=gd).bfloat16()
    a_q, a_s = ops.quantize_rows(a)
    a_q_row, a_s_row = ops.quantize_rows(a, mode="row")
    b_q, b_s = ops.quantize_blocks(torch.randn(G, N, K, device=device, generator=gd).bfloat16())
    flops = 2.0 * R * N * K

    def rate(fn):
        for _ in range(warmup):
            fn()
        ms = time_kernel(fn, reps=steps)
        return {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12}

    result = {"workload": cfg["name"], "rows_per_group_min_max": [int(counts.min()), int(counts.max())],
              "flop": flops,
              "b200_1x128_scales": rate(lambda: ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets)),
              "b200_row_scales": rate(lambda: ops.grouped_gemm_fp8(a_q_row, a_s_row, b_q, b_s, offsets))}
    for entry in ("b200_1x128_scales", "b200_row_scales"):
        result[entry]["frac_of_2x_bf16_sustained"] = result[entry]["tflops"] / (2.0 * peaks["bf16_tflops_sustained"])
        if fp8_peak.get("sustained"):
            result[entry]["frac_of_measured_fp8_sustained"] = result[entry]["tflops"] / fp8_peak["sustained"]
    ops.check_status(device)
    mlops = reference_package()
    if mlops is None:
        result["reference_triton_grouped_block_gemm"] = {"unavailable": "reference package not at oracle/_ref"}
        return result
    try:
        from mlops.kernels.block_fp8 import grouped_block_gemm

        run = lambda: grouped_block_gemm(a_q_row, b_q, b_s, offsets, row_scale=a_s_row.reshape(-1).contiguous())  # noqa: E731
        out_ref = run()
        out_own = ops.grouped_gemm_fp8(a_q_row, a_s_row, b_q, b_s, offsets)
        diff = (out_ref.float() - out_own.float()).abs().max().item() / out_own.float().abs().max().item()
        entry = rate(run)
        entry["max_abs_diff_over_max_abs"] = diff
        entry["kernel"] = "mlops.kernels.block_fp8.grouped_block_gemm (Triton, row scales, its launch defaults)"
        result["reference_triton_grouped_block_gemm"] = entry
    except Exception as error:  # Triton missing or refusing this GPU: say so, do not hide it
        result["reference_triton_grouped_block_gemm"] = {"unavailable": repr(error)[:300]}
    return result


def extras(device, peaks, fp8_peak):
    """The configurations the headline does not cover, three timed steps each."""
    out = {}
    out["c2"] = run_c2(device, peaks, fp8_peak)
    from mlops_b200 import provider

    for key, bias_std in (("c3", BALANCED_BIAS_STD), ("c5", BALANCED_BIAS_STD), ("c4_skewed", SKEWED_BIAS_STD),
                          ("c4_fp8_weight_gradients", BALANCED_BIAS_STD), ("c3_bf16_experts", BALANCED_BIAS_STD)):
        cfg = dict(WORKLOADS["c4" if key.startswith("c4_") else "c3" if key.startswith("c3") else key])
        gc.collect()
        torch.cuda.empty_cache()
        layer = Layer(cfg, device, bias_std=bias_std, bf16_weights=key == "c3_bf16_experts")
        # the optional recipe with E4M3 operands for the expert weight gradients (not the headline's)
        previous = provider.set_weight_gradient_operands("fp8" if key == "c4_fp8_weight_gradients" else "bf16")
        try:
            ms, _launches, gemms = run_layer(layer, 3, 2, device)
        finally:
            provider.set_weight_gradient_operands(previous)
        _out, _gx, _aux, counts = layer.step(layer.x, layer.dy)
        routed, shared = layer.flops()
        entry = {"workload": cfg["name"], "ms_per_step": ms, "tokens_per_s": cfg["T"] / (ms * 1e-3),
                 "tflops_per_gpu": (routed + shared) / (ms * 1e-3) / 1e12, "fp8_gemm_tflops": gemms["fp8_tflops"],
                 "fp8_frac_of_2x_bf16_sustained": (gemms["fp8_tflops"] or 0.0) / (2.0 * peaks["bf16_tflops_sustained"]),
                 "wgrad_tflops": gemms["wgrad_tflops"],
                 "rows_per_expert_min_max": [int(counts.min()), int(counts.max())], "steps": 3, "warmup": 2}
        if fp8_peak.get("sustained"):
            entry["fp8_frac_of_measured_fp8_sustained"] = (gemms["fp8_tflops"] or 0.0) / fp8_peak["sustained"]
        if key == "c5":
            entry["lora_rank_products_ms_per_step"] = gemms["bf16_ms_per_step"]
        if key == "c4_skewed":
            entry["router_bias"] = f"N(0, {SKEWED_BIAS_STD}): skewed load"
        if key == "c3_bf16_experts":
            entry["compute"] = "plain bf16 expert weights: bf16 grouped GEMMs, nothing quantised"
            for key_ in ("fp8_gemm_tflops", "fp8_frac_of_2x_bf16_sustained", "fp8_frac_of_measured_fp8_sustained"):
                entry.pop(key_, None)
            entry["bf16_gemm_tflops"] = gemms["bf16_tflops"]
            entry["bf16_gemm_frac_of_bf16_sustained"] = (gemms["bf16_tflops"] or 0.0) / peaks["bf16_tflops_sustained"]
        if key == "c4_fp8_weight_gradients":
            entry["weight_grads"] = ("E4M3 operands, one scale per expert and column (quantised per step), fp32 sums; "
                                     "wgrad_tflops counts the GEMMs only, ms_per_step includes the quantisation")
        out[key] = entry
        del layer
    gc.collect()
    torch.cuda.empty_cache()
    return out


def gpu_arm(args, cfg):
    from mlops_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    group = None
    ep_check = None
    if distributed:
        import torch.distributed as dist

        # the all-to-all kernels run beside the GEMMs on at most this many SMs; the FP8 GEMMs draw
        # their tiles dynamically and take whatever SMs are left
        comm_sms = int(os.environ.get("B200MOE_EP_COMM_SMS", "32"))
        os.environ.setdefault("NCCL_MAX_CTAS", str(comm_sms))
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # keeps NCCL's version banner off stdout: one JSON line only
        # the collectives of a step are short and on its critical path: their kernels go ahead of the
        # GEMMs' CTAs when SMs free up
        options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=device, pg_options=options)
        group = dist.group.WORLD
        from mlops_b200 import ep as ep_module

        # correctness first: the expert-parallel layer against the single-GPU layer on the
        # gathered weights (a small case of the workload's routing), asserted on every rank
        ep_check = ep_module.parity_check(group, device, routing_mode=cfg["mode"], n_group=cfg["n_group"],
                                          topk_group=cfg["topk_group"], routed_scaling=cfg["scaling"],
                                          shared=cfg["shared"],
                                          presum=os.environ.get("B200MOE_EP_PRESUM", "1") == "1",
                                          transport=os.environ.get("B200MOE_EP_TRANSPORT",
                                                                   "peer" if world <= 4 else "nccl"))
    if args.workload == "c2":
        peaks, peak_kind = measured_peaks()
        fp8_peak = measure_fp8_peak(device)
        print(json.dumps({"metric": "grouped_gemm_fp8_tflops", "unit": "TFLOP/s", "n_gpus": 1,
                          "config": {"workload": WORKLOADS["c2"]["name"]}, "peak_measured_fp8": fp8_peak,
                          **run_c2(device, peaks, fp8_peak, steps=max(args.steps, 1), warmup=max(args.warmup, 1))}))
        return
    T, D, E, F, K = cfg["T"], cfg["D"], cfg["E"], cfg["F"], cfg["K"]
    layer = Layer(cfg, device, world=world, rank=rank, group=group)
    step = layer.step

    # ---- device-resident timing (the `value`)
    for _ in range(args.warmup):
        step(layer.x, layer.dy)
    ops.check_status(device)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ops.GEMM_TIMINGS = []
    launches_before = ops.LAUNCHES
    ms_per_step = timed_steps(lambda: step(layer.x, layer.dy), args.steps, device, distributed)
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
    buffers = [(layer.x, layer.dy), (torch.empty_like(layer.x), torch.empty_like(layer.dy))]
    uploaded = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    state = dict(i=0, steps=0)

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])  # the step that read this buffer has finished
            buffers[slot][0].copy_(layer.x_host, non_blocking=True)
            buffers[slot][1].copy_(layer.dy_host, non_blocking=True)
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
    e2e_ms = timed_steps(e2e_step, args.steps, device, distributed)
    h2d = layer.x_host.numel() * 2 + layer.dy_host.numel() * 2
    d2h = host_result.numel() * 4

    per_rank_rows = phases = None
    if distributed:
        import torch.distributed as dist

        mine = torch.tensor([layer.rows_received[-1]], device=device, dtype=torch.int64)
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        per_rank_rows = [int(t.item()) for t in gathered]
        # one more step with phase marks (rank 0's view; outside every timed region)
        layer.ep.profile = True
        step(layer.x, layer.dy)
        merged: dict[str, float] = {}
        for name, ms in layer.ep.phase_times():
            merged[name] = merged.get(name, 0.0) + ms
        layer.ep.profile = False
        phases = {name: round(ms, 3) for name, ms in merged.items()}
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    gemms = gemm_summary(timings, args.steps)
    achieved = gemms["fp8_tflops"] or 0.0
    peak_fp8 = 2.0 * peaks["bf16_tflops_sustained"]
    routed_flops, shared_flops = layer.flops()
    tokens_total = T * world
    rows_local = T * K  # per rank on average
    experts_local = E // world
    # algorithmic bytes of the four FP8 launches of a step: A once (+ its scales), the weights
    # once, the bf16 output once
    gemm_shapes = ((D, 2 * F), (F, D), (D, F), (2 * F, D))  # (K, N) of up, down, dgrad-down, dgrad-up
    algorithmic = [rows_local * k + 4.0 * rows_local * k / 128 + experts_local * n * k + 2.0 * rows_local * n
                   for k, n in gemm_shapes]
    traffic = None
    if args.workload in ("c4", "c4p") and world == 1:
        scale = 8.0 if args.workload == "c4" else 1.0
        traffic = scale * sum(GEMM_DRAM_BYTES_C4P) / len(GEMM_DRAM_BYTES_C4P)
    line = {
        "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": tokens_total / (ms_per_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["name"], "tokens_per_gpu": T, "hidden": D, "experts": E, "intermediate": F,
                   "top_k": K, "routing": cfg["mode"],
                   "router_bias": (f"N(0, {layer.bias_std}), balanced load (N(0, 0.1), skewed, is reported as "
                                   "workloads.c4_skewed)") if layer.bias is not None else None,
                   "shared_expert": bool(cfg["shared"]), "call": "provider.apply + torch.autograd.grad"
                   if not distributed else "ExpertParallelMoE.forward_backward",
                   "expert_parallel": world, "expert_map": layer.ep.config.expert_map if distributed else "local",
                   "dedup_dispatch": bool(distributed and layer.ep.config.dedup),
                   "presum_return": bool(distributed and layer.ep.config.presum),
                   "dispatch_transport": (layer.ep.config.transport if distributed else None),
                   "rows_per_rank": per_rank_rows, "weights": "block-FP8 e4m3 128x128, random N(0,0.02)",
                   "activations": "e4m3 1x128 blocks", "weight_grads": "bf16 operands, fp32 sums, bf16 out",
                   "l2": "inputs exceed L2 (no flush needed)" if T * D * 2 > (126 << 20) else "inputs fit L2"},
        "tflops_per_gpu": (routed_flops + shared_flops) / (ms_per_step * 1e-3) / 1e12,
        "gpu_launches": launches,
        "e2e": {"value": tokens_total / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "returned": "four fp32 scalars (sums of the output and of grad_x, aux, max count): a training "
                            "step returns its loss-like summary, no tensor, to the host"},
        "roofline": {"kernel": "grouped_gemm_fp8_kernel", "bound": "tensor", "achieved": achieved,
                     "peak": peak_fp8, "unit": "TFLOP/s", "frac": achieved / peak_fp8 if peak_fp8 else None,
                     "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_kind}); "
                                    "FP8 issues at twice the bf16 rate",
                     "frac_of_nominal_fp8": achieved / NOMINAL_FP8_TFLOPS,
                     "launches_timed": gemms["fp8_launches"], "ms_in_kernel_per_step": gemms["fp8_ms_per_step"],
                     "traffic": traffic,
                     "traffic_source": None if traffic is None else
                     "dram__bytes_read.sum + dram__bytes_write.sum per launch (mean of the step's four launches) "
                     "of the ncu capture at profiling size, scaled by rows and experts",
                     "algorithmic_bytes": sum(algorithmic) / len(algorithmic)},
        "wgrad": {"kernel": "grouped_wgrad_pair_kernel", "achieved_tflops": gemms["wgrad_tflops"],
                  "ms_in_kernel_per_step": gemms["wgrad_ms_per_step"],
                  "peak_bf16_sustained": peaks["bf16_tflops_sustained"],
                  "frac": (gemms["wgrad_tflops"] or 0.0) / peaks["bf16_tflops_sustained"]},
        "clocks": clocks,
    }
    if distributed:
        line["ep_check"] = ep_check
        line["ep_phases_ms"] = phases
    if world == 1:
        del layer, buffers
        gc.collect()
        torch.cuda.empty_cache()
        fp8_peak = {} if args.no_extras else measure_fp8_peak(device)  # (a profiling run leaves it out)
        line["roofline"]["peak_measured_fp8"] = fp8_peak or None
        if fp8_peak.get("sustained"):
            line["roofline"]["frac_of_measured_fp8_sustained"] = achieved / fp8_peak["sustained"]
        if not args.no_extras and args.workload == "c4":
            line["hbm_kernels"] = hbm_kernels(cfg, device, peaks)
            line["workloads"] = extras(device, peaks, fp8_peak)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(cfg)
    print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--no-extras", action="store_true", help="skip the other workloads, the HBM kernels and the FP8 peak measurement")
    args = parser.parse_args()
    cfg = dict(WORKLOADS[args.workload])
    if args.workload == "c2" and args.impl == "reference":
        cfg = dict(WORKLOADS["c4"])
    if args.impl == "reference":
        reference_arm(args, cfg)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the CUDA path has no CPU fallback)")
    gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
