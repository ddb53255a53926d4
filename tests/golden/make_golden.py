"""Generates the golden fixtures in this folder by running the REFERENCE implementation
(als244/mlops, imported from its source tree) on seeded CPU inputs.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference/src

The reference cannot travel to the GPU machine, so its outputs are committed here as
small fixtures (`*.pt`, torch.save of a dict of tensors); the tests load the fixtures and
never import the reference. Small inputs are stored with the outputs; the larger ones come
from the seeded factories in `inputs.py`, and the fixture records their checksum.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import inputs  # noqa: E402


def main(reference_src: str) -> None:
    sys.path.insert(0, reference_src)
    import mlops
    from mlops.block_fp8 import BlockFP8Weight
    from mlops.dispatch import use_implementation
    from mlops.expert_parallel.reference import expert_computation
    from mlops.kernels.block_fp8 import dequantize_blocks, quantize_blocks
    from mlops.kernels.moe_dispatch import combine, sort_assignments
    from mlops.kernels.moe_router import route, route_torch
    from mlops.kernels.quack_moe.quantize_rows import quantize_rows_fp8_reference
    from mlops.providers.moe_common import routing_gradient, routing_statistics

    torch.set_num_threads(1)  # fixed summation order in the fixtures' float outputs

    # ------------------------------------------------------------------ routing + sort
    cases = []
    specs = [
        ("softmax_then_topk", 96, 8, 2, 1, 1, 1.0),
        ("topk_then_softmax", 96, 8, 2, 1, 1, 1.0),
        ("softmax_then_topk", 64, 128, 8, 1, 1, 1.0),
        ("sigmoid_noaux_tc", 64, 256, 8, 8, 4, 2.5),
        ("sigmoid_noaux_tc", 48, 64, 6, 4, 2, 1.0),
        ("sigmoid_noaux_tc", 48, 64, 6, 1, 1, 1.0),   # group stage skipped
        ("sigmoid_noaux_tc", 40, 96, 4, 8, 3, 1.5),   # 12 experts per group
        ("topk_then_softmax", 16, 1024, 32, 1, 1, 1.0),
    ]
    for index, (mode, tokens, experts, top_k, n_group, topk_group, scaling) in enumerate(specs):
        g = torch.Generator().manual_seed(100 + index)
        logits = torch.randn(tokens, experts, generator=g)
        logits[:3] = 0.25                      # all experts tied
        logits[3, : experts // 2] = 1.0        # half tied high, half random
        bias = torch.randn(experts, generator=g) * 0.1 if mode == "sigmoid_noaux_tc" else None
        kwargs = dict(bias=bias, n_group=n_group, topk_group=topk_group, routed_scaling=scaling)
        weights, ids = route(logits, top_k, mode, **kwargs)
        weights_t, ids_t = route_torch(logits, top_k, mode, **kwargs)
        assert torch.equal(ids, ids_t), "reference route and route_torch disagree"
        order, offsets, slots = sort_assignments(ids, experts)
        lengths = (tokens,) if index % 2 == 0 else (tokens // 2, tokens - tokens // 2)
        aux, counts, psum = routing_statistics(
            logits, ids, routing_mode=mode, lengths=lengths, experts=experts
        )
        grad_w = torch.randn(tokens, top_k, generator=g)
        grad_aux = torch.tensor(0.7)
        grad_psum = torch.randn(experts, generator=g)
        grad_logits = routing_gradient(
            grad_aux, grad_psum, grad_w, weights, ids, logits, routing_mode=mode, lengths=list(lengths)
        )
        cases.append(
            dict(mode=mode, top_k=top_k, n_group=n_group, topk_group=topk_group, scaling=scaling,
                 logits=logits, bias=bias, weights=weights, ids=ids, order=order, offsets=offsets,
                 slots=slots, lengths=lengths, aux=aux, counts=counts, psum=psum, grad_w=grad_w,
                 grad_aux=grad_aux, grad_psum=grad_psum, grad_logits=grad_logits)
        )
    torch.save(cases, HERE / "routing.pt")

    # ------------------------------------------------------------------- quantisers
    quant = {}
    w = inputs.block_weight()
    for name, value in (("w_fp32", w), ("w_bf16", w.bfloat16())):
        data, scale = quantize_blocks(value)
        quant[name + "_data"] = data.view(torch.uint8)
        quant[name + "_scale"] = scale
        quant[name + "_dequant_bf16"] = dequantize_blocks(data, scale, dtype=torch.bfloat16)
    x, gather = inputs.activation_rows()
    q, s = quantize_rows_fp8_reference(x, gather=gather)
    quant.update(rows_data=q.view(torch.uint8), rows_scale=s, checksum=inputs.checksum(w, x, gather))
    torch.save(quant, HERE / "quantize.pt")

    # ----------------------------------------------------------------------- combine
    g = torch.Generator().manual_seed(9)
    tokens, top_k, width = 24, 3, 64
    source = torch.randn(tokens * top_k, width, generator=g).bfloat16()
    slots = torch.randperm(tokens * top_k, generator=g).view(tokens, top_k).to(torch.int32)
    weights = torch.rand(tokens, top_k, generator=g)
    residual = torch.randn(tokens, width, generator=g).bfloat16()
    torch.save(
        dict(source=source, slots=slots, weights=weights, residual=residual,
             output=combine(source, slots, weights, residual)),
        HERE / "combine.pt",
    )

    # ------------------------------------- config 1 through the reference's CPU provider
    c1 = inputs.config1()
    torch.set_num_threads(8)
    x_in = c1["x"].clone().requires_grad_(True)
    router_in = c1["router"].clone().requires_grad_(True)
    q13 = BlockFP8Weight.quantize(c1["w13"]).requires_grad_(True)
    q2 = BlockFP8Weight.quantize(c1["w2"]).requires_grad_(True)
    with use_implementation("moe", "native_torch.moe"):
        out, aux, counts, psum = mlops.moe(
            x_in, c1["residual"], router_in, q13, q2, top_k=c1["top_k"],
            routing_mode=c1["routing_mode"], compute_precision="bf16",
        )
    loss = (out.float() * c1["dy"].float()).sum()
    gx, grouter, g13, g2 = torch.autograd.grad(loss, (x_in, router_in, q13, q2))
    torch.save(
        dict(checksum=inputs.checksum(c1["x"], c1["router"], c1["w13"], c1["w2"], c1["dy"]),
             w13_scale=q13._scale, w2_scale=q2._scale,
             w13_data_checksum=inputs.checksum(q13._data), w2_data_checksum=inputs.checksum(q2._data),
             output=out.detach(), aux=aux.detach(), counts=counts, psum=psum.detach(),
             grad_x=gx, grad_router=grouter,
             grad_w13_sample=g13[:, ::16, ::8].contiguous(), grad_w13_norm=g13.float().norm(),
             grad_w2_sample=g2[:, ::8, ::16].contiguous(), grad_w2_norm=g2.float().norm()),
        HERE / "config1_native_torch.pt",
    )

    # ----------------------------------------- expert-parallel reference, fixed routes
    ep = inputs.ep_case()
    y = expert_computation(ep["x"], ep["ids"], ep["p"], ep["gate"], ep["up"], ep["down"])
    torch.save(dict(checksum=inputs.checksum(*(ep[k] for k in ("x", "gate", "up", "down", "ids", "p"))), y=y),
               HERE / "ep_reference.pt")
    # --------------------------------- expert LoRA through the reference's builtin composition
    from mlops.lora.experts import expert_lora

    lc = inputs.lora_case()
    leaves = {k: lc[k].clone().requires_grad_(True) for k in ("x", "router", "a13", "b13", "a2", "b2")}
    g13 = BlockFP8Weight.quantize(lc["w13"])
    g2 = BlockFP8Weight.quantize(lc["w2"])
    out, aux, counts, psum = expert_lora(
        leaves["x"], lc["residual"], leaves["router"], g13, g2, leaves["a13"], leaves["b13"], leaves["a2"],
        leaves["b2"], top_k=lc["top_k"], routing_mode=lc["routing_mode"], scale=lc["scale"],
        implementation="builtin", compute_precision="bf16")
    grads = torch.autograd.grad((out.float() * lc["dy"].float()).sum(), list(leaves.values()))
    base_out, *_ = mlops.moe(lc["x"], lc["residual"], lc["router"], g13, g2, top_k=lc["top_k"],
                             routing_mode=lc["routing_mode"], compute_precision="bf16")
    torch.save(
        dict(checksum=inputs.checksum(*(lc[k] for k in ("x", "residual", "router", "w13", "w2", "a13", "b13",
                                                         "a2", "b2", "dy"))),
             output=out.detach(), base_output=base_out.detach(), counts=counts, aux=aux.detach(),
             **{"grad_" + k: g for k, g in zip(leaves, grads)}),
        HERE / "lora_builtin.pt",
    )
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2 and "MLOPS_REFERENCE_SRC" not in os.environ:
        raise SystemExit("usage: make_golden.py /path/to/reference/src  (or set MLOPS_REFERENCE_SRC)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["MLOPS_REFERENCE_SRC"])
