"""Parity of the quantisers, SwiGLU rows and combine kernels through the C ABI: E4M3 bytes
and fp32 scales bit-exact against the oracle and the reference's fixtures."""

import pytest
import torch

import inputs
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
U8 = torch.uint8


def _ops():
    from mlops_b200 import ops

    return ops


def test_weight_blocks_match_reference_fixture(golden):
    ops = _ops()
    fixture = golden("quantize.pt")
    w = inputs.block_weight()
    for name, value in (("w_fp32", w), ("w_bf16", w.bfloat16())):
        data, scale = ops.quantize_blocks(value.to(DEV))
        assert torch.equal(data.cpu().view(U8), fixture[name + "_data"])
        assert torch.equal(scale.cpu(), fixture[name + "_scale"])


def test_row_quantiser_matches_reference_fixture(golden):
    ops = _ops()
    fixture = golden("quantize.pt")
    x, gather = inputs.activation_rows()
    data, scale = ops.quantize_rows(x.to(DEV), gather=gather.to(DEV), gather_div=1, mode="row")
    assert torch.equal(data.cpu().view(U8), fixture["rows_data"])
    assert torch.equal(scale.cpu()[:, 0], fixture["rows_scale"])


@pytest.mark.parametrize("rows,width", [(300, 256), (64, 192), (1000, 7168), (33, 2048), (7, 8)])
@pytest.mark.parametrize("mode", ["1x128", "row"])
def test_quantize_rows_bit_exact(rows, width, mode):
    ops = _ops()
    g = torch.Generator().manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g).bfloat16()
    x[0] = 0                     # all-zero row keeps the 1e-12 floor
    x[rows // 2] *= 30000        # values that saturate nothing after scaling
    gather = torch.randint(0, rows, (2 * rows,), generator=g).to(torch.int32)
    q_ref, s_ref = O.quantize_rows(x, gather=torch.div(gather, 2, rounding_mode="floor"), mode=mode)
    q, s = ops.quantize_rows(x.to(DEV), gather=gather.to(DEV), gather_div=2, mode=mode)
    assert torch.equal(q.cpu().view(U8), q_ref.view(U8))
    assert torch.equal(s.cpu(), s_ref)
    q2, s2 = ops.quantize_rows(x.to(DEV), mode=mode)  # no gather
    q2_ref, s2_ref = O.quantize_rows(x, mode=mode)
    assert torch.equal(q2.cpu().view(U8), q2_ref.view(U8)) and torch.equal(s2.cpu(), s2_ref)


def test_quantize_rows_writes_the_gathered_rows_into_a_given_slice():
    """`copy_out`: the quantiser also writes the bf16 rows it gathered, into a caller's slice
    (a pitched view of a larger buffer), bit for bit; the E4M3 result does not change."""
    ops = _ops()
    g = torch.Generator().manual_seed(21)
    x = torch.randn(90, 384, generator=g).bfloat16().to(DEV)
    gather = torch.randint(0, 90 * 3, (200,), generator=g).to(torch.int32).to(DEV)
    q_ref, s_ref = ops.quantize_rows(x, gather=gather, gather_div=3)
    big = torch.full((260, 384), float("nan"), dtype=torch.bfloat16, device=DEV)
    q, s, copy = ops.quantize_rows(x, gather=gather, gather_div=3, copy_out=big[30:230])
    assert copy.data_ptr() == big[30:230].data_ptr()
    assert torch.equal(big[30:230], x[torch.div(gather, 3, rounding_mode="floor").long()])
    assert big[:30].isnan().all() and big[230:].isnan().all()
    assert torch.equal(q.view(U8), q_ref.view(U8)) and torch.equal(s, s_ref)


def test_quantize_rows_empty():
    ops = _ops()
    q, s = ops.quantize_rows(torch.zeros(0, 256, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (0, 256) and s.shape == (0, 2)


@pytest.mark.parametrize("rows,width", [(100, 512), (77, 640), (50, 80)])
@pytest.mark.parametrize("limit", [None, 1.5])
def test_swiglu_quantize(rows, width, limit):
    """fp32 SwiGLU differs from the CPU's by an ulp of expf at most, which can move a value
    across an E4M3 rounding boundary: bytes must agree on all but a 1e-3 fraction, and the
    bf16 activation within bf16 rounding."""
    ops = _ops()
    g = torch.Generator().manual_seed(rows)
    h = (torch.randn(rows, 2 * width, generator=g) * 2).bfloat16()
    act = O.swiglu(h, limit)
    q_ref, s_ref = O.quantize_rows(act, mode="1x128")
    q, s, a16 = ops.swiglu_quantize(h.to(DEV), limit=limit, quantized=True, rounded=True)
    same = (q.cpu().view(U8) == q_ref.view(U8)).float().mean().item()
    assert same > 0.999
    torch.testing.assert_close(s.cpu(), s_ref, rtol=1e-6, atol=0)
    mx, mean = O.rel_errors(a16.float().cpu(), act)
    assert mx <= 2e-2 and mean <= 2e-3


@pytest.mark.parametrize("limit", [None, 1.5])
def test_dswiglu_routed(limit):
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    rows, width = 90, 256
    h = (torch.randn(rows, 2 * width, generator=g) * 2).bfloat16()
    r = torch.randn(rows, width, generator=g).bfloat16()
    route_weights = torch.rand(rows, generator=g)
    order = torch.randperm(rows, generator=g).to(torch.int32)
    ds_ref, gh_ref, as_ref = O.dswiglu_routed(h, r, route_weights[order.long()], limit)
    ds, gq, gs, gb, a_s = ops.dswiglu_routed(
        h.to(DEV), r.to(DEV), route_weights.to(DEV), order.to(DEV), limit=limit, quantized=True,
        rounded=True, scaled_activation=True,
    )
    torch.testing.assert_close(ds.cpu(), ds_ref, rtol=1e-5, atol=1e-5)
    for actual, expected in ((gb, gh_ref), (a_s, as_ref)):
        mx, mean = O.rel_errors(actual.float().cpu(), expected)
        assert mx <= 2e-2 and mean <= 2e-3
    q_ref, s_ref = O.quantize_rows(gh_ref, mode="1x128")
    torch.testing.assert_close(gs.cpu(), s_ref, rtol=1e-5, atol=0)
    assert (gq.cpu().view(U8) == q_ref.view(U8)).float().mean().item() > 0.995


def test_combine_matches_reference_fixture_and_oracle(golden):
    ops = _ops()
    fixture = golden("combine.pt")
    out = ops.combine(*(fixture[k].to(DEV) for k in ("source", "slots", "weights", "residual")))
    assert torch.equal(out.cpu(), O.combine(fixture["source"], fixture["slots"], fixture["weights"], fixture["residual"]))
    torch.testing.assert_close(out.cpu().float(), fixture["output"].float(), rtol=2 ** -7, atol=1e-6)
    g = torch.Generator().manual_seed(3)
    tokens, top_k, width = 200, 4, 384
    src = torch.randn(tokens * top_k, width, generator=g).bfloat16()
    slots = torch.randperm(tokens * top_k, generator=g).view(tokens, top_k).to(torch.int32)
    again = ops.dispatch_backward(src.to(DEV), slots.to(DEV))
    assert torch.equal(again.cpu(), O.combine(src, slots, None, None))
    assert torch.equal(again, ops.dispatch_backward(src.to(DEV), slots.to(DEV)))  # repeatable
    order = torch.randperm(tokens * top_k, generator=g).to(torch.int32)
    x = torch.randn(tokens, width, generator=g).bfloat16()
    rows = ops.dispatch(x.to(DEV), order.to(DEV), top_k)
    assert torch.equal(rows.cpu(), x[order.long() // top_k])


def test_scatter_quantiser_equals_the_gathered_quantiser_bit_for_bit():
    """Quantising every token once and writing its row to its K expert-ordered rows gives the
    bytes, the scales and the bf16 copies of the per-output-row gather (which is pinned above
    against the reference's `quantize_rows_fp8_reference`), including a width that is not a
    multiple of 128 and a slot outside the output, which is reported and skipped."""
    from mlops_b200 import ops
    from mlops_b200._lib import NativeError

    g = torch.Generator().manual_seed(31)
    tokens, top_k, experts = 700, 8, 64
    for width in (7168, 1000):
        x = torch.randn(tokens, width, generator=g).bfloat16().to(DEV)
        ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).to(torch.int32).to(DEV)
        order, _offsets, slots, _counts = ops.sort_assignments(ids, experts)
        q_ref, s_ref, c_ref = ops.quantize_rows(x, gather=order, gather_div=top_k, with_copy=True)
        q, s, c = ops.quantize_rows_scatter(x, slots, with_copy=True)
        assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
        assert torch.equal(s, s_ref) and torch.equal(c, c_ref)
    ops.check_status(DEV)
    bad = slots.clone()
    bad[3, 2] = tokens * top_k + 5
    ops.quantize_rows_scatter(x, bad)
    with pytest.raises(NativeError):
        ops.check_status(DEV)
