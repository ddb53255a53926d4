"""Parity of the tcgen05 grouped GEMMs through the C ABI against the float64 product of the
same dequantised operands (the comparison of the reference's
tests/test_block_fp8_transpose_gemm.py:447-498). Tolerance: bf16 output, max relative error
<= 2e-2 and mean <= 2e-3 (see `oracle.moe_oracle.rel_errors`)."""

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FP8 = torch.float8_e4m3fn
MAX_REL, MEAN_REL = 2e-2, 2e-3


def _ops():
    from mlops_b200 import ops

    return ops


def _offsets(counts):
    offs = torch.zeros(len(counts) + 1, dtype=torch.int32)
    offs[1:] = torch.tensor(counts).cumsum(0).to(torch.int32)
    return offs


def _case(counts, n, k, seed, mn_major, spread=False):
    g = torch.Generator().manual_seed(seed)
    rows, groups = sum(counts), len(counts)
    a = torch.randn(rows, k, generator=g)
    b = torch.randn(groups, n, k, generator=g)
    if spread:  # block scales across 2^+-14 and one all-zero block (reference test shapes)
        b[0, :128, :128] = 0
        b[-1, :, :128] *= 2.0 ** 14
        a[:, :128] *= 2.0 ** -14
    a_q, a_s = O.quantize_rows(a, mode="1x128")
    b_q, b_s = O.quantize_blocks(b)
    if mn_major:
        b_q = b_q.view(torch.uint8).transpose(1, 2).contiguous().view(FP8)
        b_s = b_s.transpose(1, 2).contiguous()
    return a_q, a_s, b_q, b_s, _offsets(counts)


def _run(a_q, a_s, b_q, b_s, offs, mn_major, block_n, scale_layout="block_major"):
    ops = _ops()
    n = b_q.shape[2] if mn_major else b_q.shape[1]
    scales = a_s.to(DEV) if scale_layout == "row_major" else a_s.t().contiguous().to(DEV).t()
    out = torch.full((a_q.shape[0], n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.grouped_gemm_fp8(a_q.to(DEV), scales, b_q.to(DEV), b_s.to(DEV), offs.to(DEV),
                         b_mn_major=mn_major, block_n=block_n, out=out)
    ops.check_status(DEV)
    return out


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("mn_major", [False, True])
def test_integer_operands_are_exact(block_n, mn_major):
    g = torch.Generator().manual_seed(1)
    counts, n, k = [128, 64], 256, 384
    rows = sum(counts)
    a = torch.randint(-3, 4, (rows, k), generator=g).float()
    b = torch.randint(-3, 4, (2, n, k), generator=g).float()
    a_q, b_q = a.to(FP8), b.to(FP8)
    a_s = torch.ones(rows, 3)
    b_s = torch.ones(2, 2, 3)
    offs = _offsets(counts)
    ref = O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs)
    if mn_major:
        b_q = b_q.view(torch.uint8).transpose(1, 2).contiguous().view(FP8)
        b_s = b_s.transpose(1, 2).contiguous()
    out = _run(a_q, a_s, b_q, b_s, offs, mn_major, block_n)
    # integer products and sums are exact in fp32; only the bf16 store rounds
    assert torch.equal(out.cpu(), ref.float().bfloat16())


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("mn_major", [False, True])
@pytest.mark.parametrize(
    "counts,n,k",
    [
        ([128, 256], 256, 512),
        ([0, 70, 131, 15, 260], 384, 640),     # empty expert, partial M tiles
        ([1, 0, 0, 513], 128, 128),
        ([300], 2048, 7168),                   # the DeepSeek-shaped K loop (56 blocks)
    ],
)
def test_random_operands(counts, n, k, mn_major, block_n):
    a_q, a_s, b_q, b_s, offs = _case(counts, n, k, seed=n + k, mn_major=mn_major)
    out = _run(a_q, a_s, b_q, b_s, offs, mn_major, block_n)
    ref = O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs, b_mn_major=mn_major)
    assert not torch.isnan(out.float()).any()
    mx, mean = O.rel_errors(out.float().cpu(), ref)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)


@pytest.mark.parametrize("block_n", [128, 256])
def test_partial_blocks_and_scale_spread(block_n):
    """K and N that are not multiples of 128 (reference shapes D=192, F=80 scaled to the
    16-byte pitch rule), block scales spread over 2^+-14, an all-zero weight block."""
    a_q, a_s, b_q, b_s, offs = _case([5, 300, 70], 200, 192, seed=4, mn_major=False)
    out = _run(a_q, a_s, b_q, b_s, offs, False, block_n)
    mx, mean = O.rel_errors(out.float().cpu(), O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs))
    assert mx <= MAX_REL and mean <= MEAN_REL
    a_q, a_s, b_q, b_s, offs = _case([130, 70], 256, 384, seed=5, mn_major=False, spread=True)
    out = _run(a_q, a_s, b_q, b_s, offs, False, block_n)
    ref = O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs)
    for lo in range(0, 256, 128):  # per 128-column cell, as the reference's tests judge it
        mx, mean = O.rel_errors(out.float().cpu()[:, lo:lo + 128], ref[:, lo:lo + 128])
        assert mx <= MAX_REL and mean <= MEAN_REL


def test_scale_layouts_and_row_scales_agree():
    """Row-major and block-major activation scales give identical bytes; one scale per row
    (the reference's in-tree recipe) goes through the same kernel."""
    a_q, a_s, b_q, b_s, offs = _case([100, 156], 256, 512, seed=6, mn_major=False)
    o1 = _run(a_q, a_s, b_q, b_s, offs, False, 128, "block_major")
    o2 = _run(a_q, a_s, b_q, b_s, offs, False, 128, "row_major")
    assert torch.equal(o1, o2)
    g = torch.Generator().manual_seed(7)
    a = torch.randn(256, 512, generator=g)
    a_qr, a_sr = O.quantize_rows(a, mode="row")
    out = _run(a_qr, a_sr, b_q, b_s, offs, False, 256)
    mx, mean = O.rel_errors(out.float().cpu(), O.grouped_block_gemm(a_qr, a_sr, b_q, b_s, offs))
    assert mx <= MAX_REL and mean <= MEAN_REL


def test_rows_outside_every_group_are_left_untouched():
    a_q, a_s, b_q, b_s, _ = _case([200], 128, 128, seed=8, mn_major=False)
    offs = torch.tensor([10, 150], dtype=torch.int32)
    out = _run(a_q, a_s, b_q, b_s, offs, False, 128)
    assert torch.isnan(out[:10].float()).all() and torch.isnan(out[150:].float()).all()
    assert not torch.isnan(out[10:150].float()).any()


def test_malformed_offsets_are_reported():
    ops = _ops()
    from mlops_b200._lib import NativeError

    a_q, a_s, b_q, b_s, _ = _case([128], 128, 128, seed=9, mn_major=False)
    bad = torch.tensor([0, 4096], dtype=torch.int32)  # past the last row
    _ = ops.grouped_gemm_fp8(a_q.to(DEV), a_s.to(DEV), b_q.to(DEV), b_s.to(DEV), bad.to(DEV))
    with pytest.raises(NativeError):
        ops.check_status(DEV)


def test_repeatable_bitwise():
    a_q, a_s, b_q, b_s, offs = _case([0, 70, 131, 15, 260], 384, 640, seed=10, mn_major=False)
    assert torch.equal(_run(a_q, a_s, b_q, b_s, offs, False, 256), _run(a_q, a_s, b_q, b_s, offs, False, 256))


def test_config2_shape_linearity_and_sampled_parity():
    """Benchmark configuration 2 (the standalone grouped GEMM) at full size (32 groups, Zipf split of 65536 rows, K=4096, N=2048):
    sampled rows against float64, plus linearity in the activation scales
    (gemm(2 * a_scale) == 2 * gemm(a_scale) exactly, a power-of-two factor)."""
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    p = torch.arange(1, 33).float().pow(-1.1)
    counts = torch.bincount(torch.multinomial(p / p.sum(), 65536, replacement=True, generator=g), minlength=32)
    offs = _offsets(counts.tolist()).to(DEV)
    a = torch.randn(65536, 4096, device=DEV, dtype=torch.bfloat16)
    a_q, a_s = ops.quantize_rows(a)
    b_q, b_s = ops.quantize_blocks(torch.randn(32, 2048, 4096, device=DEV, dtype=torch.bfloat16))
    out = ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offs, block_n=256)
    doubled = ops.grouped_gemm_fp8(a_q, (a_s * 2).t().contiguous().t(), b_q, b_s, offs, block_n=256)
    assert torch.equal(doubled.float(), out.float() * 2)
    ops.check_status(DEV)
    offs_cpu = offs.cpu().tolist()
    for group in (0, 5, 31):
        lo, hi = offs_cpu[group], offs_cpu[group + 1]
        if hi == lo:
            continue
        rows = slice(lo, min(hi, lo + 64))
        ref = O.grouped_block_gemm(
            a_q[rows].cpu(), a_s[rows].cpu(), b_q[group:group + 1].cpu(), b_s[group:group + 1].cpu(),
            torch.tensor([0, rows.stop - rows.start], dtype=torch.int32),
        )
        mx, mean = O.rel_errors(out[rows].float().cpu(), ref)
        assert mx <= MAX_REL and mean <= MEAN_REL


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(
    "counts,m,n",
    [([64], 128, 256), ([128, 64], 128, 256), ([0, 70, 131, 15, 260], 256, 512),
     ([0, 70, 131, 15, 260], 384, 320), ([1000, 3, 0, 500], 1024, 768)],
)
def test_wgrad(counts, m, n, out_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(m + n)
    rows, groups = sum(counts), len(counts)
    grad = torch.randn(rows, m, generator=g).bfloat16()
    x = torch.randn(rows, n, generator=g).bfloat16()
    offs = _offsets(counts)
    out = ops.grouped_wgrad(grad.to(DEV), x.to(DEV), offs.to(DEV), groups, out_dtype)
    ops.check_status(DEV)
    ref = O.grouped_wgrad(grad, x, offs, groups)
    for e, count in enumerate(counts):
        if count == 0:
            assert int(torch.count_nonzero(out[e])) == 0      # exact zeros for an empty expert
        else:
            mx, mean = O.rel_errors(out[e].float().cpu(), ref[e])
            assert mx <= (1e-5 if out_dtype == torch.float32 else MAX_REL), mx
            assert mean <= (1e-6 if out_dtype == torch.float32 else MEAN_REL), mean


@pytest.mark.parametrize("m,n", [(256, 512), (128, 256)])  # the CTA-pair kernel and the single-CTA kernel
def test_wgrad_groups_are_isolated_from_a_neighbours_inf_and_nan(m, n):
    """The last K block of a group is loaded together with the first rows of the next group;
    both operand tiles are zeroed past the group's end, so an Inf or NaN there cannot reach
    this group's gradient (0 x Inf would be NaN if only one operand were zeroed)."""
    ops = _ops()
    g = torch.Generator().manual_seed(77)
    counts = [70, 131, 40]
    rows = sum(counts)
    grad = torch.randn(rows, m, generator=g).bfloat16()
    x = torch.randn(rows, n, generator=g).bfloat16()
    offs = _offsets(counts)
    clean = ops.grouped_wgrad(grad.to(DEV), x.to(DEV), offs.to(DEV), 3, torch.float32)
    grad_bad, x_bad = grad.clone(), x.clone()
    x_bad[70] = float("inf")          # first row of group 1, X operand
    grad_bad[71, :5] = float("nan")   # second row of group 1, G operand
    x_bad[201, 3] = float("-inf")     # first row of group 2
    dirty = ops.grouped_wgrad(grad_bad.to(DEV), x_bad.to(DEV), offs.to(DEV), 3, torch.float32)
    ops.check_status(DEV)
    assert torch.equal(dirty[0], clean[0])           # group 0 never sees group 1's rows
    assert not bool(torch.isfinite(dirty[1]).all())  # group 1 owns them
    assert bool(torch.isnan(dirty[2][:, 3]).any() | torch.isinf(dirty[2][:, 3]).any())
    keep = torch.ones(n, dtype=torch.bool)
    keep[3] = False
    assert torch.equal(dirty[2][:, keep.to(DEV)], clean[2][:, keep.to(DEV)])


@pytest.mark.parametrize("b_mn_major", [False, True])
@pytest.mark.parametrize(
    "counts,n,k",
    [([128], 256, 64), ([128], 256, 512), ([0, 70, 131, 15, 260], 512, 192), ([0, 70, 131, 15, 260], 320, 456),
     ([1000, 3, 0, 500], 768, 1024),
     # one narrow side: the rank-r products of expert LoRA (project: N = r, expand: K = r)
     ([0, 70, 131, 15, 260], 16, 456), ([1000, 3, 0, 500], 8, 2048), ([0, 70, 131, 15, 260], 320, 16),
     ([1000, 3, 0, 500], 1536, 24)],
)
def test_grouped_gemm_bf16(counts, n, k, b_mn_major):
    """The bf16 forward / input-gradient product against float64 of the same operands: one rounding
    to bf16 is the only difference, so the bound is bf16's half ulp. Empty experts, partial row
    tiles, N and K that are no multiples of the tile, both operand orders of the stored weight."""
    ops = _ops()
    g = torch.Generator().manual_seed(n + k + int(b_mn_major))
    rows, groups = sum(counts), len(counts)
    a = torch.randn(rows, k, generator=g).bfloat16()
    b = (torch.randn(groups, k, n, generator=g) if b_mn_major else torch.randn(groups, n, k, generator=g)).bfloat16()
    addend = torch.randn(rows, n, generator=g).bfloat16()
    offs = _offsets(counts)
    out = ops.grouped_gemm_bf16(a.to(DEV), b.to(DEV), offs.to(DEV), b_mn_major=b_mn_major)
    out_add = ops.grouped_gemm_bf16(a.to(DEV), b.to(DEV), offs.to(DEV), b_mn_major=b_mn_major, addend=addend.to(DEV))
    ops.check_status(DEV)
    ref = O.grouped_mm(a, b, offs, b_mn_major=b_mn_major)
    assert torch.equal(out.cpu(), ref.bfloat16()) or O.rel_errors(out.float().cpu(), ref)[0] <= 4e-3
    mx, mean = O.rel_errors(out.float().cpu(), ref)
    assert mx <= 4e-3 and mean <= 1.5e-3, (mx, mean)
    mx, mean = O.rel_errors(out_add.float().cpu(), ref + addend.double())
    assert mx <= 4e-3 and mean <= 1.5e-3, (mx, mean)


def test_bf16_gemm_and_fp8_weight_gradient_at_layer_size():
    """The two newer tensor-core kernels at the size of a DeepSeek-V3-shaped layer slice (32
    experts with a Zipf split of 32768 rows, D=7168, 2F=4096): size-independent properties and
    sampled pieces against float64. bf16 GEMM: exact linearity in a power-of-two factor of the
    weights, sampled rows. FP8 weight gradient: exact linearity in the column scales, sampled
    output blocks, and the all-experts sum against one dense product of the quantised operands."""
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    p = torch.arange(1, 33).float().pow(-1.1)
    counts = torch.bincount(torch.multinomial(p / p.sum(), 32768, replacement=True, generator=g), minlength=32)
    offs = _offsets(counts.tolist()).to(DEV)
    gd = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(32768, 7168, device=DEV, generator=gd).bfloat16()
    w13 = (torch.randn(32, 4096, 7168, device=DEV, generator=gd) * 0.05).bfloat16()
    h = ops.grouped_gemm_bf16(x, w13, offs)
    assert torch.equal(ops.grouped_gemm_bf16(x, w13 * 4, offs).float(), h.float() * 4)
    back = ops.grouped_gemm_bf16(h, w13, offs, b_mn_major=True)   # dx-shaped product on the same weight
    ops.check_status(DEV)
    offs_cpu = offs.cpu().tolist()
    for group in (0, 7, 31):
        lo, hi = offs_cpu[group], offs_cpu[group + 1]
        if hi == lo:
            continue
        rows = slice(lo, min(hi, lo + 48))
        local = torch.tensor([0, rows.stop - rows.start], dtype=torch.int32)
        ref = O.grouped_mm(x[rows].cpu(), w13[group:group + 1].cpu(), local)
        mx, mean = O.rel_errors(h[rows].float().cpu(), ref)
        assert mx <= 4e-3 and mean <= 1.5e-3, (mx, mean)
        ref = O.grouped_mm(h[rows].cpu(), w13[group:group + 1].cpu(), local, b_mn_major=True)
        mx, mean = O.rel_errors(back[rows].float().cpu(), ref)
        assert mx <= 4e-3 and mean <= 1.5e-3, (mx, mean)
    # FP8 weight gradient dW13 = dh^T x per expert
    dh = torch.randn(32768, 4096, device=DEV, generator=gd).bfloat16()
    dh_q, dh_s = ops.quantize_columns(dh, offs, 32)
    x_q, x_s = ops.quantize_columns(x, offs, 32)
    dw = ops.grouped_wgrad_fp8(dh_q, dh_s, x_q, x_s, offs, 32, torch.float32)
    assert torch.equal(ops.grouped_wgrad_fp8(dh_q, dh_s * 2, x_q, x_s * 0.5, offs, 32, torch.float32), dw)
    ops.check_status(DEV)
    for group in (0, 7, 31):
        lo, hi = offs_cpu[group], offs_cpu[group + 1]
        if hi == lo:
            assert int(torch.count_nonzero(dw[group])) == 0
            continue
        local = torch.tensor([0, hi - lo], dtype=torch.int32)
        ref = O.grouped_wgrad_fp8(dh_q[lo:hi, 128:192].cpu(), dh_s[group:group + 1, 128:192].cpu(),
                                  x_q[lo:hi, 7040:7168].cpu(), x_s[group:group + 1, 7040:7168].cpu(), local, 1)
        mx, mean = O.rel_errors(dw[group, 128:192, 7040:7168].cpu(), ref[0])
        assert mx <= 1e-4 and mean <= 1e-5, (mx, mean)
    # checksum over experts: with unit scales, the sum of all experts' products is one dense product
    ones_m, ones_n = torch.ones_like(dh_s), torch.ones_like(x_s)
    total = ops.grouped_wgrad_fp8(dh_q, ones_m, x_q, ones_n, offs, 32, torch.float32).sum(0)
    dense = dh_q[:, :256].float().t() @ x_q[:, :512].float()
    mx, mean = O.rel_errors(total[:256, :512].cpu(), dense.double().cpu())
    assert mx <= 1e-3 and mean <= 1e-4, (mx, mean)


@pytest.mark.parametrize("counts,width", [([64], 128), ([0, 70, 131, 15, 260], 384), ([300, 1, 0, 555], 1024)])
def test_quantize_columns_is_bit_exact(counts, width):
    """Column-scaled E4M3 (one scale per expert and column over the expert's rows): bytes and
    scales bit-for-bit against the CPU restatement, including an empty group (scale 1e-12), a
    one-row group, groups that end inside a 32-row warp piece, and a scale spread of 2^+-14."""
    ops = _ops()
    g = torch.Generator().manual_seed(width + len(counts))
    rows, groups = sum(counts), len(counts)
    x = torch.randn(rows, width, generator=g)
    x *= torch.exp2(torch.randint(-14, 15, (1, width), generator=g).float())     # per-column spread
    x[:, 5] = 0.0                                                               # an all-zero column
    x = x.bfloat16()
    offs = _offsets(counts)
    q, scales = ops.quantize_columns(x.to(DEV), offs.to(DEV), groups)
    ops.check_status(DEV)
    q_ref, s_ref = O.quantize_columns(x, offs, groups)
    assert torch.equal(scales.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(
    "counts,m,n",
    [([128], 128, 256), ([64], 128, 256), ([0, 70, 131, 15, 260], 256, 512),
     ([0, 70, 131, 15, 260], 384, 320), ([1000, 3, 0, 500], 1024, 768)],
)
def test_wgrad_fp8(counts, m, n, out_dtype):
    """The FP8 weight gradient on given column-scaled operands against float64 of the same
    dequantised operands; then the whole recipe against the bf16 product at the reference's own
    bound for FP8 weight gradients (6e-2 relative Frobenius, tests/test_sonicmoe_fp8.py:114-124)."""
    ops = _ops()
    g = torch.Generator().manual_seed(m + n + 1)
    rows, groups = sum(counts), len(counts)
    grad = torch.randn(rows, m, generator=g).bfloat16()
    x = torch.randn(rows, n, generator=g).bfloat16()
    offs = _offsets(counts)
    g_q, g_s = ops.quantize_columns(grad.to(DEV), offs.to(DEV), groups)
    x_q, x_s = ops.quantize_columns(x.to(DEV), offs.to(DEV), groups)
    out = ops.grouped_wgrad_fp8(g_q, g_s, x_q, x_s, offs.to(DEV), groups, out_dtype)
    ops.check_status(DEV)
    ref = O.grouped_wgrad_fp8(g_q.cpu(), g_s.cpu(), x_q.cpu(), x_s.cpu(), offs, groups)
    exact = O.grouped_wgrad(grad, x, offs, groups)
    for e, count in enumerate(counts):
        if count == 0:
            assert int(torch.count_nonzero(out[e])) == 0
            continue
        mx, mean = O.rel_errors(out[e].float().cpu(), ref[e])
        assert mx <= (1e-5 if out_dtype == torch.float32 else MAX_REL), mx
        assert mean <= (1e-6 if out_dtype == torch.float32 else MEAN_REL), mean
        frob = ((out[e].double().cpu() - exact[e]).norm() / exact[e].norm()).item()
        assert frob <= 6e-2, frob
    # accumulate into a caller's buffer, scaled
    base = torch.randn(groups, m, n, generator=g).to(out_dtype)
    acc = ops.grouped_wgrad_fp8(g_q, g_s, x_q, x_s, offs.to(DEV), groups, accumulate_into=base.to(DEV).clone(), scale=0.5)
    expect = base.double() + 0.5 * ref
    mx, mean = O.rel_errors(acc.float().cpu(), expect)
    assert mx <= (1e-5 if out_dtype == torch.float32 else MAX_REL), mx


def test_wgrad_fp8_groups_are_isolated_from_a_neighbours_nan():
    ops = _ops()
    g = torch.Generator().manual_seed(78)
    counts, m, n = [70, 131, 40], 128, 256
    rows = sum(counts)
    grad = torch.randn(rows, m, generator=g).bfloat16()
    x = torch.randn(rows, n, generator=g).bfloat16()
    offs = _offsets(counts).to(DEV)
    g_q, g_s = ops.quantize_columns(grad.to(DEV), offs, 3)
    x_q, x_s = ops.quantize_columns(x.to(DEV), offs, 3)
    clean = ops.grouped_wgrad_fp8(g_q, g_s, x_q, x_s, offs, 3, torch.float32)
    x_bad = x_q.clone()
    x_bad.view(torch.uint8)[70] = 0x7F   # E4M3 NaN in the first row of group 1
    dirty = ops.grouped_wgrad_fp8(g_q, g_s, x_bad, x_s, offs, 3, torch.float32)
    ops.check_status(DEV)
    assert torch.equal(dirty[0], clean[0]) and torch.equal(dirty[2], clean[2])
    assert bool(torch.isnan(dirty[1]).any())


def test_segmented_layout_matches_expert_sorted_layout():
    """Rows laid out [source][expert] (what an expert-parallel exchange delivers): the GEMM
    with `weights < groups` and the weight gradient with `segments > 1` must equal the plain
    expert-sorted computation on the regrouped rows."""
    ops = _ops()
    g = torch.Generator().manual_seed(12)
    experts, sources, n, k = 3, 4, 256, 384
    counts = torch.randint(0, 90, (sources, experts), generator=g)
    counts[1, 2] = 0
    seg_offs = _offsets(counts.reshape(-1).tolist())
    rows = int(counts.sum())
    a = torch.randn(rows, k, generator=g)
    a_q, a_s = O.quantize_rows(a, mode="1x128")
    b_q, b_s = O.quantize_blocks(torch.randn(experts, n, k, generator=g))
    out = _run(a_q, a_s, b_q, b_s, seg_offs, False, 256)
    # reference: per segment against weight (segment index % experts)
    ref = torch.zeros(rows, n, dtype=torch.float64)
    offs = seg_offs.tolist()
    for s in range(sources * experts):
        lo, hi = offs[s], offs[s + 1]
        if hi > lo:
            e = s % experts
            ref[lo:hi] = O.grouped_block_gemm(a_q[lo:hi], a_s[lo:hi], b_q[e:e + 1], b_s[e:e + 1],
                                              torch.tensor([0, hi - lo], dtype=torch.int32))
    mx, mean = O.rel_errors(out.float().cpu(), ref)
    assert mx <= MAX_REL and mean <= MEAN_REL
    grad = torch.randn(rows, 128, generator=g).bfloat16()
    x = torch.randn(rows, 256, generator=g).bfloat16()
    dw = ops.grouped_wgrad(grad.to(DEV), x.to(DEV), seg_offs.to(DEV), experts, torch.float32)
    ops.check_status(DEV)
    for e in range(experts):
        expected = torch.zeros(128, 256, dtype=torch.float64)
        for s in range(sources):
            lo, hi = offs[s * experts + e], offs[s * experts + e + 1]
            expected += grad[lo:hi].double().t() @ x[lo:hi].double()
        mx, mean = O.rel_errors(dw[e].cpu(), expected)
        assert mx <= 1e-5, mx


@pytest.mark.parametrize("limit", [None, 0.75])
@pytest.mark.parametrize("counts,inner,k", [([0, 70, 131, 15, 260], 256, 384), ([300, 212], 128, 7168), ([40], 384, 128)])
def test_fused_swiglu_epilogue_equals_the_two_kernel_form(counts, inner, k, limit):
    """Up GEMM with the SwiGLU + quantisation epilogue: h13, E4M3 activation bytes and scales
    must equal `grouped_gemm_fp8` followed by `swiglu_quantize` bit for bit."""
    ops = _ops()
    a_q, a_s, b_q, b_s, offs = _case(counts, 2 * inner, k, seed=inner + k, mn_major=False)
    dev = [t.to(DEV) for t in (a_q, a_s.t().contiguous().t(), b_q, b_s, offs)]
    dev[1] = a_s.t().contiguous().to(DEV).t()
    h13 = ops.grouped_gemm_fp8(dev[0], dev[1], dev[2], dev[3], dev[4])
    act_q, act_s, _ = ops.swiglu_quantize(h13, limit=limit)
    rows = sum(counts)
    fused = torch.full((rows, 2 * inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    h13_f, act_q_f, act_s_f = ops.grouped_gemm_fp8_swiglu(dev[0], dev[1], dev[2], dev[3], dev[4], limit=limit, out=fused)
    ops.check_status(DEV)
    assert torch.equal(h13_f, h13)
    assert torch.equal(act_s_f, act_s)
    assert torch.equal(act_q_f.view(torch.uint8), act_q.view(torch.uint8))


@pytest.mark.parametrize("counts,n,k,top_k", [([0, 70, 131, 15, 260], 256, 384, 2), ([300, 212], 384, 512, 4),
                                               ([64, 64, 64, 64], 7168, 256, 8)])
def test_fused_combine_store_matches_gemm_then_combine(counts, n, k, top_k):
    """Down GEMM with the combine fused into its store against `grouped_gemm_fp8` followed by
    `combine`. The fused sum is formed with fp32 atomics in arrival order, so the two results are
    bf16 roundings of fp32 sums whose order differs; the parity metric is checked as well."""
    ops = _ops()
    a_q, a_s, b_q, b_s, offs = _case(counts, n, k, seed=n + k + top_k, mn_major=False)
    dev = [t.to(DEV) for t in (a_q, a_s, b_q, b_s, offs)]
    rows = sum(counts)
    tokens = rows // top_k
    g = torch.Generator().manual_seed(7)
    order = torch.randperm(tokens * top_k, generator=g)[:rows].to(torch.int32)  # row -> assignment
    slots = torch.full((tokens * top_k,), 0, dtype=torch.int32)
    slots[order.long()] = torch.arange(rows, dtype=torch.int32)
    route_weights = torch.rand(tokens, top_k, generator=g) + 0.1
    residual = torch.randn(tokens, n, generator=g).bfloat16()
    assert rows == tokens * top_k  # every assignment has a row in these cases
    y = ops.grouped_gemm_fp8(*dev)
    expected = ops.combine(y, slots.reshape(tokens, top_k).to(DEV), route_weights.to(DEV), residual.to(DEV))
    fused = ops.grouped_gemm_fp8_combine(*dev, order.to(DEV), route_weights.to(DEV), tokens,
                                         residual=residual.to(DEV))
    ops.check_status(DEV)
    # one bf16 rounding of fp32 sums that differ only in order: at most one ulp of the sum of
    # the terms' magnitudes
    magnitude = ops.combine(y.abs(), slots.reshape(tokens, top_k).to(DEV), route_weights.to(DEV),
                            residual.abs().to(DEV)).float()
    diff = (fused.float() - expected.float()).abs()
    assert (diff <= magnitude * 2.0 ** -7 + 1e-6).all(), diff.max().item()
    mx, mean = O.rel_errors(fused.cpu(), expected.double().cpu())
    assert mx <= MAX_REL and mean <= MEAN_REL


@pytest.mark.parametrize("mn_major", [False, True])
def test_scattered_store_places_rows_by_the_map(mn_major):
    """`row_map`: product row r lands at out[row_map[r]], bit-identical to the plain store."""
    ops = _ops()
    counts = [70, 0, 131, 15, 260]
    a_q, a_s, b_q, b_s, offs = _case(counts, 384, 256, seed=11, mn_major=mn_major)
    dev = [t.to(DEV) for t in (a_q, a_s, b_q, b_s, offs)]
    rows = sum(counts)
    plain = ops.grouped_gemm_fp8(*dev, b_mn_major=mn_major)
    row_map = torch.randperm(rows, generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV)
    out = torch.full((rows, 384), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.grouped_gemm_fp8(*dev, b_mn_major=mn_major, out=out, row_map=row_map)
    ops.check_status(DEV)
    assert torch.equal(out[row_map.long()], plain)


# ------------------------------------------------------------ the CTA-pair form of the GEMM
@pytest.fixture
def pair_form():
    """Forces the CTA-pair form of the wide tile (normally chosen by shape) for one test."""
    ops = _ops()
    ops.set_gemm_pair(1)
    yield ops
    ops.set_gemm_pair(-1)


@pytest.mark.parametrize("mn_major", [False, True])
@pytest.mark.parametrize(
    "counts,n,k",
    [
        ([256, 512], 256, 512),
        ([0, 70, 131, 15, 260, 300], 384, 640),   # empty expert, tiles whose second CTA has no rows
        ([1, 0, 0, 513], 128, 128),               # one column half beyond N
        ([700], 2048, 7168),                      # the DeepSeek-shaped K loop (56 blocks)
        ([130, 70], 200, 192),                    # K and N that are not multiples of 128
    ],
)
def test_pair_form_matches_float64_and_the_single_cta_form(pair_form, counts, n, k, mn_major):
    if mn_major and n % 16:
        pytest.skip("an input gradient needs N % 16 == 0")
    a_q, a_s, b_q, b_s, offs = _case(counts, n, k, seed=n + k + 1, mn_major=mn_major)
    out = _run(a_q, a_s, b_q, b_s, offs, mn_major, 256)
    ref = O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs, b_mn_major=mn_major)
    assert not torch.isnan(out.float()).any()
    mx, mean = O.rel_errors(out.float().cpu(), ref)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    pair_form.set_gemm_pair(0)
    single = _run(a_q, a_s, b_q, b_s, offs, mn_major, 256)
    assert torch.equal(out, single)  # the same sums in the same order: bit-identical


@pytest.mark.parametrize("mn_major", [False, True])
def test_pair_form_integer_operands_scatter_and_addend(pair_form, mn_major):
    ops = pair_form
    g = torch.Generator().manual_seed(12)
    counts, n, k = [300, 212], 512, 384
    rows = sum(counts)
    a = torch.randint(-3, 4, (rows, k), generator=g).float()
    b = torch.randint(-3, 4, (2, n, k), generator=g).float()
    a_q, b_q = a.to(FP8), b.to(FP8)
    a_s, b_s = torch.ones(rows, 3), torch.ones(2, 4, 3)
    offs = _offsets(counts)
    ref = O.grouped_block_gemm(a_q, a_s, b_q, b_s, offs)
    if mn_major:
        b_q = b_q.view(torch.uint8).transpose(1, 2).contiguous().view(FP8)
        b_s = b_s.transpose(1, 2).contiguous()
    out = _run(a_q, a_s, b_q, b_s, offs, mn_major, 256)
    assert torch.equal(out.cpu(), ref.float().bfloat16())
    addend = torch.randint(-8, 9, (rows, n), generator=g).bfloat16()
    row_map = torch.randperm(rows, generator=g).to(torch.int32)
    scattered = ops.grouped_gemm_fp8(a_q.to(DEV), a_s.to(DEV), b_q.to(DEV), b_s.to(DEV), offs.to(DEV),
                                     b_mn_major=mn_major, addend=addend.to(DEV), row_map=row_map.to(DEV))
    ops.check_status(DEV)
    expected = torch.empty_like(ref)
    expected[row_map.long()] = ref + addend.double()
    assert torch.equal(scattered.cpu(), expected.float().bfloat16())


_STORE_FORMS_SNIPPET = """
import hashlib, sys, torch
sys.path.insert(0, {root!r})
from mlops_b200 import ops
g = torch.Generator(device="cuda").manual_seed(5)
counts = [0, 130, 1, 255, 64, 33, 300, 97]   # warps with all 32 rows in the group, with fewer, with none
rows, n, k = sum(counts), 544, 384            # 544 = 2 x 256 + 32: the last tile is one 32-column block wide
a = torch.randn(rows, k, device="cuda", generator=g).bfloat16()
w = torch.randn(len(counts), n, k, device="cuda", generator=g).bfloat16()
a_q, a_s = ops.quantize_rows(a)
w_q, w_s = ops.quantize_blocks(w)
offs = torch.tensor([0] + counts, dtype=torch.int32).cumsum(0).to(torch.int32).cuda()
out = ops.grouped_gemm_fp8(a_q, a_s, w_q, w_s, offs)
# the fused SwiGLU form stores h13 the same way
w13 = torch.randn(len(counts), 512, k, device="cuda", generator=g).bfloat16()
w13_q, w13_s = ops.quantize_blocks(w13)
fused = ops.grouped_gemm_fp8_swiglu(a_q, a_s, w13_q, w13_s, offs)
ops.check_status(torch.device("cuda"))
torch.cuda.synchronize()
digest = hashlib.sha256(out.view(torch.int16).cpu().numpy().tobytes())
digest.update(fused[0].view(torch.int16).cpu().numpy().tobytes())
print("DIGEST", digest.hexdigest(), float(out.float().abs().sum()))
"""


def test_tma_store_and_register_store_write_the_same_bytes():
    """The output of the FP8 GEMM leaves through TMA stores where a warp's 32 rows all belong
    to the group and from registers elsewhere; with B200MOE_GEMM_TMA_STORE=0 (read once per
    process, hence the child processes) everything leaves from registers. Same bytes."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parent.parent)
    digests = []
    for switch in ("1", "0"):
        env = dict(os.environ, B200MOE_GEMM_TMA_STORE=switch)
        done = subprocess.run([sys.executable, "-c", _STORE_FORMS_SNIPPET.format(root=root)], env=env,
                              capture_output=True, text=True, timeout=300)
        assert done.returncode == 0, done.stderr[-2000:]
        line = [l for l in done.stdout.splitlines() if l.startswith("DIGEST")][-1].split()
        assert float(line[2]) > 0
        digests.append(line[1])
    assert digests[0] == digests[1]
