"""tcgen05 GEMM kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(got, want):
    return ((got.float() - want).norm() / want.norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 1024),
                                   (300, 520, 264), (1024, 3584, 2048), (77, 40, 72)])
def test_gemm_bf16_matches_fp32(m, n, k):
    from aboleth_b200.ops import check_gemm_status, gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    a = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn(n, k, generator=g, device="cuda").to(torch.bfloat16)
    out = gemm_bf16(a, b)
    torch.cuda.synchronize()
    check_gemm_status("cuda")
    want = a.float() @ b.float().t()
    assert _rel_err(out, want) < 5e-3
    # An exact case: small integers are exact in bf16 and in the fp32 accumulator.
    ai = torch.randint(-3, 4, (m, k), generator=g, device="cuda").to(torch.bfloat16)
    bi = torch.randint(-3, 4, (n, k), generator=g, device="cuda").to(torch.bfloat16)
    exact = (ai.float() @ bi.float().t())
    got = gemm_bf16(ai, bi).float()
    torch.cuda.synchronize()
    assert torch.equal(got, exact.to(torch.bfloat16).float())


def test_grouped_gemm_matches_loop_of_matmuls():
    from aboleth_b200.ops import check_gemm_status, grouped_gemm_bf16

    experts, n, k = 6, 512, 320
    counts = torch.tensor([0, 5, 128, 200, 1, 131], dtype=torch.int32, device="cuda")
    align = 8
    padded = (counts + align - 1) // align * align
    offsets = (torch.cumsum(padded, 0) - padded).to(torch.int32)
    rows = int(padded.sum())
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(rows, k, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(experts, n, k, generator=g, device="cuda").to(torch.bfloat16)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm_bf16(a, w, counts, offsets, out)
    torch.cuda.synchronize()
    check_gemm_status("cuda")
    for e in range(experts):
        lo, cnt = int(offsets[e]), int(counts[e])
        want = a[lo:lo + cnt].float() @ w[e].float().t()
        if cnt:
            assert _rel_err(out[lo:lo + cnt], want) < 5e-3
        pad = out[lo + cnt:lo + int(padded[e])]
        assert bool((pad == 7.0).all())  # rows outside the expert are never written


def test_grouped_gemm_large_experts_use_wide_tiles():
    """Averages of >= 512 rows per expert take the 256-row tile path; ragged counts, many columns."""
    from aboleth_b200.ops import check_gemm_status, grouped_gemm_bf16

    experts, n, k = 4, 1288, 256  # 6 tile columns, the last one partial
    counts = torch.tensor([700, 0, 1031, 517], dtype=torch.int32, device="cuda")
    padded = (counts + 7) // 8 * 8
    offsets = (torch.cumsum(padded, 0) - padded).to(torch.int32)
    rows = int(padded.sum())
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn(rows, k, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(experts, n, k, generator=g, device="cuda").to(torch.bfloat16)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm_bf16(a, w, counts, offsets, out)
    torch.cuda.synchronize()
    check_gemm_status("cuda")
    for e in range(experts):
        lo, cnt = int(offsets[e]), int(counts[e])
        if cnt:
            want = a[lo:lo + cnt].float() @ w[e].float().t()
            assert _rel_err(out[lo:lo + cnt], want) < 5e-3
        assert bool((out[lo + cnt:lo + int(padded[e])] == 7.0).all())


@pytest.mark.parametrize("m,n,k", [(512, 256, 256), (1000, 520, 384), (4096, 4096, 2048)])
def test_gemm_e4m3_matches_fp32(m, n, k):
    """e4m3 x e4m3 products are exact in fp32, so only the accumulation order and the final bf16
    rounding separate the kernel from an fp32 matmul of the dequantised operands."""
    from aboleth_b200.ops import check_gemm_status, gemm_e4m3

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, generator=g, device="cuda").to(torch.float8_e4m3fn)
    out = gemm_e4m3(a, b, alpha=0.5)
    torch.cuda.synchronize()
    check_gemm_status(a.device)
    want = 0.5 * (a.float() @ b.float().t())
    assert _rel_err(out, want) < 5e-3
    # small integers: every partial sum is exact
    ai = torch.randint(-2, 3, (m, k), generator=g, device="cuda").float().to(torch.float8_e4m3fn)
    bi = torch.randint(-2, 3, (n, k), generator=g, device="cuda").float().to(torch.float8_e4m3fn)
    got = gemm_e4m3(ai, bi).float()
    torch.cuda.synchronize()
    assert torch.equal(got, (ai.float() @ bi.float().t()).to(torch.bfloat16).float())


@pytest.mark.parametrize("m,n,k,pow2", [(256, 384, 512, True), (1000, 520, 384, False)])
def test_block_scaled_e4m3_gemm_matches_fp32(m, n, k, pow2):
    """1 x 128 activation scales and 128 x 128 weight scales: the expansion to bf16 is the fp32
    product rounded once (exact for power-of-two scales), and the GEMM over it matches an fp32
    matmul of the dequantised operands."""
    from aboleth_b200.ops import check_gemm_status
    from aboleth_b200.ops.gemm import dequant_block_scaled, gemm_e4m3_block_scaled
    from aboleth_b200.ops.moe_ops import quant_fp8

    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    a_q, a_s = quant_fp8(x, round_scale=pow2)
    w = 0.02 * torch.randn(n, k, generator=g, device="cuda")
    rows_b, cols_b = -(-n // 128), k // 128
    padded = torch.zeros(rows_b * 128, k, device="cuda")
    padded[:n] = w
    amax = padded.view(rows_b, 128, cols_b, 128).abs().amax(dim=(1, 3)).clamp_min(1e-10)
    b_s = amax / 448.0
    if pow2:
        b_s = torch.exp2(torch.ceil(torch.log2(b_s)))
    b_full = b_s.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)
    b_q = (w / b_full).clamp(-448, 448).to(torch.float8_e4m3fn)
    a_full = a_s.repeat_interleave(128, dim=1)

    a_deq = dequant_block_scaled(a_q, a_s)
    b_deq = dequant_block_scaled(b_q, b_s.contiguous(), block=(128, 128))
    torch.cuda.synchronize()
    assert torch.equal(a_deq, (a_q.float() * a_full).to(torch.bfloat16))
    assert torch.equal(b_deq, (b_q.float() * b_full).to(torch.bfloat16))
    if pow2:  # nothing was rounded
        assert torch.equal(a_deq.float(), a_q.float() * a_full)

    # Power-of-two scales go to the tensor core as ue8m0 (no expansion); others take the expansion.
    out = gemm_e4m3_block_scaled(a_q, a_s, b_q, b_s.contiguous(), path="mx" if pow2 else "expand")
    torch.cuda.synchronize()
    check_gemm_status(out.device)
    want = (a_q.float() * a_full) @ (b_q.float() * b_full).t()
    assert _rel_err(out, want) < 5e-3
    if pow2:
        # fp32 accumulation of exact products of e4m3 values and power-of-two scales: the two paths
        # differ only in the order of additions
        other = gemm_e4m3_block_scaled(a_q, a_s, b_q, b_s.contiguous(), path="expand")
        torch.cuda.synchronize()
        assert _rel_err(out, other.float()) < 2e-3
    # A strided view (rows of a wider buffer) goes through the same kernel.
    wide = torch.zeros(m, k + 64, dtype=torch.float8_e4m3fn, device="cuda")
    wide[:, :k] = a_q
    assert torch.equal(dequant_block_scaled(wide[:, :k], a_s), a_deq)


@pytest.mark.parametrize("tile,m,n,k", [("1", 300, 640, 512),     # 128 x 256 tiles: partial rows, 2.5 column tiles
                                         ("2", 300, 640, 512),     # 256 x 192 tiles: tiles start at odd granules
                                         ("2", 700, 1000, 384)])   # three row tiles, ragged last column tile
def test_block_scaled_mx_gemm_is_exact_on_integers_and_flags_bad_scales(tile, m, n, k, monkeypatch):
    """Small integers and power-of-two scales: every product and partial sum is exact, so the
    tensor-core path must reproduce the fp32 result bit for bit (after the bf16 rounding of the
    output) - this pins the scale-factor layout: a wrong row or K segment changes the sum."""
    from aboleth_b200.ops import check_gemm_status, gemm_e4m3_block_scaled
    from aboleth_b200.ops.gemm import gemm_status

    monkeypatch.setenv("ABOLETH_GEMM_MX_TILE", tile)
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randint(-2, 3, (m, k), generator=g, device="cuda").float()
    b = torch.randint(-2, 3, (n, k), generator=g, device="cuda").float()
    a_s = torch.exp2(torch.randint(-3, 4, (m, k // 128), generator=g, device="cuda").float())
    b_s = torch.exp2(torch.randint(-3, 4, (-(-n // 128), k // 128), generator=g, device="cuda").float())
    a_q, b_q = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)
    out = gemm_e4m3_block_scaled(a_q, a_s, b_q, b_s)
    torch.cuda.synchronize()
    check_gemm_status(out.device)
    a_full = a_s.repeat_interleave(128, dim=1)
    b_full = b_s.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)
    want = ((a * a_full) @ (b * b_full).t()).to(torch.bfloat16)
    assert torch.equal(out, want)
    # a scale that is not a power of two cannot be carried as ue8m0: reported, not silently rounded
    bad = a_s.clone()
    bad[5, 1] = 0.3
    gemm_e4m3_block_scaled(a_q, bad, b_q, b_s)
    torch.cuda.synchronize()
    assert gemm_status(out.device)[:2].tolist() == [3, 0x3500]
    gemm_status(out.device).zero_()


@pytest.mark.parametrize("counts", [[0, 5, 128, 200, 1, 131],        # small experts: 128-row tiles
                                    [700, 0, 1031, 517, 300, 260]])   # 256-row tiles, ragged
def test_grouped_block_scaled_gemm_is_exact_on_integers(counts):
    """Expert-contiguous e4m3 rows (every expert on a 128-row boundary) times e4m3 expert weights, scales
    applied by the tensor core.  Small integers and power-of-two scales make the result exact."""
    from aboleth_b200.ops import check_gemm_status, grouped_gemm_e4m3_mx, pack_scales_mx

    experts, n, k = len(counts), 640, 384
    counts = torch.tensor(counts, dtype=torch.int32, device="cuda")
    padded = (counts + 127) // 128 * 128
    offsets = (torch.cumsum(padded, 0) - padded).to(torch.int32)
    rows = int(padded.sum())
    g = torch.Generator(device="cuda").manual_seed(17)
    a = torch.randint(-2, 3, (rows, k), generator=g, device="cuda").float()
    w = torch.randint(-2, 3, (experts, n, k), generator=g, device="cuda").float()
    a_s = torch.exp2(torch.randint(-2, 3, (rows, k // 128), generator=g, device="cuda").float())
    w_s = torch.exp2(torch.randint(-2, 3, (experts, n // 128, k // 128), generator=g, device="cuda").float())
    fp8 = torch.float8_e4m3fn
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm_e4m3_mx(a.to(fp8), pack_scales_mx(a_s, rows, k, weight=False), w.to(fp8),
                         pack_scales_mx(w_s.view(experts * n // 128, k // 128), experts * n, k, weight=True),
                         counts, offsets, out)
    torch.cuda.synchronize()
    check_gemm_status("cuda")
    a_full = a * a_s.repeat_interleave(128, dim=1)
    for e in range(experts):
        lo, cnt = int(offsets[e]), int(counts[e])
        w_full = w[e] * w_s[e].repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
        assert torch.equal(out[lo:lo + cnt], (a_full[lo:lo + cnt] @ w_full.t()).to(torch.bfloat16))
        assert bool((out[lo + cnt:lo + int(padded[e])] == 7.0).all())   # padding rows are never written
