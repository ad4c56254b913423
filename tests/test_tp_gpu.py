"""Fused tensor-parallel GEMM + collective kernels, ranks emulated on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(got, want):
    return ((got.float() - want).norm() / want.norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("world,m_local,k,n_local", [(2, 256, 256, 256), (4, 512, 512, 384), (3, 256, 1024, 520),
                                                   (2, 512, 16384, 2000)])  # last: two raster groups
def test_all_gather_gemm_matches_fp32(world, m_local, k, n_local):
    from aboleth_b200.parallel import LocalTpGroup

    g = torch.Generator(device="cuda").manual_seed(world)
    a = [torch.randn(m_local, k, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    b = [torch.randn(n_local, k, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    group = LocalTpGroup(world, m_local, k, 256)
    for _ in range(3):  # alternating buffers and advancing epochs
        outs = group.ag_gemm(a, b)
        torch.cuda.synchronize()
    full = torch.cat(a).float()
    for r in range(world):
        group.ag[r].check()
        assert _rel(outs[r], full @ b[r].float().t()) < 5e-3


@pytest.mark.parametrize("world,m_local,k_local,n", [(2, 256, 256, 256), (4, 256, 384, 520), (3, 512, 128, 1024),
                                                   (2, 512, 16384, 2000)])  # last: two raster groups
def test_gemm_reduce_scatter_matches_fp32(world, m_local, k_local, n):
    from aboleth_b200.parallel import LocalTpGroup

    g = torch.Generator(device="cuda").manual_seed(10 + world)
    a = [torch.randn(world * m_local, k_local, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    b = [torch.randn(n, k_local, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    group = LocalTpGroup(world, m_local, 64, n)
    for _ in range(3):
        outs = group.gemm_rs(a, b)
        torch.cuda.synchronize()
    total = sum(a[r].float() @ b[r].float().t() for r in range(world))
    for r in range(world):
        group.rs[r].check()
        want = total[r * m_local:(r + 1) * m_local]
        assert _rel(outs[r], want) < 8e-3  # partials travel as bf16


def test_block_scaled_activations_through_both_fused_ops():
    """e4m3 activations with 1 x 128 scales enter the fused kernels through the bf16 expansion."""
    from aboleth_b200.ops.moe_ops import quant_fp8
    from aboleth_b200.parallel import LocalTpGroup
    from aboleth_b200.parallel.tp import CONSUME, PRODUCE

    world, m_local, k, n = 2, 256, 256, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    group = LocalTpGroup(world, m_local, k, n)
    b = [torch.randn(n, k, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]

    shards = [quant_fp8(torch.randn(m_local, k, generator=g, device="cuda").to(torch.bfloat16), round_scale=True)
              for _ in range(world)]
    outs = [op.block_scaled(*shards[r], b[r], phases=PRODUCE) for r, op in enumerate(group.ag)]
    outs = [op.block_scaled(*shards[r], b[r], outs[r], phases=CONSUME, advance=False)
            for r, op in enumerate(group.ag)]
    torch.cuda.synchronize()
    full = torch.cat([q.float() * s.repeat_interleave(128, dim=1) for q, s in shards])
    for r in range(world):
        group.ag[r].check()
        assert _rel(outs[r], full @ b[r].float().t()) < 5e-3

    parts = [quant_fp8(torch.randn(world * m_local, k, generator=g, device="cuda").to(torch.bfloat16))
             for _ in range(world)]
    outs = [op.block_scaled(*parts[r], b[r], phases=PRODUCE) for r, op in enumerate(group.rs)]
    outs = [op.block_scaled(*parts[r], b[r], outs[r], phases=CONSUME, advance=False)
            for r, op in enumerate(group.rs)]
    torch.cuda.synchronize()
    total = sum((parts[r][0].float() * parts[r][1].repeat_interleave(128, dim=1)) @ b[r].float().t()
                for r in range(world))
    for r in range(world):
        group.rs[r].check()
        assert _rel(outs[r], total[r * m_local:(r + 1) * m_local]) < 8e-3


def _mx_operands(rows, cols_n, k, g):
    """Small-integer e4m3 operands with random power-of-two block scales: every product and every
    fp32 partial sum is exact, so a wrong scale-factor row, K block or rank offset shows as a
    mismatch rather than as noise."""
    from aboleth_b200.ops import pack_scales_mx

    a = torch.randint(-2, 3, (rows, k), generator=g, device="cuda").float()
    b = torch.randint(-2, 3, (cols_n, k), generator=g, device="cuda").float()
    a_s = torch.exp2(torch.randint(-2, 3, (rows, k // 128), generator=g, device="cuda").float())
    b_s = torch.exp2(torch.randint(-2, 3, (-(-cols_n // 128), k // 128), generator=g, device="cuda").float())
    fp8 = torch.float8_e4m3fn
    packed = (a.to(fp8), pack_scales_mx(a_s, rows, k, weight=False), b.to(fp8),
              pack_scales_mx(b_s, cols_n, k, weight=True))
    a_full = a * a_s.repeat_interleave(128, dim=1)
    b_full = b * b_s.repeat_interleave(128, dim=0)[:cols_n].repeat_interleave(128, dim=1)
    return packed, a_full, b_full


@pytest.mark.parametrize("world,m_local,k,n_local", [(2, 256, 256, 256), (4, 512, 512, 520), (3, 256, 1024, 1000)])
def test_all_gather_gemm_block_scaled_e4m3_is_exact(world, m_local, k, n_local):
    """The shards cross as e4m3 with their scale-factor atoms and are multiplied by the
    block-scaled MMA: no expansion to bf16 anywhere."""
    from aboleth_b200.parallel import LocalTpGroup

    g = torch.Generator(device="cuda").manual_seed(20 + world)
    ranks = [_mx_operands(m_local, n_local, k, g) for _ in range(world)]
    group = LocalTpGroup(world, m_local, k, 256)
    args = [[ranks[r][0][i] for r in range(world)] for i in range(4)]
    for _ in range(3):
        outs = group.ag_gemm_mx(*args)
        torch.cuda.synchronize()
    full = torch.cat([ranks[r][1] for r in range(world)])
    for r in range(world):
        group.ag[r].check()
        assert torch.equal(outs[r], (full @ ranks[r][2].t()).to(torch.bfloat16))


@pytest.mark.parametrize("world,m_local,k_local,n", [(2, 256, 256, 256), (4, 256, 384, 520), (3, 512, 128, 1000)])
def test_gemm_reduce_scatter_block_scaled_e4m3(world, m_local, k_local, n):
    from aboleth_b200.parallel import LocalTpGroup

    g = torch.Generator(device="cuda").manual_seed(30 + world)
    ranks = [_mx_operands(world * m_local, n, k_local, g) for _ in range(world)]
    group = LocalTpGroup(world, m_local, 64, n)
    args = [[ranks[r][0][i] for r in range(world)] for i in range(4)]
    for _ in range(3):
        outs = group.gemm_rs_mx(*args)
        torch.cuda.synchronize()
    # each rank's partial is rounded to bf16 before it travels; the sum over ranks is fp32
    total = sum((ranks[r][1] @ ranks[r][2].t()).to(torch.bfloat16).float() for r in range(world))
    for r in range(world):
        group.rs[r].check()
        want = total[r * m_local:(r + 1) * m_local].to(torch.bfloat16)
        assert torch.equal(outs[r], want)
