"""The tcgen05/TMA matrix product against a plain fp64 product, at sizes that are not the engine's:
row, column and reduction tails, every tile width, every epilogue."""
import pytest
import torch

from plain import kernels_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def _k():
    from forge_b200 import kernels
    return kernels


SHAPES = [(128, 256, 64), (1, 48, 8), (7, 100, 72), (130, 257, 200), (300, 515, 1032), (64, 2560, 2048),
          (1000, 384, 96), (257, 130, 4104)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("tile_n", [0, 16, 32, 64, 128, 160, 192, 224, 256])
def test_plain_product_every_tile_width(M, N, K, tile_n):
    k = _k()
    a, w = _rand(M, K), _rand(N, K, seed=1)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2)).to(DEV)
    ref = R.gemm_ref(a, w, bias)
    got = k.gemm_sm100(a, w, bias=bias, tile_n=tile_n)
    k.check_kernel_status()
    # fp32 accumulation of exact bf16 products: the error is a few fp32 roundings of the row's magnitude
    assert (got - ref).abs().max() <= 1e-5 * ref.abs().max() * max(1.0, (K / 64) ** 0.5)


@pytest.mark.parametrize("M,N,K", [(5, 64, 64), (200, 330, 264), (129, 2048, 520)])
def test_epilogues(M, N, K):
    k = _k()
    a, w = _rand(M, K), _rand(N, K, seed=1, scale=0.2)
    ref = R.gemm_ref(a, w)
    tol = 1e-5 * ref.abs().max() * 3
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(DEV)
    got = k.gemm_sm100(a, w, accumulate_into=res.clone())
    assert (got - (res + ref)).abs().max() <= tol + 1e-6 * res.abs().max()
    got = k.gemm_sm100(a, w, epilogue="cast")
    assert got.dtype == torch.bfloat16 and (got.float() - ref).abs().max() <= 8e-3 * ref.abs().max()
    got = k.gemm_sm100(a, w, epilogue="swiglu")
    want = R.silu_mul_interleaved_ref(ref)
    assert got.shape == (M, N // 2) and (got.float() - want).abs().max() <= 8e-3 * want.abs().max() + 1e-6
    k.check_kernel_status()


def test_many_tiles_per_cta_and_both_accumulators():
    """More tiles than SMs, so every CTA walks several tiles and alternates its two accumulators."""
    k = _k()
    a, w = _rand(1536, 256), _rand(4096, 256, seed=1)
    ref = R.gemm_ref(a, w)
    for tile_n in (128, 160, 224, 256):
        got = k.gemm_sm100(a, w, tile_n=tile_n)
        assert (got - ref).abs().max() <= 2e-5 * ref.abs().max()
    k.check_kernel_status()


@pytest.mark.parametrize("tile_n", [128, 160, 192, 224, 256, 512])
@pytest.mark.parametrize("M,N,K", [(300, 1000, 136), (129, 36, 64), (1100, 2052, 72)])
def test_fp32_results_through_shared_memory_and_tma(M, N, K, tile_n):
    """The wide tiles store fp32 results with TMA and add into the residual with the L2's reduction: row and
    column tails that a box overhangs (1000 = 31 boxes of 32 + 8 columns), a bias, and two additions into the
    same buffer, which must count each product once."""
    k = _k()
    a, w = _rand(M, K), _rand(N, K, seed=1, scale=0.3)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2)).to(DEV)
    ref = R.gemm_ref(a, w, bias)
    tol = 1e-5 * ref.abs().max() * max(1.0, (K / 64) ** 0.5)
    guard = torch.full((M + 2, N), 7.0, device=DEV)            # the rows around the result must stay as they are
    got = k.gemm_sm100(a, w, bias=bias, tile_n=tile_n, out=guard[1:M + 1])
    assert (got - ref).abs().max() <= tol
    assert (guard[0] == 7.0).all() and (guard[M + 1] == 7.0).all()
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(DEV)
    acc = res.clone()
    k.gemm_sm100(a, w, bias=bias, accumulate_into=acc, tile_n=tile_n)
    assert (acc - (res + ref)).abs().max() <= tol + 1e-6 * res.abs().max()
    k.gemm_sm100(a, w, bias=bias, accumulate_into=acc, tile_n=tile_n)
    assert (acc - (res + 2 * ref)).abs().max() <= 2 * tol + 1e-6 * res.abs().max()
    k.check_kernel_status()


@pytest.mark.parametrize("tile_n", [0, 1002, 1004])
@pytest.mark.parametrize("M,N,K", [(512, 2048, 2048), (129, 36, 64), (300, 1000, 136), (512, 2048, 5632), (700, 515, 1032),
                                   (257, 130, 4104), (1100, 2052, 72), (1024, 2048, 2048), (384, 300, 192)])
def test_k_cut_across_a_cluster_for_some_hundred_rows(M, N, K, tile_n):
    """Tiles of 128 x 128 whose K is shared by 2 or 4 CTAs, two k-blocks per copy where K is a multiple of 64, partial
    sums added through distributed shared memory in rank order: fp32 store and the addition into the residual (each product counted once), bias, row, column and
    reduction tails (a last k-block that is partly zeros, CTAs of a cluster with no k-block at all: K = 64 or 72 with 4
    CTAs), and the same bits every time."""
    k = _k()
    a, w = _rand(M, K), _rand(N, K, seed=1, scale=0.3)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2)).to(DEV)
    ref = R.gemm_ref(a, w, bias)
    tol = 1e-5 * ref.abs().max() * max(1.0, (K / 64) ** 0.5)
    guard = torch.full((M + 2, N), 7.0, device=DEV)            # the rows around the result must stay as they are
    got = k.gemm_sm100(a, w, bias=bias, tile_n=tile_n, out=guard[1:M + 1])
    assert (got - ref).abs().max() <= tol
    assert (guard[0] == 7.0).all() and (guard[M + 1] == 7.0).all()
    for _ in range(3):
        assert torch.equal(k.gemm_sm100(a, w, bias=bias, tile_n=tile_n), got)
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(DEV)
    acc = res.clone()
    k.gemm_sm100(a, w, bias=bias, accumulate_into=acc, tile_n=tile_n)
    assert (acc - (res + ref)).abs().max() <= tol + 1e-6 * res.abs().max()
    first = acc.clone()
    k.gemm_sm100(a, w, bias=bias, accumulate_into=acc, tile_n=tile_n)
    assert (acc - (res + 2 * ref)).abs().max() <= 2 * tol + 1e-6 * res.abs().max()
    again = res.clone()
    k.gemm_sm100(a, w, bias=bias, accumulate_into=again, tile_n=tile_n)
    assert torch.equal(again, first)                           # the additions do not depend on the CTAs' timing
    k.check_kernel_status()


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (130, 257, 200), (300, 515, 1032), (2048, 2560, 2048), (1000, 384, 96),
                                   (257, 130, 4104), (4608, 4608, 128)])
def test_two_ctas_on_one_tile(M, N, K):
    """The cta_group::2 kernel: a pair of CTAs on a [256 x 256] tile, every epilogue; row, column and reduction
    tails; (4608, 4608): 324 tiles for 74 pairs, so every pair walks several tiles and both accumulators."""
    k = _k()
    a, w = _rand(M, K), _rand(N, K, seed=1, scale=0.3)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2)).to(DEV)
    ref = R.gemm_ref(a, w, bias)
    tol = 1e-5 * ref.abs().max() * max(1.0, (K / 64) ** 0.5)
    got = k.gemm_sm100(a, w, bias=bias, tile_n=512)
    assert (got - ref).abs().max() <= tol
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(DEV)
    got = k.gemm_sm100(a, w, bias=bias, accumulate_into=res.clone(), tile_n=512)
    assert (got - (res + ref)).abs().max() <= tol + 1e-6 * res.abs().max()
    got = k.gemm_sm100(a, w, bias=bias, epilogue="cast", tile_n=512)
    assert (got.float() - ref).abs().max() <= 8e-3 * ref.abs().max()
    if N % 2 == 0:
        got = k.gemm_sm100(a, w, bias=bias, epilogue="swiglu", tile_n=512)
        want = R.silu_mul_interleaved_ref(ref)
        assert got.shape == (M, N // 2) and (got.float() - want).abs().max() <= 8e-3 * want.abs().max() + 1e-6
    # the same pair of CTAs on tiles of 192 and 128 columns (K in whole pairs of k-blocks only; other K are refused)
    for tile_n in (1192, 1128):
        if K % 64 != 0 or K < 128:
            with pytest.raises(k.KernelError, match="K % 64"):
                k.gemm_sm100(a, w, bias=bias, tile_n=tile_n)
            continue
        got = k.gemm_sm100(a, w, bias=bias, tile_n=tile_n)
        assert (got - ref).abs().max() <= tol, tile_n
        got = k.gemm_sm100(a, w, bias=bias, accumulate_into=res.clone(), tile_n=tile_n)
        assert (got - (res + ref)).abs().max() <= tol + 1e-6 * res.abs().max(), tile_n
        if N % 2 == 0:
            got = k.gemm_sm100(a, w, bias=bias, epilogue="swiglu", tile_n=tile_n)
            assert (got.float() - want).abs().max() <= 8e-3 * want.abs().max() + 1e-6, tile_n
    k.check_kernel_status()
    with pytest.raises(k.KernelError, match="two-CTA"):
        k.gemm_sm100(_rand(64, 64), _rand(128, 64), tile_n=512)


@pytest.mark.parametrize("M", [1, 8, 16, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 64), (48, 8), (2560, 2048), (257, 200), (2048, 5632), (1000, 1032)])
@pytest.mark.parametrize("cluster", [0, -1, -2, -3, -4, -5, -6, -7, -8, -100, -8004, -6402, -9601, -11203, -6408, -6401])
def test_few_rows_kernel_with_k_cut_across_a_cluster(M, N, K, cluster):
    """The decode-shaped kernels (weights as the MMA's M operand) for every epilogue: K cut over a cluster of
    1 to 8 CTAs with partial sums added through distributed shared memory, tiles of fewer than 128 weight rows
    (-(100 * rows + cluster)), and (-100) units of work dealt out evenly to persistent CTAs with partial sums added
    through a workspace."""
    k = _k()
    a, w = _rand(M, K), _rand(N, K, seed=1, scale=0.3)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2)).to(DEV)
    if cluster == -100 and M > 64:                       # the evenly dealt kernel stops at 64 rows and says so
        with pytest.raises(k.KernelError, match="at most 64 rows"):
            k.gemm_sm100(a, w, bias=bias, tile_n=cluster)
        return
    ref = R.gemm_ref(a, w, bias)
    tol = 1e-5 * ref.abs().max() * max(1.0, (K / 64) ** 0.5)
    got = k.gemm_sm100(a, w, bias=bias, tile_n=cluster)
    assert (got - ref).abs().max() <= tol
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(3)).to(DEV)
    got = k.gemm_sm100(a, w, bias=bias, accumulate_into=res.clone(), tile_n=cluster)
    assert (got - (res + ref)).abs().max() <= tol + 1e-6 * res.abs().max()
    got = k.gemm_sm100(a, w, bias=bias, epilogue="cast", tile_n=cluster)
    assert (got.float() - ref).abs().max() <= 8e-3 * ref.abs().max()
    if N % 2 == 0:
        got = k.gemm_sm100(a, w, bias=bias, epilogue="swiglu", tile_n=cluster)
        want = R.silu_mul_interleaved_ref(ref)
        assert got.shape == (M, N // 2) and (got.float() - want).abs().max() <= 8e-3 * want.abs().max() + 1e-6
    k.check_kernel_status()


def test_few_rows_kernel_is_deterministic():
    k = _k()
    a, w = _rand(8, 2048), _rand(2048, 2048, seed=1)
    first = k.gemm_sm100(a, w)
    for _ in range(5):
        assert torch.equal(k.gemm_sm100(a, w), first)


def test_refuses_what_it_cannot_do():
    k = _k()
    with pytest.raises(k.KernelError, match="64, 80, 96, 112 or 128"):      # shorter tiles would let the MMA read past the CTA's shared memory
        k.gemm_sm100(_rand(4, 64), _rand(128, 64), tile_n=-1601)
    with pytest.raises(k.KernelError, match="multiple of 8"):
        k.gemm_sm100(_rand(4, 12), _rand(8, 12))
    with pytest.raises(k.KernelError, match="even"):
        k.gemm_sm100(_rand(4, 16), _rand(7, 16), epilogue="swiglu")
    assert not k.gemm_sm100_supports(64, 12) and k.gemm_sm100_supports(64, 16)


@pytest.mark.parametrize("M,K,nh,nkv,hd,ps,bias,rotary", [
    (300, 512, 8, 2, 64, 16, False, True),      # a tile of 128 columns holds two heads
    (2048, 2048, 32, 4, 64, 64, False, True),   # the benchmark's prompt: 2560 columns
    (257, 3584 // 7, 7, 1, 128, 8, True, True),  # head size 128, bias, columns that are no multiple of 256
    (513, 192, 5, 5, 64, 16, True, False),      # no rotation (keys are stored as projected)
])
def test_projection_whose_epilogue_rotates_and_stores(M, K, nh, nkv, hd, ps, bias, rotary):
    """x . [Wq; Wk; Wv]^T with rotary encoding and the paged cache write in the product's epilogue, against the plain
    product followed by the plain rotate-and-store; some rows have no slot (their keys must not be written)."""
    from forge_b200 import kernels as k
    from plain import kernels_ref as R
    g = torch.Generator().manual_seed(M + K)
    N = (nh + 2 * nkv) * hd
    x = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    b = torch.randn(N, generator=g) * 0.3 if bias else None
    positions = torch.randint(0, 5000, (M,), generator=g, dtype=torch.int32)
    pages = -(-M // ps) + 3
    slots = torch.randperm(pages * ps, generator=g)[:M].to(torch.int32)
    slots[5] = -1
    slots[M - 1] = -1
    cache0 = torch.randn(pages, 2, nkv, ps, hd, generator=g).to(torch.bfloat16)
    qkv = R.gemm_ref(x, w, b)
    q_ref, cache_ref = R.rope_kv_write_ref(qkv, positions, slots, cache0, nh, nkv, hd, ps, 10000.0, rotary)
    dev = "cuda:0"
    cache = cache0.clone().to(dev)
    table = k.rope_table(positions.to(dev), hd, 10000.0, by_pair=True) if rotary else None
    # the library's own choice, then every tile it has: one CTA on 128 or 256 columns, a pair of CTAs on 128, 192 or 256
    for tile in (0, 128, 256, 1128, 1192, 1256):
        cache = cache0.clone().to(dev)
        args = (x.to(dev), w.to(dev), None if b is None else b.to(dev), table, slots.to(dev), cache, nh, nkv, hd, ps)
        if tile == 1192 and hd == 128:
            with pytest.raises(k.KernelError, match="not available"):      # 192 columns are no whole heads of 128
                k.gemm_sm100_qkv_rope(*args, tile=tile)
            continue
        q = k.gemm_sm100_qkv_rope(*args, tile=tile)
        k.check_kernel_status()
        assert (q.float().cpu() - q_ref).abs().max() <= 2e-2 * q_ref.abs().max(), tile
        assert (cache.float().cpu() - cache_ref).abs().max() <= 2e-2 * cache_ref.abs().max(), tile
        assert torch.equal(cache.cpu()[cache_ref == cache0.float()], cache0[cache_ref == cache0.float()]), tile
