"""Each CUDA kernel alone against a plain PyTorch restatement, at sizes other than the engine's."""
import math

import pytest
import torch

from plain import kernels_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _k():
    from forge_b200 import kernels
    return kernels


def _rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,V,H", [(1, 7, 24), (37, 1001, 200), (5, 64, 2056)])
def test_embedding(dtype, T, V, H):
    k = _k()
    table = _rand(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out = k.embedding(ids, table)
    assert torch.equal(out, R.embedding_ref(ids, table))


def test_embedding_flags_bad_id():
    k = _k()
    table = _rand(10, 8)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = k.embedding(torch.tensor([3, 10, -1], dtype=torch.int32, device=DEV), table, status=status)
    assert int(status.item()) & 1
    assert torch.all(out[1:] == 0) and torch.equal(out[0], table[3])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,eps", [(3, 24, 1e-5), (17, 1000, 1e-6), (2, 5000, 1e-2)])
def test_rmsnorm(out_dtype, T, H, eps):
    k = _k()
    x, w = _rand(T, H, scale=3.0), _rand(H, seed=1) + 1.0
    ref = R.rmsnorm_ref(x, w, eps)
    got = k.rmsnorm(x, w, eps, out_dtype).float()
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert (got - ref).abs().max() <= tol * ref.abs().max()
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    got2 = k.rmsnorm(x, w, eps, out_dtype, rows=rows).float()
    assert torch.equal(got2, got[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,ps,theta", [(4, 2, 16, 16, 1e4), (3, 1, 48, 8, 5e5), (7, 7, 128, 32, 1e6)])
def test_rope_kv_write(dtype, nh, nkv, hd, ps, theta):
    k = _k()
    T, pages = 21, 9
    qkv = _rand(T, (nh + 2 * nkv) * hd, scale=2.0)
    positions = torch.randint(0, 3000, (T,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * ps)[:T].to(torch.int32).to(DEV)
    slots[4] = -1
    cache = torch.zeros(pages, 2, nkv, ps, hd, dtype=dtype, device=DEV)
    q = k.rope_kv_write(qkv, positions, slots, cache, nh, nkv, hd, ps, theta, dtype)
    q_ref, cache_ref = R.rope_kv_write_ref(qkv, positions, slots, cache * 0, nh, nkv, hd, ps, theta)
    tol = 2e-4 if dtype == torch.float32 else 1e-2     # fp32 angles at positions up to 3000
    assert (q.float() - q_ref).abs().max() <= tol * q_ref.abs().max()
    assert (cache.float() - cache_ref).abs().max() <= tol * cache_ref.abs().max()
    # with the step's cos/sin table instead of angles computed per head: the same numbers
    cache2 = torch.zeros_like(cache)
    q_t = k.rope_kv_write(qkv, positions, slots, cache2, nh, nkv, hd, ps, theta, dtype, table=k.rope_table(positions, hd, theta))
    assert torch.equal(q_t, q) and torch.equal(cache2, cache)
    # no rotation: a plain copy
    q2 = k.rope_kv_write(qkv, positions, None, None, nh, nkv, hd, ps, theta, dtype, rotary=False)
    assert torch.equal(q2.float(), qkv[:, :nh * hd].to(dtype).float())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_silu_mul_interleaved(out_dtype):
    k = _k()
    gu = _rand(13, 2 * 177, scale=4.0)
    ref = R.silu_mul_interleaved_ref(gu)
    got = k.silu_mul_interleaved(gu, out_dtype).float()
    tol = 1e-6 if out_dtype == torch.float32 else 1e-2
    assert (got - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (70, 130, 50), (33, 257, 1000), (128, 64, 16)])
def test_gemm_simt(dtype, M, N, K):
    k = _k()
    a, w, b = _rand(M, K, dtype=dtype), _rand(N, K, dtype=dtype, seed=1), _rand(N, seed=2)
    ref = R.gemm_ref(a, w, b)
    got = k.gemm_simt(a, w, bias=b)
    assert (got - ref).abs().max() <= 2e-6 * math.sqrt(K) * ref.abs().max() + 1e-6
    acc = _rand(M, N, seed=3)
    got2 = k.gemm_simt(a, w, bias=None, out=acc.clone(), accumulate=True)
    assert (got2 - (acc + R.gemm_ref(a, w))).abs().max() <= 2e-6 * math.sqrt(K) * ref.abs().max() + 1e-6


def _paged_case(nh, nkv, hd, ps, lens, dtype, seed=0):
    """Requests of the given lengths scattered over shuffled pages; queries for the last few positions."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // ps) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max(-(-n // ps) for n in lens)
    table = torch.full((len(lens), max_pages), -1, dtype=torch.int32)
    cache = (torch.randn(n_pages, 2, nkv, ps, hd, generator=g)).to(dtype)
    tok_req, positions = [], []
    for r, n in enumerate(lens):
        for i in range(-(-n // ps)):
            table[r, i] = perm.pop()
        for p in sorted({0, n // 2, max(0, n - ps - 1), n - 2, n - 1} & set(range(n))):
            tok_req.append(r)
            positions.append(p)
    T = len(tok_req)
    q = (torch.randn(T, nh * hd, generator=g)).to(dtype)
    dev = lambda t: t.to(DEV)
    return (dev(q), dev(cache), dev(table), dev(torch.tensor(tok_req, dtype=torch.int32)),
            dev(torch.tensor(positions, dtype=torch.int32)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 16, 0), (3, 1, 32, 8, 0), (6, 2, 80, 16, 0),
                                                 (8, 1, 128, 32, 0), (4, 4, 64, 16, 37), (2, 1, 256, 64, 0)])
def test_paged_attention_simt(dtype, nh, nkv, hd, ps, window):
    k = _k()
    q, cache, table, tok_req, positions = _paged_case(nh, nkv, hd, ps, [1, ps, ps + 1, 5 * ps - 1, 300], dtype)
    ref = R.paged_attention_ref(q, cache, table, tok_req, positions, nh, nkv, hd, ps, window)
    got = k.paged_attention_simt(q, cache, table, tok_req, positions, nh, nkv, hd, ps, window=window).float()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (got - ref).abs().max() <= tol * ref.abs().max()


def test_paged_attention_far_key_stands_out():
    """One key among hundreds, on an early page, carries nearly all the weight: a kernel that skips or
    misplaces that page cannot pass."""
    k = _k()
    nh, nkv, hd, ps = 2, 1, 32, 16
    q, cache, table, tok_req, positions = _paged_case(nh, nkv, hd, ps, [700], torch.float32, seed=3)
    far = 21                                            # position of the far key (page 1, slot 5)
    page = int(table[0, far // ps])
    cache[page, 0, 0, far % ps, :] = q[-1, :hd] * 4.0   # aligned with head 0 of the last query
    ref = R.paged_attention_ref(q, cache, table, tok_req, positions, nh, nkv, hd, ps)
    got = k.paged_attention_simt(q, cache, table, tok_req, positions, nh, nkv, hd, ps)
    v_far = cache[page, 1, 0, far % ps, :]
    assert (ref[-1, :hd] - v_far).abs().max() < 1e-3    # the construction works: output is that value
    assert (got - ref).abs().max() <= 1e-5 * ref.abs().max()


def test_argmax_lowest_index_wins():
    k = _k()
    logits = _rand(5, 1003)
    logits[0, 17] = logits[0, 900] = 50.0
    logits[1, 1002] = 60.0
    logits[2, 0] = 60.0
    got = k.argmax(logits)
    assert got.tolist() == torch.argmax(logits, dim=-1).tolist()
    assert got[0].item() == 17


@pytest.mark.parametrize("V", [1531, 32000, 60000])      # keys in shared memory (a partial chunk; whole chunks of 32), keys in global memory
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 0, 1.0), (0.8, 40, 1.0), (1.3, 0, 0.9),
                                                      (0.7, 40, 0.9), (1.0, 1, 1.0), (0.9, 3000, 0.95)])
def test_sample_picks_the_token_whose_interval_holds_u(temperature, top_k, top_p, V):
    """(0.9, 3000, 0.95): more kept entries than the kernel gathers, so top-p is found digit by digit as without top-k."""
    k = _k()
    R_ = 16
    logits = _rand(R_, V, scale=3.0)
    logits[3, 100:140] = logits[3].max() + 0.5             # ties at the top: all of them are kept
    us = torch.linspace(0.01, 0.99, R_)
    got = k.sample(logits, torch.full((R_,), temperature, device=DEV), torch.full((R_,), top_k, dtype=torch.int32, device=DEV),
                   torch.full((R_,), top_p, device=DEV), us.to(DEV))
    for r in range(R_):
        p = R.sample_probabilities_ref(logits[r].cpu(), temperature, top_k, top_p)
        cdf = torch.cumsum(p, 0)
        i = int(got[r])
        assert p[i] > 0, "a token outside the kept set was drawn"
        lo = float(cdf[i - 1]) if i > 0 else 0.0
        assert lo - 1e-5 <= float(us[r]) <= float(cdf[i]) + 1e-5


def test_repeat_penalty():
    k = _k()
    logits = _rand(2, 50)
    before = logits.clone()
    tokens = torch.tensor([3, 7, 9], dtype=torch.int32, device=DEV)
    counts = torch.tensor([1, 2, 1], dtype=torch.int32, device=DEV)
    offsets = torch.tensor([0, 2, 3], dtype=torch.int32, device=DEV)
    pen = torch.tensor([1.5, 2.0], device=DEV)
    k.repeat_penalty(logits, tokens, counts, offsets, pen)
    def f(v, p, c):
        for _ in range(c):
            v = v / p if v > 0 else v * p
        return v
    want = before.clone()
    want[0, 3] = f(before[0, 3].item(), 1.5, 1)
    want[0, 7] = f(before[0, 7].item(), 1.5, 2)
    want[1, 9] = f(before[1, 9].item(), 2.0, 1)
    assert torch.allclose(logits, want, rtol=1e-6, atol=0)
