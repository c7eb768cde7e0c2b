"""The tensor-core paged attention kernel alone, against a plain fp64 restatement: head sizes in steps of
16, groups that are no power of two, page sizes, windows, steps that mix prompt portions with decode
tokens, and key ranges cut into slices."""
from types import SimpleNamespace

import pytest
import torch

from plain import kernels_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_case(nh, nkv, hd, ps, reqs, seed=0):
    """reqs: list of (context_before, q_len).  Pages are scattered; returns everything the kernel needs
    plus flat per-token (request, position) for the reference."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-(c + q) // ps) for c, q in reqs) + 2
    perm = torch.randperm(total_pages, generator=g).tolist()
    max_pages = max(-(-(c + q) // ps) for c, q in reqs)
    table = torch.full((len(reqs), max_pages), -1, dtype=torch.int32)
    cache = torch.randn(total_pages, 2, nkv, ps, hd, generator=g).to(torch.bfloat16)
    q_start, tok_req, positions = [0], [], []
    for s, (c, q) in enumerate(reqs):
        for i in range(-(-(c + q) // ps)):
            table[s, i] = perm.pop()
        tok_req += [s] * q
        positions += list(range(c, c + q))
        q_start.append(q_start[-1] + q)
    T = q_start[-1]
    q = torch.randn(T, nh * hd, generator=g).to(torch.bfloat16)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(num_requests=len(reqs), host_q_start=q_start, host_context_before=[c for c, _ in reqs],
                            q_start=i32(q_start), context_before=i32([c for c, _ in reqs]), attention_plan={})
    group = SimpleNamespace(block_table=table.to(DEV))
    return q.to(DEV), cache.to(DEV), group, batch, i32(tok_req), i32(positions)


SHAPES = [(4, 2, 16, 16), (3, 1, 32, 8), (32, 4, 64, 16), (8, 1, 128, 32), (6, 2, 80, 16), (7, 1, 48, 16),
          (2, 1, 256, 64), (40, 2, 64, 16)]
MIXED = [(0, 1), (0, 77), (130, 1), (63, 2), (200, 40), (5, 1), (64, 64), (511, 1)]


@pytest.mark.parametrize("nh,nkv,hd,ps", SHAPES)
@pytest.mark.parametrize("window", [0, 50])
def test_mixed_step(nh, nkv, hd, ps, window):
    from forge_b200 import kernels as k
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, MIXED)
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps, window)
    got = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps, window=window).float()
    err = (got - ref).abs().amax(dim=1)
    bad = torch.nonzero(err > 1e-2 * ref.abs().max())
    assert len(bad) == 0, f"first wrong token {int(bad[0])} (request {int(tok_req[bad[0]])}, position {int(positions[bad[0]])})"


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 4, 64, 16), (3, 1, 32, 8), (16, 2, 128, 16)])
@pytest.mark.parametrize("splits", [1, 2, 5, 16])
def test_decode_tokens_with_sliced_keys(nh, nkv, hd, ps, splits):
    from forge_b200 import kernels as k
    reqs = [(0, 1), (63, 1), (64, 1), (65, 1), (300, 1), (1000, 1)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=1)
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps)
    got = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps, num_splits=splits).float()
    assert (got - ref).abs().max() <= 1e-2 * ref.abs().max()
    auto = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps).float()      # the heuristic's choice
    assert (auto - ref).abs().max() <= 1e-2 * ref.abs().max()


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 4, 64, 16), (6, 2, 80, 16), (2, 1, 256, 64), (4, 4, 16, 16)])
@pytest.mark.parametrize("splits", [40, 150, 300])
def test_long_contexts_in_many_slices(nh, nkv, hd, ps, splits):
    """Hundreds of slices per request (a long context spread over the whole GPU): the merge deals them to the threads
    of a CTA, one to four warps; short requests leave most slices without a key; one far key carries the weight."""
    from forge_b200 import kernels as k
    reqs = [(5000, 1), (9000, 1), (100, 1), (0, 1)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=6)
    far = 4321
    page = int(group.block_table[1, far // ps])
    cache[page, 0, 0, far % ps, :] = (q[1, :hd].float() * 4.0).to(torch.bfloat16)
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps)
    got = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps, num_splits=splits).float()
    k.check_kernel_status()
    err = (got - ref).abs().amax(dim=1)
    assert float(err.max()) <= 1e-2 * float(ref.abs().max()), err.tolist()


def test_far_key_and_page_edges():
    """One early key gets nearly all the weight of the last query; contexts end exactly on, one before and
    one after a page's edge and a key tile's edge."""
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 8, 2, 64, 16
    reqs = [(c, 1) for c in (15, 16, 17, 63, 64, 65, 127, 128, 129)] + [(700, 3)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=2)
    far = 21
    page = int(group.block_table[len(reqs) - 1, far // ps])
    cache[page, 0, 0, far % ps, :] = (q[-1, :hd].float() * 4.0).to(torch.bfloat16)
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps)
    v_far = cache[page, 1, 0, far % ps, :].float()
    assert (ref[-1, :hd] - v_far).abs().max() < 5e-2
    for splits in (1, 4):
        got = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps, num_splits=splits).float()
        assert (got - ref).abs().max() <= 1e-2 * ref.abs().max()


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 4, 64, 16), (3, 1, 32, 8), (16, 2, 128, 16), (6, 2, 80, 16), (4, 4, 16, 16)])
@pytest.mark.parametrize("window,rotary", [(0, True), (40, True), (0, False)])
def test_decode_step_in_one_kernel(nh, nkv, hd, ps, window, rotary):
    """Rotary encoding + cache write + attention of one new token per request in one launch, against the
    plain rope-and-write followed by the plain attention; contexts on and around page and tile edges, few
    and many requests (8 or 4 warps per CTA)."""
    from forge_b200 import kernels as k
    theta = 5e5
    for ctxs in ([0, 15, 16, 31, 32, 33, 63, 64, 300, 1000], [7] * 70 + [129], [2500, 3100]):     # the last: many tiles per warp, 4 CTAs per request
        reqs = [(c, 1) for c in ctxs]
        q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=4)
        S = len(reqs)
        qkv = torch.randn(S, (nh + 2 * nkv) * hd, generator=torch.Generator().manual_seed(9)).to(q.device) * 1.5
        slots = torch.tensor([int(group.block_table[s, c // ps]) * ps + c % ps for s, c in enumerate(ctxs)],
                             dtype=torch.int32, device=q.device)
        q_ref, cache_ref = R.rope_kv_write_ref(qkv, positions, slots, cache, nh, nkv, hd, ps, theta, rotary)
        cache_ref = cache_ref.to(torch.bfloat16)                  # the engine's cache holds bf16
        ref = R.paged_attention_ref(q_ref.to(torch.bfloat16), cache_ref, group.block_table, tok_req, positions, nh, nkv, hd, ps, window)
        # max_context steers how many CTAs share a request's keys (1, 2 or 4): unknown, the real bound, a huge one
        for max_context in (0, max(ctxs) + 1, 100000):
            work = cache.clone()
            got = k.decode_attention_fused(qkv, work, group.block_table, positions, slots, nh, nkv, hd, ps, theta,
                                           rotary=rotary, window=window, max_context=max_context).float()
            assert (got - ref).abs().max() <= 1e-2 * ref.abs().max(), max_context
            assert (work.float() - cache_ref.float()).abs().max() <= 1e-2 * cache_ref.float().abs().max()   # k, v landed in their slots


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 4, 64, 64), (32, 4, 64, 16), (14, 2, 128, 64), (16, 2, 128, 32), (3, 1, 64, 32), (16, 1, 64, 64)])
@pytest.mark.parametrize("window,rotary", [(0, True), (100, True), (0, False)])
def test_decode_step_with_the_cache_streamed_through_a_ring(nh, nkv, hd, ps, window, rotary):
    """The decode attention whose keys and values come by TMA into a ring of 64-key tiles, against the plain
    rope-and-write followed by the plain attention: contexts on and around page and tile edges (the new token is the
    first, the last, the only row of its tile), few and many requests (8 or 4 consumer warps), 1 to 16 CTAs per request,
    more tiles than the ring holds, a window that cuts the first tile, and one far key that carries the weight."""
    from forge_b200 import kernels as k
    theta = 5e5
    for ctxs in ([0, 15, 16, 31, 32, 33, 63, 64, 65, 127, 128, 300, 1000], [7] * 70 + [129, 640], [2500, 3100], [5000]):
        reqs = [(c, 1) for c in ctxs]
        q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=4)
        S = len(reqs)
        qkv = torch.randn(S, (nh + 2 * nkv) * hd, generator=torch.Generator().manual_seed(9)).to(q.device) * 1.5
        slots = torch.tensor([int(group.block_table[s, c // ps]) * ps + c % ps for s, c in enumerate(ctxs)],
                             dtype=torch.int32, device=q.device)
        q_ref, cache_ref = R.rope_kv_write_ref(qkv, positions, slots, cache, nh, nkv, hd, ps, theta, rotary)
        if window == 0 and max(ctxs) >= 2500:
            # one early key gets nearly all the weight of the last request's first head
            far = 77
            page = int(group.block_table[S - 1, far // ps])
            cache_ref[page, 0, 0, far % ps, :] = q_ref[S - 1, :hd].float() * 4.0
            cache[page, 0, 0, far % ps, :] = cache_ref[page, 0, 0, far % ps, :].to(torch.bfloat16)
        cache_ref = cache_ref.to(torch.bfloat16)                  # the engine's cache holds bf16
        ref = R.paged_attention_ref(q_ref.to(torch.bfloat16), cache_ref, group.block_table, tok_req, positions, nh, nkv, hd, ps, window)
        for ksplit, max_context in ((0, 0), (0, max(ctxs) + 1), (1, 0), (2, 0), (4, 0), (8, 0), (16, 0)):
            if (ksplit > 1 and S * nkv * ksplit > 2048) or (ksplit == 16 and S > 4):
                continue
            work = cache.clone()
            got = k.decode_attention_stream(qkv, work, group.block_table, positions, slots, nh, nkv, hd, ps, theta,
                                            rotary=rotary, window=window, max_context=max_context, ksplit=ksplit).float()
            k.check_kernel_status()
            err = (got - ref).abs().amax(dim=1)
            assert float(err.max()) <= 1e-2 * float(ref.abs().max()), (ksplit, max_context, err.tolist())
            assert (work.float() - cache_ref.float()).abs().max() <= 1e-2 * cache_ref.float().abs().max()   # k, v landed in their slots
