"""The tcgen05/TMEM attention kernel for prompt portions (head sizes 64 and 128, groups that do and do not divide
the tile's 128 rows) against a plain fp64 restatement, alone and through the dispatcher that sends requests with few
rows to the mma.sync kernel."""
import pytest
import torch

from plain import kernels_ref as R
from test_attention_mma_gpu import make_case

pytestmark = pytest.mark.gpu

SHAPES = [(32, 4, 64, 16), (8, 8, 64, 16), (16, 1, 64, 8), (4, 2, 64, 64), (6, 3, 64, 32),
          (32, 8, 128, 16),      # head size 128, group of 4 (the Llama-3-8B shape)
          (28, 4, 128, 64),      # head size 128, group of 7: a tile holds 18 tokens = 126 rows (the Qwen2.5-7B shape)
          (6, 2, 64, 16),        # group of 3: 42 tokens = 126 rows
          (5, 1, 128, 8),        # group of 5: 25 tokens = 125 rows
          (40, 2, 64, 16)]       # group of 20: 6 tokens = 120 rows
PORTIONS = [(0, 100), (130, 17), (0, 300), (63, 65), (500, 16), (64, 64)]


def _rows_of_big(reqs, group, min_rows):
    rows, t = [], 0
    for c, q in reqs:
        if q * group >= min_rows:
            rows += list(range(t, t + q))
        t += q
    return torch.tensor(rows, dtype=torch.long)


@pytest.mark.parametrize("nh,nkv,hd,ps", SHAPES)
@pytest.mark.parametrize("window", [0, 70])
def test_prompt_portions(nh, nkv, hd, ps, window):
    from forge_b200 import kernels as k
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, PORTIONS)
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps, window)
    out = torch.full_like(q, float("nan"))
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, window=window, out=out)
    k.check_kernel_status()
    big = _rows_of_big(PORTIONS, nh // nkv, k.TC_MIN_ROWS).to(q.device)
    assert n > 0 and len(big) > 0
    err = (got.float()[big] - ref[big]).abs().amax(dim=1)
    bad = torch.nonzero(~(err <= 1e-2 * ref.abs().max()))
    assert len(bad) == 0, f"first wrong token {int(big[bad[0]])} (request {int(tok_req[big[bad[0]]])}, position {int(positions[big[bad[0]]])})"


def test_shapes_it_takes():
    from forge_b200 import kernels as k
    for hd, g in ((128, 4), (128, 7), (64, 3), (64, 8), (128, 128)):
        assert k.attention_sm100_supports(hd, g, 16), (hd, g)
    assert not k.attention_sm100_supports(96, 4, 16) and not k.attention_sm100_supports(64, 4, 128)


@pytest.mark.parametrize("nh,nkv,hd,ps", SHAPES[:3] + SHAPES[5:8])
def test_dispatcher_covers_every_token(nh, nkv, hd, ps):
    """Portions of prompts beside decode tokens: big requests by tcgen05, small ones by mma.sync, no row missed."""
    from forge_b200 import kernels as k
    reqs = PORTIONS + [(700, 1), (3, 1), (64, 2)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=5)
    batch.tok_req, batch.positions = tok_req, positions
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps)
    got = k.paged_attention(q, cache, group, batch, nh, nkv, hd, ps).float()
    k.check_kernel_status()
    assert not torch.isnan(got).any()
    assert (got - ref).abs().max() <= 1e-2 * ref.abs().max()


def test_long_causal_prompt_heaviest_tiles_first():
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 32, 4, 64, 16
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, [(0, 1100)], seed=7)
    ref = R.paged_attention_ref(q[-40:], cache, group.block_table, tok_req[-40:], positions[-40:], nh, nkv, hd, ps)
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps)
    k.check_kernel_status()
    assert n == -(-1100 * 8 // 128)
    # the same with head size 128 and 7 query heads per kv head
    nh, nkv, hd, ps = 14, 2, 128, 32
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, [(0, 700)], seed=8)
    ref = R.paged_attention_ref(q[-40:], cache, group.block_table, tok_req[-40:], positions[-40:], nh, nkv, hd, ps)
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps)
    k.check_kernel_status()
    assert n == -(-700 // 18)
    assert (got.float()[-40:] - ref).abs().max() <= 1e-2 * ref.abs().max()
    assert (got.float()[-40:] - ref).abs().max() <= 1e-2 * ref.abs().max()


@pytest.mark.parametrize("window", [0, 400])
def test_block_table_longer_than_one_window_and_a_far_key(window):
    """285 pages of 8 tokens: the kernel stages block-table entries 256 at a time, so this request needs two
    windows.  One key near the start (position 21, in the first window) and one just past the window's seam
    (position 2050) are made to stand out for the last tokens: a page taken from the wrong window, or a
    reference exponent moved at the wrong time, shows in those rows."""
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 8, 2, 64, 8
    reqs = [(2200, 80), (0, 40)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=11)
    table = group.block_table
    for pos, gain in ((21, 3.0), (2050, 2.0)):
        page, slot = int(table[0, pos // ps]), pos % ps
        for kvh in range(nkv):
            # head kvh * 4 of the last 8 tokens looks straight at this key
            direction = q[72:80, kvh * 4 * hd:(kvh * 4 + 1) * hd].float().mean(dim=0)
            cache[page, 0, kvh, slot] = (gain * direction / direction.norm() * hd ** 0.5).to(torch.bfloat16)
    ref = R.paged_attention_ref(q, cache, table, tok_req, positions, nh, nkv, hd, ps, window)
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, window=window)
    k.check_kernel_status()
    assert n == -(-80 * 4 // 128) + -(-40 * 4 // 128)
    err = (got.float() - ref).abs().amax(dim=1)
    bad = torch.nonzero(~(err <= 1e-2 * ref.abs().max()))
    assert len(bad) == 0, f"first wrong token {int(bad[0])} (request {int(tok_req[bad[0]])}, position {int(positions[bad[0]])})"
