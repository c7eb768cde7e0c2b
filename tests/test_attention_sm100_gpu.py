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
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, shares=1)
    k.check_kernel_status()
    assert n == -(-1100 * 8 // 128)
    # the same with head size 128 and 7 query heads per kv head
    nh, nkv, hd, ps = 14, 2, 128, 32
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, [(0, 700)], seed=8)
    ref = R.paged_attention_ref(q[-40:], cache, group.block_table, tok_req[-40:], positions[-40:], nh, nkv, hd, ps)
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, shares=1)
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
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, window=window, shares=1)
    k.check_kernel_status()
    assert n == -(-80 * 4 // 128) + -(-40 * 4 // 128)
    err = (got.float() - ref).abs().amax(dim=1)
    bad = torch.nonzero(~(err <= 1e-2 * ref.abs().max()))
    assert len(bad) == 0, f"first wrong token {int(bad[0])} (request {int(tok_req[bad[0]])}, position {int(positions[bad[0]])})"


CUT_SHAPES = [(32, 4, 64, 16), (28, 4, 128, 64), (6, 2, 64, 16), (16, 1, 64, 8), (8, 2, 128, 32)]


@pytest.mark.parametrize("nh,nkv,hd,ps", CUT_SHAPES)
@pytest.mark.parametrize("shares", [2, 3, 7, 32])
@pytest.mark.parametrize("window", [0, 70])
def test_keys_cut_into_shares(nh, nkv, hd, ps, shares, window):
    """Every tile's keys cut into (up to) ``shares`` parts, each by a CTA of its own, added up by the second kernel.
    The portions include rows that see no key of a share (positions 63.. with the second share starting at key 64,
    shares wholly outside the window): those shares must count as nothing."""
    from forge_b200 import kernels as k
    reqs = PORTIONS + [(1500, 40), (1000, 130)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=3)
    ref = R.paged_attention_ref(q, cache, group.block_table, tok_req, positions, nh, nkv, hd, ps, window)
    out = torch.full_like(q, float("nan"))
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, window=window, out=out, shares=shares)
    k.check_kernel_status()
    plain_out, n1 = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, window=window, shares=1)
    assert n > n1 > 0
    big = _rows_of_big(reqs, nh // nkv, k.TC_MIN_ROWS).to(q.device)
    err = (got.float()[big] - ref[big]).abs().amax(dim=1)
    bad = torch.nonzero(~(err <= 1e-2 * ref.abs().max()))
    assert len(bad) == 0, f"first wrong token {int(big[bad[0]])} (request {int(tok_req[big[bad[0]]])}, position {int(positions[big[bad[0]]])})"
    # and the same as the uncut kernel up to the rounding of the last bfloat16 bit
    assert (got.float()[big] - plain_out.float()[big]).abs().max() <= 2e-2 * ref.abs().max()


@pytest.mark.parametrize("shares", [4, None])
def test_a_far_key_in_another_share(shares):
    """A short portion on a long context with one early key that stands out: it lies in the first share, the rows'
    own neighbourhood in the last; a share dropped or weighted wrongly in the sum shows at once.  ``None``: the
    plan's own choice, which cuts such a step by itself (4 tiles x 2 kv heads for some hundred places)."""
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 8, 2, 64, 16
    reqs = [(5000, 64), (0, 70)]
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=13)
    table = group.block_table
    for pos, gain in ((21, 3.0), (2600, 2.0)):
        page, slot = int(table[0, pos // ps]), pos % ps
        for kvh in range(nkv):
            direction = q[56:64, kvh * 4 * hd:(kvh * 4 + 1) * hd].float().mean(dim=0)
            cache[page, 0, kvh, slot] = (gain * direction / direction.norm() * hd ** 0.5).to(torch.bfloat16)
    ref = R.paged_attention_ref(q, cache, table, tok_req, positions, nh, nkv, hd, ps, 0)
    got, n = k.paged_attention_sm100(q, cache, group, batch, nh, nkv, hd, ps, shares=shares)
    k.check_kernel_status()
    tiles = -(-64 * 4 // 128) + -(-70 * 4 // 128)
    if shares is None:
        assert n > tiles, "the plan was meant to cut the long request's keys"
        assert n * nkv <= 2 * torch.cuda.get_device_properties(0).multi_processor_count
    else:
        assert n == 2 * shares + 1 + 1 + 2       # the short request's three tiles have 1, 1 and 2 key tiles
    err = (got.float() - ref).abs().amax(dim=1)
    bad = torch.nonzero(~(err <= 1e-2 * ref.abs().max()))
    assert len(bad) == 0, f"first wrong token {int(bad[0])} (request {int(tok_req[bad[0]])}, position {int(positions[bad[0]])})"
