"""The host side of the prompt attention's key shares (kernels.attention_plan_tc), without a GPU: which tiles are cut,
into how many shares, and that the lists the kernels read agree with each other."""
from types import SimpleNamespace

import pytest
import torch

from forge_b200 import kernels


@pytest.fixture()
def on_cpu(monkeypatch):
    monkeypatch.setattr(kernels, "_sm_count", lambda device: 148)
    monkeypatch.setattr(kernels, "new_ints", lambda values, device: torch.tensor(values, dtype=torch.int32))
    monkeypatch.setattr(kernels, "new_tensor", lambda shape, dtype, device, whole_step=False: torch.empty(tuple(shape), dtype=dtype))


def plan_of(reqs, group, n_kv_heads, head_dim, window=0, shares=None):
    q_start = [0]
    for _, q in reqs:
        q_start.append(q_start[-1] + q)
    batch = SimpleNamespace(num_requests=len(reqs), host_q_start=q_start, host_context_before=[c for c, _ in reqs],
                            attention_plan={})
    return kernels.attention_plan_tc(batch, group, "cpu", n_kv_heads, head_dim, window, shares)


def entries_of(plan):
    cut = plan["tile_cut"].view(-1, 3).tolist() if plan["tile_cut"] is not None else [[0, 1, 0]] * plan["num_tiles"]
    return list(zip(plan["tile_req"].tolist(), plan["tile_row0"].tolist(), cut))


def check_consistent(plan, n_kv_heads, head_dim):
    """Every tile's shares 0..z-1 are listed once each, point at z consecutive slots of their own, and the list of
    tiles to add up names exactly the cut tiles."""
    by_tile = {}
    for req, row0, (share, shares, slot) in entries_of(plan):
        by_tile.setdefault((req, row0), []).append((share, shares, slot))
    merges = {} if plan["merge_list"] is None else {(r, r0): (s0, z) for r, r0, s0, z in plan["merge_list"].view(-1, 4).tolist()}
    used = set()
    for key, parts in by_tile.items():
        z = parts[0][1]
        assert sorted(p[0] for p in parts) == list(range(z)) and all(p[1] == z for p in parts)
        if z == 1:
            assert key not in merges
            continue
        assert 2 <= z <= kernels.TC_MAX_SHARES
        slot0 = parts[0][2]
        assert all(p[2] == slot0 for p in parts) and merges[key] == (slot0, z)
        slots = set(range(slot0, slot0 + z))
        assert not (slots & used)
        used |= slots
    assert len(merges) == plan["num_merge"] == sum(1 for parts in by_tile.values() if parts[0][1] > 1)
    if used:
        assert max(used) + 1 == len(used)          # the slots are packed
        assert plan["part_o"].numel() == len(used) * n_kv_heads * kernels.TC_ROWS * head_dim
        assert plan["part_ml"].numel() == len(used) * n_kv_heads * kernels.TC_ROWS * 2


def test_a_whole_prompt_is_left_alone(on_cpu):
    plan = plan_of([(0, 2048)], 8, 4, 64)
    assert plan["num_tiles"] == 128 and plan["num_merge"] == 0 and plan["tile_cut"] is None


@pytest.mark.parametrize("reqs,group,nkv,hd", [([(20000, 512)], 8, 4, 64), ([(20000, 256)], 8, 4, 64), ([(8000, 64)], 8, 4, 64),
                                               ([(8000, 200), (100, 1), (3000, 1)], 8, 4, 64), ([(8000, 128)], 7, 4, 128),
                                               ([(5000, 64), (0, 70)], 4, 2, 64)])
def test_short_portions_on_long_contexts_are_cut_to_fill_the_places(on_cpu, reqs, group, nkv, hd):
    plan = plan_of(reqs, group, nkv, hd)
    places = 148 * (2 if hd <= 64 else 1)
    assert plan["num_merge"] > 0
    assert plan["num_tiles"] * nkv <= places, "the shares must not need a second wave of CTAs"
    uncut = plan_of(reqs, group, nkv, hd, shares=1)
    assert plan["num_tiles"] > uncut["num_tiles"]
    check_consistent(plan, nkv, hd)
    # longest first: a share's work never grows along the list
    work = {}
    for req, row0, (share, shares, slot) in entries_of(plan):
        ctx, q = reqs[req]
        tile_rows = (kernels.TC_ROWS // group) * group
        kv_hi = ctx + (min(q * group, row0 + tile_rows) - 1) // group + 1
        work[(req, row0, share)] = -(-kv_hi // kernels.KV_TILE) / shares
    listed = [work[(r, r0, c[0])] for r, r0, c in entries_of(plan)]
    assert listed == sorted(listed, reverse=True)


def test_short_contexts_are_not_cut(on_cpu):
    # 128 new tokens on 300 cached: 7 key tiles a tile at most, fewer than a share holds at least
    plan = plan_of([(300, 128)], 8, 4, 64)
    assert plan["num_merge"] == 0


def test_more_than_half_of_the_places_taken_is_left_alone(on_cpu):
    plan = plan_of([(20000, 512)], 7, 4, 128)          # 29 tiles x 4 kv heads = 116 of 148 places
    assert plan["num_merge"] == 0 and plan["num_tiles"] == 29


@pytest.mark.parametrize("shares", [2, 5, 32, 100])
def test_forced_shares_never_exceed_a_tiles_key_tiles(on_cpu, shares):
    reqs = [(63, 65), (500, 16), (0, 300)]
    plan = plan_of(reqs, 4, 2, 64, shares=shares)
    check_consistent(plan, 2, 64)
    for req, row0, (share, z, slot) in entries_of(plan):
        ctx, q = reqs[req]
        kv_hi = ctx + (min(q * 4, row0 + 128) - 1) // 4 + 1
        assert z <= min(shares, -(-kv_hi // kernels.KV_TILE), kernels.TC_MAX_SHARES)


def test_the_window_shortens_what_a_tile_is_worth(on_cpu):
    # with a window of 256 keys a tile on a long context has 5 key tiles: nothing to share out
    assert plan_of([(20000, 64)], 8, 4, 64, window=256)["num_merge"] == 0
    assert plan_of([(20000, 64)], 8, 4, 64)["num_merge"] > 0
