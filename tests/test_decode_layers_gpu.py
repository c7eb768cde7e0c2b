"""The persistent kernel that runs all layers of a decode step, alone, against plain functions: several layers,
widths that are no powers of two, groups of 1 to 8 query heads, q/k/v bias, a window, contexts on and around page
and tile edges, 1 to 16 tokens; and its grid barrier's time limit."""
import math

import pytest
import torch

from plain import kernels_ref as R
from plain import llama as P
from test_attention_mma_gpu import make_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layers(n_layers, H, I, nh, nkv, hd, bias, seed):
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s, scale: (torch.randn(*s, generator=g) * scale)
    out = []
    for _ in range(n_layers):
        out.append(dict(wq=rnd((nh + 2 * nkv) * hd, H, scale=H ** -0.5).to(torch.bfloat16),
                        wo=rnd(H, nh * hd, scale=0.5 * (nh * hd) ** -0.5).to(torch.bfloat16),
                        wg=rnd(I, H, scale=H ** -0.5).to(torch.bfloat16), wu=rnd(I, H, scale=H ** -0.5).to(torch.bfloat16),
                        wd=rnd(H, I, scale=0.5 * I ** -0.5).to(torch.bfloat16),
                        n1=1.0 + rnd(H, scale=0.1), n2=1.0 + rnd(H, scale=0.1),
                        b=rnd((nh + 2 * nkv) * hd, scale=0.3) if bias else None))
    return out


def _plain_layers(layers, resid, caches, table, positions, slots, nh, nkv, hd, ps, theta, eps, window):
    """float64 on the CPU, with the one rounding that the cache imposes (keys and values are stored in bfloat16)."""
    x = resid.double()
    S = x.shape[0]
    tok_req = torch.arange(S, dtype=torch.int32)
    new_caches = []
    for L, cache in zip(layers, caches):
        y = P.rms_norm(x, L["n1"].double(), eps)
        qkv = P.linear(y, L["wq"].double(), None if L["b"] is None else L["b"].double())
        q, cache2 = R.rope_kv_write_ref(qkv, positions, slots, cache, nh, nkv, hd, ps, theta, True)
        cache2 = cache2.to(torch.bfloat16)
        new_caches.append(cache2)
        a = R.paged_attention_ref(q, cache2, table, tok_req, positions, nh, nkv, hd, ps, window).double()
        x = x + P.linear(a.reshape(S, nh * hd), L["wo"].double())
        x = x + P.swiglu(P.rms_norm(x, L["n2"].double(), eps), L["wg"].double(), L["wu"].double(), L["wd"].double())
    return x, new_caches


@pytest.mark.parametrize("H,I,nh,nkv,hd,bias,window", [
    (256, 320, 4, 2, 64, False, 0),         # small: a CTA gets less than one unit of some matrices
    (2048, 5632, 32, 4, 64, False, 0),      # the benchmark's widths
    (192, 448, 6, 2, 32, True, 0),          # group of 3, bias, widths that are multiples of 64 only
    (512, 1408, 8, 1, 64, True, 70),        # one kv head (group of 8), a window
    (1024, 1536, 8, 2, 128, False, 0),      # head size 128
])
def test_all_layers_of_a_decode_step(H, I, nh, nkv, hd, bias, window):
    from forge_b200 import kernels as k
    ps, theta, eps, n_layers = 16, 30000.0, 1e-3, 3
    assert k.DecodeLayers.supports(H, I, nh, nkv, hd)
    layers = _layers(n_layers, H, I, nh, nkv, hd, bias, seed=H)
    # 10 requests (keys of a request shared by several CTAs), one, 16 (the most), and three with many tiles a warp
    for ctxs in ([0, 15, 16, 31, 32, 33, 63, 64, 300, 700], [0], [5] * 9 + [129] + [64] * 6, [1500, 1, 2100]):
        reqs = [(c, 1) for c in ctxs]
        S = len(reqs)
        _, cache0, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=S)
        caches = [(cache0.float().cpu() * (0.5 + 0.25 * i)).to(torch.bfloat16) for i in range(n_layers)]
        slots = torch.tensor([int(group.block_table[s, c // ps]) * ps + c % ps for s, c in enumerate(ctxs)], dtype=torch.int32)
        resid = torch.randn(S, H, generator=torch.Generator().manual_seed(3)) * 1.3
        want, want_caches = _plain_layers(layers, resid, caches, group.block_table.cpu(), positions.cpu(), slots, nh, nkv, hd, ps,
                                          theta, eps, window)
        dev_caches = [c.to(DEV) for c in caches]
        dev_layers = [dict(wqkv=L["wq"].to(DEV), wo=L["wo"].to(DEV),
                           wgu=torch.stack([L["wg"], L["wu"]], dim=1).reshape(2 * I, H).contiguous().to(DEV), wdown=L["wd"].to(DEV),
                           norm1=L["n1"].float().to(DEV), norm2=L["n2"].float().to(DEV),
                           bias=None if L["b"] is None else L["b"].float().to(DEV), kv=c) for L, c in zip(layers, dev_caches)]
        dl = k.DecodeLayers(dev_layers, H, I, nh, nkv, hd, ps, theta, True, eps, window=window)
        for rep in range(2):                    # the second run finds the scratch as the first left it
            for c, c0 in zip(dev_caches, caches):
                c.copy_(c0)
            got = resid.clone().to(DEV)
            dl.run(got, group.block_table, positions, slots.to(DEV))
            torch.cuda.synchronize()
            k.check_kernel_status(DEV)
            assert dl.barrier.tolist() == [0, 0, 0, 0]
            err = (got.double().cpu() - want).abs().max() / want.abs().max()
            assert err <= 2e-2, (ctxs[:4], rep, float(err))
            for c, cw in zip(dev_caches, want_caches):      # keys and values landed in their slots
                assert (c.float().cpu() - cw.float()).abs().max() <= 2e-2 * cw.float().abs().max()


def test_sizes_it_does_not_take_are_refused():
    from forge_b200 import kernels as k
    assert not k.DecodeLayers.supports(96, 256, 3, 1, 32)        # a width that is not a multiple of 64
    assert not k.DecodeLayers.supports(2048, 5632, 34, 2, 64)    # 17 query heads per kv head
    assert not k.DecodeLayers.supports(2048, 5632, 32, 4, 64, tokens=17)


def test_grid_barrier_gives_up_after_its_time_limit():
    """One CTA arrives at a barrier that expects two arrivals and nothing ever brings the second: after the limit
    (here 2 ms) the kernel must raise its status bits and return, leaving the device usable."""
    from forge_b200 import kernels as k
    lib = k.library("decode_layers", {"FORGE_ATT_HD": 64})
    barrier = torch.zeros(4, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0[0].record()
    rc = lib.forge_decode_layers_barrier_probe(barrier.data_ptr(), status.data_ptr(), 2_000_000, torch.cuda.current_stream().cuda_stream)
    t0[1].record()
    assert rc == 0
    torch.cuda.synchronize()
    assert 1.5 <= t0[0].elapsed_time(t0[1]) <= 500
    s = int(status.item())
    assert s & 2 and s & (1 << 20)
    assert barrier.tolist()[:2] == [1, 1]            # one arrival, and the word that tells other CTAs to leave
    assert torch.ones(4, device=DEV).sum().item() == 4.0


@pytest.mark.parametrize("page_size", [16, 64])
def test_whole_model_with_all_layers_in_one_kernel(page_size, tmp_path_factory):
    """The engine with the persistent kernel switched on (it is off by default): a model of head size 64 whose last
    tokens are decoded one by one, alone and four requests at a time, through the CUDA graph, against the plain
    implementation at every position."""
    import schedules
    from helpers import TINY, TOL, make_model_dir, random_tokens
    from plain.llama import PlainLlama
    from test_engine_gpu import first_bad, run_schedule
    from forge_b200.engine import ModelRunner
    d = make_model_dir(tmp_path_factory, "C")
    plain = PlainLlama(d)
    reqs = {f"r{i}": random_tokens(n, TINY["C"]["vocab_size"], seed=60 + i) for i, n in enumerate([150, 40, 300, 77, 64])}
    want = {rid: plain.logits(t).float() for rid, t in reqs.items()}
    for steps in (schedules.last_one_by_one(reqs), schedules.mixed(reqs, max_live=4, decode_tail=20)):
        runner = ModelRunner(d, dtype="bfloat16", page_size=page_size, cache_tokens=schedules.peak_tokens(reqs, steps, round_to=page_size),
                             max_requests=4, fused_decode=True)
        assert runner.fused_decode
        got = run_schedule(runner, reqs, steps)
        msg = first_bad(got, want, TOL["bfloat16"])
        assert msg is None, msg
