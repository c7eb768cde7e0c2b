"""forge_paged_attention_mma_static, the attention entry point that allocates nothing, called through its
exported C symbol the way a foreign runtime would call it: with raw device pointers it owns and a stream.
Its scratch is an array inside the library, so the test checks it against the ordinary entry point (which
gets its scratch from the caller) on two calls in a row, the second of which finds the array dirty with
the first call's partial results and works on different inputs.  Collected last on purpose: if it fails,
a run that stops at the first failure has already run everything else."""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from test_attention_mma_gpu import make_case

pytestmark = pytest.mark.gpu


def _static_entry(head_dim):
    from forge_b200.kernels.build import build_library
    lib = ctypes.CDLL(build_library("attention_mma", defines={"FORGE_ATT_HD": head_dim}))
    fn = lib.forge_paged_attention_mma_static
    fn.argtypes = [c_void_p] * 8 + [c_int] * 9 + [c_float, c_void_p]
    fn.restype = c_int
    lib.forge_last_error.restype = ctypes.c_char_p
    return lib, fn


def _call(fn, lib, q, cache, group, batch, plan, nh, nkv, hd, ps, splits):
    out = torch.full_like(q, float("nan"))
    rc = fn(q.data_ptr(), cache.data_ptr(), out.data_ptr(), group.block_table.data_ptr(), plan["tile_req"].data_ptr(),
            plan["tile_row0"].data_ptr(), batch.q_start.data_ptr(), batch.context_before.data_ptr(), plan["num_tiles"],
            plan["max_rows"], nh, nkv, hd, ps, group.block_table.shape[1], 0, splits, hd ** -0.5,
            torch.cuda.current_stream().cuda_stream)
    return rc, out, lib.forge_last_error().decode()


def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row():
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 32, 4, 64, 16
    lib, fn = _static_entry(hd)
    for call, (reqs, splits, seed) in enumerate([([(300, 1), (64, 1), (1000, 1), (5, 1)], 8, 1),
                                                 ([(17, 1), (511, 1), (130, 1)], 3, 2)]):
        q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=seed)
        plan = k.attention_plan(batch, nh // nkv, q.device)
        want = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps, num_splits=splits)
        rc, got, msg = _call(fn, lib, q, cache, group, batch, plan, nh, nkv, hd, ps, splits)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any(), f"call {call}: some rows were never written"
        # the same kernels on the same inputs: the tolerance of the attention tests, 1e-2 of the scale
        assert (got.float() - want.float()).abs().max() <= 1e-2 * want.float().abs().max(), f"call {call}"


def test_static_scratch_entry_refuses_what_does_not_fit():
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 32, 4, 64, 16
    lib, fn = _static_entry(hd)
    q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, [(40, 1)] * 64, seed=3)
    plan = k.attention_plan(batch, nh // nkv, q.device)
    rc, _, msg = _call(fn, lib, q, cache, group, batch, plan, nh, nkv, hd, ps, 2000)   # 64*4*2000*16*66 floats
    assert rc != 0 and "scratch floats needed" in msg and "holds" in msg
    # sizes whose product would wrap round 64 bits must not slip under the limit either (nothing is launched:
    # the refusal comes before any pointer is looked at)
    rc = fn(None, None, None, None, None, None, None, None, 2 ** 28, 16, nh, 2 ** 15, hd, ps, 4, 0, 2 ** 15, 0.125, None)
    assert rc != 0


def test_static_scratch_entry_with_prompt_portions():
    """Requests that bring many rows (the four-warp layout of the scratch, 64 rows a tile) with their keys cut
    into slices; and a long prompt in one slice, which needs no scratch at all and must not be refused for a
    size it does not use."""
    from forge_b200 import kernels as k
    nh, nkv, hd, ps = 32, 4, 64, 16
    lib, fn = _static_entry(hd)
    for reqs, splits in (([(200, 9), (40, 3), (0, 7)], 3), ([(0, 2048)], 1), ([(100, 24), (700, 1)], 2)):
        q, cache, group, batch, tok_req, positions = make_case(nh, nkv, hd, ps, reqs, seed=5)
        plan = k.attention_plan(batch, nh // nkv, q.device)
        assert plan["max_rows"] > 16
        want = k.paged_attention_mma(q, cache, group, batch, nh, nkv, hd, ps, num_splits=splits)
        rc, got, msg = _call(fn, lib, q, cache, group, batch, plan, nh, nkv, hd, ps, splits)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        assert (got.float() - want.float()).abs().max() <= 1e-2 * want.float().abs().max(), (reqs, splits)
