"""The index predicates of the checks build (csrc/checks.cuh), on the CPU: they are plain functions of integers,
compiled here as host code, and are given the bad page ids and slots that no GPU is ever given."""
import ctypes
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = r'''
#include "checks.cuh"
extern "C" int page_in_pool(long long page, long long num_pages) { return forge::page_in_pool(page, num_pages); }
extern "C" int slot_in_pool(long long slot, long long num_pages, long long page_size) { return forge::slot_in_pool(slot, num_pages, page_size); }
extern "C" int token_in_step(long long t, long long n) { return forge::token_in_step(t, n); }
'''


@pytest.fixture(scope="module")
def predicates(tmp_path_factory):
    d = tmp_path_factory.mktemp("checks")
    src, so = d / "shim.cpp", d / "shim.so"
    src.write_text(SHIM)
    subprocess.check_call(["g++", "-std=c++17", "-shared", "-fPIC", "-I", os.path.join(ROOT, "forge_b200", "csrc"), str(src), "-o", str(so)])
    lib = ctypes.CDLL(str(so))
    for f in (lib.page_in_pool, lib.slot_in_pool, lib.token_in_step):
        f.argtypes = [ctypes.c_longlong] * (3 if f is lib.slot_in_pool else 2)
        f.restype = ctypes.c_int
    return lib


def test_page_ids(predicates):
    ok = predicates.page_in_pool
    assert ok(0, 10) and ok(9, 10)
    assert not ok(10, 10) and not ok(-1, 10) and not ok(2 ** 31, 10) and not ok(-2 ** 31, 10) and not ok(0, 0)


def test_slots(predicates):
    ok = predicates.slot_in_pool
    assert ok(0, 4, 16) and ok(63, 4, 16)
    assert not ok(64, 4, 16) and not ok(-1, 4, 16) and not ok(5, 0, 16) and not ok(5, 4, 0)
    assert ok(2 ** 33, 2 ** 30, 16) and not ok(2 ** 34, 2 ** 30, 16)          # no wrap in 32 bits


def test_token_indices(predicates):
    ok = predicates.token_in_step
    assert ok(0, 1) and ok(2047, 2048) and not ok(2048, 2048) and not ok(-1, 2048) and not ok(0, 0)
