"""The tile geometry of csrc/geometry.h against a brute-force mask (CPU, the header compiled with g++).

For a set of (seqlen_q, seqlen_k, causal, window) cases, both tile walks -- query tiles per key tile
(five-GEMM kernel) and key tiles per query tile (dQ kernel) -- must cover every visible pair, tiles
reported as mask-free must be fully visible, and the per-row ranges used for masking in registers
must reproduce oracle.golden.band_mask element by element."""
import ctypes
import subprocess

import numpy as np
import pytest

from oracle.golden import band_mask
from tests.conftest import ROOT

SRC = r'''
#include "geometry.h"
using namespace fa3b200;
extern "C" {
int g_first_q(int kt, int sq, int sk, int c, int wl, int wr) { return first_q_tile(kt, make_band(sq, sk, c, wl, wr)); }
int g_last_q(int kt, int sq, int sk, int c, int wl, int wr) { return last_q_tile(kt, make_band(sq, sk, c, wl, wr)); }
int g_first_k(int qt, int sq, int sk, int c, int wl, int wr) { return first_k_tile(qt, make_band(sq, sk, c, wl, wr)); }
int g_last_k(int qt, int sq, int sk, int c, int wl, int wr) { return last_k_tile(qt, make_band(sq, sk, c, wl, wr)); }
int g_needs_mask(int kt, int qt, int sq, int sk, int c, int wl, int wr) {
    return tile_needs_mask(kt, qt, make_band(sq, sk, c, wl, wr));
}
void g_query_range(int key, int q0, int sq, int sk, int c, int wl, int wr, int* lo, int* hi) {
    query_range_of_key(key, q0, make_band(sq, sk, c, wl, wr), lo, hi);
}
void g_key_range(int query, int k0, int sq, int sk, int c, int wl, int wr, int* lo, int* hi) {
    key_range_of_query(query, k0, make_band(sq, sk, c, wl, wr), lo, hi);
}
}
'''

CASES = [
    (256, 256, True, (-1, -1)), (300, 300, True, (-1, -1)), (300, 700, True, (-1, -1)),
    (700, 300, True, (-1, -1)), (1, 384, True, (-1, -1)), (130, 1000, False, (-1, -1)),
    (777, 1000, False, (50, 300)), (900, 400, True, (64, -1)), (512, 2048, False, (5, 5)),
    (256, 1024, False, (8, 64)), (640, 640, False, (128, 128)), (1024, 1024, True, (100, -1)),
    (384, 384, True, (383, 500)), (200, 200, False, (0, 0)),
]


@pytest.fixture(scope="module")
def lib(tmp_path_factory):
    d = tmp_path_factory.mktemp("geom")
    (d / "g.cpp").write_text(SRC)
    so = d / "libgeom.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I",
                    str(ROOT / "flash_attention3_b200/csrc"), str(d / "g.cpp"), "-o", str(so)], check=True)
    return ctypes.CDLL(str(so))


@pytest.mark.parametrize("sq,sk,causal,window", CASES)
def test_tile_walks_cover_the_band_and_masks_match(lib, sq, sk, causal, window):
    args = (sq, sk, int(causal), window[0], window[1])
    masked = band_mask(sq, sk, causal, window)
    visible = np.ones((sq, sk), bool) if masked is None else ~masked
    nq, nk = (sq + 127) // 128, (sk + 127) // 128
    lo, hi = ctypes.c_int(), ctypes.c_int()
    idx = np.arange(128)

    covered = np.zeros_like(visible)
    for kt in range(nk):
        for qt in range(lib.g_first_q(kt, *args), lib.g_last_q(kt, *args) + 1):
            assert 0 <= qt < nq
            block = visible[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128]
            if not lib.g_needs_mask(kt, qt, *args):
                assert block.all() and block.shape[1] == 128
            for key in range(kt * 128, min(sk, (kt + 1) * 128)):
                lib.g_query_range(key, qt * 128, *args, ctypes.byref(lo), ctypes.byref(hi))
                keep = (idx >= lo.value) & (idx <= hi.value)
                assert np.array_equal(keep[:block.shape[0]], block[:, key - kt * 128])
            if (kt + 1) * 128 > sk:  # a key past the end of the sequence survives nowhere
                lib.g_query_range(sk, qt * 128, *args, ctypes.byref(lo), ctypes.byref(hi))
                assert not ((idx >= lo.value) & (idx <= hi.value)).any()
            covered[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128] = True
    assert not (visible & ~covered).any()

    covered[:] = False
    for qt in range(nq):
        for kt in range(lib.g_first_k(qt, *args), lib.g_last_k(qt, *args) + 1):
            assert 0 <= kt < nk
            block = visible[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128]
            for query in range(qt * 128, min(sq, (qt + 1) * 128)):
                lib.g_key_range(query, kt * 128, *args, ctypes.byref(lo), ctypes.byref(hi))
                keep = (idx >= lo.value) & (idx <= hi.value)
                assert np.array_equal(keep[:block.shape[1]], block[query - qt * 128])
                assert not keep[block.shape[1]:].any()
            covered[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128] = True
    assert not (visible & ~covered).any()
