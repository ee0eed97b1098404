"""Host-side logic that needs no GPU: how the skinny-M kernels split K, and the descriptor
bit fields the kernels are launched with (compiled from the library's own headers with g++)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "blaze_b200", "csrc")

PROGRAM = r'''
#include <cstdio>
#include <initializer_list>
#include "decode_split.h"
int main() {
    // every (tiles, stages, max_split, forced) combination of interest: print the split
    const int sms = 148;
    for (int n_tiles : {1, 2, 8, 32, 33, 86, 96, 148, 172, 1024})
        for (int k_stages : {1, 2, 3, 5, 16, 17, 32, 43, 86, 344})
            for (int max_split : {1, 2, 4, 8})
                for (int forced : {0, 1, 2, 3, 8})
                    std::printf("%d %d %d %d %d\n", n_tiles, k_stages, max_split, forced,
                                blz::decode_pick_split(n_tiles, k_stages, sms, max_split, forced));
    // tiles per CTA of the W4A16 kernel: (tiles, instruction N, split, forced)
    for (int n_tiles : {96, 148, 149, 172, 300, 1000})
        for (int mma_n : {16, 32})
            for (int split : {1, 2})
                for (int forced : {0, 1, 2, 5})
                    std::printf("tiles %d %d %d %d %d\n", n_tiles, mma_n, split, forced, blz::decode_tiles_per_cta(n_tiles, sms, mma_n, split, forced));
    std::printf("max %d %d %d %d\n", blz::decode_max_split(16), blz::decode_max_split(32), blz::decode_max_split(64), blz::decode_max_split(128));
    return 0;
}
'''


@pytest.fixture(scope="module")
def split_table(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    d = tmp_path_factory.mktemp("split")
    src = d / "split.cpp"
    src.write_text(PROGRAM)
    exe = d / "split"
    subprocess.run([gxx, "-std=c++17", "-O1", "-I", CSRC, "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines()
    rows = [tuple(int(x) for x in l.split()) for l in out if not l.startswith(("max", "tiles"))]
    limits = [int(x) for x in out[-1].split()[1:]]
    tiles = {tuple(int(x) for x in l.split()[1:5]): int(l.split()[5]) for l in out if l.startswith("tiles")}
    return rows, limits, tiles


def test_split_is_a_power_of_two_within_limits(split_table):
    rows, _, _ = split_table
    for n_tiles, k_stages, max_split, forced, s in rows:
        assert s >= 1 and s & (s - 1) == 0, (n_tiles, k_stages, max_split, forced, s)
        assert s <= max_split
        if forced > 0:
            assert s <= forced


def test_no_split_is_empty_and_every_split_has_two_stages(split_table):
    rows, _, _ = split_table
    for n_tiles, k_stages, max_split, forced, s in rows:
        per = -(-k_stages // s)
        assert (s - 1) * per < k_stages, "an empty split would leave a CTA of the cluster without work"
        if s > 1:
            assert k_stages // s >= 2


def test_split_fills_the_device_when_tiles_are_few(split_table):
    rows, _, _ = split_table
    table = {(a, b, c, d): s for a, b, c, d, s in rows}
    assert table[(96, 16, 8, 0)] == 1          # 96 tiles: 0.65 CTAs per SM is enough
    assert table[(32, 16, 8, 0)] == 4          # 32 tiles of 16 stages: 128 CTAs
    assert table[(32, 43, 8, 0)] == 4
    assert table[(172, 16, 8, 0)] == 1
    assert table[(1, 344, 8, 0)] == 8
    assert table[(1, 1, 8, 0)] == 1


def test_max_split_by_activation_tile(split_table):
    _, limits, _ = split_table
    assert limits == [8, 4, 2, 2]


def test_tiles_per_cta_of_the_w4a16_kernel(split_table):
    _, _, TILES = split_table
    assert TILES[(96, 16, 1, 0)] == 1 and TILES[(148, 16, 1, 0)] == 1      # one wave: one tile per CTA
    assert TILES[(149, 16, 1, 0)] == 2 and TILES[(172, 16, 1, 0)] == 2    # beyond one wave: two (86 CTAs for 172 tiles)
    assert TILES[(1000, 16, 1, 0)] == 2                                   # never more than the accumulator columns hold
    assert TILES[(172, 32, 1, 0)] == 1                                    # instruction N 32: one tile
    assert TILES[(172, 16, 2, 0)] == 1                                    # not combined with a K split by itself
    assert TILES[(96, 16, 2, 2)] == 2 and TILES[(96, 16, 1, 5)] == 2 and TILES[(96, 32, 1, 5)] == 1   # forced, clamped
