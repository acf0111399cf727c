"""The work list of the two-block tiling of the grouped GEMMs, enumerated on the host by the same
code the kernel's scheduler runs (``b200moe_gemm_two_block_schedule``): no GPU needed.

Checked for many block distributions: every (M block, N tile) pair of every expert is processed
exactly once; an item never crosses an expert boundary; the busiest CTA stays within a few units of
the ideal share (every tile costs two units, so the round-robin deal keeps the CTAs in step)."""
import random

import numpy as np
import pytest

from electrock_infer_b200 import _lib


def schedule(blocks, n_tiles, m_group, grid, slots):
    lib = _lib.load()
    b = np.asarray(blocks, dtype=np.int32)
    per_cta = []
    for cta in range(grid):
        n = lib.b200moe_gemm_two_block_schedule(b.ctypes.data, len(blocks), n_tiles, m_group, slots, grid, cta,
                                                None, 0)
        assert n >= 0
        buf = np.zeros((max(n, 1), 4), dtype=np.int32)
        m = lib.b200moe_gemm_two_block_schedule(b.ctypes.data, len(blocks), n_tiles, m_group, slots, grid,
                                                cta, buf.ctypes.data, n)
        assert m == n
        per_cta.append(buf[:n])
    return per_cta


def check(blocks, n_tiles, m_group, grid, slots=1):
    per_cta = schedule(blocks, n_tiles, m_group, grid, slots)
    off = np.concatenate([[0], np.cumsum(blocks)])
    seen = np.zeros((off[-1], n_tiles), dtype=np.int32)
    costs = []
    for items in per_cta:
        cost = 0
        for e, m, n, k in items:
            assert k in (1, 2) and 0 <= n < n_tiles
            for j in range(k):
                assert off[e] <= m + j < off[e + 1], "an item crosses an expert boundary"
                seen[m + j, n] += 1
            cost += k
        costs.append(cost)
    assert (seen == 1).all(), "every (M block, N tile) exactly once"
    ideal = -(-int(off[-1]) * n_tiles // grid)
    return max(costs), ideal


def test_every_block_and_tile_exactly_once_random_shapes():
    rng = random.Random(1)
    for _ in range(150):
        experts = rng.choice([1, 2, 3, 8])
        blocks = [rng.choice([0, 0, 1, 2, 3, 5, 8, 13, 29, 50]) for _ in range(experts)]
        if sum(blocks) == 0:
            continue
        slots = rng.choice([0, 1])
        busiest, ideal = check(blocks, rng.choice([1, 2, 3, 7, 16, 112]), rng.choice([0, 4, 10, 40]),
                               rng.choice([1, 2, 7, 148]), slots)
        if slots:  # every tile costs two units: the deal is balanced
            assert busiest <= ideal + 3


@pytest.mark.parametrize("blocks,n_tiles,m_group", [
    ([50, 29, 20, 12, 11, 6, 3, 1], 112, 40),   # first GEMM, T=8192 with the skewed routing
    ([50, 29, 20, 12, 11, 6, 3, 1], 16, 10),    # second GEMM, same batch
    ([13, 8, 5, 3, 3, 2, 1, 1], 112, 40),       # T=2048
    ([33] * 8, 112, 40),                        # T=16384, near-uniform
    ([33], 16, 10),                             # one expert per rank (expert parallel over 8)
])
def test_mixtral_shapes_reach_the_ideal_share(blocks, n_tiles, m_group):
    busiest, ideal = check(blocks, n_tiles, m_group, 148, slots=1)
    assert busiest == ideal
    check(blocks, n_tiles, m_group, 148, slots=0)  # coverage only: one-block tiles cost half


def test_bad_arguments_are_refused():
    lib = _lib.load()
    b = np.asarray([1, -2], dtype=np.int32)
    assert lib.b200moe_gemm_two_block_schedule(b.ctypes.data, 2, 4, 0, 1, 148, 0, None, 0) < 0
    assert lib.b200moe_gemm_two_block_schedule(None, 2, 4, 0, 1, 148, 0, None, 0) < 0
    assert lib.b200moe_gemm_two_block_schedule(b.ctypes.data, 2, 4, 0, 0, 148, 148, None, 0) < 0
