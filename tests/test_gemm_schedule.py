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


def choice(blocks, n_tiles, k, slots, ctas=148):
    b = np.asarray(blocks, dtype=np.int32)
    return _lib.load().b200moe_gemm_two_block_choice(b.ctypes.data, len(blocks), n_tiles, k, slots, ctas)


# Block counts per expert of the skewed benchmark routing (mixtral_prefill_t8192_skew cut to T
# tokens) and of near-uniform routing, with what interleaved runs on a B200 measured as the faster
# tiling of each grouped GEMM (1 = two M blocks per tile).  Sizes where the two tilings measured
# within run-to-run noise are left out.
MEASURED = [
    ("skew T=2048", [13, 8, 5, 3, 3, 2, 1, 1], 0, 0),
    ("skew T=3072", [19, 11, 8, 5, 5, 3, 2, 1], 0, 0),
    ("skew T=4096", [25, 15, 10, 6, 6, 3, 2, 1], None, 1),
    ("skew T=6144", [37, 22, 15, 8, 9, 5, 3, 1], None, 1),
    ("skew T=8192", [50, 29, 20, 12, 11, 6, 3, 1], 1, 1),
    ("uniform T=2048", [5, 4, 4, 5, 4, 4, 5, 4], None, 0),
    ("uniform T=3072", [7, 6, 7, 6, 6, 7, 6, 7], None, 0),
    ("uniform T=16384", [33] * 8, 1, 1),
]


@pytest.mark.parametrize("name,blocks,first,second", MEASURED, ids=[m[0] for m in MEASURED])
def test_tiling_choice_follows_the_measurements(name, blocks, first, second):
    """The device-side rule (estimated finishing times of the two tilings), evaluated on the host
    for Mixtral-8x7B's two GEMMs: N tiles 14336/128 and 4096/256, K 4096 and 14336."""
    if first is not None:
        assert choice(blocks, 112, 4096, 1) == first
    if second is not None:
        assert choice(blocks, 16, 14336, 0) == second


def test_tiling_choice_edge_cases():
    assert choice([1, 1, 1, 1, 1, 1, 1, 1], 112, 4096, 1) == 0      # no pair of blocks anywhere
    assert choice([0, 0, 0, 0, 0, 0, 0, 0], 16, 14336, 0) == 0
    assert choice([33] * 8, 16, 1792, 0) == 0                        # short K: never two-block tiles
    assert choice([33], 16, 14336, 0) == 1                           # one expert per rank (eight GPUs)
    assert choice([33], 16, 14336, 0, ctas=0) < 0 and choice([-1], 16, 14336, 0) < 0
