"""Static tile order of the fused expert-parallel MoE kernels, walked on the host.

The persistent CTAs of `ep_moe_forward_kernel` / `ep_moe_backward_kernel` take tiles from a counter in this order and
start them in order; a tile only ever waits for tiles that come EARLIER in the order, which is what makes the
scheme deadlock-free. `torch.ops.b200.moe_tile_order` runs the kernels' own table-building and decoding code
compiled for the host (csrc/moe_common.cuh:build_tile_order, decode_tile; csrc/moe_kernels.cu:decode_bwd_tile), so
these checks are about the code that runs on the GPU, not a restatement of it.
"""
import collections

import pytest
import torch


def _ops():
    from jax_gpt_b200 import _ext
    try:
        return _ext.ops()
    except Exception as e:  # no compiler and no prebuilt library
        pytest.skip(f"extension unavailable: {e}")


def _order(rows, D, I, grid, backward):
    tiles, lag = _ops().moe_tile_order(torch.tensor(rows, dtype=torch.int32), D, I, grid, backward)
    return [tuple(t) for t in tiles.tolist()], lag


def _expected_forward(rows, D, I):
    exp = set()
    for el, r in enumerate(rows):
        mt = (r + 127) // 128
        exp |= {(el, 0, m, n) for m in range(mt) for n in range(I // 128)}
        exp |= {(el, 1, m, n) for m in range(mt) for n in range(D // 256)}
    return exp


def _expected_backward(rows, D, I):
    exp = set()
    for el, r in enumerate(rows):
        mt = (r + 127) // 128
        if mt == 0:
            continue      # an expert without rows has no gradient tiles at all
        exp |= {(el, 0, m, n) for m in range(mt) for n in range(I // 256)}
        exp |= {(el, 1, m, n) for m in range(mt) for n in range(D // 256)}
        exp |= {(el, 2, m, n) for m in range(I // 128) for n in range(D // 256)}
        exp |= {(el, 3, m, n) for m in range(D // 128) for n in range(2 * I // 256)}
    return exp


ROWS = [
    [640] * 64,                                   # the Qwen3.5 benchmark layer on one rank
    [1024] * 32,                                  # one rank's share of the DeepSeek-V3 layer
    [0, 0, 5, 0, 1300, 129, 0, 64, 0, 0, 0, 2],   # skewed routing, several empty experts
    [0] * 7 + [80] + [0] * 504,                   # decode: 512 local experts, almost all empty
    [1],
    [0, 0, 0],
]


@pytest.mark.parametrize("rows", ROWS)
@pytest.mark.parametrize("backward", [False, True])
def test_every_tile_once_and_dependencies_point_backwards(rows, backward):
    D, I, grid = 2048, 512, 148
    tiles, lag = _order(rows, D, I, grid, backward)
    expected = (_expected_backward if backward else _expected_forward)(rows, D, I)
    assert len(tiles) == len(expected) and set(tiles) == expected          # every tile exactly once
    assert 1 <= lag <= len(rows)
    at = {t: i for i, t in enumerate(tiles)}
    last_producer_m = collections.defaultdict(lambda: -1)    # (expert, m-tile) -> position of its last GEMM1 / dAct tile
    last_producer_e = collections.defaultdict(lambda: -1)    # expert -> same over all its m-tiles
    for (el, ph, m, n), i in at.items():
        if ph == 0:
            last_producer_m[(el, m)] = max(last_producer_m[(el, m)], i)
            last_producer_e[el] = max(last_producer_e[el], i)
    for (el, ph, m, n), i in at.items():
        if ph == 1:                                   # down GEMM / dX waits for the producers of its m-tile
            assert last_producer_m[(el, m)] < i
        if backward and ph == 3:                      # dW_gate|up waits for every dAct tile of its expert
            assert last_producer_e[el] < i


@pytest.mark.parametrize("backward", [False, True])
@pytest.mark.parametrize("shape", [(2048, 512, [640] * 64), (7168, 2048, [1024] * 32)])
def test_consumers_follow_their_producers_by_more_than_the_tiles_in_flight(shape, backward):
    """With enough experts for the lag not to be clamped, a tile's consumers come more than two rounds of the grid
    after it even at the start of the order, where the slots hold (full-depth) producer tiles only; in the steady
    state the distance is the lag times the tiles of an expert."""
    D, I, rows = shape
    grid = 148
    tiles, lag = _order(rows, D, I, grid, backward)
    assert lag < len(rows)
    at = {t: i for i, t in enumerate(tiles)}
    gaps = []
    for (el, ph, m, n), i in at.items():
        if ph == 1:
            prod = [at[(el, 0, m, k)] for k in range((I // 256) if backward else (I // 128))]
            gaps.append(i - max(prod))
    assert min(gaps) >= 2 * grid, (min(gaps), lag)
    per_expert = len(tiles) // len(rows)
    assert max(gaps) >= (lag - 1) * per_expert, (max(gaps), lag, per_expert)


def test_rejected_shapes():
    with pytest.raises(RuntimeError):
        _ops().moe_tile_order(torch.tensor([128], dtype=torch.int32), 2048 + 64, 512, 148, False)


def test_random_routings_keep_the_invariants():
    """Property check over random expert counts, row counts (many empty experts, a few huge ones), widths and grid
    sizes: every tile exactly once, every dependency earlier in the order, the lag within [1, experts]."""
    hyp = pytest.importorskip("hypothesis")
    st = pytest.importorskip("hypothesis.strategies")

    rows_st = st.lists(st.one_of(st.just(0), st.integers(1, 200), st.integers(200, 3000)), min_size=1, max_size=40)

    @hyp.settings(max_examples=60, deadline=None)
    @hyp.given(rows=rows_st, d_mult=st.integers(1, 4), i_mult=st.integers(1, 4), grid=st.sampled_from([1, 8, 132, 148]),
               backward=st.booleans())
    def check(rows, d_mult, i_mult, grid, backward):
        D, I = 256 * d_mult, 256 * i_mult
        tiles, lag = _order(rows, D, I, grid, backward)
        expected = (_expected_backward if backward else _expected_forward)(rows, D, I)
        assert len(tiles) == len(expected) and set(tiles) == expected
        assert 1 <= lag <= len(rows)
        at = {t: i for i, t in enumerate(tiles)}
        for (el, ph, m, n), i in at.items():
            if ph == 1:
                n_prod = (I // 256) if backward else (I // 128)
                assert all(at[(el, 0, m, k)] < i for k in range(n_prod))
            if backward and ph == 3:
                mt = (rows[el] + 127) // 128
                assert all(at[(el, 0, mm, k)] < i for mm in range(mt) for k in range(I // 256))

    check()
