"""The packed shuffle tree of the half-row dense kernel (csrc/step_tma_half.cuh: tree_pack /
tree_rows) restated in numpy float32: reducing 8 (4, 2) rows together with one shuffle per level
and row pair performs, for every row, exactly the additions of the single-row xor tree
(_shared.cuh:59-60), so the sums are bit-identical.  No GPU needed: this pins the argument, the
-m gpu tests pin the kernel."""
import numpy as np
import pytest

LANES = np.arange(32)


def xor_tree(p):
    """The reference's reduction: five rounds of p += shfl_xor(p, off); every lane ends with the sum."""
    p = p.astype(np.float32).copy()
    for off in (16, 8, 4, 2, 1):
        p = (p + p[LANES ^ off]).astype(np.float32)
    return p


def tree_pack(a, b, off):
    up = (LANES & off) != 0
    keep, send = np.where(up, b, a), np.where(up, a, b)
    return (keep + send[LANES ^ off]).astype(np.float32)


def tree_rows(acc):
    rb = len(acc)
    if rb == 8:
        a, b = tree_pack(acc[0], acc[1], 16), tree_pack(acc[2], acc[3], 16)
        c, d = tree_pack(acc[4], acc[5], 16), tree_pack(acc[6], acc[7], 16)
        v = tree_pack(tree_pack(a, b, 8), tree_pack(c, d, 8), 4)
        rest = (2, 1)
    elif rb == 4:
        v = tree_pack(tree_pack(acc[0], acc[1], 16), tree_pack(acc[2], acc[3], 16), 8)
        rest = (4, 2, 1)
    else:
        v = tree_pack(acc[0], acc[1], 16)
        rest = (8, 4, 2, 1)
    for off in rest:
        v = (v + v[LANES ^ off]).astype(np.float32)
    return v


def lane_of(r):
    return ((r & 1) << 4) | (((r >> 1) & 1) << 3) | (((r >> 2) & 1) << 2)


@pytest.mark.parametrize("rb", [2, 4, 8])
def test_packed_tree_equals_the_single_row_tree(rb):
    rng = np.random.default_rng(rb)
    for trial in range(200):
        scale = np.float32(10.0 ** rng.integers(-20, 20))
        acc = [(rng.standard_normal(32) * scale).astype(np.float32) for _ in range(rb)]
        if trial % 7 == 0:
            acc[0][rng.integers(32)] = np.float32(np.inf)
        if trial % 11 == 0:
            acc[-1][:] = np.float32(0.0)
            acc[-1][3] = np.float32(-0.0)
        with np.errstate(invalid="ignore", over="ignore"):
            v = tree_rows(acc)
            for r in range(rb):
                want = xor_tree(acc[r])
                assert np.all(want.view(np.int32) == want.view(np.int32)[0]) or np.isnan(want).any()
                np.testing.assert_array_equal(v[lane_of(r)].view(np.int32), want[0].view(np.int32))
