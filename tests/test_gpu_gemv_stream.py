"""Batch-1 streaming GEMV (K a multiple of 512): exact-integer and edge cases. Needs a B200."""

import numpy as np
import pytest

from oracle import c_oracle
from oracle import tq1_oracle as o
from tests.gpu_util import POWERS, random_blocks, run_linear

pytestmark = pytest.mark.gpu


def ones_scale(groups):
    return np.full(groups, 1.0, dtype=np.float16).view(np.uint8).reshape(-1, 2)


def test_all_243_bytes_at_every_slot_of_every_group_position():
    """Byte value v in slot s of group g, positional activations: the group sum is v - 121.

    K = 3584 = 7 chunks of 512, so the 28 groups cover all four positions in a chunk.
    """
    rows, groups = 243, 28
    columns = groups * 128
    for slot_shift in range(0, 25, 6):
        trits = np.ones((rows, groups, 128), dtype=np.uint8)
        x = np.zeros((groups, columns), dtype=np.float32)
        for value in range(rows):
            digits = [(value // p) % 3 for p in (1, 3, 9, 27, 81)]
            for grp in range(groups):
                slot = (grp + slot_shift) % 25
                trits[value, grp, 5 * slot:5 * slot + 5] = digits
        for grp in range(groups):
            slot = (grp + slot_shift) % 25
            x[grp, grp * 128 + 5 * slot: grp * 128 + 5 * slot + 5] = POWERS
        blocks = o.encode_blocks(ones_scale(rows * groups), trits.reshape(-1, 128)).reshape(rows, groups, 28)
        want = np.arange(rows, dtype=np.float32) - 121.0
        for grp in range(groups):
            got = run_linear(blocks, x[grp:grp + 1])[0]
            np.testing.assert_array_equal(got, want, err_msg=f"group {grp} shift {slot_shift}")


def test_all_27_tail_bytes_in_each_group_position():
    rows, groups = 27, 4
    for grp in range(groups):
        trits = np.ones((rows, groups, 128), dtype=np.uint8)
        for value in range(rows):
            trits[value, grp, 125:] = [(value // p) % 3 for p in (1, 3, 9)]
        blocks = o.encode_blocks(ones_scale(rows * groups), trits.reshape(-1, 128)).reshape(rows, groups, 28)
        x = np.zeros((1, 512), dtype=np.float32)
        x[0, grp * 128 + 125: grp * 128 + 128] = POWERS[:3]
        got = run_linear(blocks, x)[0]
        np.testing.assert_array_equal(got, np.arange(rows, dtype=np.float32) - 13.0)


def test_every_fp16_scale_pattern_reaches_the_output():
    rows = 1 << 16
    trits = np.ones((rows, 4, 128), dtype=np.uint8)
    trits[:, 2, 7] = 2                      # one +1 weight in group 2
    scale_bits = np.zeros((rows, 4), dtype=np.uint16)
    scale_bits[:, 2] = np.arange(rows, dtype=np.uint16)
    scale_bits[:, 0] = 0x3C00               # finite scales elsewhere (their group sums are zero)
    blocks = o.encode_blocks(scale_bits.reshape(-1).view(np.uint8).reshape(-1, 2),
                             trits.reshape(-1, 128)).reshape(rows, 4, 28)
    x = np.zeros((1, 512), dtype=np.float32)
    x[0, 2 * 128 + 7] = 1.0
    got = run_linear(blocks, x)[0]
    with np.errstate(invalid="ignore"):
        want = np.arange(rows, dtype=np.uint16).view(np.float16).astype(np.float32)
    finite = np.isfinite(want)
    np.testing.assert_array_equal(got[finite], want[finite])
    assert np.all(np.isnan(got[np.isnan(want)]))
    np.testing.assert_array_equal(got[np.isinf(want)], want[np.isinf(want)])


@pytest.mark.parametrize(("rows", "columns"), ((256, 512), (300, 1024), (512, 5120)))
def test_non_finite_activations_propagate_like_the_reference(rows, columns):
    blocks, _ = random_blocks(rows, columns, seed=31, dist="tests")
    cases = {
        "all_nan": np.full(columns, np.nan),
        "all_inf": np.full(columns, np.inf),
        "nan_first": np.zeros(columns),
        "nan_tail": np.zeros(columns),
        "neg_inf_last": np.zeros(columns),
        "inf_among_normals": np.random.default_rng(1).standard_normal(columns),
    }
    cases["nan_first"][0] = np.nan
    cases["nan_tail"][125] = np.nan
    cases["neg_inf_last"][columns - 1] = -np.inf
    cases["inf_among_normals"][columns // 2 + 3] = np.inf
    for name, xv in cases.items():
        x = xv.astype(np.float16)[None, :]
        with np.errstate(invalid="ignore"):
            want = o.reference_matmul(blocks, x.astype(np.float32), rows=rows, columns=columns)
        got = run_linear(blocks, x)
        assert np.array_equal(o.nonfinite_classes(got), o.nonfinite_classes(want)), name
        assert not np.isfinite(got).any(), name


def test_wide_dynamic_range_within_a_group():
    """Activations spanning the whole FP16 range inside every group: the block fixed point
    keeps 22 bits below the group maximum, which matches FP32 accumulation."""
    rows, columns = 512, 2048
    blocks, rng = random_blocks(rows, columns, seed=9, dist="tests")
    x = (rng.standard_normal(columns) * 2.0 ** rng.integers(-24, 15, size=columns)).astype(np.float16)
    want = o.float64_matmul(blocks, x[None, :], rows=rows, columns=columns)
    assert o.normalised_error(run_linear(blocks, x[None, :]), want) < 1e-5
    # subnormal-only and huge-only vectors
    for fill in (np.float16(6e-8), np.float16(65504.0), np.float16(-3.0e-5)):
        xv = np.full((1, columns), fill, dtype=np.float16)
        want = o.float64_matmul(blocks, xv, rows=rows, columns=columns)
        assert o.normalised_error(run_linear(blocks, xv), want) < 1e-5


@pytest.mark.parametrize(("rows", "columns"), ((1, 512), (15, 512), (17, 1024), (33, 1536), (100, 4096), (4000, 512)))
def test_ragged_row_counts(rows, columns):
    blocks, rng = random_blocks(rows, columns, seed=rows * 7 + columns, dist="bench")
    x = rng.standard_normal((1, columns)).astype(np.float16)
    want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
    got = run_linear(blocks, x)
    assert got.shape == (1, rows)
    assert o.normalised_error(got, want) < 1e-5


def test_workspace_is_reusable_across_shapes():
    """Alternating shapes on one workspace: the partial-sum slots must be clear again after each call."""
    shapes = ((5120, 5120), (64, 512), (1024, 5120), (5120, 17408), (48, 5120))
    cases = []
    for rows, columns in shapes:
        blocks, rng = random_blocks(rows, columns, seed=rows + columns)
        x = rng.standard_normal((1, columns)).astype(np.float16)
        cases.append((blocks, x, run_linear(blocks, x)))
    for _ in range(3):
        for blocks, x, first in cases:
            assert np.array_equal(run_linear(blocks, x), first)


def test_workspace_is_shared_with_the_batched_kernels():
    """Batch-1 and batched calls alternate on one workspace without disturbing each other."""
    blocks, rng = random_blocks(1024, 5120, seed=12)
    x1 = rng.standard_normal((1, 5120)).astype(np.float16)
    x8 = rng.standard_normal((8, 5120)).astype(np.float16)
    x300 = rng.standard_normal((300, 5120)).astype(np.float16)
    first1, first8 = run_linear(blocks, x1), run_linear(blocks, x8)
    for _ in range(2):
        run_linear(blocks, x300)
        assert np.array_equal(run_linear(blocks, x1), first1)
        assert np.array_equal(run_linear(blocks, x8), first8)


def test_very_tall_matrix_runs_as_row_ranges():
    """An output head taller than one launch's slot region (16 MiB / (8 B x K chunks) rows) is split
    into row ranges; a tall, narrow stand-in keeps the oracle fast."""
    rows, columns = 300_000, 512 * 8          # 8 chunks: 262,144 rows per launch
    rng = np.random.default_rng(11)
    blocks = np.empty((rows, columns // 128, 28), dtype=np.uint8)
    blocks[:, :, 0:2] = rng.standard_normal((rows, columns // 128)).astype(np.float16).view(np.uint8).reshape(
        rows, columns // 128, 2)
    blocks[:, :, 2:27] = rng.integers(0, 243, (rows, columns // 128, 25), dtype=np.uint8)
    blocks[:, :, 27] = rng.integers(0, 27, (rows, columns // 128), dtype=np.uint8)
    x = rng.standard_normal((1, columns)).astype(np.float16)
    want = c_oracle.matmul_f32(blocks, x.astype(np.float32), rows=rows, columns=columns)
    got = run_linear(blocks, x)
    assert got.shape == (1, rows)
    assert o.normalised_error(got, want) < 1e-5
