"""Batched linear (tcgen05 path, K a multiple of 512) against the oracle. Needs a B200."""

import numpy as np
import pytest
import torch

from oracle import c_oracle, tq1_oracle as o
from tests.gpu_util import POWERS, random_blocks, run_linear

pytestmark = pytest.mark.gpu

# The required bound is 1e-3 (max |got - want| / max |want|). The tensor cores add the FP16 products of a
# 5120- to 17408-long row in FP32 within one accumulator, which lands between 3e-6 and 1.1e-5 on these cases.
F32_TOL = 5e-5
F16_TOL = 2e-3


def ones_scale(groups):
    return np.full(groups, 1.0, dtype=np.float16).view(np.uint8).reshape(-1, 2)


def test_all_243_bytes_at_every_slot_exactly():
    """28 groups (K = 3584), batch 28: activation row g is positional inside group g only."""
    rows, groups = 243, 28
    columns = groups * 128
    for shift in (0, 7, 19):
        trits = np.ones((rows, groups, 128), dtype=np.uint8)
        x = np.zeros((groups, columns), dtype=np.float32)
        for value in range(rows):
            digits = [(value // p) % 3 for p in (1, 3, 9, 27, 81)]
            for grp in range(groups):
                slot = (grp + shift) % 25
                trits[value, grp, 5 * slot:5 * slot + 5] = digits
        for grp in range(groups):
            slot = (grp + shift) % 25
            x[grp, grp * 128 + 5 * slot: grp * 128 + 5 * slot + 5] = POWERS
        blocks = o.encode_blocks(ones_scale(rows * groups), trits.reshape(-1, 128)).reshape(rows, groups, 28)
        want = np.tile(np.arange(rows, dtype=np.float32) - 121.0, (groups, 1))
        np.testing.assert_array_equal(run_linear(blocks, x), want)
        np.testing.assert_array_equal(run_linear(blocks, x[:5]), want[:5])


def test_all_27_tail_bytes_exactly():
    rows, groups = 27, 4
    trits = np.ones((rows, groups, 128), dtype=np.uint8)
    x = np.zeros((groups, 512), dtype=np.float32)
    for grp in range(groups):
        x[grp, grp * 128 + 125: grp * 128 + 128] = POWERS[:3]
        for value in range(rows):
            trits[value, grp, 125:] = [(value // p) % 3 for p in (1, 3, 9)]
    blocks = o.encode_blocks(ones_scale(rows * groups), trits.reshape(-1, 128)).reshape(rows, groups, 28)
    want = np.tile(np.arange(rows, dtype=np.float32) - 13.0, (groups, 1))
    np.testing.assert_array_equal(run_linear(blocks, x), want)


def test_finite_scale_patterns_reach_the_output():
    """Every finite FP16 scale, one +1 and one -1 weight: outputs are exactly +-scale."""
    rows = 1 << 16
    trits = np.ones((rows, 4, 128), dtype=np.uint8)
    trits[:, 1, 3] = 2
    trits[:, 1, 77] = 0
    scale_bits = np.zeros((rows, 4), dtype=np.uint16)
    scale_bits[:, 1] = np.arange(rows, dtype=np.uint16)
    blocks = o.encode_blocks(scale_bits.reshape(-1).view(np.uint8).reshape(-1, 2),
                             trits.reshape(-1, 128)).reshape(rows, 4, 28)
    x = np.zeros((2, 512), dtype=np.float32)
    x[0, 128 + 3] = 1.0
    x[1, 128 + 77] = 1.0
    got = run_linear(blocks, x)
    with np.errstate(invalid="ignore"):
        s = np.arange(rows, dtype=np.uint16).view(np.float16).astype(np.float32)
    finite = np.isfinite(s)
    np.testing.assert_array_equal(got[0][finite], s[finite])
    np.testing.assert_array_equal(got[1][finite], -s[finite])


@pytest.mark.parametrize("batch", (2, 3, 16, 17, 31, 64, 100, 128, 130, 300))
@pytest.mark.parametrize(("rows", "columns"), ((1000, 1536), (128, 512), (5120, 5120)))
def test_random_against_float64(rows, columns, batch):
    blocks, rng = random_blocks(rows, columns, seed=rows + columns + batch, dist="tests")
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
    got = run_linear(blocks, x)
    assert got.shape == (batch, rows)
    assert o.normalised_error(got, want) < F32_TOL
    assert o.normalised_error(run_linear(blocks, x, out_dtype=torch.float16), want) < F16_TOL


@pytest.mark.parametrize("batch", (2, 16, 300))
def test_worst_observed_error_is_pinned(batch):
    """The batched kernel misses the reference's own FP32 bound of 1e-5 (src/ternel_mlx/kernel_gate.py:105) on
    long rows: FP16 products of up to 17408 terms are added in ONE FP32 accumulator inside the tensor cores,
    where the reference's kernels add per-group FP32 sums. The worst values measured are 1.03e-5 .. 1.1e-5
    (5120 x 5120, batch 300); this pins them so that a drift towards the loose 5e-5 bound cannot pass unseen."""
    for rows, columns in ((5120, 5120), (1024, 17408)):
        blocks, rng = random_blocks(rows, columns, seed=rows + columns + batch, dist="tests")
        x = rng.standard_normal((batch, columns)).astype(np.float16)
        want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
        assert o.normalised_error(run_linear(blocks, x), want) < 1.5e-5


@pytest.mark.parametrize(("rows", "columns", "batch"), ((256, 17408, 4), (384, 17408, 16), (5120, 17408, 8),
                                                          (1024, 5120, 2), (17408, 5120, 16)))
def test_split_k_shapes(rows, columns, batch):
    """Few output tiles and long K: K is split over CTAs and the partials are added in a fixed order."""
    blocks, rng = random_blocks(rows, columns, seed=rows + batch)
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    want = c_oracle.matmul_f32(blocks, x.astype(np.float32), rows=rows, columns=columns)
    got = run_linear(blocks, x)
    assert o.normalised_error(got, want) < F32_TOL
    assert np.array_equal(run_linear(blocks, x), got)          # run-to-run identical


def test_pm_one_data_is_exact():
    rng = np.random.default_rng(3)
    for rows, columns, batch in ((256, 5120, 16), (128, 17408, 5), (300, 1024, 130)):
        groups = rows * columns // 128
        trits = (rng.integers(0, 2, size=(groups, 128)) * 2).astype(np.uint8)
        blocks = o.encode_blocks(ones_scale(groups), trits).reshape(rows, columns // 128, 28)
        x = (rng.integers(0, 2, size=(batch, columns)) * 2 - 1).astype(np.float16)
        want = x.astype(np.int64) @ (trits.reshape(rows, columns).astype(np.int64) - 1).T
        np.testing.assert_array_equal(run_linear(blocks, x), want.astype(np.float32))


def test_non_finite_activations_reach_every_output():
    rows, columns = 256, 1024
    blocks, _ = random_blocks(rows, columns, seed=31, dist="tests")
    x = np.zeros((3, columns), dtype=np.float16)
    x[0, 0] = np.nan
    x[1, 700] = np.inf
    x[2, 125] = -np.inf
    got = run_linear(blocks, x)
    with np.errstate(invalid="ignore"):
        want = o.reference_matmul(blocks, x.astype(np.float32), rows=rows, columns=columns)
    assert np.array_equal(o.nonfinite_classes(got), o.nonfinite_classes(want))
    assert not np.isfinite(got).any()


@pytest.mark.parametrize(("rows", "columns"), ((17408, 5120), (5120, 17408)))
@pytest.mark.parametrize("batch", (512, 2048))
def test_prefill_shapes_full_size(rows, columns, batch):
    """Prefill configuration: sampled activation rows against the C oracle, and y(2x) = 2 y(x)."""
    blocks, rng = random_blocks(rows, columns, seed=rows + batch)
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    got = run_linear(blocks, x, out_dtype=torch.float16)
    sample = np.array([0, 1, batch // 2, batch - 1, 77 % batch, 300 % batch])
    want = c_oracle.matmul_f32(blocks, x[sample].astype(np.float32), rows=rows, columns=columns)
    assert o.normalised_error(got[sample], want) < 1e-3           # FP16 out: the published gate
    got32 = run_linear(blocks, x[:128])
    want32 = c_oracle.matmul_f32(blocks, x[:8].astype(np.float32), rows=rows, columns=columns)
    assert o.normalised_error(got32[:8], want32) < F32_TOL
    doubled = run_linear(blocks, (x[:128].astype(np.float32) * 2).astype(np.float16))
    np.testing.assert_array_equal(doubled, got32 * 2)


@pytest.mark.parametrize(("rows", "columns", "batch"), ((1000, 1536, 17), (5120, 5120, 100), (640, 5120, 300)))
def test_every_token_tile_gives_the_right_answer(rows, columns, batch):
    """The dispatch rule may pick any token tile for a batch size: all five must be correct for it."""
    from ternel_b200 import _native
    lib = _native.lib()
    blocks, rng = random_blocks(rows, columns, seed=rows + batch)
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
    try:
        for tile in (16, 32, 64, 128, 256):
            assert lib.tq1_debug_force_token_tile(tile) == 0
            assert o.normalised_error(run_linear(blocks, x), want) < F32_TOL, tile
        assert lib.tq1_debug_force_token_tile(48) == _native.TQ1_ERR_INVALID
    finally:
        assert lib.tq1_debug_force_token_tile(0) == 0
