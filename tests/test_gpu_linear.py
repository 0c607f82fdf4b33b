"""Parity of the CUDA linear path (through the C ABI) with the oracle. Needs a B200."""

import numpy as np
import pytest
import torch

from oracle import c_oracle, tq1_oracle as o
from tests.gpu_util import POWERS, random_blocks, run_linear, to_dev

pytestmark = pytest.mark.gpu

# FP32 accumulation against the float64 product, normalised per activation case by max|y|
# (the reference's own bound for an FP32 store; the published gate is 1e-3).
F32_TOL = 1e-5
F16_TOL = 2e-3   # one narrowing of the result to FP16


def ones_scale(groups):
    return np.full(groups, 1.0, dtype=np.float16).view(np.uint8).reshape(-1, 2)


def test_all_243_bytes_decode_at_every_slot_exactly():
    rows, groups = 243, 25
    columns = groups * 128
    trits = np.ones((rows, groups, 128), dtype=np.uint8)
    for value in range(rows):
        digits = [(value // p) % 3 for p in (1, 3, 9, 27, 81)]
        for slot in range(groups):
            trits[value, slot, 5 * slot:5 * slot + 5] = digits
    blocks = o.encode_blocks(ones_scale(rows * groups), trits.reshape(-1, 128)).reshape(rows, groups, 28)
    x = np.zeros((groups, columns), dtype=np.float32)
    for slot in range(groups):
        begin = slot * 128 + 5 * slot
        x[slot, begin:begin + 5] = POWERS
    want = np.tile(np.arange(rows, dtype=np.float32) - 121.0, (groups, 1))
    for m0 in (0, 1, 9):       # batch 25, batch 1 and batch 16 launches all go through
        got = run_linear(blocks, x[m0:m0 + (25 if m0 == 0 else 1 if m0 == 1 else 16)])
        np.testing.assert_array_equal(got, want[m0:m0 + got.shape[0]])


def test_all_27_tail_bytes_decode_exactly():
    rows = 27
    trits = np.ones((rows, 128), dtype=np.uint8)
    for value in range(rows):
        for d, p in enumerate((1, 3, 9)):
            trits[value, 125 + d] = (value // p) % 3
    blocks = o.encode_blocks(ones_scale(rows), trits).reshape(rows, 1, 28)
    x = np.zeros((1, 128), dtype=np.float32)
    x[0, 125:] = POWERS[:3]
    got = run_linear(blocks, x)
    np.testing.assert_array_equal(got, (np.arange(rows, dtype=np.float32) - 13.0).reshape(1, rows))


def test_every_fp16_scale_pattern_reaches_the_output():
    rows = 1 << 16
    trits = np.ones((rows, 128), dtype=np.uint8)
    trits[:, 0] = 2
    scale_bits = np.arange(rows, dtype=np.uint16).view(np.uint8).reshape(-1, 2)
    blocks = o.encode_blocks(scale_bits, trits).reshape(rows, 1, 28)
    x = np.zeros((1, 128), dtype=np.float32)
    x[0, 0] = 1.0
    got = run_linear(blocks, x)[0]
    with np.errstate(invalid="ignore"):
        want = np.arange(rows, dtype=np.uint16).view(np.float16).astype(np.float32)
    finite = np.isfinite(want)
    np.testing.assert_array_equal(got[finite], want[finite])
    assert np.all(np.isnan(got[np.isnan(want)]))
    np.testing.assert_array_equal(got[np.isinf(want)], want[np.isinf(want)])


def test_golden_cases_from_the_reference(golden_cases):
    for name, c in golden_cases.items():
        got = run_linear(c["blocks"], c["x"])
        assert o.normalised_error(got, c["y_f64"]) < F32_TOL, name
        assert o.normalised_error(got, c["y_gemv"]) < F32_TOL, name
        got16 = run_linear(c["blocks"], c["x"], out_dtype=torch.float16)
        assert o.normalised_error(got16, c["y_f64"]) < F16_TOL, name


SHAPES = ((48, 5120), (256, 640), (512, 384), (1024, 5120), (300, 256), (5120, 5120), (4096, 4096),
          (1000, 1536), (17, 128), (1, 2048))


@pytest.mark.parametrize(("rows", "columns"), SHAPES)
@pytest.mark.parametrize("batch", (1, 2, 3, 8, 16))
def test_random_shapes_against_float64(rows, columns, batch):
    blocks, rng = random_blocks(rows, columns, seed=rows * 31 + columns, dist="tests")
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
    got = run_linear(blocks, x)
    assert got.shape == (batch, rows)
    assert o.normalised_error(got, want) < F32_TOL
    got16 = run_linear(blocks, x, out_dtype=torch.float16)
    assert o.normalised_error(got16, want) < F16_TOL


@pytest.mark.parametrize("batch", (17, 33, 64, 100, 128, 257))
def test_large_batches_against_float64(batch):
    rows, columns = 640, 1024
    blocks, rng = random_blocks(rows, columns, seed=batch, dist="bench")
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
    assert o.normalised_error(run_linear(blocks, x), want) < F32_TOL


@pytest.mark.parametrize("dist", ("bench", "real", "tests"))
def test_single_matrix_configuration(dist):
    """The 4096x4096 configuration: FP16 in, FP32 accumulate, against the NumPy decode-and-dot."""
    if dist == "bench":
        blocks, x = o.synth_matrix(4096, 4096, seed=0)
        want = np.load("tests/golden/single_matrix_4096.npz")["y"]
    else:
        blocks, rng = random_blocks(4096, 4096, seed=3, dist=dist)
        x = rng.standard_normal(4096).astype(np.float16)
        want = c_oracle.matmul_f32(blocks, x.astype(np.float32), rows=4096, columns=4096)[0]
    got = run_linear(blocks, x[None, :])[0]
    assert o.normalised_error(got, want) < 1e-5
    got16 = run_linear(blocks, x[None, :], out_dtype=torch.float16)[0]
    assert o.normalised_error(got16, want) < 1e-3       # the published gate, FP16 out


def edge_activations(columns, rng):
    idx = np.arange(columns)
    edges = {
        "zeros": np.zeros(columns),
        "ones": np.ones(columns),
        "alternating": np.where(idx % 2 == 0, 1.0, -1.0),
        "hot_first": np.eye(1, columns, 0)[0],
        "hot_last": np.eye(1, columns, columns - 1)[0],
        "hot_tail": np.eye(1, columns, 125)[0],
        "fp16_max": np.full(columns, 65504.0),
        "fp16_max_alternating": np.where(idx % 2 == 0, 65504.0, -65504.0),
        "fp16_min_normal": np.full(columns, 6.103515625e-05),
        "fp16_subnormal": np.full(columns, 1e-7),
        "mixed_magnitudes": rng.standard_normal(columns) * 10.0 ** rng.integers(-6, 4, size=columns),
    }
    return list(edges), np.stack(list(edges.values())).astype(np.float16)


@pytest.mark.parametrize(("rows", "columns"), ((256, 384), (512, 5120)))
def test_edge_activations(rows, columns):
    blocks, rng = random_blocks(rows, columns, seed=29, dist="tests")
    labels, x = edge_activations(columns, rng)
    want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
    for m in (len(labels), 1):
        got = run_linear(blocks, x[:m])
        for i in range(m):
            assert o.normalised_error(got[i], want[i]) < F32_TOL, labels[i]
    for i, label in enumerate(labels):      # one launch per case exercises the batch-1 kernel
        got = run_linear(blocks, x[i:i + 1])
        assert o.normalised_error(got[0], want[i]) < F32_TOL, label


def test_non_finite_activations_propagate_like_the_reference():
    rows, columns = 256, 384
    blocks, _ = random_blocks(rows, columns, seed=31, dist="tests")
    cases = {
        "all_nan": np.full(columns, np.nan),
        "all_inf": np.full(columns, np.inf),
        "nan_first": np.zeros(columns),
        "nan_tail": np.zeros(columns),
        "neg_inf_last": np.zeros(columns),
    }
    cases["nan_first"][0] = np.nan
    cases["nan_tail"][125] = np.nan
    cases["neg_inf_last"][columns - 1] = -np.inf
    x = np.stack(list(cases.values())).astype(np.float16)
    with np.errstate(invalid="ignore"):
        want = o.reference_matmul(blocks, x.astype(np.float32), rows=rows, columns=columns)
    for batch in (x, x[2:3], x[4:5]):
        got = run_linear(blocks, batch)
        ref = want if batch.shape[0] == 5 else (want[2:3] if np.isnan(batch[0, 0]) else want[4:5])
        assert np.array_equal(o.nonfinite_classes(got), o.nonfinite_classes(ref))
        assert not np.isfinite(got).any()


def test_runs_are_bit_identical():
    blocks, rng = random_blocks(1024, 5120, seed=8)
    for batch in (1, 4, 16):
        x = rng.standard_normal((batch, 5120)).astype(np.float16)
        first = run_linear(blocks, x)
        for _ in range(3):
            assert np.array_equal(run_linear(blocks, x), first)


def test_pm_one_data_is_exact():
    """+-1 weights, unit scales and +-1 activations: every partial sum is a small integer."""
    rng = np.random.default_rng(77)
    for rows, columns in ((256, 5120), (128, 17408), (96, 6144)):
        groups = rows * columns // 128
        trits = (rng.integers(0, 2, size=(groups, 128)) * 2).astype(np.uint8)
        blocks = o.encode_blocks(ones_scale(groups), trits).reshape(rows, columns // 128, 28)
        for batch in (1, 2, 5, 16):
            x = (rng.integers(0, 2, size=(batch, columns)) * 2 - 1).astype(np.float16)
            w = trits.reshape(rows, columns).astype(np.int64) - 1
            want = x.astype(np.int64) @ w.T
            np.testing.assert_array_equal(run_linear(blocks, x), want.astype(np.float32))


@pytest.mark.parametrize(("rows", "columns"), ((5120, 5120), (1024, 5120), (17408, 5120), (5120, 17408)))
def test_layer_shapes_full_size(rows, columns):
    """Full benchmark shapes: C oracle for values, linearity as a size-independent property."""
    blocks, rng = random_blocks(rows, columns, seed=rows + columns)
    x = rng.standard_normal((2, columns)).astype(np.float16)
    want = c_oracle.matmul_f32(blocks, x.astype(np.float32), rows=rows, columns=columns)
    got = run_linear(blocks, x[:1])
    assert o.normalised_error(got, want[:1]) < F32_TOL
    got2 = run_linear(blocks, x)
    assert o.normalised_error(got2, want) < F32_TOL
    # y(2x) == 2 y(x) exactly (scaling by two is exact in FP16 and FP32)
    doubled = run_linear(blocks, (x[:1].astype(np.float32) * 2).astype(np.float16))
    np.testing.assert_array_equal(doubled, got * 2)


def test_module_matches_kernel_and_keeps_leading_dims():
    from ternel_b200.layout import PackedTensorLayout
    from ternel_b200.modules import PackedEmbedding, PackedLinear
    rows, columns = 512, 640
    blocks, rng = random_blocks(rows, columns, seed=5)
    layout = PackedTensorLayout.for_tensor(rows, columns)
    lin = PackedLinear(layout).cuda()
    lin.load_blocks(blocks)
    x = torch.from_numpy(rng.standard_normal((2, 3, columns)).astype(np.float16)).cuda()
    y = lin(x)
    assert y.shape == (2, 3, rows) and y.dtype == torch.float16
    want = o.float64_matmul(blocks, x.reshape(-1, columns).cpu().numpy(), rows=rows, columns=columns)
    assert o.normalised_error(y.reshape(-1, rows).float().cpu().numpy(), want) < F16_TOL
    emb = PackedEmbedding(layout).cuda()
    emb.load_blocks(to_dev(blocks))
    assert torch.equal(emb.as_linear(x), y)       # the tied head is the same kernel, bit for bit
    bad = blocks.copy()
    bad[5, 2, 9] = 250
    with pytest.raises(ValueError, match="regular=1, tail=0"):
        lin.load_blocks(to_dev(bad))


def test_device_byte_scan_counts_every_illegal_byte():
    """The load-time scan on the device: exact counts of code bytes above 242 and tail bytes above 26,
    whatever their place in the block, and a clean pass on legal data (scale bytes are never counted)."""
    from ternel_b200 import FormatError
    from ternel_b200.ops import validate_device_blocks
    rows, columns = 1000, 1536
    blocks, rng = random_blocks(rows, columns, seed=77)
    blocks[:, :, 0:2] = 0xff                               # scale bytes may hold anything
    dev = torch.from_numpy(blocks).cuda()
    validate_device_blocks(dev)                            # legal: no exception
    bad = blocks.copy().reshape(-1, 28)
    picks = rng.choice(bad.shape[0], size=300, replace=False)
    n_full = n_tail = 0
    for n, g in enumerate(picks):
        if n % 3 == 0:
            bad[g, 27] = 27 + n % 200                      # tail byte above 26
            n_tail += 1
        else:
            bad[g, 2 + n % 25] = 243 + n % 13              # a regular code byte above 242
            n_full += 1
            if n % 7 == 0:
                bad[g, 2 + (n + 11) % 25] = 255
                n_full += (n + 11) % 25 != n % 25
    with pytest.raises(FormatError, match=f"regular={n_full}, tail={n_tail}"):
        validate_device_blocks(torch.from_numpy(bad.reshape(blocks.shape)).cuda())
    counts = torch.ops.ternel.tq1_validate(torch.from_numpy(bad.reshape(blocks.shape)).cuda()).cpu().tolist()
    assert counts == [n_full, n_tail]


def test_two_rows_in_one_launch_equal_two_batch_1_calls():
    """Batches the dispatch sends through the batch-1 kernel (one launch, one pass per activation row) give, row
    by row, the bits of separate batch-1 calls."""
    from ternel_b200.dispatch import looped_tokens
    from ternel_b200.ops import tq1_matmul
    tokens = looped_tokens()
    if tokens < 2:
        pytest.skip("the dispatch sends no batch through the batch-1 kernel")
    blocks, rng = random_blocks(1040, 1024, seed=77)
    x = rng.standard_normal((tokens, 1024)).astype(np.float16)
    bd, xd = to_dev(blocks), to_dev(x)
    both = tq1_matmul(bd, xd, out_dtype=torch.float32)
    for m in range(tokens):
        one = tq1_matmul(bd, xd[m:m + 1], out_dtype=torch.float32)
        assert torch.equal(both[m:m + 1], one)
    want = o.float64_matmul(blocks, x.astype(np.float32), rows=1040, columns=1024)
    assert o.normalised_error(both.cpu().numpy(), want) < 1e-5


def test_check_status_reads_the_shared_workspace():
    from ternel_b200 import ops
    blocks, rng = random_blocks(64, 512, seed=5)
    x = rng.standard_normal((1, 512)).astype(np.float16)
    ops.tq1_matmul(to_dev(blocks), to_dev(x))
    ops.check_status()                                   # nothing ran out
    buf = ops._workspaces[torch.cuda.current_device()]
    buf[:4].view(torch.int32)[0] = 5                     # what a slot wait that ran out would leave
    with pytest.raises(RuntimeError, match="status 5"):
        ops.check_status()
    assert int(buf[:4].view(torch.int32)[0].item()) == 0
    y = ops.tq1_matmul(to_dev(blocks), to_dev(x), out_dtype=torch.float32)      # and later calls are clean
    want = o.float64_matmul(blocks, x.astype(np.float32), rows=64, columns=512)
    assert o.normalised_error(y.cpu().numpy(), want) < 1e-5
