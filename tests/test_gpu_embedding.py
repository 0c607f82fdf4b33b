"""Parity of the packed-embedding gather with the oracle: exact equality. Needs a B200."""

import numpy as np
import pytest
import torch

from oracle import tq1_oracle as o
from tests.gpu_util import random_blocks, to_dev

pytestmark = pytest.mark.gpu


def gather(blocks, ids, dtype):
    from ternel_b200.ops import tq1_get_rows
    out = tq1_get_rows(to_dev(blocks), torch.as_tensor(ids).cuda(), dtype=dtype)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_golden_rows(golden_cases):
    for name, c in golden_cases.items():
        ids = c["ids"].astype(np.int64)
        assert np.array_equal(gather(c["blocks"], ids, torch.float16), c["rows_f16"]), name
        assert np.array_equal(gather(c["blocks"], ids, torch.float32), c["rows_f32"]), name


@pytest.mark.parametrize(("rows", "columns"), ((48, 5120), (300, 256), (4096, 5120), (7, 128)))
@pytest.mark.parametrize("dtype", (torch.float16, torch.float32))
def test_rows_equal_the_oracle(rows, columns, dtype):
    blocks, rng = random_blocks(rows, columns, seed=rows + columns, dist="tests")
    ids = rng.integers(0, rows, size=33)
    npdt = np.float16 if dtype == torch.float16 else np.float32
    want = o.get_rows(blocks, ids, rows=rows, columns=columns, dtype=npdt)
    assert np.array_equal(gather(blocks, ids, dtype), want)


def test_every_byte_value_and_every_scale_pattern():
    g = np.load("tests/golden/codec_bytes.npz")
    blocks = g["blocks"].reshape(243, 1, 28)
    ids = np.arange(243)
    want = o.get_rows(blocks, ids, rows=243, columns=128, dtype=np.float32)
    got = gather(blocks, ids, torch.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(np.nan_to_num(got, nan=7.0).view(np.uint32), np.nan_to_num(want, nan=7.0).view(np.uint32))
    # all 65,536 scale patterns, one weight of each sign and a zero
    rows = 1 << 16
    trits = np.ones((rows, 128), dtype=np.uint8)
    trits[:, 0], trits[:, 1] = 2, 0
    scale_bits = np.arange(rows, dtype=np.uint16).view(np.uint8).reshape(-1, 2)
    blocks = o.encode_blocks(scale_bits, trits).reshape(rows, 1, 28)
    with np.errstate(invalid="ignore"):
        want = o.get_rows(blocks, np.arange(rows), rows=rows, columns=128, dtype=np.float16)
    got = gather(blocks, np.arange(rows), torch.float16)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    finite = ~np.isnan(want)
    assert np.array_equal(got[finite].view(np.uint16), want[finite].view(np.uint16))


def test_out_of_range_ids_give_zero_rows():
    blocks, rng = random_blocks(64, 256, seed=2)
    ids = np.array([0, 63, 64, -1, 1 << 40, -(1 << 40), 5], dtype=np.int64)
    got = gather(blocks, ids, torch.float16)
    ok = (ids >= 0) & (ids < 64)
    want = o.get_rows(blocks, ids[ok], rows=64, columns=256, dtype=np.float16)
    assert np.array_equal(got[ok], want)
    assert not got[~ok].any()


def test_module_keeps_index_shape_and_dtype():
    from ternel_b200.layout import PackedTensorLayout
    from ternel_b200.modules import PackedEmbedding
    blocks, rng = random_blocks(300, 384, seed=4)
    emb = PackedEmbedding(PackedTensorLayout.for_tensor(300, 384), dtype=torch.float16).cuda()
    emb.load_blocks(blocks)
    for dtype in (torch.int32, torch.int64, torch.int16, torch.uint8):
        ids = torch.from_numpy(rng.integers(0, 200, size=(2, 5))).to(dtype).cuda()
        out = emb(ids)
        assert out.shape == (2, 5, 384) and out.dtype == torch.float16
        want = o.get_rows(blocks, ids.cpu().numpy().reshape(-1).astype(np.int64), rows=300, columns=384,
                          dtype=np.float16)
        assert np.array_equal(out.reshape(-1, 384).cpu().numpy(), want)
    with pytest.raises(ValueError, match="integer"):
        emb(torch.zeros(3, device="cuda"))


def test_full_vocabulary_table_round_trip():
    """151936 x 5120 table: gather-then-reencode is the identity on the gathered rows."""
    rows, columns = 151936, 5120
    rng = np.random.default_rng(0)
    groups = rows * columns // 128
    # build bytes directly (legal values) instead of via trits: the table is 170 MB
    blocks = rng.integers(0, 243, size=(groups, 28), dtype=np.uint8)
    blocks[:, 27] %= 27
    blocks[:, 1] &= 0x3F            # keep scales finite and modest
    blocks = blocks.reshape(rows, columns // 128, 28)
    ids = np.array([0, 1, rows - 1, 77777, 151935, 12345, 151936], dtype=np.int64)
    got = gather(blocks, ids, torch.float16)
    want = o.get_rows(blocks, ids[:-1], rows=rows, columns=columns, dtype=np.float16)
    assert np.array_equal(got[:-1].view(np.uint16), want.view(np.uint16))
    assert not got[-1].any()
