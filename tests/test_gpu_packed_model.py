"""The swapped torch model against its dense twin, and the 27B model's shape census. Needs a B200."""

import numpy as np
import pytest
import torch
from torch import nn

from oracle import c_oracle
from oracle import tq1_oracle as o
from ternel_b200.layout import MODEL_LINEAR_SHAPES
from ternel_b200.modules import PackedEmbedding, PackedLinear
from ternel_b200.packed_model import blocks_from_ternary, dense_from_ternary, expect_counts, replace_with_packed
from tests.gpu_util import run_linear
from tests.test_packed_model_host import Toy

pytestmark = pytest.mark.gpu


def fast_blocks(rows, columns, rng):
    """Random legal blocks without the Python-side packer (the head has 9.9 M groups)."""
    groups = columns // 128
    blocks = np.empty((rows, groups, 28), dtype=np.uint8)
    blocks[:, :, 0:2] = (np.abs(rng.standard_normal((rows, groups))) * 0.02).astype(np.float16).view(np.uint8).reshape(
        rows, groups, 2)
    blocks[:, :, 2:27] = rng.integers(0, 243, (rows, groups, 25), dtype=np.uint8)
    blocks[:, :, 27] = rng.integers(0, 27, (rows, groups), dtype=np.uint8)
    return blocks


@pytest.mark.parametrize("shape", MODEL_LINEAR_SHAPES, ids=lambda s: f"{s.rows}x{s.columns}")
@pytest.mark.parametrize("batch", (1, 4))
def test_every_linear_shape_of_the_model(shape, batch):
    """All nine distinct shapes a decoded token issues, including 48 rows and the 248,320-row head."""
    rng = np.random.default_rng(shape.rows + batch)
    blocks = fast_blocks(shape.rows, shape.columns, rng)
    x = rng.standard_normal((batch, shape.columns)).astype(np.float16)
    want = c_oracle.matmul_f32(blocks, x.astype(np.float32), rows=shape.rows, columns=shape.columns)
    got = run_linear(blocks, x)
    assert got.shape == (batch, shape.rows)
    assert o.normalised_error(got, want) < 5e-5
    got16 = run_linear(blocks, x, out_dtype=torch.float16)
    assert o.normalised_error(got16, want) < 2e-3


def test_swapped_model_matches_its_dense_twin():
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    dense = Toy(vocab=1024, hidden=512, ffn=1024, layers=2).cuda().half()
    packed = Toy(vocab=1024, hidden=512, ffn=1024, layers=2)
    packed.load_state_dict(dense.state_dict())
    packed = packed.cuda().half()
    counts = replace_with_packed(packed, dtype=torch.float16)
    expect_counts(counts)
    assert counts == {"linear": 5, "embedding": 1}
    for path, module in packed.named_modules():
        if isinstance(module, (PackedLinear, PackedEmbedding)):
            lay = module.layout
            trits = rng.integers(-1, 2, (lay.rows, lay.columns))
            scales = (np.abs(rng.standard_normal((lay.rows, lay.columns // 128))) * 0.03 + 0.01).astype(np.float16)
            module.load_blocks(blocks_from_ternary(trits, scales))
            twin = dense.get_submodule(path)
            with torch.no_grad():
                twin.weight.copy_(dense_from_ternary(trits, scales).to(twin.weight))
    ids = torch.randint(0, 1024, (3, 7), device="cuda")
    with torch.no_grad():
        want = dense(ids).float()
        got = packed(ids).float()
    assert got.shape == want.shape == (3, 7, 1024)
    # the embedding is exact; every linear layer narrows to FP16 once in both models
    assert torch.equal(packed.embed(ids), dense.embed(ids))
    err = (got - want).abs().max() / want.abs().max()
    assert err < 1e-2, float(err)
    # batch-1 decode shape goes through the streaming kernel, the rest through the batched one
    one = packed(ids[:1, :1]).float()
    assert (one - dense(ids[:1, :1]).float()).abs().max() / want.abs().max() < 1e-2
