"""On-disk forms written by the reference, loaded and run on the GPU. Needs a B200.

tests/golden/sidecar_small.tq1g128 and .lut23 were written by the reference's own writers
(src/bonsai_tq1/format.py:149-246, src/bonsai_tq1/lut23_reorder.py:42-123,323-334; see make_golden.py).
Each tensor goes reader -> PackedLinear.load_blocks (device scan) -> tq1_matmul and is compared with the
oracle, at batch 1 and 5.
"""

import numpy as np
import pytest
import torch

from oracle import tq1_oracle as o
from ternel_b200 import loaders
from tests.conftest import GOLDEN

pytestmark = pytest.mark.gpu

NAMES = ("blk.0.ffn_down.weight", "blk.0.ssm_a.weight")


def _run(blocks, name):
    from ternel_b200.layout import PackedTensorLayout
    from ternel_b200.modules import PackedLinear
    rows, columns = blocks.shape[0], blocks.shape[1] * 128
    layer = PackedLinear(PackedTensorLayout.for_tensor(rows, columns), device="cuda", out_dtype=torch.float32)
    layer.load_blocks(blocks)                      # runs the fail-closed byte scan on the device
    rng = np.random.default_rng(len(name))
    for batch in (1, 5):
        x = rng.standard_normal((batch, columns)).astype(np.float16)
        got = layer(torch.from_numpy(x).cuda()).cpu().numpy()
        want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
        assert got.shape == (batch, rows)
        assert o.normalised_error(got, want) < 1e-5, (name, batch)


def test_sidecar_tensors_run_on_the_gpu():
    _, manifest = loaders.read_sidecar(GOLDEN / "sidecar_small.tq1g128")
    for name in NAMES:
        _run(loaders.load_sidecar_tensor(GOLDEN / "sidecar_small.tq1g128", manifest, name), name)


def test_lut23_sidecar_tensors_run_on_the_gpu():
    _, manifest = loaders.read_lut23_sidecar(GOLDEN / "sidecar_small.lut23")
    for name in NAMES:
        _run(loaders.load_lut23_tensor(GOLDEN / "sidecar_small.lut23", manifest, name), name)
