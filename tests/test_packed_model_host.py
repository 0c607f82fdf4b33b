"""Graph swap of a torch model (host logic only): counts, shapes, bias rejection, state-dict loading."""

import numpy as np
import pytest
import torch
from torch import nn

from ternel_b200 import FormatError
from ternel_b200.layout import DISPATCHES_PER_TOKEN, MODEL_LINEAR_SHAPES, PackedTensorLayout, pack_blocks
from ternel_b200.modules import PackedEmbedding, PackedLinear
from ternel_b200.packed_model import blocks_from_ternary, dense_from_ternary, expect_counts, replace_with_packed


class Block(nn.Module):
    def __init__(self, hidden, ffn):
        super().__init__()
        self.up = nn.Linear(hidden, ffn, bias=False)
        self.down = nn.Linear(ffn, hidden, bias=False)
        self.norm = nn.LayerNorm(hidden)

    def forward(self, x):
        return x + self.down(torch.nn.functional.silu(self.up(self.norm(x))))


class Toy(nn.Module):
    def __init__(self, vocab=512, hidden=256, ffn=384, layers=2):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        self.layers = nn.ModuleList(Block(hidden, ffn) for _ in range(layers))
        self.head = nn.Linear(hidden, vocab, bias=False)

    def forward(self, ids):
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x)
        return self.head(x)


def test_swap_counts_and_shapes():
    model = Toy()
    counts = replace_with_packed(model, dtype=torch.float16)
    assert counts == {"linear": 5, "embedding": 1}
    expect_counts(counts)
    assert isinstance(model.embed, PackedEmbedding) and model.embed.layout.blocks_shape == (512, 2, 28)
    assert isinstance(model.layers[1].down, PackedLinear)
    assert model.layers[1].down.layout.rows == 256 and model.layers[1].down.layout.columns == 384
    assert isinstance(model.layers[0].norm, nn.LayerNorm)          # everything else is left alone
    names = set(model.state_dict())
    assert "layers.0.up.blocks" in names and "head.blocks" in names and "embed.blocks" in names


def test_skip_and_sanity_checks():
    model = Toy()
    counts = replace_with_packed(model, skip=("head", "embed"))
    assert counts == {"linear": 4, "embedding": 0}
    assert isinstance(model.head, nn.Linear)
    with pytest.raises(FormatError, match="embedding"):
        expect_counts(counts)
    with pytest.raises(FormatError, match="no linear"):
        expect_counts({"linear": 0, "embedding": 1})


def test_bias_is_rejected():
    model = nn.Sequential(nn.Linear(128, 128, bias=True))
    with pytest.raises(FormatError, match="bias"):
        replace_with_packed(model)


def test_state_dict_of_a_converted_checkpoint_loads():
    """`<path>.codes` / `<path>.scales` pairs (the converted artifact's naming) fill the swapped modules."""
    rng = np.random.default_rng(5)
    model = Toy(vocab=256, hidden=128, ffn=256, layers=1)
    replace_with_packed(model)
    state, want = {}, {}
    for path, module in model.named_modules():
        if isinstance(module, (PackedLinear, PackedEmbedding)):
            lay = module.layout
            trits = rng.integers(-1, 2, (lay.rows, lay.columns))
            scales = (np.abs(rng.standard_normal((lay.rows, lay.columns // 128))) * 0.05).astype(np.float16)
            blocks = blocks_from_ternary(trits, scales)
            codes, sc = pack_blocks(blocks, layout=lay)
            state[f"{path}.codes"] = torch.from_numpy(codes)
            state[f"{path}.scales"] = torch.from_numpy(sc.view(np.int16))
            want[path] = blocks
    state.update({k: v for k, v in model.state_dict().items() if "norm" in k})
    result = model.load_state_dict(state, strict=True)
    assert not result.missing_keys and not result.unexpected_keys
    for path, blocks in want.items():
        assert np.array_equal(model.get_submodule(path).blocks.numpy(), blocks)
    del state["head.scales"]
    with pytest.raises(RuntimeError, match="head.scales"):
        model.load_state_dict(state, strict=True)


def test_blocks_from_ternary_matches_the_dense_matrix():
    from oracle import tq1_oracle as o
    rng = np.random.default_rng(1)
    trits = rng.integers(-1, 2, (6, 256))
    scales = rng.standard_normal((6, 2)).astype(np.float16)
    blocks = blocks_from_ternary(trits, scales)
    dense = o.decode_dense(blocks) if hasattr(o, "decode_dense") else None
    x = rng.standard_normal((3, 256)).astype(np.float16)
    want = x.astype(np.float64) @ dense_from_ternary(trits, scales).double().numpy().T
    got = o.float64_matmul(blocks, x, rows=6, columns=256)
    assert np.allclose(got, want, rtol=0, atol=1e-9)
    with pytest.raises(FormatError):
        blocks_from_ternary(np.full((1, 128), 2), np.ones((1, 1), np.float16))


def test_shape_census_accounts_for_a_token():
    assert sum(s.dispatches_per_token for s in MODEL_LINEAR_SHAPES) == DISPATCHES_PER_TOKEN == 497
    for shape in MODEL_LINEAR_SHAPES:
        lay = shape.layout()
        assert isinstance(lay, PackedTensorLayout) and lay.payload_bytes == 28 * shape.rows * shape.columns // 128
    assert MODEL_LINEAR_SHAPES[0].layout().tile == 48          # no padded rows: the tile is the row count
