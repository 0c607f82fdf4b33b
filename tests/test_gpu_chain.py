"""Chains of batch-1 products in one persistent launch: every link against the oracle, fed with the
activations the GPU actually handed over, plus the bookkeeping that lets a chain be replayed. Needs a B200."""

import numpy as np
import pytest
import torch

from oracle import tq1_oracle as o
from tests.gpu_util import random_blocks, to_dev

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5          # FP32 output, the reference's own bound (src/ternel_mlx/kernel_gate.py:105)


def silu_mul(gate, up):
    gate = gate.astype(np.float32)
    return gate / (np.float32(1.0) + np.exp(-gate)) * up.astype(np.float32)


def oracle_link(blocks, x, *, swiglu=False, out_scale=1.0):
    rows, columns = blocks.shape[0], blocks.shape[1] * 128
    y = o.float64_matmul(blocks, x.astype(np.float32)[None, :], rows=rows, columns=columns)[0]
    if swiglu:
        y = silu_mul(y[0::2], y[1::2])
    return (y * np.float32(out_scale)).astype(np.float32)


def check_chain(specs, x0, *, plan=True, repeats=2):
    """specs: list of dicts(blocks, source, source_offset, swiglu, out_scale, x). Runs the chain, then checks each
    link against the oracle applied to the FP16 values the GPU produced for its source."""
    from ternel_b200.chain import ChainPlan, Link, chain_workspace_bytes, linear_chain

    links, outs32, outs16 = [], [], []
    for spec in specs:
        blocks = spec["blocks"]
        n_out = blocks.shape[0] // 2 if spec.get("swiglu") else blocks.shape[0]
        y32 = torch.full((n_out,), float("nan"), dtype=torch.float32, device="cuda")
        outs32.append(y32)
        links.append(Link(blocks=to_dev(blocks),
                          x=to_dev(spec["x"].astype(np.float16)) if spec.get("x") is not None else None,
                          source=spec.get("source", -1), source_offset=spec.get("source_offset", 0), y=y32,
                          swiglu=bool(spec.get("swiglu")), out_scale=spec.get("out_scale", 1.0)))
    if plan:
        runner = ChainPlan(links)
        run = runner.run
        workspace = runner.workspace
    else:
        workspace = torch.zeros(chain_workspace_bytes(links), dtype=torch.uint8, device="cuda")
        run = lambda: linear_chain(links, workspace)
    first = None
    for _ in range(repeats):
        for y in outs32:
            y.fill_(float("nan"))
        run()
        torch.cuda.synchronize()
        assert int(workspace[:4].view(torch.int32)[0].item()) == 0, "a bounded device wait ran out"
        got = [y.cpu().numpy() for y in outs32]
        if first is None:
            first = got
        else:                               # replays are bit-identical
            for a, b in zip(first, got):
                assert np.array_equal(a, b)
    for i, spec in enumerate(specs):
        if spec.get("x") is not None:
            x = spec["x"].astype(np.float16)
        else:
            src = first[spec["source"]].astype(np.float16)      # what the next link was handed: the FP16 rounding
            k = spec["blocks"].shape[1] * 128
            x = src[spec.get("source_offset", 0): spec.get("source_offset", 0) + k]
        want = oracle_link(spec["blocks"], x, swiglu=bool(spec.get("swiglu")), out_scale=spec.get("out_scale", 1.0))
        err = o.normalised_error(first[i][None, :], want[None, :])
        assert err < F32_TOL, f"link {i}: {err}"
    return first


def test_single_link_equals_the_plain_entry_point():
    from ternel_b200.ops import tq1_matmul
    blocks, rng = random_blocks(1024, 5120, seed=3)
    x = rng.standard_normal(5120).astype(np.float16)
    got = check_chain([dict(blocks=blocks, x=x)], x, plan=False)[0]
    plain = tq1_matmul(to_dev(blocks), to_dev(x[None, :]), out_dtype=torch.float32).cpu().numpy()[0]
    assert np.array_equal(got, plain)


@pytest.mark.parametrize("plan", (False, True))
def test_dependent_links_hand_their_output_over(plan):
    """qkv -> o (reads the q part) -> gate|up with SiLU*mul -> down, each reading its predecessor."""
    hidden, ffn = 1024, 1536
    rng = np.random.default_rng(5)
    qkv, _ = random_blocks(hidden + 512, hidden, seed=11)
    wo, _ = random_blocks(hidden, hidden, seed=12)
    gate_up, _ = random_blocks(2 * ffn, hidden, seed=13)
    down, _ = random_blocks(hidden, ffn, seed=14)
    x = rng.standard_normal(hidden).astype(np.float16)
    specs = [
        dict(blocks=qkv, x=x, out_scale=2.0),
        dict(blocks=wo, source=0, source_offset=0, out_scale=1.5),
        dict(blocks=gate_up, source=1, swiglu=True, out_scale=4.0),
        dict(blocks=down, source=2, out_scale=0.5),
    ]
    check_chain(specs, x, plan=plan, repeats=3)


def test_two_layers_of_model_shapes_in_one_plan():
    """Eight links shaped like two decoder layers (scaled down): every link depends on the one before."""
    hidden, ffn, kv = 1536, 4608, 256
    rng = np.random.default_rng(8)
    x = rng.standard_normal(hidden).astype(np.float16)
    specs = []
    for layer in range(2):
        qkv, _ = random_blocks(hidden + 2 * kv, hidden, seed=100 + layer)
        wo, _ = random_blocks(hidden, hidden, seed=200 + layer)
        gate_up, _ = random_blocks(2 * ffn, hidden, seed=300 + layer)
        down, _ = random_blocks(hidden, ffn, seed=400 + layer)
        base = 4 * layer
        specs += [
            dict(blocks=qkv, out_scale=1.0 / 0.45, **(dict(x=x) if layer == 0 else dict(source=base - 1))),
            dict(blocks=wo, source=base, out_scale=1.0 / 0.45),
            dict(blocks=gate_up, source=base + 1, swiglu=True, out_scale=6.0),
            dict(blocks=down, source=base + 2, out_scale=1.0 / 0.8),
        ]
    check_chain(specs, x, plan=True, repeats=2)


def test_fan_out_and_independent_links():
    """Three links read the same earlier output, two more read activations that exist before the launch."""
    rng = np.random.default_rng(21)
    first, _ = random_blocks(1536, 1024, seed=31)
    a, _ = random_blocks(512, 1536, seed=32)
    b, _ = random_blocks(48, 1536, seed=33)            # N not a multiple of 16
    c, _ = random_blocks(2000, 1024, seed=34)
    d, _ = random_blocks(300, 512, seed=35)
    x = rng.standard_normal(1024).astype(np.float16)
    x2 = rng.standard_normal(512).astype(np.float16)
    specs = [
        dict(blocks=first, x=x),
        dict(blocks=a, source=0),
        dict(blocks=b, source=0),
        dict(blocks=c, source=0, source_offset=512),
        dict(blocks=d, x=x2),
        dict(blocks=c, x=x),
    ]
    check_chain(specs, x, plan=True, repeats=2)
    check_chain(specs, x, plan=False, repeats=2)


def test_many_links_reuse_both_slot_regions():
    """Sixteen dependent square links: the two slot regions alternate and the arrival counters gate the reuse."""
    size = 1024
    rng = np.random.default_rng(40)
    x = rng.standard_normal(size).astype(np.float16)
    specs = []
    for i in range(16):
        blocks, _ = random_blocks(size, size, seed=500 + i)
        specs.append(dict(blocks=blocks, out_scale=1.0 / 0.4, **(dict(x=x) if i == 0 else dict(source=i - 1))))
    check_chain(specs, x, plan=True, repeats=3)


def test_non_finite_values_travel_through_the_hand_off():
    blocks0, _ = random_blocks(1024, 1024, seed=61, dist="tests")
    blocks1, _ = random_blocks(512, 1024, seed=62, dist="tests")
    x = np.random.default_rng(2).standard_normal(1024).astype(np.float16)
    x[77] = np.inf
    from ternel_b200.chain import ChainPlan, Link
    y0 = torch.zeros(1024, dtype=torch.float32, device="cuda")
    y1 = torch.zeros(512, dtype=torch.float32, device="cuda")
    plan = ChainPlan([Link(blocks=to_dev(blocks0), x=to_dev(x), y=y0), Link(blocks=to_dev(blocks1), source=0, y=y1)])
    plan.run()
    torch.cuda.synchronize()
    assert plan.status() == 0
    with np.errstate(invalid="ignore", over="ignore"):
        want0 = o.reference_matmul(blocks0, x.astype(np.float32)[None, :], rows=1024, columns=1024)
        got0 = y0.cpu().numpy()[None, :]
        assert np.array_equal(o.nonfinite_classes(got0), o.nonfinite_classes(want0))
        want1 = o.reference_matmul(blocks1, got0.astype(np.float16).astype(np.float32), rows=512, columns=1024)
    assert np.array_equal(o.nonfinite_classes(y1.cpu().numpy()[None, :]), o.nonfinite_classes(want1))


def test_chain_shares_its_workspace_with_single_calls():
    """Single batch-1 calls through the C ABI on the chain's workspace between replays of the chain."""
    import ctypes
    from ternel_b200 import _native
    from ternel_b200.chain import ChainPlan, Link
    from ternel_b200.format import check
    lib = _native.lib()
    blocks0, rng = random_blocks(1024, 1024, seed=71)
    blocks1, _ = random_blocks(768, 1024, seed=72)
    x = rng.standard_normal(1024).astype(np.float16)
    y0 = torch.zeros(1024, dtype=torch.float32, device="cuda")
    y1 = torch.zeros(768, dtype=torch.float32, device="cuda")
    xd, b0, b1 = to_dev(x), to_dev(blocks0), to_dev(blocks1)
    plan = ChainPlan([Link(blocks=b0, x=xd, y=y0), Link(blocks=b1, source=0, y=y1)])
    plan.run()
    torch.cuda.synchronize()
    first = y1.cpu().numpy().copy()
    single = torch.zeros(1024, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        check(lib.tq1_linear_f16(b0.data_ptr(), xd.data_ptr(), single.data_ptr(), 1, 1, 1024, 1024,
                                 plan.workspace.data_ptr(), plan.workspace.numel(), stream))
        plan.run()
        torch.cuda.synchronize()
        assert np.array_equal(single.cpu().numpy(), y0.cpu().numpy())
        assert np.array_equal(y1.cpu().numpy(), first)
    assert plan.status() == 0


def test_bad_links_are_refused_before_any_launch():
    from ternel_b200.chain import ChainPlan, Link
    from ternel_b200.format import FormatError
    blocks, rng = random_blocks(256, 1024, seed=81)
    x = to_dev(rng.standard_normal(1024).astype(np.float16))
    b = to_dev(blocks)
    with pytest.raises(FormatError):
        ChainPlan([Link(blocks=b, source=0)])                              # the first link has nothing to read
    with pytest.raises((FormatError, ValueError)):
        ChainPlan([Link(blocks=b, x=x), Link(blocks=b, source=0)])         # 256 outputs cannot feed K = 1024
    with pytest.raises((FormatError, ValueError)):
        ChainPlan([Link(blocks=to_dev(random_blocks(256, 640, seed=1)[0]), x=x[:640].contiguous())])   # K % 512


@pytest.mark.parametrize(("rows", "columns"), ((16, 512), (300, 1536), (1024, 5120), (5000, 2048)))
def test_panel_layout_is_a_lossless_permutation(rows, columns):
    """blocks -> panels -> blocks restores every byte; a panel is the chunk's [rows][112] slice, zero padded."""
    from ternel_b200.chain import blocks_to_panels, panels_to_blocks
    blocks, _ = random_blocks(rows, columns, seed=rows + columns, dist="tests")
    dev = to_dev(blocks)
    panels = blocks_to_panels(dev)
    torch.cuda.synchronize()
    host = panels.cpu().numpy()
    pad = (rows + 15) // 16 * 16
    assert host.shape == (columns // 512, pad, 112)
    want = blocks.reshape(rows, columns // 512, 112).transpose(1, 0, 2)
    assert np.array_equal(host[:, :rows], want)
    assert not host[:, rows:].any()
    back = panels_to_blocks(panels, rows)
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy(), blocks)


def test_chain_over_panels_equals_chain_over_canonical_blocks():
    """The same dependent chain streamed from either layout gives bit-identical outputs."""
    from ternel_b200.chain import ChainPlan, Link, blocks_to_panels
    rng = np.random.default_rng(77)
    shapes = ((1536, 1024), (1000, 1536), (2048, 512), (48, 2048))        # ragged row counts, several chunks
    x = to_dev(rng.standard_normal(1024).astype(np.float16))
    weights = [to_dev(random_blocks(n, k, seed=900 + i)[0]) for i, (n, k) in enumerate(shapes)]
    results = []
    for use_panels in (False, True):
        links, outs = [], []
        for i, ((n, k), w) in enumerate(zip(shapes, weights)):
            y = torch.zeros(n, dtype=torch.float32, device="cuda")
            outs.append(y)
            kwargs = dict(x=x) if i == 0 else dict(source=i - 1)
            if use_panels:
                links.append(Link(blocks=blocks_to_panels(w), panel_rows=n, y=y, out_scale=2.0, **kwargs))
            else:
                links.append(Link(blocks=w, y=y, out_scale=2.0, **kwargs))
        plan = ChainPlan(links)
        for _ in range(2):
            plan.run()
        torch.cuda.synchronize()
        assert plan.status() == 0
        results.append([y.cpu().numpy() for y in outs])
    for a, b in zip(*results):
        assert np.isfinite(a).all() and np.abs(a).max() > 0
        assert np.array_equal(a, b)


def test_row_shards_are_pushed_into_every_ranks_hand_off_area():
    """Two ranks emulated one after the other on one GPU (a kernel here never waits for the other rank): each runs
    a one-link chain over its half of the rows with both hand-off areas as peers. Afterwards BOTH areas hold the
    whole output as {FP16 bits, tag} words and each rank's y holds its own rows."""
    import ctypes
    from ternel_b200 import _native
    from ternel_b200.chain import ChainPlan, Link
    lib = _native.lib()
    rows, columns = 1024, 1536
    blocks, rng = random_blocks(rows, columns, seed=314)
    x = rng.standard_normal(columns).astype(np.float16)
    want = o.float64_matmul(blocks, x[None, :], rows=rows, columns=columns)[0]
    xd = to_dev(x)
    half = rows // 2
    shards = [to_dev(blocks[:half]), to_dev(blocks[half:])]
    ys = [torch.zeros(half, dtype=torch.float16, device="cuda") for _ in range(2)]
    probe = [Link(blocks=shards[0], x=xd, y=ys[0])]
    from ternel_b200.chain import _pack_links
    nbytes = lib.tq1_chain_handoff_bytes(_pack_links(probe), 1, 2)
    areas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    plans = [ChainPlan([Link(blocks=shards[r], x=xd, y=ys[r])], peers=(r, 2, [a.data_ptr() for a in areas]))
             for r in range(2)]
    for step in range(2):
        for r in range(2):
            plans[r].run()
        torch.cuda.synchronize()
        for r in range(2):
            assert plans[r].status() == 0
            got = ys[r].float().cpu().numpy()
            assert o.normalised_error(got[None, :], want[None, r * half:(r + 1) * half]) < 2e-3
        full = np.concatenate([ys[0].cpu().numpy(), ys[1].cpu().numpy()])
        for area in areas:
            words = area[: rows * 8].view(torch.int64).cpu().numpy()
            values = (words & 0xffff).astype(np.uint16).view(np.float16)
            tags = (words >> 32).astype(np.uint32)
            assert np.array_equal(values, full)                  # every row, from both ranks, in both areas
            assert len(set(tags.tolist())) == 1 and tags[0] == step + 1      # one tag per call of the chain


def test_column_shards_hand_over_partial_sums_that_the_reader_adds():
    """Rank 0 of two, alone on the GPU: its o-like link holds all rows and the first half of the columns, so its
    output is a partial sum that travels as an FP32 word. The other rank's partial sums are written into rank 0's
    hand-off area by the test (same tag), so the next link finds both and must read their sum, rounded once to
    FP16. A single-rank chain with a column-sharded link (one part) is checked the same way."""
    from ternel_b200 import _native
    from ternel_b200.chain import ChainPlan, Link, _pack_links
    lib = _native.lib()
    rows, columns, next_rows = 1024, 1024, 528
    rng = np.random.default_rng(99)
    w_part, _ = random_blocks(rows, columns // 2, seed=5)            # columns [0, 512) of the o-like matrix
    w_next, _ = random_blocks(next_rows, rows, seed=6)
    x_local = rng.standard_normal(columns // 2).astype(np.float16)
    other = (rng.standard_normal(rows) * 0.3).astype(np.float32)      # what rank 1 would have pushed
    part_want = o.float64_matmul(w_part, x_local[None, :].astype(np.float32), rows=rows, columns=columns // 2)[0] * 0.5
    for world in (2, 1):
        y_part = torch.zeros(rows, dtype=torch.float32, device="cuda")
        y_next = torch.zeros(next_rows, dtype=torch.float32, device="cuda")
        links = [Link(blocks=to_dev(w_part), x=to_dev(x_local), y=y_part, partial=True, out_scale=0.5),
                 Link(blocks=to_dev(w_next), source=0, y=y_next)]
        if world == 2:
            nbytes = lib.tq1_chain_handoff_bytes(_pack_links(links), len(links), 2)
            areas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
            words = (np.int64(1) << 32) | other.view(np.uint32).astype(np.int64)          # tag 1: link 0 of the first launch
            areas[0][rows * 8: 2 * rows * 8].copy_(torch.from_numpy(words.view(np.uint8)).cuda())
            plan = ChainPlan(links, peers=(0, 2, [a.data_ptr() for a in areas]))
        else:
            plan = ChainPlan(links)
        plan.run()
        torch.cuda.synchronize()
        assert plan.status() == 0
        got_part = y_part.cpu().numpy()
        assert o.normalised_error(got_part[None, :], part_want[None, :].astype(np.float32)) < 1e-5
        total = got_part + other if world == 2 else got_part
        x_next = total.astype(np.float16)
        want = o.float64_matmul(w_next, x_next[None, :].astype(np.float32), rows=next_rows, columns=rows)[0]
        assert o.normalised_error(y_next.cpu().numpy()[None, :], want[None, :].astype(np.float32)) < 1e-5
        if world == 2:      # rank 1's area received rank 0's partial sums as FP32 words
            pushed = areas[1][: rows * 8].view(torch.int64).cpu().numpy()
            assert np.array_equal((pushed & 0xffffffff).astype(np.uint32).view(np.float32), got_part)


def test_tags_close_to_wrapping_are_reported_and_results_stay_good():
    """Word 2 of the workspace is the tag base. Once it passes 0xF0000000 a launch still computes correctly but
    leaves status 7, which asks the caller to zero the workspace before the 32-bit tags wrap."""
    from ternel_b200.chain import Link, chain_workspace_bytes, linear_chain
    blocks, rng = random_blocks(528, 1024, seed=12)
    x = rng.standard_normal(1024).astype(np.float16)
    y0 = torch.zeros(528, dtype=torch.float32, device="cuda")
    y1 = torch.zeros(528, dtype=torch.float32, device="cuda")
    blocks2, _ = random_blocks(528, 512, seed=13)
    links = [Link(blocks=to_dev(blocks), x=to_dev(x), y=y0), Link(blocks=to_dev(blocks2), source=0, y=y1)]
    ws = torch.zeros(chain_workspace_bytes(links), dtype=torch.uint8, device="cuda")
    words = ws[:16].view(torch.int32)
    words[2] = -0x10000000 - 1                   # 0xEFFFFFFF: one launch of two links takes the base past 0xF0000000
    linear_chain(links, ws)
    torch.cuda.synchronize()
    assert int(words[0].item()) == 7
    want0 = o.float64_matmul(blocks, x[None, :].astype(np.float32), rows=528, columns=1024)[0]
    assert o.normalised_error(y0.cpu().numpy()[None, :], want0[None, :].astype(np.float32)) < 1e-5
    x1 = y0.cpu().numpy().astype(np.float16)[:512]
    want1 = o.float64_matmul(blocks2, x1[None, :].astype(np.float32), rows=528, columns=512)[0]
    assert o.normalised_error(y1.cpu().numpy()[None, :], want1[None, :].astype(np.float32)) < 1e-5
    ws.zero_()                                   # what the caller does on status 7
    linear_chain(links, ws)
    torch.cuda.synchronize()
    assert int(words[0].item()) == 0
