"""The library's kernel/tile choice replayed against the recorded B200 sweep (no GPU needed): for every
recorded (batch, shape) the chosen token tile must be within 10% of the best recorded one, the way the
reference replays its dispatch rules against committed sweeps (tests/test_mlx_modules.py:553-1084 there)."""

import pytest

from ternel_b200.dispatch import LOOPED_MAX, SWEEP_BATCHES, SWEEP_SHAPES, chosen_over_best, load_sweep, plan


def test_rule_is_near_the_best_recorded_option_everywhere():
    sweep = load_sweep()
    assert len(sweep["cases"]) == len(SWEEP_BATCHES) * len(SWEEP_SHAPES)
    worst = 1.0
    for case in sweep["cases"]:
        assert ("us_looped" in case) == (case["batch"] <= LOOPED_MAX)       # both arms recorded where both exist
        ratio, chosen = chosen_over_best(case)
        assert chosen.kernel in ("tensor_core", "stream_gemv")
        assert ratio <= 1.10, (case, chosen)
        worst = max(worst, ratio)
    assert 1.0 <= worst <= 1.10


def test_plan_boundaries():
    assert plan(1, 5120, 5120).kernel == "stream_gemv"
    assert plan(1, 5120, 5120, aligned=False).kernel == "rows"
    assert plan(1, 5120, 640).kernel == "rows"                 # K not a multiple of 512
    assert plan(4, 100, 640).kernel == "rows"
    assert plan(2, 17408, 5120).kernel == "stream_gemv"       # two passes of the batch-1 kernel in one launch
    small = plan(5, 17408, 5120)
    assert (small.kernel, small.token_tile, small.parts) == ("tensor_core", 16, 2) and small.ctas == 272
    for batch in range(5, 17):
        assert plan(batch, 5120, 17408).token_tile == 16       # up to 16 rows: always the 16-row tile
    big = plan(2048, 17408, 5120)
    assert big.token_tile == 256 and big.parts == 0 and big.ctas == 148       # stream-K over one CTA per SM
    assert plan(192, 17408, 5120).token_tile == 256            # one 256-row tile beats two 128-row tiles
    with pytest.raises(ValueError):
        plan(0, 128, 512)
