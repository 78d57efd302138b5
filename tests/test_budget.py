"""Read budgets: plan compilation and byte pricing (reference tests/test_budget.py)."""

import json

import pytest

from cfm_b200.reader.budget import (
    PaidRound,
    compile_budget,
    load_layer_budgets,
    sketch_code_stride,
    sketch_storage_bytes,
)


@pytest.mark.parametrize("screen_keep,coordinates", [(1.0, 128), (0.625, 80)])
def test_plan_rounds_and_prices(screen_keep, coordinates):
    plan = compile_budget(
        hidden_size=2048, expert_width=1024, top_k=8, retention=0.15, screen_keep=screen_keep
    )
    n, h, f = 8192, 2048, plan.final_count
    assert plan.rounds == (PaidRound(0, 0, n, f), PaidRound(0, h, f, f))
    assert plan.screen_coordinates == coordinates
    assert plan.sketch_read_bytes() == 8 * 16 * (coordinates * 416 + 2 * 4096)
    assert plan.sketch_read_bytes(sectors=False) == 8 * 16 * (coordinates * 410 + 2 * 4096)
    assert plan.sketch_read_bytes(residual=False) == 8 * 16 * (coordinates * 416 + 4096)
    assert plan.selected_weight_bytes() == 2 * h * 3 * f
    assert plan.selection_read_bytes() == 12 * n
    assert plan.selection_read_bytes(False) == 4 * n
    assert plan.native_read_bytes() == 6 * n * h
    assert plan.recovery_read_bytes(32) == 64 * (n - f + h)


def test_benchmark_config_prices():
    # Per-token read cost of the Qwen3-30B-A3B-shaped layer at the deployed budget.
    plan = compile_budget(
        hidden_size=2048, expert_width=768, top_k=8, retention=0.123046875, screen_keep=0.625
    )
    assert (plan.final_count, plan.screen_coordinates) == (756, 80)
    assert plan.selected_weight_bytes() == 9_289_728
    assert plan.sketch_read_bytes(residual=False) == 3_670_016
    assert plan.recovery_read_bytes(64) == 951_808
    assert plan.selection_read_bytes(False) == 24_576
    assert plan.native_read_bytes() == 75_497_472


def test_dense_bypass():
    dense = compile_budget(hidden_size=128, expert_width=32, top_k=4, retention=1)
    assert dense.rounds == (PaidRound(0, 128, 128, 128),)
    assert dense.sketch_read_bytes() == 0
    assert dense.selection_read_bytes() == 0


@pytest.mark.parametrize(("retention", "f"), [(2.5 / 32, 2), (3.5 / 32, 4), (3 / 32, 3)])
def test_half_even_rounding(retention, f):
    plan = compile_budget(hidden_size=128, expert_width=16, top_k=2, retention=retention)
    assert (plan.final_count, plan.completion_count) == (f, f)


@pytest.mark.parametrize("screen_keep", [0.625, 1.0])
def test_width_not_multiple_of_16_rejected(screen_keep):
    with pytest.raises(ValueError, match=r"divisible by 16.*sketch metadata"):
        compile_budget(
            hidden_size=128, expert_width=88, top_k=1, retention=0.125, screen_keep=screen_keep
        )


@pytest.mark.parametrize(
    ("hidden", "width", "retention"),
    [(0, 16, 0.1), (64, 16, 0.1), (128, 0, 0.1), (128, 16, 0), (128, 16, float("nan")),
     (128, 16, 0.01), (128, 16, 1.5)],
)
def test_invalid_budgets(hidden, width, retention):
    with pytest.raises(ValueError):
        compile_budget(hidden_size=hidden, expert_width=width, top_k=2, retention=retention)


def test_partial_screen_needs_pruning():
    with pytest.raises(ValueError):
        compile_budget(hidden_size=128, expert_width=16, top_k=2, retention=1.0, screen_keep=0.5)


def test_strides_and_storage():
    assert [sketch_code_stride(2 * i) for i in (768, 1024, 512, 1536)] == [320, 416, 208, 624]
    assert sketch_storage_bytes(2 * 768, 2048) == 655_360
    # I = 512: six whole tiles and one shared tail sector per coordinate pair of blocks.
    assert sketch_storage_bytes(2 * 512, 256) == 2 * 128 * 192 + 128 * 32


def test_layer_budgets(tmp_path):
    path = tmp_path / "allocation.json"
    path.write_text(json.dumps({"final_counts": [4, 8], "screen_keep": 0.625}))
    plans = load_layer_budgets(
        path, layers=2, hidden_size=128, expert_width=16, top_k=2, screen_keep=0.625
    )
    assert [p.final_count for p in plans] == [4, 8]
    path.write_text(json.dumps({"final_counts": [4]}))
    with pytest.raises(ValueError):
        load_layer_budgets(
            path, layers=2, hidden_size=128, expert_width=16, top_k=2, screen_keep=0.625
        )
    path.write_text(json.dumps({"final_counts": [4, 32]}))
    with pytest.raises(ValueError):
        load_layer_budgets(
            path, layers=2, hidden_size=128, expert_width=16, top_k=2, screen_keep=0.625
        )
