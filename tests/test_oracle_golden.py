"""Pin the CPU oracle against golden vectors made by the reference's own PyTorch reader.

The goldens come from `tests/golden/make_golden.py`, which runs the reference's
`_reference_screen` / `_reference_output` (tests/test_progressive_reader.py:102-267)
unmodified.  Selections must be identical; outputs agree to the reference's own
tolerance (rtol 0.025, atol 0.02, :823) and within 1e-2 relative L2; sketch
projections to 2e-4 (:429-433).
"""

import numpy as np
import pytest
import torch

import cases
from helpers import bf16_from_bits, golden, prepared, relative_l2, run_oracle

FAST = [n for n in cases.NAMES if n != "olmoe-t1"]


@pytest.mark.parametrize("name", FAST + ["olmoe-t1"])
def test_oracle_matches_reference_golden(oracle, name):
    item = prepared(name)
    case, expected = item["case"], golden(name)
    got = run_oracle(oracle, item)
    plan = case.plan
    tokens, n, f = case.hidden.shape[0], plan.candidate_count, plan.final_count
    active = torch.ones(tokens, dtype=torch.bool)
    if case.padding is not None:
        active = ~case.padding
    agrees = torch.from_numpy(expected["rotation_agrees"])
    # Selection: bit-exact wherever the reference's two rotations agree with each other.
    comparable = active & agrees
    assert comparable.any()
    ids = torch.from_numpy(expected["selected_ids"])
    assert torch.equal(got["candidate_ids"][comparable], ids[comparable])
    if case.threshold is None:
        assert (got["selected"].sum(1)[active] == f).all()
    else:
        assert torch.equal(
            got["selected"].sum(1)[active],
            torch.from_numpy(expected["selected_count"]).long()[active],
        )
    # Output.
    reference_out = bf16_from_bits(expected["output_bits"]).float()
    torch.testing.assert_close(
        got["output"][comparable], reference_out[comparable], rtol=0.025, atol=0.02
    )
    assert relative_l2(got["output"][comparable], reference_out[comparable]) < 1e-2
    if case.padding is not None:
        assert not got["output"][case.padding].any()
    # Sketch projections and scores on the stored subsample.
    if plan.completion_count < n:
        step = int(expected["sample_step"])
        rows = comparable.repeat_interleave(n)[::step]
        projections = got["partial"].permute(1, 0, 2).reshape(2, -1)[:, ::step]
        torch.testing.assert_close(
            projections[:, rows], torch.from_numpy(expected["projections"])[:, rows],
            rtol=2e-4, atol=2e-5,
        )
        scores = got["scores"].reshape(-1)[::step]
        torch.testing.assert_close(
            scores[rows], torch.from_numpy(expected["scores"])[rows], rtol=0.025, atol=2e-5
        )


def test_zero_input_selects_first_candidates(oracle):
    item = prepared("zero-input-ties")
    got = run_oracle(oracle, item)
    f = item["case"].plan.final_count
    assert torch.equal(got["candidate_ids"], torch.arange(f, dtype=torch.int32).expand(2, -1))
    assert not got["output"].any()


def test_fp32_evaluation_within_one_percent(oracle):
    for name in ("tiny", "qwen3-e16-t8", "gemma-gelu"):
        item = prepared(name)
        rounded = run_oracle(oracle, item)
        exact = run_oracle(oracle, item, fp32=True)
        assert torch.equal(rounded["selected"], exact["selected"])
        assert relative_l2(rounded["output"], exact["output"]) < 1e-2


def test_oracle_is_thread_count_invariant(oracle):
    item = prepared("qwen35-e16-t4")
    one = run_oracle(oracle, item, threads=1)
    many = run_oracle(oracle, item, threads=4)
    for key in ("scores", "candidate_ids", "output", "partial"):
        assert torch.equal(one[key], many[key])
