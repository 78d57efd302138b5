"""The oracle's kept channels against the reference's on 576 tokens (`flip_study.npz`).

`tests/golden/make_flip_study.py` stored, for 288 tokens of each of two layer
shapes, what the reference's own PyTorch reader keeps.  The oracle computes its
block dot products in 22-bit fixed point and its scores in pinned FP32
arithmetic, the reference in torch FP32 with its own reduction trees, so a
candidate whose score sits within rounding of the cut may be kept by one and
dropped by the other.  This test counts those flips and requires every one of
them to be explained the way the reference's own test explains flips between
its kernel and its oracle (tests/test_progressive_reader.py:630-639): the
flipped candidate's score lies within twice the largest score difference of the
cut; or the token is one where the reference's two rotations already disagree
about the kept coordinates.  The counts are printed (run with -s).
"""

import numpy as np
import pytest
import torch

from helpers import GOLDEN, prepared_case, run_oracle

import make_flip_study as study


def cells():
    return [(config, experts, seed) for config, experts in study.STUDY for seed in study.SEEDS]


@pytest.fixture(scope="module")
def stored():
    with np.load(GOLDEN / "flip_study.npz") as data:
        return {key: data[key] for key in data.files}


@pytest.mark.parametrize("config,experts,seed", cells())
def test_flips_against_the_reference_are_boundary_cases(oracle, stored, config, experts, seed):
    case = study.study_case(config, experts, seed)
    plan = case.plan
    n, f = plan.candidate_count, plan.final_count
    got = run_oracle(oracle, prepared_case(case))
    key = f"{config}/{seed}"
    want = torch.from_numpy(np.unpackbits(stored[f"{key}/selected"], axis=1)[:, :n]).bool()
    window_ids = torch.from_numpy(stored[f"{key}/window_ids"].astype(np.int64))
    window_scores = torch.from_numpy(stored[f"{key}/window_scores"])
    agrees = torch.from_numpy(stored[f"{key}/rotation_agrees"])
    assert torch.equal(want.sum(1), torch.full((study.TOKENS,), f))
    assert torch.equal(got["selected"].sum(1), want.sum(1))
    flipped = got["selected"] ^ want
    tokens_with_flips = flipped.any(1)
    boundary = rotation = 0
    for token in tokens_with_flips.nonzero().flatten().tolist():
        channels = flipped[token].nonzero().flatten()
        if not bool(agrees[token]):
            rotation += len(channels) // 2
            continue
        ids, reference_scores = window_ids[token], window_scores[token]
        mine = got["scores"][token][ids]
        error = (reference_scores - mine).abs().max()
        cutoff = reference_scores[study.WINDOW - 1]  # the F-th largest score
        for channel in channels.tolist():
            at = (ids == channel).nonzero().flatten()
            assert len(at) == 1, f"token {token}: flipped channel {channel} is far from the cut"
            assert abs(float(reference_scores[at[0]] - cutoff)) <= 2 * float(error), (
                f"token {token}: channel {channel} flipped away from the cut")
        boundary += len(channels) // 2
    # Away from rotation ties the scores agree to FP32 rounding on the window around the cut.
    comparable = agrees.nonzero().flatten()
    ids = window_ids[comparable]
    torch.testing.assert_close(got["scores"][comparable].gather(1, ids), window_scores[comparable],
                               rtol=0.025, atol=2e-5)
    print(f"{key}: {study.TOKENS} tokens x {f} kept channels: "
          f"{int(tokens_with_flips.sum())} tokens with a flip, {boundary} boundary flips, "
          f"{rotation} flips on tokens with a rotation tie")
