"""Write `tests/golden/flip_study.npz`: the reference's kept channels on many tokens.

Run once, in a checkout that has the reference repository importable:

    PYTHONPATH=/path/to/calibration-free-moe python tests/golden/make_flip_study.py

The golden cases of `make_golden.py` pin the selection on about sixty tokens.
This study widens that to 288 tokens per layer shape: the Qwen3-30B-A3B-shaped
layer (inputs with 1 % of the dimensions scaled by 20) and the Qwen3.5-35B-A3B-shaped
layer (Student-t inputs, biased router), 16 experts each, three seeds of 96
tokens.  For every token it runs, unmodified, the reference's independent PyTorch
reader (`tests/test_progressive_reader.py::_reference_output`, which selects with
the scores of `_reference_screen`) through a `ProgressiveReader` instance created
without its constructor, and stores

* the kept-channel mask (bit-packed),
* the reference's scores of the 64 candidates ranked around the cut (ranks
  F - 32 .. F + 31 by descending score, ties in candidate order) with their ids,
  which is where a flip can happen and what the reference's own boundary rule
  (tests/test_progressive_reader.py:630-639) needs, and
* whether the reference's two rotations (butterfly and dense matrix) keep the
  same coordinates for the token.

`tests/test_flip_study.py` compares the CPU oracle with it.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import cases  # noqa: E402
from make_golden import _reference_tests  # noqa: E402

STUDY = (("qwen3-30b-a3b", 16), ("qwen3.5-35b-a3b", 16))
SEEDS = (11, 12, 13)
TOKENS = 96
WINDOW = 32


def study_case(config: str, experts: int, seed: int, tokens: int = TOKENS):
    """The seeded inputs of one (shape, seed) cell; shared with the test."""
    return cases._synthetic(f"{config}-s{seed}", config, tokens, experts, seed)


def main() -> None:
    from calibration_free_moe.reader.progressive import ProgressiveReader, channel_major_down
    from calibration_free_moe.reader.sketch import (
        block_hadamard_signs, build_sketch, rotate_blocks,
    )

    reference = _reference_tests()
    stored = {}
    for config, experts in STUDY:
        for seed in SEEDS:
            case = study_case(config, experts, seed)
            plan = case.plan
            h, n, f = plan.hidden_size, plan.candidate_count, plan.final_count
            signs = block_hadamard_signs(h, "cpu")
            codes, statistics = build_sketch(case.gate_up, signs)
            down = channel_major_down(case.down)
            reader = object.__new__(ProgressiveReader)
            reader.plan = plan
            reader.sketch_signs = signs
            reader.sketch_codes, reader.sketch_statistics = codes, statistics
            reader.norms = down.float().square().sum(1).sqrt()
            reader.recovery_geometry = None
            reader.selection_score = "point"
            reader.activation = "silu"
            reader.selection_threshold = None
            _, selected, _ = reference._reference_output(
                reader, case.gate_up, case.down, case.encoder, case.decoder, case.hidden,
                case.ids, case.weights, None,
            )
            _, _, scores = reference._reference_screen(reader, case.hidden, case.ids, case.weights)
            order = scores.argsort(dim=1, descending=True, stable=True)
            window = order[:, f - WINDOW : f + WINDOW]
            assert torch.equal(
                torch.zeros_like(selected).scatter_(1, order[:, :f], True), selected)
            keep = plan.screen_coordinates
            dense = case.hidden.float() @ reference._dense_block_rotation(signs).T
            blocks = dense.reshape(TOKENS, -1, 128)
            top = blocks.abs().argsort(dim=-1, descending=True, stable=True)[..., :keep]
            dense_support = torch.zeros_like(blocks, dtype=torch.bool).scatter(-1, top, True)
            ranks = rotate_blocks(case.hidden, signs).reshape(TOKENS, -1, 128).abs()
            kept = ranks.argsort(dim=-1, descending=True, stable=True)[..., :keep]
            butterfly_support = torch.zeros_like(dense_support).scatter(-1, kept, True)
            key = f"{config}/{seed}"
            stored[f"{key}/selected"] = np.packbits(selected.numpy(), axis=1)
            stored[f"{key}/window_ids"] = window.to(torch.int16).numpy()
            stored[f"{key}/window_scores"] = scores.gather(1, window).numpy()
            stored[f"{key}/rotation_agrees"] = (
                (dense_support == butterfly_support).flatten(1).all(1).numpy())
            print(f"{key}: T={TOKENS} N={n} F={f} rotation ties: "
                  f"{int((~stored[f'{key}/rotation_agrees']).sum())}", flush=True)
    np.savez_compressed(Path(__file__).resolve().parent / "flip_study.npz", **stored)


if __name__ == "__main__":
    main()
