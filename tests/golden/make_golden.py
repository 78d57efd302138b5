"""Write the golden vectors of `tests/golden/` from the reference's own code.

Run once, in a checkout that has the reference repository importable:

    PYTHONPATH=/path/to/calibration-free-moe python tests/golden/make_golden.py

For every case of `cases.py` this runs, unmodified, the reference's sketch
builder (`calibration_free_moe.reader.sketch.build_sketch`) and its independent
PyTorch reader (`tests/test_progressive_reader.py::_reference_screen` and
`_reference_output`) on the CPU, through a `ProgressiveReader` instance created
without its constructor and given only the attributes those functions read.
The stored expectations are: the kept candidate ids per token, the BF16 output,
the sketch projections and scores (subsampled for large cases), digests of the
sketch bytes, and, per token, whether the two rotations the reference uses (the
butterfly of `rotate_blocks` and the dense Sylvester matrix of its tests) keep
the same coordinates.  A token where they disagree is one the reference's own
kernel and test oracle would also disagree on; tests skip the selection
comparison for exactly those tokens.
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

import importlib.util

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import cases  # noqa: E402  (tests/golden/cases.py)


def _reference_tests():
    """Import the reference's tests/test_progressive_reader.py by file path."""
    import calibration_free_moe

    path = Path(calibration_free_moe.__file__).resolve().parents[1] / "tests" / "test_progressive_reader.py"
    spec = importlib.util.spec_from_file_location("reference_reader_tests", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def main() -> None:
    from calibration_free_moe.reader.progressive import ProgressiveReader, channel_major_down
    from calibration_free_moe.reader.sketch import (
        block_hadamard_signs,
        build_sketch,
        mask_rotated_blocks,
        rotate_blocks,
    )

    reference = _reference_tests()
    out_dir = Path(__file__).resolve().parent
    for name in cases.NAMES:
        case = cases.build(name)
        plan = case.plan
        h, n = plan.hidden_size, plan.candidate_count
        signs = block_hadamard_signs(h, "cpu")
        codes, statistics = build_sketch(case.gate_up, signs)
        down = channel_major_down(case.down)
        reader = object.__new__(ProgressiveReader)
        reader.plan = plan
        reader.sketch_signs = signs
        reader.sketch_codes, reader.sketch_statistics = codes, statistics
        reader.norms = down.float().square().sum(1).sqrt()
        reader.recovery_geometry = None
        if case.score != "point" and case.decoder is not None:
            # The geometry the reference constructor prepares (progressive.py:3359-3373),
            # evaluated here on the CPU with the same tensor operations.
            geometry = torch.zeros(case.gate_up.shape[0], plan.expert_width, 2)
            decoder_rows = case.decoder.float().T
            for expert in range(case.gate_up.shape[0]):
                original = down[expert].float().T
                response = case.encoder[expert].transpose(0, 1).contiguous().float() @ decoder_rows
                norm = reader.norms[expert]
                alpha = (original * response).sum(-1) / torch.where(
                    norm > 0, norm, torch.ones_like(norm)
                )
                beta = (response.square().sum(-1) - alpha.square()).clamp_min(0).sqrt()
                geometry[expert, :, 0] = alpha
                geometry[expert, :, 1] = beta
            reader.recovery_geometry = geometry
        reader.selection_score = case.score
        reader.activation = case.activation
        reader.selection_threshold = (
            torch.tensor([case.threshold], dtype=torch.float32)
            if case.threshold is not None
            else None
        )
        rank = case.decoder.shape[1] if case.decoder is not None else 0
        e = case.gate_up.shape[0]
        encoder = case.encoder if rank else torch.zeros(e, 1, plan.expert_width)
        decoder = case.decoder if rank else torch.zeros(h, 1)
        output, selected, _ = reference._reference_output(
            reader, case.gate_up, case.down, encoder, decoder, case.hidden, case.ids,
            case.weights, case.padding,
        )
        tokens = case.hidden.shape[0]
        stored = {
            "output_bits": output.view(torch.int16).numpy(),
            "selected_ids": np.stack(
                [
                    np.pad(row.nonzero().flatten().int().numpy(), (0, plan.final_count),
                           constant_values=-1)[: plan.final_count]
                    for row in selected
                ]
            ),
            "selected_count": selected.sum(1).int().numpy(),
            "codes_sha256": np.frombuffer(
                hashlib.sha256(codes.numpy().tobytes()).digest(), dtype=np.uint8
            ),
            "statistics_sha256": np.frombuffer(
                hashlib.sha256(
                    statistics.permute(0, 2, 3, 1).contiguous().view(torch.int16).numpy().tobytes()
                ).digest(),
                dtype=np.uint8,
            ),
        }
        if plan.completion_count < n:
            projected, _, scores = reference._reference_screen(
                reader, case.hidden, case.ids, case.weights
            )
            step = max(1, (tokens * n) // 16384)
            stored["sample_step"] = np.array(step)
            stored["scores"] = scores.reshape(-1)[::step].numpy()
            stored["projections"] = projected.permute(1, 0, 2).reshape(2, -1)[:, ::step].numpy()
            dense = case.hidden.float() @ reference._dense_block_rotation(signs).T
            blocks = dense.reshape(tokens, -1, 128)
            keep = plan.screen_coordinates
            top = blocks.abs().argsort(dim=-1, descending=True, stable=True)[..., :keep]
            dense_support = torch.zeros_like(blocks, dtype=torch.bool).scatter(-1, top, True)
            butterfly = mask_rotated_blocks(rotate_blocks(case.hidden, signs), keep)
            if keep == 128:
                butterfly_support = torch.ones_like(dense_support)
            else:
                # A kept coordinate may itself be exactly zero only for all-zero blocks.
                ranks = rotate_blocks(case.hidden, signs).reshape(tokens, -1, 128).abs()
                order = ranks.argsort(dim=-1, descending=True, stable=True)[..., :keep]
                butterfly_support = torch.zeros_like(dense_support).scatter(-1, order, True)
                assert torch.equal(
                    torch.where(butterfly_support, ranks, 0.0),
                    butterfly.reshape(tokens, -1, 128).abs(),
                )
            stored["rotation_agrees"] = (
                (dense_support == butterfly_support).flatten(1).all(1).numpy()
            )
        else:
            stored["rotation_agrees"] = np.ones(tokens, dtype=bool)
        np.savez_compressed(out_dir / f"{name}.npz", **stored)
        print(
            f"{name}: T={tokens} N={n} F={plan.final_count} "
            f"rotation_agrees={stored['rotation_agrees'].tolist()}"
        )


if __name__ == "__main__":
    main()
