"""Helpers shared by the parity tests."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import cases
from cfm_b200.reader.progressive import channel_major_down, recovery_geometry
from cfm_b200.reader.sketch import block_hadamard_signs, build_sketch

GOLDEN = Path(__file__).resolve().parent / "golden"


def golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as data:
        return {key: data[key] for key in data.files}


def prepared(name: str) -> dict:
    """A named case's inputs plus its CPU-built sketch and channel-major down weight."""
    return prepared_case(cases.build(name))


def prepared_case(case) -> dict:
    """A case's inputs plus its CPU-built sketch and channel-major down weight."""
    signs = block_hadamard_signs(case.plan.hidden_size, "cpu")
    codes, statistics = build_sketch(case.gate_up, signs)
    down = channel_major_down(case.down)
    geometry = None
    if case.score != "point" and case.decoder is not None:
        geometry = recovery_geometry(
            down, case.encoder.transpose(1, 2).contiguous(), case.decoder,
            down.float().square().sum(1).sqrt(),
        )
    return {
        "case": case,
        "signs": signs,
        "codes": codes,
        "statistics": statistics,
        "down": down,
        "geometry": geometry,
    }


def run_oracle(oracle, item: dict, **overrides) -> dict:
    case = item["case"]
    arguments = dict(
        plan=case.plan, gate_up=case.gate_up, down=item["down"], codes=item["codes"],
        statistics=item["statistics"], signs=item["signs"], hidden=case.hidden, ids=case.ids,
        weights=case.weights, encoder=case.encoder, decoder=case.decoder,
        padding=case.padding, activation=case.activation, score=case.score,
        geometry=item.get("geometry"), threshold=case.threshold,
    )
    arguments.update(overrides)
    return oracle.forward(**arguments)


def relative_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    denominator = expected.float().norm().item()
    return (actual.float() - expected.float()).norm().item() / max(denominator, 1e-30)


def bf16_from_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)
