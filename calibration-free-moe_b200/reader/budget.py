"""Read budgets of the sparse decode reader and their per-token byte prices.

Host-side integer arithmetic only.  Mirrors the interface of the reference's
`calibration_free_moe/reader/budget.py` (`sketch_code_stride` :13,
`sketch_storage_bytes` :22, `PaidRound` :36, `BudgetPlan` :52,
`compile_budget` :150, `load_layer_budgets` :209) so a plan compiled by either
package compares equal field by field.

Symbols: H hidden size, I channels per expert, K experts per token,
N = K * I candidate channels per token, F channels kept per token.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

SECTOR = 32  # bytes; the unit the read cost is priced in
ROTATION_BLOCK = 128  # coordinates per Hadamard block


def _ceil_to(value: int, unit: int) -> int:
    return (value + unit - 1) // unit * unit


def _code_pairs(width: int) -> int:
    """Useful code bytes of one rotated coordinate: a gate byte and an up byte per five channels."""
    return 2 * ((width + 4) // 5)


def sketch_code_stride(rows: int) -> int:
    """Code bytes stored per rotated coordinate for `rows` = 2 I sketch rows.

    Reference layout (reader/budget.py:13): byte pairs (gate, up) of five trits
    each, padded up to a multiple of 16 bytes.
    """
    return _ceil_to(_code_pairs(rows // 2), 16)


def sketch_storage_bytes(rows: int, hidden: int) -> int:
    """Packed code bytes of one expert in the reference layout (reader/budget.py:22).

    Whole 32-byte tiles are stored coordinate-major.  When the stride leaves a
    16-byte remainder, the remainders of two neighbouring rotation blocks share
    one 32-byte sector per coordinate.
    """
    stride = sketch_code_stride(rows)
    blocks = hidden // ROTATION_BLOCK
    body, tail = stride // SECTOR * SECTOR, stride % SECTOR
    block_pairs = (blocks + 1) // 2
    return blocks * ROTATION_BLOCK * body + block_pairs * ROTATION_BLOCK * 2 * tail


@dataclass(frozen=True)
class PaidRound:
    """One stage of a plan (reference reader/budget.py:36).

    `entering_count` channels come in, the best `retained_count` go on.  The
    stage reads native input coordinates [input_start, input_end): an empty
    range is the sketch screen, the full range [0, H) an exact evaluation.
    """

    input_start: int
    input_end: int
    entering_count: int
    retained_count: int


@dataclass(frozen=True)
class BudgetPlan:
    """Token-independent read plan of one MoE layer (reference reader/budget.py:52)."""

    hidden_size: int
    expert_width: int
    top_k: int
    completion_count: int
    final_count: int
    rounds: tuple[PaidRound, ...]
    screen_coordinates: int = ROTATION_BLOCK

    def __post_init__(self) -> None:
        if self.expert_width % 16:
            raise ValueError(
                "Reader expert width must be divisible by 16 "
                "for sector-aligned sketch metadata"
            )

    # -- sizes -----------------------------------------------------------
    @property
    def candidate_count(self) -> int:
        """N = K * I."""
        return self.top_k * self.expert_width

    @property
    def screened(self) -> bool:
        """True when the sketch screen runs (fewer channels computed than candidates)."""
        return self.completion_count < self.candidate_count

    # -- prices, bytes per token ----------------------------------------
    def native_read_bytes(self) -> int:
        """Dense routed-expert BF16 bytes: gate, up and down rows of all N channels."""
        return 6 * self.candidate_count * self.hidden_size

    def selected_weight_bytes(self) -> int:
        """BF16 gate+up rows of the exactly computed channels plus down rows of the kept ones."""
        rows = 2 * self.completion_count + self.final_count
        return 2 * self.hidden_size * rows

    def sketch_read_bytes(self, residual: bool = True, sectors: bool = True) -> int:
        """Sketch bytes the batch-one screen of one token reads (reference :102).

        Per routed expert and rotation block: the code run of every kept
        coordinate, the FP16 scale plane of all 2 I rows and, with `residual`,
        the FP16 residual-variance plane.  `sectors` rounds every contiguous run
        up to 32 bytes.
        """
        if not self.screened:
            return 0

        def run(size: int) -> int:
            return _ceil_to(size, SECTOR) if sectors else size

        blocks = self.hidden_size // ROTATION_BLOCK
        code_run = run(_code_pairs(self.expert_width))
        plane = run(2 * 2 * self.expert_width)
        per_block = self.screen_coordinates * code_run + plane * (2 if residual else 1)
        return self.top_k * blocks * per_block

    def recovery_read_bytes(self, rank: int) -> int:
        """BF16 encoder rows of the N - F skipped channels and the H x R decoder."""
        return 2 * rank * (self.candidate_count - self.final_count + self.hidden_size)

    def selection_read_bytes(self, geometry: bool = True) -> int:
        """FP32 down-column norm per candidate (+ two geometry values with `geometry`)."""
        if not self.screened:
            return 0
        return (12 if geometry else 4) * self.candidate_count


def _require_positive_int(name: str, value: object) -> None:
    if type(value) is not int or value <= 0:
        raise ValueError(f"{name} must be a positive integer")


def _require_fraction(name: str, value: object) -> None:
    ok = isinstance(value, (int, float)) and math.isfinite(value) and 0 < value <= 1
    if not ok:
        raise ValueError(f"{name} must be finite and in (0, 1]")


def compile_budget(
    *,
    hidden_size: int,
    expert_width: int,
    top_k: int,
    retention: float,
    screen_keep: float = 1.0,
) -> BudgetPlan:
    """Turn a retention fraction into a plan (reference reader/budget.py:150).

    F = round(retention * N) with Python's half-to-even rounding, 1 <= F <= N.
    F < N gives two stages, screen (N -> F) then exact (F -> F); F == N gives
    the single dense stage with no screen.  `screen_keep` < 1 lets the screen
    read only ceil(128 * screen_keep) rotated coordinates per block.
    Violations raise ValueError.
    """
    _require_positive_int("hidden_size", hidden_size)
    _require_positive_int("expert_width", expert_width)
    _require_positive_int("top_k", top_k)
    _require_fraction("retention", retention)
    _require_fraction("screen_keep", screen_keep)

    candidates = top_k * expert_width
    kept_channels = round(retention * candidates)
    if kept_channels < 1 or kept_channels > candidates:
        raise ValueError("Rounded budgets must satisfy 1 <= F <= N")
    if hidden_size % ROTATION_BLOCK:
        raise ValueError("Sketch hidden width must be divisible by 128")
    coordinates = math.ceil(screen_keep * ROTATION_BLOCK)
    dense = kept_channels == candidates
    if dense and coordinates < ROTATION_BLOCK:
        raise ValueError(
            "A partial-sketch screen needs fewer selected than candidate channels"
        )
    exact = PaidRound(0, hidden_size, kept_channels, kept_channels)
    if dense:
        rounds: tuple[PaidRound, ...] = (
            PaidRound(0, hidden_size, candidates, kept_channels),
        )
    else:
        rounds = (PaidRound(0, 0, candidates, kept_channels), exact)
    return BudgetPlan(
        hidden_size,
        expert_width,
        top_k,
        kept_channels,
        kept_channels,
        rounds,
        coordinates,
    )


def load_layer_budgets(
    path: str | Path,
    *,
    layers: int,
    hidden_size: int,
    expert_width: int,
    top_k: int,
    screen_keep: float,
) -> list[BudgetPlan]:
    """Compile one plan per MoE layer from an allocation JSON (reference :209).

    The file holds `final_counts` (one F per layer, 1 <= F < N) and may hold
    `dimensions` and `screen_keep`, which must agree with the arguments.
    """
    allocation = json.loads(Path(path).read_text())
    counts = allocation["final_counts"]
    if not isinstance(counts, list) or len(counts) != layers:
        raise ValueError("Layer allocation must give one count per MoE layer")
    expected = {
        "num_hidden_layers": layers,
        "hidden_size": hidden_size,
        "expert_width": expert_width,
        "num_experts_per_tok": top_k,
    }
    dimensions = allocation.get("dimensions")
    if dimensions is not None:
        for key, value in expected.items():
            if dimensions.get(key) != value:
                raise ValueError("Layer allocation dimensions do not match the model")
    if "screen_keep" in allocation:
        theirs = math.ceil(ROTATION_BLOCK * allocation["screen_keep"])
        if theirs != math.ceil(ROTATION_BLOCK * screen_keep):
            raise ValueError("Layer allocation screen_keep does not match the reader")
    candidates = top_k * expert_width
    for count in counts:
        if type(count) is not int or not 1 <= count < candidates:
            raise ValueError("Layer counts must be integers in [1, candidate_count)")
    return [
        compile_budget(
            hidden_size=hidden_size,
            expert_width=expert_width,
            top_k=top_k,
            retention=count / candidates,
            screen_keep=screen_keep,
        )
        for count in counts
    ]
