"""Seeded parity cases shared by the golden-vector generator and the tests.

Each case rebuilds its inputs on the CPU from a seed, so only the expected
outputs need to be stored (`tests/golden/*.npz`, written by `make_golden.py`
from the reference's own PyTorch functions).  Shapes follow the reference's
reader tests (tests/test_progressive_reader.py: seeds 77, 181, 417, 421) and
the benchmark configurations.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import Tensor

import cfm_b200  # noqa: F401  (registers the package alias)
from cfm_b200 import synthetic
from cfm_b200.reader.budget import BudgetPlan, compile_budget


@dataclass
class Case:
    name: str
    plan: BudgetPlan
    gate_up: Tensor  # bf16 [E, 2I, H]
    down: Tensor  # bf16 logical [E, H, I], contiguous (not yet channel-major)
    encoder: Tensor | None  # bf16 [E, R, I]
    decoder: Tensor | None  # bf16 [H, R]
    hidden: Tensor  # bf16 [T, H]
    ids: Tensor  # int32 [T, K]
    weights: Tensor  # f32 [T, K]
    padding: Tensor | None = None
    activation: str = "silu"
    score: str = "point"
    threshold: float | None = None
    notes: dict = field(default_factory=dict)


def _plan(h: int, i: int, k: int, retention: float, keep: float) -> BudgetPlan:
    return compile_budget(
        hidden_size=h, expert_width=i, top_k=k, retention=retention, screen_keep=keep
    )


def _synthetic(name: str, config: str, tokens: int, experts: int | None, seed: int = 0,
               **budget) -> Case:
    shape = synthetic.CONFIGS[config]
    layer, generator = synthetic.make_layer(shape, seed, experts)
    hidden, ids, weights = synthetic.make_batch(layer, tokens, generator)
    plan = _plan(
        shape.hidden, shape.width, shape.top_k,
        budget.get("retention", shape.retention), budget.get("screen_keep", shape.screen_keep),
    )
    return Case(name, plan, layer.gate_up, layer.down, layer.encoder, layer.decoder,
                hidden, ids, weights)


def _random(name: str, seed: int, h: int, i: int, e: int, k: int, rank: int, tokens: int,
            retention: float, keep: float, activation: str = "silu",
            routes: list[list[int]] | None = None, padding: list[bool] | None = None,
            zero_input: bool = False, equal_experts: bool = False,
            score: str = "point", threshold: float | None = None) -> Case:
    g = torch.Generator().manual_seed(seed)
    gate_up = (torch.randn(e, 2 * i, h, generator=g) / h**0.5).bfloat16()
    down = (torch.randn(e, h, i, generator=g) / i**0.5).bfloat16()
    encoder = decoder = None
    if rank:
        encoder = (torch.randn(e, rank, i, generator=g) / i**0.5).bfloat16()
        decoder = (torch.randn(h, rank, generator=g) / rank**0.5).bfloat16()
    if equal_experts:
        gate_up[1:k] = gate_up[:1]
        down[1:k] = down[:1]
    hidden = torch.randn(tokens, h, generator=g).bfloat16()
    if zero_input:
        hidden.zero_()
    if routes is None:
        ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(tokens)]).int()
    else:
        ids = torch.tensor(routes, dtype=torch.int32)
    weights = torch.rand(tokens, k, generator=g) * 0.6 + 0.2
    if equal_experts:
        ids = torch.arange(k - 1, -1, -1, dtype=torch.int32).expand(tokens, -1).contiguous()
        weights = torch.full((tokens, k), 1.0 / k)
    pad = torch.tensor(padding) if padding is not None else None
    return Case(name, _plan(h, i, k, retention, keep), gate_up, down, encoder, decoder,
                hidden, ids, weights.float(), pad, activation, score, threshold)


def build(name: str) -> Case:
    """Rebuild the named case's inputs."""
    return _CASES[name]()


_CASES = {
    # Benchmark-shaped layers.
    "tiny": lambda: _synthetic("tiny", "tiny", 4, None),
    "olmoe-t1": lambda: _synthetic("olmoe-t1", "olmoe", 1, None),
    "qwen3-e16-t8": lambda: _synthetic("qwen3-e16-t8", "qwen3-30b-a3b", 8, 16),
    "qwen35-e16-t4": lambda: _synthetic("qwen35-e16-t4", "qwen3.5-35b-a3b", 4, 16),
    "wide-e8-t2": lambda: _synthetic("wide-e8-t2", "wide", 2, 8, retention=0.125,
                                     screen_keep=0.5),
    # Shapes of the reference's own reader tests.
    "nonpower-full": lambda: _random("nonpower-full", 77, 384, 160, 4, 2, 8, 2, 0.125, 1.0,
                                     routes=[[2, 0], [1, 3]]),
    "nonpower-half-gelu": lambda: _random("nonpower-half-gelu", 77, 384, 160, 4, 2, 8, 2,
                                          0.125, 0.5, "gelu_tanh", routes=[[2, 0], [1, 3]]),
    "dense-bypass": lambda: _random("dense-bypass", 77, 384, 160, 4, 2, 8, 2, 1.0, 1.0,
                                    routes=[[2, 0], [1, 3]]),
    "graph-routes": lambda: _random("graph-routes", 181, 128, 64, 4, 2, 8, 2, 0.25, 1.0,
                                    routes=[[3, 1], [2, 0]], padding=[False, True]),
    "no-bank-i528": lambda: _random("no-bank-i528", 417, 128, 528, 8, 8, 0, 4, 0.125, 0.625,
                                    equal_experts=False),
    "zero-input-ties": lambda: _random("zero-input-ties", 417, 128, 528, 8, 8, 0, 2, 0.125,
                                       0.625, zero_input=True),
    "equal-experts": lambda: _random("equal-experts", 421, 256, 96, 8, 4, 16, 3, 0.123046875,
                                     0.625, equal_experts=True),
    "gemma-gelu": lambda: _random("gemma-gelu", 419, 256, 704, 4, 2, 32, 4, 0.125, 0.625,
                                  "gelu_tanh", routes=[[0, 2], [2, 0], [1, 2], [2, 1]]),
    # The recovery-aware (Gauss-Hermite) score, with and without a recovery map.
    "gh-full": lambda: _random("gh-full", 419, 256, 512, 4, 2, 32, 4, 0.2, 1.0,
                               routes=[[0, 2], [2, 0], [1, 2], [2, 1]], score="recovery-aware"),
    "gh-keep80-gelu": lambda: _random("gh-keep80-gelu", 503, 256, 704, 4, 2, 32, 2, 0.125, 0.625,
                                      "gelu_tanh", routes=[[3, 1], [0, 2]],
                                      score="recovery-aware"),
    "gh-no-bank": lambda: _random("gh-no-bank", 257, 128, 528, 8, 8, 0, 2, 0.125, 0.625,
                                  score="recovery-aware"),
    # Threshold mode (reference tests/test_progressive_reader.py:1178-1304): F = N - 1 so the
    # cap never binds; 0.008925 sits in a wide gap of the scores (kept counts differ per token);
    # zero keeps the cap; the largest float keeps nothing.
    "threshold-mid": lambda: _random("threshold-mid", 257, 384, 160, 6, 3, 8, 4, 479 / 480, 0.625,
                                     threshold=0.008925),
    "threshold-zero": lambda: _random("threshold-zero", 257, 384, 160, 6, 3, 8, 4, 479 / 480,
                                      0.625, threshold=0.0),
    "threshold-max-gh": lambda: _random("threshold-max-gh", 257, 384, 160, 6, 3, 8, 2, 479 / 480,
                                        1.0, score="recovery-aware",
                                        threshold=3.4028234663852886e38),
}

NAMES = tuple(_CASES)
