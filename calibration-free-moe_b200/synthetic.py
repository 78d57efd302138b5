"""Seeded synthetic MoE layers and decode batches.

Stand-ins for real checkpoints and evaluation panels, which this repository
does not ship: random BF16 expert weights of a named model's layer shape,
random-orthonormal recovery factors, hidden states of a stated distribution and
router outputs computed from them.  All draws come from one CPU
`torch.Generator` in a fixed order (gate/up, down, router, decoder, encoder,
hidden, bias), in FP32, then cast, so a (config, seed, tokens) triple names the
same tensors on every machine.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor


@dataclass(frozen=True)
class LayerShape:
    """Dimensions and budget of one benchmark configuration."""

    name: str
    hidden: int
    experts: int
    width: int
    top_k: int
    rank: int
    sigma: float
    retention: float = 0.123046875
    screen_keep: float = 0.625
    renormalize: bool = True
    input_kind: str = "normal"  # normal | outliers | student_t
    router_bias: bool = False


# The layer shapes the benchmark configurations name.
CONFIGS = {
    "olmoe": LayerShape("olmoe", 2048, 64, 1024, 8, 64, 0.02, renormalize=False),
    "qwen3-30b-a3b": LayerShape(
        "qwen3-30b-a3b", 2048, 128, 768, 8, 64, 0.02, input_kind="outliers"
    ),
    "qwen3.5-35b-a3b": LayerShape(
        "qwen3.5-35b-a3b", 2048, 256, 512, 8, 64, 0.02, input_kind="student_t",
        router_bias=True,
    ),
    "wide": LayerShape("wide", 4096, 128, 1536, 8, 128, 0.015),
    # A small shape with the structure of the above, for quick checks.
    "tiny": LayerShape("tiny", 256, 8, 64, 2, 8, 0.05, retention=0.125),
}


@dataclass
class SyntheticLayer:
    shape: LayerShape
    gate_up: Tensor  # bf16 [E, 2I, H]
    down: Tensor  # bf16 logical [E, H, I] (not yet channel-major)
    router: Tensor  # bf16 [E, H]
    decoder: Tensor  # bf16 [H, R]
    encoder: Tensor  # bf16 [E, R, I]


def _orthonormal(rows: int, columns: int, generator: torch.Generator) -> Tensor:
    q, _ = torch.linalg.qr(torch.randn(rows, columns, generator=generator))
    return q


def make_layer(shape: LayerShape, seed: int = 0, experts: int | None = None) -> tuple[SyntheticLayer, torch.Generator]:
    """Draw one layer's weights on the CPU; returns them and the generator for the inputs.

    `experts` overrides the expert count (the draw order keeps the first experts
    of a smaller layer different from those of the full one; it only shortens
    test time).
    """
    g = torch.Generator().manual_seed(seed)
    e = experts if experts is not None else shape.experts
    h, i, r = shape.hidden, shape.width, shape.rank
    gate_up = (torch.randn(e, 2 * i, h, generator=g) * shape.sigma).bfloat16()
    down = (torch.randn(e, h, i, generator=g) * shape.sigma).bfloat16()
    router = (torch.randn(e, h, generator=g) * shape.sigma).bfloat16()
    decoder = _orthonormal(h, r, g).bfloat16()
    encoder = torch.stack([_orthonormal(i, r, g).T for _ in range(e)]).bfloat16()
    return SyntheticLayer(shape, gate_up, down, router, decoder, encoder), g


def make_batch(layer: SyntheticLayer, tokens: int, generator: torch.Generator) -> tuple[Tensor, Tensor, Tensor]:
    """Draw hidden states and route them: (hidden bf16 [T,H], ids int32 [T,K], weights f32 [T,K])."""
    shape = layer.shape
    h, k = shape.hidden, shape.top_k
    if shape.input_kind == "student_t":
        # Student-t with 3 degrees of freedom, scaled to unit variance.
        z = torch.randn(tokens, h, generator=generator)
        chi = torch.randn(tokens, h, 3, generator=generator).square().sum(-1)
        x = z / (chi / 3).sqrt() / math.sqrt(3.0)
    else:
        x = torch.randn(tokens, h, generator=generator)
        if shape.input_kind == "outliers":
            count = math.ceil(0.01 * h)
            dims = torch.randperm(h, generator=generator)[:count]
            x[:, dims] *= 20.0
    hidden = x.bfloat16()
    logits = hidden.float() @ layer.router.float().T
    if shape.router_bias:
        logits = logits + torch.randn(layer.router.shape[0], generator=generator)
    probabilities = torch.softmax(logits, dim=-1, dtype=torch.float32)
    weights, ids = probabilities.topk(k, dim=-1)
    if shape.renormalize:
        weights = weights / weights.sum(-1, keepdim=True)
    return hidden, ids.int(), weights.float().contiguous()
