"""Gate nonlinearities of the routed experts (reference calibration_free_moe/activation.py:10-28)."""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

GatedActivation = Literal["silu", "gelu_tanh"]

# Integer codes passed through the C ABI.
ACTIVATION_CODES = {"silu": 0, "gelu_tanh": 1}


def model_activation(config: object) -> GatedActivation:
    """Map a Hugging Face `hidden_activation` to the reader's name; SiLU when absent."""
    name = getattr(config, "hidden_activation", "silu")
    if name in ("silu", "swiglu"):
        return "silu"
    if name in ("gelu_tanh", "gelu_pytorch_tanh"):
        return "gelu_tanh"
    raise ValueError(f"Unsupported routed expert activation: {name}")


def activate(gate: Tensor, activation: GatedActivation) -> Tensor:
    """phi(gate): SiLU, or GELU in its tanh approximation."""
    if activation == "gelu_tanh":
        return torch.nn.functional.gelu(gate, approximate="tanh")
    return torch.nn.functional.silu(gate)
