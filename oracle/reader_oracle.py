"""ctypes front end of the CPU oracle (`reader_oracle.c`).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
module; the product path never does.  All tensors are CPU torch tensors.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import torch
from torch import Tensor

_HERE = Path(__file__).resolve().parent
_LIBRARY = _HERE / "_build" / "libreader_oracle.so"
_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


class _Layer(ctypes.Structure):
    _fields_ = [
        ("hidden", ctypes.c_int32),
        ("width", ctypes.c_int32),
        ("experts", ctypes.c_int32),
        ("top_k", ctypes.c_int32),
        ("final_count", ctypes.c_int32),
        ("keep", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("activation", ctypes.c_int32),
        ("global_experts", ctypes.c_int32),
        ("recovery_owner", ctypes.c_int32),
        ("gate_up", ctypes.c_void_p),
        ("down", ctypes.c_void_p),
        ("codes", ctypes.c_void_p),
        ("code_bytes", ctypes.c_int64),
        ("statistics", ctypes.c_void_p),
        ("norms", ctypes.c_void_p),
        ("encoder", ctypes.c_void_p),
        ("decoder", ctypes.c_void_p),
        ("signs", ctypes.c_void_p),
        ("expert_map", ctypes.c_void_p),
        ("score", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("geometry", ctypes.c_void_p),
        ("threshold", ctypes.c_void_p),
    ]


class _Result(ctypes.Structure):
    _fields_ = [
        (name, ctypes.c_void_p)
        for name in (
            "partial",
            "scores",
            "selected",
            "candidate_ids",
            "sorted_ids",
            "sorted_weights",
            "planes",
            "coordinates",
            "latent",
            "output",
            "routed",
            "given_scores",
            "given_selected",
        )
    ]


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc (through oracle/Makefile) if it is not built yet."""
    source = _HERE / "reader_oracle.c"
    stale = not _LIBRARY.exists() or _LIBRARY.stat().st_mtime < source.stat().st_mtime
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _LIBRARY


_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load (building first if needed) the oracle library."""
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(build()))
        lib.oracle_forward.restype = ctypes.c_int
        lib.oracle_forward.argtypes = [
            ctypes.POINTER(_Layer),
            ctypes.c_int,
            ctypes.c_void_p,
            ctypes.c_void_p,
            ctypes.c_void_p,
            ctypes.c_void_p,
            ctypes.c_int,
            ctypes.c_int,
            ctypes.POINTER(_Result),
        ]
        _lib = lib
    return _lib


def _cpu(tensor: Tensor | None, dtype: torch.dtype | None = None) -> Tensor | None:
    if tensor is None:
        return None
    tensor = tensor.detach().cpu()
    if dtype is not None:
        tensor = tensor.to(dtype)
    return tensor.contiguous()


def forward(
    *,
    plan,
    gate_up: Tensor,
    down: Tensor,
    codes: Tensor,
    statistics: Tensor,
    signs: Tensor,
    hidden: Tensor,
    ids: Tensor,
    weights: Tensor,
    encoder: Tensor | None = None,
    decoder: Tensor | None = None,
    norms: Tensor | None = None,
    padding: Tensor | None = None,
    expert_map: Tensor | None = None,
    recovery_owner: bool = True,
    activation: str = "silu",
    fp32: bool = False,
    threads: int | None = None,
    given_scores: Tensor | None = None,
    given_selected: Tensor | None = None,
    score: str = "point",
    geometry: Tensor | None = None,
    threshold: float | None = None,
) -> dict[str, Tensor]:
    """Run the oracle on T tokens.

    gate_up is BF16 `[E, 2I, H]`; down the channel-major down weight (logical
    `[E, H, I]`, stride `(H I, 1, H)`); codes/statistics the reference-layout
    sketch from `build_sketch`; encoder `[E, R, I]`, decoder `[H, R]` BF16 or
    None.  Returns projections, scores, selection, the per-token candidate list,
    the latent and the output (`[T, H]` FP32 holding BF16-rounded values, or the
    unrounded FP32 evaluation with `fp32=True`).  `given_scores` `[T, N]` replaces
    the computed scores for the selection (expert parallelism: the sum over
    ranks); `given_selected` `[T, N]` is a kept-channel mask used instead of any
    selection; `score` picks the selection score and `geometry` `[E, I, 2]` holds
    the recovery geometry of the recovery-aware score (zeros if None); `threshold`
    switches to the threshold mode (scores at or above it, at most F per token); `routed` in the result is the FP32 router-weighted sum of the
    local slots before the decoder term.
    """
    lib = load()
    h, i, k = plan.hidden_size, plan.expert_width, plan.top_k
    f, keep = plan.final_count, plan.screen_coordinates
    e = gate_up.shape[0]
    n, blocks = k * i, h // 128
    rank = decoder.shape[1] if decoder is not None else 0
    tokens = hidden.shape[0]

    gate_up = _cpu(gate_up, torch.bfloat16)
    down_rows = _cpu(down.transpose(1, 2), torch.bfloat16)  # physical [E, I, H]
    codes = _cpu(codes, torch.uint8)
    stats = _cpu(statistics.permute(0, 2, 3, 1), torch.float16)  # [E, B, 2, 2I]
    if norms is None:
        norms = down.float().square().sum(1).sqrt()
    norms = _cpu(norms, torch.float32)
    encoder = _cpu(encoder, torch.bfloat16)
    decoder = _cpu(decoder, torch.bfloat16)
    signs = _cpu(signs, torch.int8)
    hidden = _cpu(hidden, torch.bfloat16)
    ids64 = _cpu(ids, torch.int64)
    weights32 = _cpu(weights, torch.float32)
    pad = _cpu(padding, torch.uint8) if padding is not None else None
    emap = _cpu(expert_map, torch.int32) if expert_map is not None else None
    geometry32 = _cpu(geometry, torch.float32) if geometry is not None else None
    threshold32 = torch.tensor([threshold], dtype=torch.float32) if threshold is not None else None

    def pointer(tensor: Tensor | None) -> int | None:
        return tensor.data_ptr() if tensor is not None else None

    layer = _Layer(
        h, i, e, k, f, keep, rank, _ACTIVATIONS[activation],
        emap.numel() if emap is not None else 0, int(recovery_owner),
        pointer(gate_up), pointer(down_rows), pointer(codes), codes.shape[1],
        pointer(stats), pointer(norms), pointer(encoder), pointer(decoder),
        pointer(signs), pointer(emap),
        {"point": 0, "recovery-aware": 1}[score], 0, pointer(geometry32), pointer(threshold32),
    )
    out = {
        "partial": torch.zeros(tokens, 2, n),
        "scores": torch.zeros(tokens, n),
        "selected": torch.zeros(tokens, n, dtype=torch.uint8),
        "candidate_ids": torch.zeros(tokens, f, dtype=torch.int32),
        "sorted_ids": torch.zeros(tokens, k, dtype=torch.int32),
        "sorted_weights": torch.zeros(tokens, k),
        "planes": torch.zeros(tokens, blocks, keep),
        "coordinates": torch.zeros(tokens, blocks, keep, dtype=torch.int32),
        "latent": torch.zeros(tokens, max(rank, 1)),
        "output": torch.zeros(tokens, h),
        "routed": torch.zeros(tokens, h),
    }
    given = _cpu(given_scores, torch.float32) if given_scores is not None else None
    mask = _cpu(given_selected, torch.uint8) if given_selected is not None else None
    result = _Result(
        *(out[name].data_ptr() for name, _ in _Result._fields_[:-2]),
        given.data_ptr() if given is not None else None,
        mask.data_ptr() if mask is not None else None,
    )
    if threads is None:
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    code = lib.oracle_forward(
        ctypes.byref(layer), tokens, pointer(hidden), pointer(ids64), pointer(weights32),
        pointer(pad), int(fp32), int(threads), ctypes.byref(result),
    )
    if code:
        raise ValueError("oracle rejected the dimensions")
    out["selected"] = out["selected"].bool()
    out["latent"] = out["latent"][:, :rank]
    out["threads"] = min(int(threads), tokens)
    return out
