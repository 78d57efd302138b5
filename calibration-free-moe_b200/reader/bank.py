"""The data-free recovery map of one layer, from its down projections alone.

Mirrors `subspace_bank` of the reference's builder
(`scripts/build_weight_recovery_bank.py:80-94`): the decoder U holds the top-r
left singular vectors of D = [D_0 ... D_{E-1}] (every expert's down columns,
`[H, E I]`), the encoder of expert e is B_e = U^T D_e, and no calibration data
enter.  The left singular vectors are the eigenvectors of D D^T (H x H, FP64).
Here that Gram matrix is accumulated one expert at a time, so nothing of size
H x E I is ever held, and everything runs on the device the weights are on.
"""

from __future__ import annotations

import torch
from torch import Tensor


def subspace_bank(down: Tensor, rank: int) -> tuple[Tensor, Tensor, float]:
    """Return (U `[H, r]`, U^T D_e `[E, r, I]`, captured energy fraction) for down `[E, H, I]`.

    FP64 throughout, as the reference; the caller casts to BF16
    (`ProgressiveReader` takes encoder `[E, r, I]` and decoder `[H, r]`).  The sign
    of an eigenvector is whatever the eigensolver returns; U B_e, which is what the
    reader adds, does not depend on it.
    """
    experts, hidden, width = down.shape
    if not 1 <= rank <= hidden:
        raise ValueError("Recovery rank must lie between 1 and the hidden size")
    gram = torch.zeros((hidden, hidden), device=down.device, dtype=torch.float64)
    for expert in range(experts):
        columns = down[expert].double()
        gram.addmm_(columns, columns.T)
    eigenvalues, eigenvectors = torch.linalg.eigh(gram)
    decoder = eigenvectors[:, -rank:].flip(-1)
    captured = float(eigenvalues[-rank:].sum() / eigenvalues.sum())
    encoder = torch.empty((experts, rank, width), device=down.device, dtype=torch.float64)
    for expert in range(experts):
        torch.matmul(decoder.T, down[expert].double(), out=encoder[expert])
    return decoder, encoder, captured
