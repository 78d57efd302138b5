"""The reader's caller inside a serving engine, without the engine.

Mirrors the reader branch of the reference's vLLM binding
(`calibration_free_moe/runtime/experts.py`: `reader_rows` :334-378,
`ProgressiveExperts.prepare_reader_input` :402-427, `forward_modular` :429-485,
`policy` :487-516, `reader_work_report` :110-188) as engine-neutral code: the
three fields the reference's vLLM patch adds to the forward context arrive as a
`PhaseContext`, and the stock fused-MoE path that serves prefill rows is a
callable.  The reference binds vLLM 0.29 with two patches; that engine version is
not what this package is tied to, so the binding to a concrete engine is one
small adapter that builds a `PhaseContext` and passes the engine's fused-MoE call.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterable

import torch
from torch import Tensor

from ..activation import GatedActivation, activate
from ..reader.progressive import ProgressiveReader

StockExperts = Callable[[Tensor, Tensor, Tensor], Tensor]  # (x, topk_weights, topk_ids) -> out


@dataclass
class PhaseContext:
    """Which rows of a forward batch take the sparse policy.

    The fields of the reference's phase-metadata patch
    (patches/vllm-0.29.0-phase-metadata.patch): decode rows come first, so policy
    rows are the prefix `[0, num_decode_tokens)` unless a prefill recomputes
    generated tokens, when `generated_prefill_split` lists (policy rows, stock
    rows); `is_padding` marks padded rows of a captured batch.
    """

    num_decode_tokens: int
    generated_prefill_split: tuple[Tensor, Tensor] | None = None
    is_padding: Tensor | None = None


def reader_rows(
    reader: ProgressiveReader,
    x: Tensor,
    ids: Tensor,
    weights: Tensor,
    padding: Tensor | None,
    rows: int,
) -> Tensor:
    """Run the reader on any token count, in calls of at most `rows` (reference :334-378).

    Each token's output depends only on its own state and routing, and this
    reader's selections do not depend on the batch, so chunking changes nothing
    but the order of FP32 partial sums in the outputs.  Chunks are written into
    their rows of one output, in order, on the caller's stream.
    """
    if x.shape[0] <= rows:
        return reader(x, ids, weights, padding)
    output = torch.empty_like(x)
    for start in range(0, x.shape[0], rows):
        end = start + rows
        reader(
            x[start:end],
            ids[start:end],
            weights[start:end],
            padding[start:end] if padding is not None else None,
            out=output[start:end],
        )
    return output


def dense_routed_experts(
    gate_up: Tensor, down: Tensor, activation: GatedActivation = "silu"
) -> StockExperts:
    """A plain PyTorch routed-expert MLP for rows outside the policy (prefill).

    Stands where the engine's stock fused MoE is in the reference; gate_up
    `[E, 2I, H]`, down logical `[E, H, I]`.  Not part of the decode hot path.
    """

    def forward(x: Tensor, topk_weights: Tensor, topk_ids: Tensor) -> Tensor:
        out = torch.zeros(x.shape, device=x.device, dtype=torch.float32)
        width = gate_up.shape[1] // 2
        for expert in topk_ids.unique().tolist():
            token, slot = (topk_ids == expert).nonzero(as_tuple=True)
            rows = x[token]
            gate, up = (rows @ gate_up[expert].T).float().split(width, dim=-1)
            hidden = (activate(gate, activation) * up).to(x.dtype)
            routed = (hidden @ down[expert].T).float()
            out.index_add_(0, token, routed * topk_weights[token, slot].float()[:, None])
        return out.to(x.dtype)

    return forward


class ProgressiveExperts:
    """Routes policy rows through the sparse reader and the rest through the stock experts."""

    def __init__(
        self,
        reader: ProgressiveReader,
        stock: StockExperts,
        max_policy_rows: int | None = None,
        sparse_prefill: bool = False,
    ) -> None:
        self.reader = reader
        self.stock = stock
        self.max_policy_rows = max_policy_rows or reader.max_tokens
        if self.max_policy_rows > reader.max_tokens:
            raise ValueError("max_policy_rows exceeds the reader's capacity")
        self.sparse_prefill = sparse_prefill
        self.reader_input_prepared = False

    def prepare_reader_input(self, x: Tensor, context: PhaseContext) -> None:
        """Start the input rotation before the router runs (reference :402-427).

        Only when all rows are policy rows of one reader call; otherwise nothing.
        """
        rows = x.shape[0]
        whole = (
            context.generated_prefill_split is None
            and (self.sparse_prefill or context.num_decode_tokens == rows)
            and rows <= self.max_policy_rows
        )
        self.reader_input_prepared = whole and self.reader.prepare_input(x, context.is_padding)

    def forward_modular(
        self, x: Tensor, topk_weights: Tensor, topk_ids: Tensor, context: PhaseContext
    ) -> Tensor:
        """Policy rows to the reader, the rest to the stock experts (reference :429-485)."""
        count, split = context.num_decode_tokens, context.generated_prefill_split
        if self.sparse_prefill:
            count, split = x.shape[0], None
        if split is not None:
            count = split[0].numel()
        if count == 0 and split is None:
            return self.stock(x, topk_weights, topk_ids)
        if split is None:
            sparse = self.policy(slice(0, count), x, topk_weights, topk_ids, context)
            if count == x.shape[0]:
                return sparse
            prefill = self.stock(x[count:], topk_weights[count:], topk_ids[count:])
            return torch.cat((sparse, prefill), dim=0)
        policy_rows, stock_rows = split
        output = torch.empty_like(x)
        output[policy_rows] = self.policy(policy_rows, x, topk_weights, topk_ids, context)
        if stock_rows.numel():
            output[stock_rows] = self.stock(
                x[stock_rows], topk_weights[stock_rows], topk_ids[stock_rows]
            )
        return output

    def policy(
        self,
        rows: slice | Tensor,
        x: Tensor,
        topk_weights: Tensor,
        topk_ids: Tensor,
        context: PhaseContext,
    ) -> Tensor:
        """Run the reader on `rows`; its read statistics include them (reference :487-516)."""
        padding = context.is_padding
        row_padding = padding[rows].contiguous() if padding is not None else None
        chunk = (x[rows].contiguous(), topk_ids[rows].contiguous(), topk_weights[rows].contiguous())
        if self.reader_input_prepared:
            self.reader_input_prepared = False
            return self.reader(*chunk, row_padding, input_prepared=True)
        return reader_rows(self.reader, *chunk, row_padding, self.max_policy_rows)


def reader_work_report(readers: Iterable[ProgressiveReader]) -> dict[str, float | None]:
    """Sum the layers' read statistics; ratios are recomputed from the sums (reference :110-188)."""
    total: dict[str, float] = {}
    for reader in readers:
        for key, value in reader.report().items():
            if isinstance(value, (int, float)) and not key.endswith("_fraction"):
                total[key] = total.get(key, 0.0) + float(value)
    reference = total.get("reference_bytes", 0.0)
    report: dict[str, float | None] = dict(total)
    report["read_fraction"] = total.get("charged_bytes", 0.0) / reference if reference else None
    report["logical_read_fraction"] = (
        total.get("logical_charged_bytes", 0.0) / reference if reference else None
    )
    return report
