"""Expert-parallel sparse decode reader: experts sharded over the ranks of one box.

Every rank holds `E / P` consecutive experts (linear placement, as the
reference's binding requires: runtime/experts.py:677-692) with their gate/up and
down rows, sketch, norms and encoder rows; the decoder is replicated.  Tokens
are data parallel: every rank brings its own `T` decode tokens and gets their
outputs back.

One layer call, on every rank:

1. dispatch   every rank's tokens, router ids and weights reach the ranks that
              own their experts (`all_gather` of the hidden rows and of one packed
              routing record per token; with K = 8 experts over at most 8 ranks
              nearly every token has an expert on every rank, so the dispatch of
              a static-shape decode step is the gather of all rows);
2. screen     each rank scores the candidate channels of its local experts for
              all `P * T` tokens; slots of remote experts score zero;
3. exchange   the per-token top-F is global over the token's K experts: the
              score rows are summed onto each token's home rank
              (`reduce_scatter`), the home rank finds the cut (the F-th largest
              score and, per slot, how many candidates tied with it are kept)
              and publishes 4 (K + 1) bytes per token (`all_gather`);
4. local      each rank repeats the selection for its own slots from the cut,
              computes those channels exactly, their down rows and its share of
              the recovery latent;
5. combine    one FP32 row per token (router-weighted partial output followed
              by the partial latent) goes back to the token's home rank
              (`reduce_scatter`), which adds the decoder term and stores BF16.

Compared with the reference's expert-parallel mode (replicated tokens, scores
all-reduced, caller all-reduces BF16 outputs: progressive.py:4245-4251,
tests/test_expert_parallel_reader.py:128-130) tokens stay sharded, the selection
runs once per token instead of once per rank, and the output is reduced in FP32
before its single BF16 rounding.  The kept channels are the same bit for bit.

The collectives are plain `torch.distributed` calls on tensors, so the same
orchestration runs over NCCL with the CUDA engine and over gloo with a CPU
engine in the tests.
"""

from __future__ import annotations

import ctypes
from typing import Protocol

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _native
from .budget import BudgetPlan
from .progressive import ProgressiveReader


def linear_expert_map(global_experts: int, world: int, rank: int) -> Tensor:
    """Global-to-local expert ids of `rank` under linear placement (-1 = remote)."""
    if global_experts % world:
        raise ValueError("Expert count must divide evenly over the expert-parallel ranks")
    local = global_experts // world
    mapping = torch.full((global_experts,), -1, dtype=torch.int32)
    mapping[rank * local : (rank + 1) * local] = torch.arange(local, dtype=torch.int32)
    return mapping


class Engine(Protocol):
    """What the orchestration needs from one rank's compute back end."""

    def screen(self, hidden: Tensor, ids: Tensor, weights: Tensor, padding: Tensor | None) -> Tensor:
        """Score buffer `[rows, N]`: the local experts' channels scored, zero elsewhere."""

    def find_cuts(self, first_row: int, rows: int) -> Tensor:
        """Cut buffer `[all rows, 1 + K]` with rows `first_row ..` filled from the summed scores."""

    def local(self) -> Tensor:
        """From the gathered cuts: FP32 rows `[all rows, H + R]` (partial output, partial latent)."""

    def finish(self, combined: Tensor) -> Tensor:
        """Home-rank output `[T, H]` BF16 from the summed rows."""


def _all_gather_rows(tensor: Tensor, world: int, group) -> Tensor:
    out = tensor.new_empty((world * tensor.shape[0], *tensor.shape[1:]))
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, tensor.contiguous(), group=group)
    else:
        dist.all_gather(list(out.chunk(world)), tensor.contiguous(), group=group)
    return out


def _all_gather_in_place(buffer: Tensor, world: int, rank: int, group) -> None:
    """Fill `buffer` (rows of all ranks) from each rank's own block of rows."""
    rows = buffer.shape[0] // world
    mine = buffer[rank * rows : (rank + 1) * rows]
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(buffer, mine, group=group)
    else:
        dist.all_gather(list(buffer.chunk(world)), mine.clone(), group=group)


def _reduce_scatter_in_place(buffer: Tensor, world: int, rank: int, group) -> Tensor:
    """Sum `buffer` over ranks; this rank's block of rows receives its sum and is returned."""
    rows = buffer.shape[0] // world
    mine = buffer[rank * rows : (rank + 1) * rows]
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(mine, buffer, group=group)
    else:  # gloo has no reduce-scatter: reduce everything
        dist.all_reduce(buffer, group=group)
    return mine


def expert_parallel_forward(
    engine: Engine,
    hidden: Tensor,
    ids: Tensor,
    weights: Tensor,
    padding: Tensor | None = None,
    group=None,
) -> Tensor:
    """One layer call under expert parallelism (see the module docstring)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    tokens, k = ids.shape
    # One routing record per token: ids, weight bits, padding flag, as int32.
    record = torch.empty((tokens, 2 * k + 1), device=ids.device, dtype=torch.int32)
    record[:, :k] = ids
    record[:, k : 2 * k] = weights.float().contiguous().view(torch.int32)
    record[:, 2 * k] = padding.to(torch.int32) if padding is not None else 0
    all_hidden = _all_gather_rows(hidden, world, group)
    all_records = _all_gather_rows(record, world, group)
    all_ids = all_records[:, :k].contiguous()
    all_weights = all_records[:, k : 2 * k].contiguous().view(torch.float32)
    all_padding = all_records[:, 2 * k].bool() if padding is not None else None
    scores = engine.screen(all_hidden, all_ids, all_weights, all_padding)
    _reduce_scatter_in_place(scores, world, rank, group)
    cuts = engine.find_cuts(rank * tokens, tokens)
    _all_gather_in_place(cuts, world, rank, group)
    combined = engine.local()
    mine = _reduce_scatter_in_place(combined, world, rank, group)
    return engine.finish(mine)


class CudaEngine:
    """The CUDA library as the compute back end of one rank."""

    def __init__(self, reader: ProgressiveReader) -> None:
        self.reader = reader
        self._call: _native.Call | None = None
        self._rows = 0
        capacity, h = reader.max_tokens, reader.plan.hidden_size
        device = reader.native_gu.device
        self._combined = torch.empty(capacity, h + reader.rank, device=device, dtype=torch.float32)
        # The recovery encoder runs beside the two gathers on its own stream.
        self._side = torch.cuda.Stream(device, priority=-1)
        self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()

    def screen(self, hidden, ids, weights, padding):
        reader = self.reader
        rows = reader._validate_input(hidden, padding)
        call = reader._call_struct(rows, hidden, ids, weights, padding, self._combined, False)
        self._keep = (hidden, ids, weights, padding)  # the call struct holds raw pointers
        screened = reader.plan.completion_count < reader.plan.candidate_count
        with torch.cuda.device(reader.native_gu.device):
            if screened:
                reader._stage("cfm_prepare_input", call)
            reader._stage("cfm_route", call)
            if screened:
                reader._stage("cfm_screen", call)
                reader._stage("cfm_score", call)
            else:
                reader.scores[0][:rows].zero_()
        self._call, self._rows = call, rows
        return reader.scores[0][:rows]

    def find_cuts(self, first_row, rows):
        reader = self.reader
        # Workspace rows (and the padding mask) are indexed by absolute row.
        home = reader._call_struct(rows, *self._keep, self._combined, False)
        home.scores_ready, home.row_offset = 3, first_row
        with torch.cuda.device(reader.native_gu.device):
            reader._stage("cfm_select", home)
        return reader.cuts[: self._rows]

    def local(self):
        reader, call = self.reader, self._call
        call.scores_ready = 2
        device = reader.native_gu.device
        with torch.cuda.device(device):
            reader._stage("cfm_select", call)
            main = torch.cuda.current_stream(device)
            if reader.rank:
                self._fork.record(main)
                with torch.cuda.stream(self._side):
                    self._side.wait_event(self._fork)
                    reader._stage("cfm_encode", call)
                    self._join.record(self._side)
            reader._stage("cfm_exact", call)
            reader._stage("cfm_down", call)
            if reader.rank:
                main.wait_event(self._join)
            reader._stage("cfm_partial_output", call)
        return self._combined[: self._rows]

    def finish(self, combined):
        reader = self.reader
        rows = combined.shape[0]
        out = torch.empty((rows, reader.plan.hidden_size), device=combined.device,
                          dtype=torch.bfloat16)
        stream = torch.cuda.current_stream(combined.device).cuda_stream
        with torch.cuda.device(combined.device):
            code = reader._library.cfm_finish(
                ctypes.byref(reader._layer), rows, combined.data_ptr(), out.data_ptr(),
                ctypes.c_void_p(stream),
            )
        _native.check(code, "cfm_finish")
        return out


class ExpertParallelReader:
    """Sparse decode operator of one MoE layer with its experts sharded over a process group.

    Arguments are those of `ProgressiveReader` for the local experts only
    (`gate_up` `[E/P, 2I, H]`, channel-major `down`, `encoder` `[E/P, R, I]`), the
    replicated `decoder`, the global expert count, and the group.  `max_tokens`
    is the per-rank batch; every rank must call with the same number of rows
    (use `padding` for ragged batches).  Router ids are global expert ids.
    """

    def __init__(
        self,
        gate_up: Tensor,
        down: Tensor,
        encoder: Tensor | None,
        decoder: Tensor | None,
        plan: BudgetPlan,
        max_tokens: int,
        *,
        global_experts: int,
        group=None,
        **reader_options,
    ) -> None:
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if gate_up.shape[0] * self.world != global_experts:
            raise ValueError("Local experts times ranks must equal the global expert count")
        self.max_tokens = max_tokens
        expert_map = linear_expert_map(global_experts, self.world, self.rank)
        self.reader = ProgressiveReader(
            gate_up, down, encoder, decoder, plan, self.world * max_tokens,
            expert_map=expert_map, ep_group=self.group, recovery_owner=True, **reader_options,
        )
        self.engine = CudaEngine(self.reader)

    @torch.no_grad()
    def __call__(self, hidden: Tensor, ids: Tensor, weights: Tensor,
                 padding: Tensor | None = None) -> Tensor:
        if hidden.shape[0] > self.max_tokens:
            raise ValueError("Sparse input exceeds the prepared token/candidate contract")
        return expert_parallel_forward(self.engine, hidden, ids, weights, padding, self.group)

    def report(self) -> dict[str, float | None]:
        """This rank's read statistics (they add across ranks)."""
        return self.reader.report()
