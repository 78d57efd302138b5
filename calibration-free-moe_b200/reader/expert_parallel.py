"""Expert-parallel sparse decode reader: experts sharded over the ranks of one box.

Every rank holds `E / P` consecutive experts (linear placement, as the
reference's binding requires: runtime/experts.py:677-692) with their gate/up and
down rows, sketch, norms and encoder rows; the decoder is replicated.  Tokens
are data parallel: every rank brings its own `T` decode tokens and gets their
outputs back.

One layer call, on every rank:

1. dispatch   every rank's tokens, router ids and weights reach the ranks that
              own their experts (`all_gather`; with K = 8 experts over at most 8
              ranks nearly every token has an expert on every rank, so the
              dispatch of a static-shape decode step is the gather of all rows);
2. screen     each rank scores the candidate channels of its local experts for
              all `P * T` tokens; slots of remote experts score zero;
3. exchange   the per-token top-F is global over the token's K experts, so the
              scores are summed across ranks (`all_reduce`) and every rank then
              keeps the same channels (reference progressive.py:4245-4251);
4. local      each rank computes its kept channels exactly, their down rows and
              its share of the recovery latent;
5. combine    the FP32 router-weighted partial outputs and partial latents go
              back to the token's home rank (`reduce_scatter`), which adds the
              decoder term and stores BF16.

Compared with the reference's expert-parallel mode (replicated tokens, caller
all-reduces BF16 outputs: tests/test_expert_parallel_reader.py:128-130) tokens
stay sharded and the output is reduced in FP32 before its single BF16 rounding.

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
        """Scores `[rows, N]` of the local experts' channels (zero elsewhere)."""

    def local(self, scores: Tensor) -> tuple[Tensor, Tensor | None]:
        """Given the summed scores: FP32 partial outputs `[rows, H]` and latents `[rows, R]`."""

    def finish(self, routed: Tensor, latent: Tensor | None) -> Tensor:
        """Home-rank output `[T, H]` BF16 from the summed partials."""


def _all_gather_rows(tensor: Tensor, world: int, group) -> Tensor:
    out = tensor.new_empty((world * tensor.shape[0], *tensor.shape[1:]))
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, tensor.contiguous(), group=group)
    else:
        dist.all_gather(list(out.chunk(world)), tensor.contiguous(), group=group)
    return out


def _reduce_scatter_rows(tensor: Tensor, world: int, rank: int, group) -> Tensor:
    """Sum `tensor` over ranks and return this rank's block of rows."""
    rows = tensor.shape[0] // world
    if dist.get_backend(group) == "nccl":
        out = tensor.new_empty((rows, *tensor.shape[1:]))
        dist.reduce_scatter_tensor(out, tensor.contiguous(), group=group)
        return out
    # gloo has no reduce-scatter: reduce everything, keep the local block.
    total = tensor.clone()
    dist.all_reduce(total, group=group)
    return total[rank * rows : (rank + 1) * rows].contiguous()


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
    all_hidden = _all_gather_rows(hidden, world, group)
    all_ids = _all_gather_rows(ids, world, group)
    all_weights = _all_gather_rows(weights, world, group)
    all_padding = None
    if padding is not None:
        all_padding = _all_gather_rows(padding.to(torch.uint8), world, group).bool()
    scores = engine.screen(all_hidden, all_ids, all_weights, all_padding)
    dist.all_reduce(scores, group=group)
    routed, latent = engine.local(scores)
    routed = _reduce_scatter_rows(routed, world, rank, group)
    if latent is not None:
        latent = _reduce_scatter_rows(latent, world, rank, group)
    return engine.finish(routed, latent)


class CudaEngine:
    """The CUDA library as the compute back end of one rank."""

    def __init__(self, reader: ProgressiveReader) -> None:
        self.reader = reader
        self._call: _native.Call | None = None
        self._rows = 0
        capacity, h = reader.max_tokens, reader.plan.hidden_size
        self._routed = torch.empty(capacity, h, device=reader.native_gu.device, dtype=torch.float32)

    def screen(self, hidden, ids, weights, padding):
        reader = self.reader
        rows = reader._validate_input(hidden, padding)
        call = reader._call_struct(rows, hidden, ids, weights, padding, self._routed, False)
        self._keep = (hidden, ids, weights, padding)  # the call struct holds raw pointers
        with torch.cuda.device(reader.native_gu.device):
            if reader.plan.completion_count < reader.plan.candidate_count:
                reader._stage("cfm_prepare_input", call)
            reader._stage("cfm_route", call)
            if reader.plan.completion_count < reader.plan.candidate_count:
                reader._stage("cfm_screen", call)
                reader._stage("cfm_score", call)
        self._call, self._rows = call, rows
        return reader.scores[0][:rows]

    def local(self, scores):
        reader, call = self.reader, self._call
        call.scores_ready = 1
        with torch.cuda.device(reader.native_gu.device):
            for stage in ("cfm_select", "cfm_exact", "cfm_down", "cfm_encode", "cfm_partial_output"):
                reader._stage(stage, call)
        latent = reader.latent[: self._rows] if reader.rank else None
        return self._routed[: self._rows], latent

    def finish(self, routed, latent):
        reader = self.reader
        out = torch.empty(routed.shape, device=routed.device, dtype=torch.bfloat16)
        stream = torch.cuda.current_stream(routed.device).cuda_stream
        with torch.cuda.device(routed.device):
            code = reader._library.cfm_finish(
                ctypes.byref(reader._layer), routed.shape[0], routed.data_ptr(),
                latent.data_ptr() if latent is not None else None, out.data_ptr(),
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
