"""Expert-parallel sparse decode reader: experts sharded over the ranks of one box.

Every rank holds `E / P` consecutive experts (linear placement, as the
reference's binding requires: runtime/experts.py:677-692) with their gate/up and
down rows; the decoder is replicated.  Tokens are data parallel: every rank
brings its own `T` decode tokens and gets their outputs back.  Two strategies
share the placement and differ in where the screen runs.

Replicated screen (default).  The sketch, its scales, the down-column norms and
the recovery encoder of ALL experts are resident on every rank (about a tenth of
the native weights, gathered once at construction), so the home rank of a token
screens, selects and encodes it alone, exactly as a single GPU does:

1. choose     the home rank rotates its tokens, screens all K experts of each,
              selects the kept channels and starts the recovery latent;
2. dispatch   hidden rows, router ids and weights and the kept candidate ids of
              every token reach all ranks (`all_gather`s; all but the last are
              started before the screen and do not wait for the selection);
3. serve      each rank cuts the lists down to the slots whose experts it owns
              and computes those channels exactly and their down rows;
4. combine    one FP32 row of router-weighted partial outputs per token goes
              back to the token's home rank (`reduce_scatter`), which adds the
              decoder term of its latent and stores BF16.

Sharded screen.  Nothing but the decoder is replicated; ranks screen their own
experts for all `P * T` tokens and exchange scores:

1. dispatch   hidden rows and routing records reach all ranks (`all_gather`);
2. screen     each rank scores the candidate channels of its local experts for
              all tokens; slots of remote experts score zero;
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
orchestration runs over NCCL with the CUDA engines and over gloo with CPU
engines in the tests.

Exchange over peer memory (`exchange="peer"`, the default on NCCL groups of one
box).  With the replicated screen the two exchanges on the critical path, the kept
lists out and the partial rows back, need no collective: every rank maps a block
of every other rank's device memory (CUDA IPC), the selection's lists are stored
straight into all ranks' blocks by a kernel of the library, the owners' partial
rows straight into the home rank's block, and the kernels that consume them wait
on a flag the last storing CTA sets.  The home rank adds the owners' rows in rank
order, so its sum no longer depends on the order of a reduction tree.  Hidden
rows and router outputs still travel by `all_gather`, started before the screen.
"""

from __future__ import annotations

import ctypes
import types
from typing import Protocol

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _native
from .budget import BudgetPlan
from .progressive import ProgressiveReader, ReaderWorkspace, recovery_geometry


def linear_expert_map(global_experts: int, world: int, rank: int) -> Tensor:
    """Global-to-local expert ids of `rank` under linear placement (-1 = remote)."""
    if global_experts % world:
        raise ValueError("Expert count must divide evenly over the expert-parallel ranks")
    local = global_experts // world
    mapping = torch.full((global_experts,), -1, dtype=torch.int32)
    mapping[rank * local : (rank + 1) * local] = torch.arange(local, dtype=torch.int32)
    return mapping


class Engine(Protocol):
    """What the sharded-screen orchestration needs from one rank's compute back end."""

    def screen(self, hidden: Tensor, ids: Tensor, weights: Tensor, padding: Tensor | None) -> Tensor:
        """Score buffer `[rows, N]`: the local experts' channels scored, zero elsewhere."""

    def find_cuts(self, first_row: int, rows: int) -> Tensor:
        """Cut buffer `[all rows, 1 + K]` with rows `first_row ..` filled from the summed scores."""

    def local(self) -> Tensor:
        """From the gathered cuts: FP32 rows `[all rows, H + R]` (partial output, partial latent)."""

    def finish(self, combined: Tensor) -> Tensor:
        """Home-rank output `[T, H]` BF16 from the summed rows."""


class HomeEngine(Protocol):
    """What the replicated-screen orchestration needs from one rank's compute back end."""

    def choose(self, hidden: Tensor, ids: Tensor, weights: Tensor, padding: Tensor | None) -> Tensor:
        """Kept candidate ids `[T, F]` int32 of this rank's own tokens (ascending, -1 padded)."""

    def serve(self, hidden: Tensor, ids: Tensor, weights: Tensor, padding: Tensor | None,
              lists: Tensor) -> Tensor:
        """FP32 rows `[all rows, H]`: router-weighted outputs of the local experts' kept channels."""

    def finish(self, routed: Tensor) -> Tensor:
        """Home-rank output `[T, H]` BF16 from the summed rows and the latent of `choose`."""


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


def _start_gather_rows(tensor: Tensor, world: int, group):
    """`_all_gather_rows` that returns at once: (gathered tensor, work to wait for)."""
    out = tensor.new_empty((world * tensor.shape[0], *tensor.shape[1:]))
    if dist.get_backend(group) == "nccl":
        work = dist.all_gather_into_tensor(out, tensor.contiguous(), group=group, async_op=True)
    else:
        work = dist.all_gather(list(out.chunk(world)), tensor.contiguous(), group=group,
                               async_op=True)
    return out, work


def _routing_record(ids: Tensor, weights: Tensor, padding: Tensor | None) -> Tensor:
    """One int32 row per token: expert ids, router weight bits, padding flag."""
    tokens, k = ids.shape
    record = torch.empty((tokens, 2 * k + 1), device=ids.device, dtype=torch.int32)
    record[:, :k] = ids
    record[:, k : 2 * k] = weights.float().contiguous().view(torch.int32)
    record[:, 2 * k] = padding.to(torch.int32) if padding is not None else 0
    return record


def replicated_screen_forward(
    engine: HomeEngine,
    hidden: Tensor,
    ids: Tensor,
    weights: Tensor,
    padding: Tensor | None = None,
    group=None,
) -> Tensor:
    """One layer call with the screen on the tokens' home ranks (see the module docstring)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    # Rows and router outputs travel while the home rank screens and selects; they are
    # gathered as they are, so nothing has to be packed before or sliced after.
    pending = [_start_gather_rows(hidden, world, group), _start_gather_rows(ids, world, group),
               _start_gather_rows(weights, world, group)]
    if padding is not None:
        pending.append(_start_gather_rows(padding.view(torch.uint8), world, group))
    lists = engine.choose(hidden, ids, weights, padding)
    peers = getattr(engine, "exchange", None) is not None
    if not peers:  # over peer memory `choose` has already stored the lists everywhere
        pending.append(_start_gather_rows(lists, world, group))
    for _, work in pending:
        work.wait()
    mark = getattr(engine, "_mark", None)
    if mark is not None:
        mark("all_gather of rows, routes" + ("" if peers else " and lists") + " complete")
    all_hidden, all_ids, all_weights = (gathered for gathered, _ in pending[:3])
    all_padding = pending[3][0].view(torch.bool) if padding is not None else None
    all_lists = None if peers else pending[-1][0]
    routed = engine.serve(all_hidden, all_ids, all_weights, all_padding, all_lists)
    if peers:  # the rows are already in the home ranks' blocks
        return engine.finish(None)
    mine = _reduce_scatter_in_place(routed, world, rank, group)
    if mark is not None:
        mark("reduce_scatter")
    return engine.finish(mine)


def expert_parallel_forward(
    engine: Engine,
    hidden: Tensor,
    ids: Tensor,
    weights: Tensor,
    padding: Tensor | None = None,
    group=None,
) -> Tensor:
    """One layer call with the screen on the experts' ranks (see the module docstring)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    tokens, k = ids.shape
    all_hidden = _all_gather_rows(hidden, world, group)
    all_records = _all_gather_rows(_routing_record(ids, weights, padding), world, group)
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


class PeerExchange:
    """One rank's exchange block and its view of the other ranks' blocks (CUDA IPC).

    Every rank allocates a block of `cfm_exchange_bytes` bytes with the library,
    publishes its IPC handle through the process group and opens the others'.
    The ranks must share one box with peer access between their GPUs; if a rank
    cannot open a block, all ranks report failure (`available` False) and the
    caller falls back to the collectives.  Blocks live until the process exits.
    """

    def __init__(self, layer: "_native.Layer", tokens: int, group) -> None:
        library = _native.load()
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.world, self.rank, self.tokens = world, rank, tokens
        self.struct = _native.Exchange()
        self.struct.world, self.struct.rank, self.struct.tokens = world, rank, tokens
        self.available = False
        if world > _native.MAX_RANKS:
            return
        size = library.cfm_exchange_bytes(ctypes.byref(layer), world, tokens)
        block = ctypes.c_void_p()
        good = size > 0 and library.cfm_peer_alloc(size, ctypes.byref(block)) == 0
        handle = (ctypes.c_ubyte * _native.PEER_HANDLE_BYTES)()
        good = good and library.cfm_peer_export(block, handle) == 0
        handles: list = [None] * world
        dist.all_gather_object(handles, bytes(handle) if good else None, group=group)
        self.bytes = int(size)
        if good and all(h is not None for h in handles):
            for peer in range(world):
                if peer == rank:
                    self.struct.blocks[peer] = block.value
                    continue
                opened = ctypes.c_void_p()
                raw = (ctypes.c_ubyte * _native.PEER_HANDLE_BYTES).from_buffer_copy(handles[peer])
                if library.cfm_peer_import(raw, ctypes.byref(opened)) != 0:
                    good = False
                    break
                self.struct.blocks[peer] = opened.value
        else:
            good = False
        verdicts: list = [None] * world
        dist.all_gather_object(verdicts, bool(good), group=group)  # also: everyone has opened
        self.available = all(verdicts)

    def status(self) -> int:
        """Bits of the waits that ran out since the block was made (synchronises)."""
        word = ctypes.c_int32()
        code = _native.load().cfm_exchange_status(ctypes.byref(self.struct), ctypes.byref(word))
        _native.check(code, "cfm_exchange_status")
        return int(word.value)


class ShardedScreenEngine:
    """The CUDA library as the sharded-screen back end of one rank."""

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
        self._lister = torch.cuda.Stream(device, priority=-1)
        self._adopted, self._listed = torch.cuda.Event(), torch.cuda.Event()

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
                ctypes.byref(reader._layer), rows, combined.data_ptr(), None, out.data_ptr(),
                ctypes.c_void_p(stream),
            )
        _native.check(code, "cfm_finish")
        return out


class _HomeScreen:
    """Screen, selection and recovery latent of a rank's own tokens over all experts.

    Holds the replicated part of an expert-parallel layer: the sketch (both kernel
    layouts), its scales, the down-column norms, the transposed recovery encoder
    and the recovery geometry of every expert, gathered from the ranks that built
    them for their own experts, and a workspace for this rank's tokens.
    """

    def __init__(self, owner: ProgressiveReader, encoder: Tensor | None, decoder: Tensor | None,
                 max_tokens: int, selection_score: str, world: int, group) -> None:
        plan, device = owner.plan, owner._device

        def gather(local: Tensor | None) -> Tensor | None:
            return _all_gather_rows(local.contiguous(), world, group) if local is not None else None

        self.sketch_words = gather(owner.sketch_words)
        self.sketch_grouped_words = gather(owner.sketch_grouped_words)
        # Physical layout of the statistics is [E, B, 2, 2I].
        self.sketch_statistics = gather(owner.sketch_statistics.permute(0, 2, 3, 1))
        self.norms = gather(owner.norms)
        self.rank = decoder.shape[1] if decoder is not None else 0
        self.encoder = self.decoder = self.recovery_geometry = None
        if encoder is not None and decoder is not None:
            local_encoder = encoder.to(device=device, dtype=torch.bfloat16).transpose(1, 2).contiguous()
            self.encoder = gather(local_encoder)
            self.decoder = decoder.to(device=device, dtype=torch.bfloat16).contiguous()
            if selection_score != "point":
                self.recovery_geometry = gather(
                    recovery_geometry(owner.down, local_encoder, self.decoder, owner.norms))
        experts = self.norms.shape[0]
        self.workspace = ReaderWorkspace(plan, experts, self.rank, max_tokens, device)
        self.read_work = torch.zeros(20, device=device, dtype=torch.float64)
        layer = _native.Layer.from_buffer_copy(owner._layer)
        layer.experts, layer.rank = experts, self.rank
        layer.global_experts, layer.recovery_owner = 0, 1
        layer.gate_up = layer.down = layer.expert_map = None
        layer.sketch = self.sketch_words.data_ptr()
        layer.sketch_grouped = (
            self.sketch_grouped_words.data_ptr() if self.sketch_grouped_words is not None else None)
        layer.statistics = self.sketch_statistics.data_ptr()
        layer.norms = self.norms.data_ptr()
        layer.geometry = (
            self.recovery_geometry.data_ptr() if self.recovery_geometry is not None else None)
        layer.encoder = self.encoder.data_ptr() if self.encoder is not None else None
        layer.decoder = self.decoder.data_ptr() if self.decoder is not None else None
        layer.read_work = self.read_work.data_ptr()
        self.layer = layer
        self.resident_bytes = sum(
            t.numel() * t.element_size()
            for t in (self.sketch_words, self.sketch_grouped_words, self.sketch_statistics,
                      self.norms, self.encoder, self.recovery_geometry) if t is not None)


class ReplicatedScreenEngine:
    """The CUDA library as the replicated-screen back end of one rank."""

    def __init__(self, owner: ProgressiveReader, home: _HomeScreen, max_tokens: int,
                 exchange: PeerExchange | None = None) -> None:
        self.owner, self.home, self.max_tokens = owner, home, max_tokens
        self.exchange = exchange
        device = owner._device
        self._routed = torch.empty(owner.max_tokens, owner.plan.hidden_size, device=device,
                                   dtype=torch.float32)
        # The recovery encoder runs beside the dispatch and the owners' work on its own stream.
        self._side = torch.cuda.Stream(device, priority=-1)
        self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
        self._lister = torch.cuda.Stream(device, priority=-1)
        self._adopted, self._listed = torch.cuda.Event(), torch.cuda.Event()
        self._library = owner._library
        # Called with a stage name after each stage is enqueued (timelines); None = off.
        self.trace = None

    def _mark(self, name: str) -> None:
        if self.trace is not None:
            self.trace(name)

    def _home_stage(self, name: str, call: _native.Call) -> None:
        home, device = self.home, self.owner._device
        code = getattr(self._library, name)(
            ctypes.byref(home.layer), home.workspace.buffer.data_ptr(), home.workspace.capacity,
            ctypes.byref(call), ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream),
        )
        _native.check(code, name)

    def choose(self, hidden, ids, weights, padding):
        owner, home, device = self.owner, self.home, self.owner._device
        rows = hidden.shape[0] if hidden.ndim == 2 else 0
        if not 1 <= rows <= self.max_tokens:
            raise ValueError("Sparse input exceeds the prepared token/candidate contract")
        owner._validate_input(hidden, padding)
        call = owner._call_struct(rows, hidden, ids, weights, padding, None, False)
        self._home_keep = (hidden, ids, weights, padding)  # the call struct holds raw pointers
        plan = owner.plan
        screened = plan.completion_count < plan.candidate_count
        with torch.cuda.device(device):
            if screened:
                # Routing and the grouping by expert do not depend on the rotated input:
                # they run on the side stream beside the rotation, as in the whole-layer call.
                main = torch.cuda.current_stream(device)
                self._fork.record(main)
                with torch.cuda.stream(self._side):
                    self._side.wait_event(self._fork)
                    self._home_stage("cfm_route", call)
                    self._join.record(self._side)
                self._home_stage("cfm_prepare_input", call)
                main.wait_event(self._join)
            else:
                self._home_stage("cfm_route", call)
            self._mark("prepare + route")
            if screened:
                self._home_stage("cfm_screen", call)
            self._mark("screen")
            if self.exchange is not None:
                # Every rank brings the same number of rows to a call (as the collectives
                # require too); the blocks are laid out for that number, up to their capacity.
                # With the exchange in the call the selection kernel ends by storing each
                # token's kept list into every rank's block (peer stores) and releasing
                # the flags.
                if rows > self.exchange.tokens:
                    raise ValueError("Sparse input exceeds the prepared token/candidate contract")
                self.exchange.struct.tokens = rows
                call.exchange = ctypes.addressof(self.exchange.struct)
            self._home_stage("cfm_select", call)
            self._mark("select" + (" + send lists (peer stores)" if self.exchange is not None else ""))
            if home.rank:
                main = torch.cuda.current_stream(device)
                self._fork.record(main)
                with torch.cuda.stream(self._side):
                    self._side.wait_event(self._fork)
                    self._home_stage("cfm_encode", call)
                    self._join.record(self._side)
        self._rows = rows
        return home.workspace.candidate_ids[:rows]

    def serve(self, hidden, ids, weights, padding, lists):
        owner = self.owner
        rows = owner._validate_input(hidden, padding)
        call = owner._call_struct(rows, hidden, ids, weights, padding, self._routed, False)
        if self.exchange is not None:
            call.exchange = ctypes.addressof(self.exchange.struct)
        else:
            call.lists = lists.data_ptr()
        self._serve_keep = (hidden, ids, weights, padding, lists)
        with torch.cuda.device(owner._device):
            main = torch.cuda.current_stream(owner._device)
            owner._stage("cfm_adopt", call)
            self._mark("adopt" + (" (waits for the lists)" if self.exchange is not None else ""))
            # The exact gather does not read the list of down tiles: one CTA builds it on
            # a second stream meanwhile.
            self._adopted.record(main)
            with torch.cuda.stream(self._lister):
                self._lister.wait_event(self._adopted)
                owner._stage("cfm_list_tiles", call)
                self._listed.record(self._lister)
            owner._stage("cfm_exact", call)
            self._mark("exact")
            main.wait_event(self._listed)
            owner._stage("cfm_down", call)
            self._mark("down")
            owner._stage("cfm_partial_output", call)
            self._mark("partial_output")
        return self._routed[:rows]

    def finish(self, routed):
        home, device = self.home, self.owner._device
        rows = routed.shape[0] if routed is not None else self._rows
        out = torch.empty((rows, self.owner.plan.hidden_size), device=device, dtype=torch.bfloat16)
        with torch.cuda.device(device):
            main = torch.cuda.current_stream(device)
            if home.rank:
                main.wait_event(self._join)
            if routed is None:  # the owners stored their rows into this rank's exchange block
                code = self._library.cfm_finish_rows(
                    ctypes.byref(home.layer), ctypes.byref(self.exchange.struct),
                    home.workspace.latent.data_ptr() if home.rank else None, out.data_ptr(),
                    ctypes.c_void_p(main.cuda_stream),
                )
                _native.check(code, "cfm_finish_rows")
                self._mark("finish (waits for the rows)")
                return out
            code = self._library.cfm_finish(
                ctypes.byref(home.layer), rows, routed.data_ptr(),
                home.workspace.latent.data_ptr() if home.rank else None, out.data_ptr(),
                ctypes.c_void_p(main.cuda_stream),
            )
        _native.check(code, "cfm_finish")
        self._mark("finish")
        return out


class ExpertParallelReader:
    """Sparse decode operator of one MoE layer with its experts sharded over a process group.

    Arguments are those of `ProgressiveReader` for the local experts only
    (`gate_up` `[E/P, 2I, H]`, channel-major `down`, `encoder` `[E/P, R, I]`), the
    replicated `decoder`, the global expert count, and the group.  `max_tokens`
    is the per-rank batch; every rank must call with the same number of rows
    (use `padding` for ragged batches).  Router ids are global expert ids.
    `screen` picks the strategy: "replicated" (default; every rank also keeps
    the sketch, norms and recovery encoder of all experts and screens its own
    tokens alone) or "sharded" (nothing but the decoder is replicated; ranks
    exchange scores).  Both keep the same channels.  `exchange` picks how the
    replicated screen moves the kept lists and the partial rows: "peer" (kernels
    of the library over memory the ranks map from each other; every call must
    then bring the same number of rows on all ranks), "collective" (`all_gather` and
    `reduce_scatter`) or "auto" (peer memory when the group runs over NCCL and
    the mapping works).
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
        screen: str = "replicated",
        exchange: str = "auto",
        **reader_options,
    ) -> None:
        if screen not in ("replicated", "sharded"):
            raise ValueError("screen must be 'replicated' or 'sharded'")
        if exchange not in ("auto", "peer", "collective"):
            raise ValueError("exchange must be 'auto', 'peer' or 'collective'")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if gate_up.shape[0] * self.world != global_experts:
            raise ValueError("Local experts times ranks must equal the global expert count")
        self.max_tokens, self.screen = max_tokens, screen
        self.exchange: PeerExchange | None = None
        expert_map = linear_expert_map(global_experts, self.world, self.rank)
        if screen == "sharded":
            self.reader = ProgressiveReader(
                gate_up, down, encoder, decoder, plan, self.world * max_tokens,
                expert_map=expert_map, ep_group=self.group, recovery_owner=True, **reader_options,
            )
            self.home = None
            self.engine = ShardedScreenEngine(self.reader)
            return
        if (encoder is None) != (decoder is None):
            raise ValueError("Expected matching recovery encoder and decoder")
        # The owner side reads native rows only: no recovery map, no latent.
        self.reader = ProgressiveReader(
            gate_up, down, None, None, plan, self.world * max_tokens,
            expert_map=expert_map, ep_group=self.group, recovery_owner=True, **reader_options,
        )
        score = reader_options.get("selection_score", "recovery-aware")
        self.home = _HomeScreen(self.reader, encoder, decoder, max_tokens, score, self.world,
                                self.group)
        # The owner's own sketch now lives inside the gathered copy.
        local, home = self.reader, self.home
        span = slice(self.rank * gate_up.shape[0], (self.rank + 1) * gate_up.shape[0])
        local.sketch_codes = None
        local.sketch_words = home.sketch_words[span]
        local._layer.sketch = local.sketch_words.data_ptr()
        if local.sketch_grouped_words is not None:
            local.sketch_grouped_words = home.sketch_grouped_words[span]
            local._layer.sketch_grouped = local.sketch_grouped_words.data_ptr()
        local.sketch_statistics = home.sketch_statistics[span].permute(0, 3, 1, 2)
        local._layer.statistics = local.sketch_statistics.data_ptr()
        local.sketch_resident_bytes = 0
        # Lists and partial rows over peer memory where the ranks can map each other's
        # memory; "peer" insists on it, "auto" falls back to the collectives.
        peer = None
        on_nccl = gate_up.is_cuda and dist.get_backend(self.group) == "nccl"
        if exchange != "collective" and on_nccl:
            peer = PeerExchange(self.home.layer, max_tokens, self.group)
            if not peer.available:
                peer = None
        if exchange == "peer" and peer is None:
            raise RuntimeError("The ranks cannot map each other's device memory (CUDA IPC)")
        self.exchange = peer
        self.engine = ReplicatedScreenEngine(self.reader, self.home, max_tokens, peer)

    @torch.no_grad()
    def __call__(self, hidden: Tensor, ids: Tensor, weights: Tensor,
                 padding: Tensor | None = None) -> Tensor:
        if hidden.shape[0] > self.max_tokens:
            raise ValueError("Sparse input exceeds the prepared token/candidate contract")
        forward = replicated_screen_forward if self.home is not None else expert_parallel_forward
        return forward(self.engine, hidden, ids, weights, padding, self.group)

    def report(self) -> dict[str, float | None]:
        """This rank's read statistics (they add across ranks).

        With the replicated screen a token is accounted whole on its home rank,
        whichever ranks read its experts' rows.
        """
        if self.home is None:
            return self.reader.report()
        owner, home = self.reader, self.home
        plan, rank = owner.plan, home.rank
        n, h = plan.candidate_count, plan.hidden_size
        whole = types.SimpleNamespace(
            read_work=home.read_work, plan=plan, ep_group=None, rank=rank, recovery_owner=True,
            sketch_resident_bytes=home.resident_bytes,
            selection_threshold=owner.selection_threshold,
            workspace_bytes=owner.workspace_bytes + home.workspace.bytes,
            matrix_macs=(2 * n * h * (plan.completion_count != n) + 2 * plan.completion_count * h
                         + h * plan.final_count + rank * (n - plan.final_count + h)),
        )
        whole._threshold_matrix_macs = types.MethodType(
            ProgressiveReader._threshold_matrix_macs, whole)
        return ProgressiveReader.report(whole)
