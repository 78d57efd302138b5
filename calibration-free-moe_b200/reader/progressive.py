"""Sparse decode operator of one MoE layer's routed experts, on B200.

Host-side mirror of the reference operator API
(`calibration_free_moe/reader/progressive.py`: `channel_major_down` :56,
`ReaderWorkspace` :2868, `ProgressiveReader` :3124 with `__init__` :3133,
`report` :3517, `prepare_input` :3829, `__call__` :3875).  The Python here
validates arguments, owns tensors and enqueues the stages of the CUDA library on
the caller's stream; all decode arithmetic is in `csrc/cfm_reader.cu`.

Symbols: H hidden size, I channels per expert, E local experts, K experts per
token, N = K * I candidates per token, F kept channels, R recovery rank.
"""

from __future__ import annotations

import ctypes
from typing import Literal

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _native
from ..activation import ACTIVATION_CODES, GatedActivation
from .budget import BudgetPlan
from .sketch import (
    block_hadamard_signs, build_sketch, build_sketch_on_device, codes_from_words, repack_sketch,
    repack_sketch_grouped,
)
from .budget import sketch_storage_bytes

SelectionScore = Literal["recovery-aware", "point"]
SCORE_CODES = {"point": 0, "recovery-aware": 1}
TENSOR_ENGINES = {"mma_sync": 0, "tcgen05": 1}
ROW_ENGINES = {"auto": 0, "per_token": 1, "expert_major": 2}

# Accepted for interface compatibility; this implementation has one execution
# path whose results do not depend on them.
GROUPED_TOKENS = 32
GROUPED_SCREEN_TOKENS = 64
# Batch size from which the library screens expert-major; readers with a smaller
# capacity do not keep the row-major sketch copy that path reads.
GROUPED_SCREEN_MIN_TOKENS = 8


def channel_major_down(weight: Tensor) -> Tensor:
    """Re-lay a down weight `[E, H, I]` so each channel's H outputs are contiguous.

    Returns the same logical tensor over physical `[E, I, H]` storage (stride
    `(H I, 1, H)`), the layout the reader gathers rows from.
    """
    return weight.transpose(1, 2).contiguous().transpose(1, 2)


def recovery_geometry(down: Tensor, encoder: Tensor, decoder: Tensor, norms: Tensor) -> Tensor:
    """Split every channel's recovery response U B_c along and across its down column.

    down is the channel-major down weight (logical `[E, H, I]`), encoder the
    transposed encoder `[E, I, R]`, decoder `[H, R]`, norms the down-column norms
    `[E, I]`.  Returns FP32 `[E, I, 2]`: alpha = <d_c, U B_c> / ||d_c|| (1 in
    place of a zero norm) and beta = sqrt(max(||U B_c||^2 - alpha^2, 0)); one
    expert at a time, nothing of the expanded response is kept
    (reference progressive.py:3359-3373).
    """
    experts, _, width = down.shape
    geometry = torch.zeros((experts, width, 2), device=down.device, dtype=torch.float32)
    decoder_rows = decoder.float().T
    for expert in range(experts):
        column = down[expert].float().T  # [I, H]
        response = encoder[expert].float() @ decoder_rows  # [I, H]
        norm = norms[expert]
        alpha = (column * response).sum(-1) / torch.where(norm > 0, norm, torch.ones_like(norm))
        beta = (response.square().sum(-1) - alpha.square()).clamp_min(0).sqrt()
        geometry[expert, :, 0] = alpha
        geometry[expert, :, 1] = beta
    return geometry


_TORCH_TYPES = {
    "ids": torch.int32, "weights": torch.float32, "norms": torch.float32,
    "planes": torch.float32, "coordinates": torch.int32, "quantized": torch.int32,
    "exponents": torch.int32, "parts": torch.float32, "counters": torch.int32,
    "partial": torch.float32, "scores": torch.float32, "selected": torch.bool,
    "completed": torch.bool, "candidate_ids": torch.int32, "counts": torch.int32,
    "starts": torch.int32, "tile_starts": torch.int32, "activations": torch.bfloat16,
    "exact": torch.float32, "down_parts": torch.float32, "encoder_parts": torch.float32,
    "latent": torch.float32, "status": torch.int32, "limbs": torch.int8,
    "group_offsets": torch.int32, "group_pairs": torch.int32, "cuts": torch.int32,
    "variances": torch.float32, "unscales": torch.float32, "zero_limbs": torch.int8,
    "tile_list": torch.int32, "tile_count": torch.int32,
}


def _dimension_layer(plan: BudgetPlan, experts: int, rank: int) -> _native.Layer:
    layer = _native.Layer()
    layer.hidden, layer.width, layer.experts = plan.hidden_size, plan.expert_width, experts
    layer.top_k, layer.final_count = plan.top_k, plan.final_count
    layer.keep, layer.rank = plan.screen_coordinates, rank
    return layer


class ReaderWorkspace:
    """Scratch of the reader for up to `capacity` tokens per call.

    One device allocation carved into the arrays the kernels exchange; the views
    below keep the reference's names where an array has a counterpart
    (reference progressive.py:3074-3109).  A workspace may be shared by layers of
    identical dimensions that run one after another on one stream; it is not
    reentrant.  The scheduling arguments of the reference signature are accepted
    and ignored.
    """

    def __init__(
        self,
        plan: BudgetPlan,
        experts: int,
        rank: int,
        capacity: int,
        device: torch.device | str,
        grouped_tokens: int = GROUPED_TOKENS,
        grouped_screen_tokens: int = GROUPED_SCREEN_TOKENS,
        radix_select: bool = True,
        screen_block_splits: int = 8,
        grouped_screen_splits: int = 2,
    ) -> None:
        if capacity < 1:
            raise ValueError("Workspace capacity must be at least one token")
        device = torch.device(device)
        self.key = (plan, experts, rank, capacity, device, grouped_tokens, grouped_screen_tokens)
        self.capacity = capacity
        self.charged = False
        layout = _native.workspace_layout(_dimension_layer(plan, experts, rank), capacity)
        self.layout = layout
        self.bytes = int(layout.bytes)
        self.experts, self.rank = experts, rank
        # Zero-initialised: the arrival counters rely on it and reset themselves.
        self.buffer = torch.zeros(self.bytes, dtype=torch.uint8, device=device)
        self._bind(self, plan, layout)

    def _bind(self, target: object, plan: BudgetPlan, layout: "_native.WorkspaceLayout") -> None:
        """Attach typed views of the buffer, laid out for `plan`, to `target`."""
        h, i, k = plan.hidden_size, plan.expert_width, plan.top_k
        n, f, keep = plan.candidate_count, plan.final_count, plan.screen_coordinates
        blocks, c, r = h // 128, self.capacity, max(self.rank, 1)
        shapes = {
            "ids": (c, k), "weights": (c, k), "norms": (c, blocks),
            "planes": (c, blocks, keep), "coordinates": (c, blocks, keep),
            "quantized": (c, blocks, keep), "exponents": (c, blocks, 2),
            "parts": (layout.parts_tokens * k, blocks, 2 * i),
            "counters": (2 * c * k + 2 * c,), "partial": (c, 2, n), "scores": (c, n),
            "selected": (c, n), "completed": (c, n), "candidate_ids": (c, f),
            "counts": (c, k), "starts": (c, k), "tile_starts": (c, k),
            "activations": (c, n), "exact": (c, 2, f),
            "down_parts": (c, layout.down_tiles, h),
            "encoder_parts": (c, k, layout.encoder_tiles, r), "latent": (c, r),
            "status": (4,), "limbs": (c, blocks, 3, 128),
            "group_offsets": (self.experts + 1,), "group_pairs": (c * k,), "cuts": (c, k + 1),
            "variances": (c, 2, n), "unscales": (c, blocks), "zero_limbs": (blocks, 3, 128),
            "tile_list": (c * (-(-f // 64) + k), 8), "tile_count": (4,),
        }
        for name, shape in shapes.items():
            setattr(target, name, self._view(layout, name, shape))
        # Reference names for the same arrays.
        target.sketch_planes, target.sketch_coordinates = target.planes, target.coordinates
        target.screen_parts = target.parts
        target.screen_counters = target.counters[: c * k]
        target.down_splits, target.encoder_splits = layout.down_tiles, layout.encoder_tiles

    def views_for(self, plan: BudgetPlan) -> object:
        """Views of this buffer laid out for a layer that keeps fewer channels.

        The library lays the workspace out from the dimensions of the layer of each
        call.  Arrays up to and including the arrival counters do not depend on F,
        so layers that differ only in F can share one buffer sized for the largest
        (reference progressive.py:3388-3397); each needs its own views.
        """
        layout = _native.workspace_layout(
            _dimension_layer(plan, self.experts, self.rank), self.capacity
        )
        if layout.bytes > self.bytes:
            raise ValueError("Shared workspace is too small for this plan")
        views = type("WorkspaceViews", (), {})()
        views.buffer, views.capacity, views.layout = self.buffer, self.capacity, layout
        self._bind(views, plan, layout)
        return views

    def _view(self, layout, name: str, shape: tuple[int, ...]) -> Tensor:
        dtype = _TORCH_TYPES[name]
        count = 1
        for extent in shape:
            count *= extent
        start = getattr(layout, name)
        size = count * (1 if dtype is torch.bool else torch.empty((), dtype=dtype).element_size())
        return self.buffer[start : start + size].view(dtype).view(shape)


class ProgressiveReader:
    """Sparse decode operator of one MoE layer's routed experts.

    Construct one per layer, then call it once per decode step with the layer's
    hidden rows and router outputs.  Reads the native weights in place.
    """

    @torch.no_grad()
    def __init__(
        self,
        gate_up: Tensor,
        down: Tensor,
        encoder: Tensor | None,
        decoder: Tensor | None,
        plan: BudgetPlan,
        max_tokens: int,
        expert_map: Tensor | None = None,
        sketch: tuple[Tensor, Tensor] | None = None,
        activation: GatedActivation = "silu",
        grouped_tokens: int = GROUPED_TOKENS,
        workspace: ReaderWorkspace | None = None,
        grouped_screen_tokens: int = GROUPED_SCREEN_TOKENS,
        selection_score: SelectionScore = "recovery-aware",
        fused_accounting: bool = True,
        radix_select: bool = True,
        screen_block_splits: int = 8,
        grouped_screen_splits: int = 2,
        selection_threshold: float | None = None,
        screen_last_block_reduction: bool = True,
        recovery_last_block_reduction: bool = True,
        pdl: bool = True,
        *,
        ep_group: "dist.ProcessGroup | None" = None,
        recovery_owner: bool | None = None,
        retain_reference_sketch: bool = True,
        tensor_engine: str = "mma_sync",
        row_engine: str = "auto",
        sketch_builder: str = "torch",
    ) -> None:
        """Prepare the sketch, norms and workspace of one layer.

        Arguments follow the reference constructor (progressive.py:3134-3157):
        gate_up BF16 `[E, 2I, H]` contiguous on a CUDA device; down the
        channel-major down weight (logical `[E, H, I]`, stride `(H I, 1, H)`);
        encoder `[E, R, I]` and decoder `[H, R]` or both None; the layer's plan;
        the largest batch; for expert parallelism the global-to-local expert map
        (-1 for remote experts); a prebuilt `(codes, statistics)` sketch.  The
        scheduling options (grouped_tokens, grouped_screen_tokens,
        fused_accounting, radix_select, the split counts, the last-block
        reductions, pdl) are accepted for compatibility and change nothing here.

        Keyword-only additions: `ep_group` (process group of the expert-parallel
        ranks; defaults to the world group when `expert_map` is given),
        `recovery_owner` (the rank that adds the decoder term; defaults to rank 0
        of the group) and `retain_reference_sketch` (keep the reference-layout
        codes resident beside the kernel layout) and `tensor_engine`, the
        tensor-core path of the expert-major screen: "mma_sync" (default, measured
        faster) or "tcgen05" (tensor-memory accumulators); both give the same bits;
        and `row_engine`, how batches of eight tokens and more read the native
        rows: "expert_major" (a row several tokens of one expert kept is read once
        for all of them), "per_token" (one gather per token, tokens of one expert
        next to each other in time so that shared rows meet in L2) or "auto"
        (the faster one on the shapes measured so far: per token).  The kept channels
        do not depend on it; outputs differ by FP32 summation order only.
        `sketch_builder` picks who builds the sketch when none is given: "torch"
        (tensor operations, byte-identical to the reference builder on the same
        device) or "cuda" (the library's kernel, straight into the kernel layouts,
        milliseconds per layer; single coordinates within rounding of the ternary
        threshold may differ from the reference builder's).

        Contract violations raise ValueError before anything is launched.
        """
        h, i, k = plan.hidden_size, plan.expert_width, plan.top_k
        n = plan.candidate_count
        e = gate_up.shape[0] if gate_up.ndim == 3 else -1
        rank = decoder.shape[1] if decoder is not None and decoder.ndim == 2 else 0
        if selection_threshold is not None and (
            not selection_threshold >= 0
            or selection_threshold == float("inf")
            or not plan.final_count == plan.completion_count < plan.candidate_count
        ):
            raise ValueError(
                "A selection threshold is finite, nonnegative and needs a screened plan"
            )
        if selection_score not in SCORE_CODES:
            raise ValueError("selection_score must be 'recovery-aware' or 'point'")
        if tensor_engine not in TENSOR_ENGINES:
            raise ValueError("tensor_engine must be 'mma_sync' or 'tcgen05'")
        if row_engine not in ROW_ENGINES:
            raise ValueError("row_engine must be 'auto', 'per_token' or 'expert_major'")
        if sketch_builder not in ("torch", "cuda"):
            raise ValueError("sketch_builder must be 'torch' or 'cuda'")
        if activation not in ACTIVATION_CODES:
            raise ValueError(f"Unsupported routed expert activation: {activation}")
        if screen_block_splits not in (1, 2, 4, 8) or grouped_screen_splits not in (1, 2, 4, 8):
            raise ValueError("Screen block splits must be 1, 2, 4 or 8")
        # The contract check below and the error texts of this constructor restate the
        # reference's (progressive.py:3234-3271, 3310, 3328, 3407): callers and the
        # reference's tests match on which inputs are rejected and on the messages.
        if (
            gate_up.shape != (e, 2 * i, h)
            or down.shape != (e, h, i)
            or (encoder is None) != (decoder is None)
            or (encoder is not None and encoder.shape != (e, rank, i))
            or (decoder is not None and (decoder.shape != (h, rank) or rank < 1))
            or not gate_up.is_cuda
            or down.device != gate_up.device
            or gate_up.dtype != torch.bfloat16
            or down.dtype != gate_up.dtype
            or not gate_up.is_contiguous()
            or down.stride() != (h * i, 1, h)
            or (expert_map is None and k > e)
            or max_tokens < 1
            or grouped_tokens < 2
        ):
            raise ValueError(
                "Expected native GU and channel-major D CUDA experts, "
                "matching recovery and capacity"
            )
        if k > 32 or (rank and (rank % 8 or 256 % rank)):
            raise ValueError("This build supports top_k <= 32 and rank in {8,16,32,64,128,256}")
        device = gate_up.device
        self.plan, self.max_tokens, self.rank = plan, max_tokens, rank
        self.activation: GatedActivation = activation
        self.selection_score: SelectionScore = selection_score
        # FP32 explicitly (callers may construct readers under a BF16 default dtype); a
        # device scalar, so it can be refilled between CUDA-graph replays.
        self.selection_threshold = (
            torch.tensor([selection_threshold], device=device, dtype=torch.float32)
            if selection_threshold is not None
            else None
        )
        self.expert_map = (
            expert_map.to(device=device, dtype=torch.int32).contiguous()
            if expert_map is not None
            else None
        )
        if self.expert_map is not None:
            if self.expert_map.ndim != 1 or int((self.expert_map >= 0).sum()) != e:
                raise ValueError("Expert map must cover exactly the native local experts")
            self.ep_group = ep_group if ep_group is not None else dist.group.WORLD
            self.recovery_owner = (
                bool(recovery_owner)
                if recovery_owner is not None
                else dist.get_rank(self.ep_group) == 0
            )
        else:
            self.ep_group = None
            self.recovery_owner = True

        self.sketch_signs = block_hadamard_signs(h, device)
        blocks = h // 128
        if sketch is None and sketch_builder == "cuda":
            # One pass of the library's kernel over the weights, straight into the kernel layouts.
            self.sketch_words, grouped, statistics = build_sketch_on_device(gate_up, self.sketch_signs)
            self.sketch_grouped_words = grouped if max_tokens >= GROUPED_SCREEN_MIN_TOKENS else None
            self.sketch_codes = (
                codes_from_words(self.sketch_words, 2 * i, h) if retain_reference_sketch else None
            )
        else:
            if sketch is None:
                sketch = build_sketch(gate_up, self.sketch_signs)
            codes, statistics = sketch
            if (
                codes.shape != (e, sketch_storage_bytes(2 * i, h))
                or codes.dtype != torch.uint8
                or codes.device != device
                or not codes.is_contiguous()
                or statistics.shape != (e, 2 * i, blocks, 2)
                or statistics.dtype != torch.float16
                or statistics.device != device
                or statistics.stride() != (4 * i * blocks, 1, 4 * i, 2 * i)
            ):
                raise ValueError("Sketch must match the local native routed experts")
            # Kernel layout: two bits per trit, [E, H, 2I/16] words.
            self.sketch_words = repack_sketch(codes, 2 * i, h)
            # Row-major copy for the expert-major screen of batches of 8 tokens and more.
            self.sketch_grouped_words = (
                repack_sketch_grouped(codes, 2 * i, h)
                if max_tokens >= GROUPED_SCREEN_MIN_TOKENS else None
            )
            self.sketch_codes = codes if retain_reference_sketch else None
        self.sketch_statistics = statistics
        self.sketch_resident_bytes = (
            self.sketch_words.numel() * 4
            + statistics.numel() * 2
            + (self.sketch_grouped_words.numel() * 4 if self.sketch_grouped_words is not None else 0)
        )

        self.norms = down.float().square().sum(1).sqrt().contiguous()
        self.native_gu = gate_up.detach()
        self.down = down.detach()
        self.encoder: Tensor | None = None
        self.decoder: Tensor | None = None
        self.recovery_geometry: Tensor | None = None
        if encoder is not None and decoder is not None:
            # Encoder rows become contiguous per channel: [E, I, R].
            self.encoder = (
                encoder.to(device=device, dtype=torch.bfloat16).transpose(1, 2).contiguous()
            )
            self.decoder = decoder.to(device=device, dtype=torch.bfloat16).contiguous()
            if selection_score != "point":
                self.recovery_geometry = recovery_geometry(self.down, self.encoder, self.decoder, self.norms)

        if workspace is None:
            workspace = ReaderWorkspace(
                plan, e, rank, max_tokens, device, grouped_tokens, grouped_screen_tokens
            )
        workspace_plan = workspace.key[0]
        compatible_plan = workspace_plan == plan or (
            workspace_plan.hidden_size == h
            and workspace_plan.expert_width == i
            and workspace_plan.top_k == k
            and workspace_plan.screen_coordinates == plan.screen_coordinates
            and plan.final_count == plan.completion_count
            and workspace_plan.final_count == workspace_plan.completion_count
            and plan.final_count <= workspace_plan.final_count < n
        )
        if not compatible_plan or workspace.key[1:5] != (e, rank, max_tokens, device):
            raise ValueError("Shared workspace must match the plan, experts and capacity")
        self.workspace = workspace
        # A layer that keeps fewer channels than the workspace was sized for sees the
        # shared buffer through views laid out for its own F.
        w = workspace if workspace_plan == plan else workspace.views_for(plan)
        self.ids, self.weights, self.partial = w.ids, w.weights, w.partial
        self.variances, self.norms_input, self.cuts = w.variances, w.norms, w.cuts
        self.sketch_planes, self.sketch_coordinates = w.sketch_planes, w.sketch_coordinates
        self.screen_parts, self.screen_counters = w.screen_parts, w.screen_counters
        self.activations, self.completed, self.selected = w.activations, w.completed, w.selected
        self.scores = [w.scores]
        self.candidate_ids = [w.candidate_ids]
        self.starts, self.counts, self.tile_starts = w.starts, w.counts, w.tile_starts
        self.down_splits, self.encoder_splits = w.down_splits, w.encoder_splits
        self.down_parts, self.encoder_parts, self.latent = (
            w.down_parts, w.encoder_parts, w.latent,
        )
        # Shared scratch is reported once, by the first reader bound to it.
        self.workspace_bytes = 0 if workspace.charged else workspace.bytes
        workspace.charged = True
        prepared = self.recovery_geometry is not None
        self.recovery_geometry_bytes = self.recovery_geometry.numel() * 4 if prepared else 0
        self.recovery_geometry_preparation_products = prepared * 2 * e * i * h
        self.recovery_geometry_preparation_reduction_adds = prepared * 2 * e * i * (h - 1)
        self.recovery_response_preparation_macs = prepared * e * i * h * rank
        self.matrix_macs = (
            2 * n * h * (plan.completion_count != n)
            + 2 * plan.completion_count * h
            + h * plan.final_count
            + rank * (n - plan.final_count + h)
        )
        # Device-side read statistics (slots as in the reference, :3507-3514).
        self.read_work = torch.zeros(20, device=device, dtype=torch.float64)

        layer = _dimension_layer(plan, e, rank)
        layer.activation = ACTIVATION_CODES[activation]
        layer.score = SCORE_CODES[selection_score]
        layer.tensor_engine = TENSOR_ENGINES[tensor_engine]
        layer.row_engine = ROW_ENGINES[row_engine]
        layer.global_experts = self.expert_map.numel() if self.expert_map is not None else 0
        layer.recovery_owner = int(self.recovery_owner)
        layer.gate_up = self.native_gu.data_ptr()
        layer.down = self.down.data_ptr()
        layer.sketch = self.sketch_words.data_ptr()
        layer.sketch_grouped = (
            self.sketch_grouped_words.data_ptr() if self.sketch_grouped_words is not None else None
        )
        layer.statistics = statistics.data_ptr()
        layer.norms = self.norms.data_ptr()
        layer.geometry = (
            self.recovery_geometry.data_ptr() if self.recovery_geometry is not None else None
        )
        layer.encoder = self.encoder.data_ptr() if self.encoder is not None else None
        layer.decoder = self.decoder.data_ptr() if self.decoder is not None else None
        layer.signs = self.sketch_signs.data_ptr()
        layer.expert_map = self.expert_map.data_ptr() if self.expert_map is not None else None
        layer.read_work = self.read_work.data_ptr()
        layer.selection_threshold = (
            self.selection_threshold.data_ptr() if self.selection_threshold is not None else None
        )
        self._layer = layer
        self._library = _native.load()
        self._device = device

    # ------------------------------------------------------------------
    def _validate_input(self, hidden: Tensor, padding: Tensor | None) -> int:
        tokens = hidden.shape[0] if hidden.ndim == 2 else 0
        bad_padding = padding is not None and (
            padding.shape != (tokens,)
            or padding.device != hidden.device
            or padding.dtype != torch.bool
            or not padding.is_contiguous()
        )
        if (
            not 1 <= tokens <= self.max_tokens
            or hidden.shape != (tokens, self.plan.hidden_size)
            or hidden.dtype != torch.bfloat16
            or hidden.device != self._device
            or not hidden.is_contiguous()
            or bad_padding
        ):
            raise ValueError("Sparse input exceeds the prepared token/candidate contract")
        return tokens

    def _call_struct(
        self,
        tokens: int,
        hidden: Tensor,
        ids: Tensor | None,
        weights: Tensor | None,
        padding: Tensor | None,
        out: Tensor | None,
        input_prepared: bool,
    ) -> _native.Call:
        call = _native.Call()
        call.tokens = tokens
        call.ids_are_int64 = int(ids is not None and ids.dtype == torch.int64)
        call.weights_are_bf16 = int(weights is not None and weights.dtype == torch.bfloat16)
        call.input_prepared = int(input_prepared)
        call.hidden = hidden.data_ptr()
        call.ids = ids.data_ptr() if ids is not None else None
        call.weights = weights.data_ptr() if weights is not None else None
        call.padding = padding.data_ptr() if padding is not None else None
        call.out = out.data_ptr() if out is not None else None
        return call

    def _stage(self, name: str, call: _native.Call) -> None:
        stream = torch.cuda.current_stream(self._device).cuda_stream
        code = getattr(self._library, name)(
            ctypes.byref(self._layer),
            self.workspace.buffer.data_ptr(),
            self.workspace.capacity,
            ctypes.byref(call),
            ctypes.c_void_p(stream),
        )
        _native.check(code, name)

    @torch.no_grad()
    def prepare_input(self, hidden: Tensor, padding: Tensor | None = None) -> bool:
        """Run the routing-independent input rotation ahead of the router.

        Returns True when the rotation was enqueued (then pass
        `input_prepared=True` to the next call with the same rows); False, with
        nothing launched, under expert parallelism or for unscreened plans
        (reference progressive.py:3829-3873).  Work is enqueued on the current
        stream.
        """
        p = self.plan
        if self.expert_map is not None or p.completion_count == p.candidate_count:
            return False
        tokens = self._validate_input(hidden, padding)
        with torch.cuda.device(self._device):
            self._stage(
                "cfm_prepare_input",
                self._call_struct(tokens, hidden, None, None, padding, None, False),
            )
        return True

    @torch.no_grad()
    def __call__(
        self,
        hidden: Tensor,
        ids: Tensor,
        weights: Tensor,
        padding: Tensor | None = None,
        out: Tensor | None = None,
        *,
        input_prepared: bool = False,
    ) -> Tensor:
        """Compute the layer's routed-expert output for a batch of decode tokens.

        hidden BF16 `[T, H]`; ids (int32 or int64) and weights (FP32 or BF16)
        `[T, K]` from the router; padding bool `[T]` marks rows that read nothing
        and produce zeros.  Writes `[T, H]` into `out` (allocated if None) and
        adds the call's read statistics to `read_work`.  Everything is enqueued
        on the current CUDA stream without synchronising.
        """
        tokens = self._validate_input(hidden, padding)
        k = self.plan.top_k
        if (
            ids.shape != (tokens, k)
            or weights.shape != ids.shape
            or ids.device != hidden.device
            or weights.device != hidden.device
            or ids.dtype not in (torch.int32, torch.int64)
            or weights.dtype not in (torch.float32, torch.bfloat16)
            or not ids.is_contiguous()
            or not weights.is_contiguous()
            or (
                out is not None
                and (
                    out.shape != hidden.shape
                    or out.dtype != hidden.dtype
                    or out.device != hidden.device
                    or not out.is_contiguous()
                )
            )
        ):
            raise ValueError("Sparse input exceeds the prepared token/candidate contract")
        if out is None:
            out = torch.empty_like(hidden)
        call = self._call_struct(tokens, hidden, ids, weights, padding, out, input_prepared)
        with torch.cuda.device(self._device):
            if self.expert_map is None:
                self._stage("cfm_reader_forward", call)
                return out
            # Expert parallel, replicated tokens: every rank screens its local
            # experts, the scores are summed across ranks so all ranks keep the
            # same channels, and the latent is summed before the owner decodes
            # (reference progressive.py:4245-4251, 4444-4445).
            screened = self.plan.completion_count < self.plan.candidate_count
            if screened:
                self._stage("cfm_prepare_input", call)
            self._stage("cfm_route", call)
            if screened:
                self._stage("cfm_screen", call)
                self._stage("cfm_score", call)
                dist.all_reduce(self.scores[0][:tokens], group=self.ep_group)
                call.scores_ready = 1
            self._stage("cfm_select", call)
            self._stage("cfm_exact", call)
            self._stage("cfm_down", call)
            self._stage("cfm_encode", call)
            if self.rank:
                dist.all_reduce(self.latent[:tokens], group=self.ep_group)
            self._stage("cfm_output", call)
        return out

    def check_status(self) -> None:
        """Raise if a kernel of this reader's workspace reported a device-side error.

        The tensor-memory screen (`tensor_engine="tcgen05"`) bounds every barrier wait;
        a wait that runs out sets a flag in the workspace and leaves the projections
        of that call unwritten, so the kept channels of that call are not to be
        trusted.  Reading the flag synchronises with the device: call this at points
        where the host waits anyway (after a decode step, before reading a report).
        """
        status = self.workspace.status.cpu().tolist()
        if any(status):
            raise RuntimeError(f"reader kernels reported a device-side error: status {status}")

    # ------------------------------------------------------------------
    def report(self) -> dict[str, float | None]:
        """Accumulated read statistics since `read_work` was last zeroed (a device sync).

        Keys and meanings follow the reference's `report` (progressive.py:3517)
        for everything that prices parameter reads: "charged_bytes" is the read
        cost in 32-byte sectors, "read_fraction" its ratio to the dense routed
        experts, "logical_*" price exact bytes, "issued_*" are the bytes the
        kernels request.  The reference's bounds on its own Triton scratch
        traffic have no counterpart here and are not reported.
        """
        work = self.read_work.cpu().tolist()
        native, reference, recovery, selection, sketch = (
            work[0], work[1], work[3], work[4], work[5],
        )
        physical_native, physical_recovery, physical_selection = work[6], work[7], work[9]
        rotation_signs, physical_sketch = work[10], work[17]
        logical = native + recovery + selection + sketch + rotation_signs
        charged = (
            physical_native + physical_recovery + physical_selection + physical_sketch
            + rotation_signs
        )
        h = self.plan.hidden_size
        ranks = dist.get_world_size(self.ep_group) if self.ep_group is not None else 1
        return {
            "charged_bytes": charged,
            "reference_bytes": reference,
            "native_expert_coefficient_bytes": native,
            "physical_native_expert_coefficient_bytes": physical_native,
            "recovery_bytes": recovery,
            "physical_recovery_bytes": physical_recovery,
            "selection_parameter_bytes": selection,
            "physical_selection_parameter_bytes": physical_selection,
            "sketch_bytes": sketch,
            "physical_sketch_bytes": physical_sketch,
            "sketch_resident_bytes": float(self.sketch_resident_bytes),
            "selection_threshold_resident_bytes": 4.0 * (self.selection_threshold is not None),
            "rotation_sign_bytes": rotation_signs,
            "rotation_sign_resident_bytes": float(h),
            "read_fraction": charged / reference if reference else None,
            "logical_charged_bytes": logical,
            "logical_read_fraction": logical / reference if reference else None,
            "issued_sketch_bytes": work[11],
            "issued_gate_up_bytes": work[12],
            "issued_down_bytes": work[13],
            "issued_recovery_encoder_bytes": work[14],
            "grouped_rows": work[16],
            "grouped_issued_matrix_macs": work[15],
            "workspace_bytes": float(self.workspace_bytes),
            "matrix_macs_per_token": float(
                (self.matrix_macs - self.rank * h) / ranks
                + (self.rank * h if self.recovery_owner else 0)
            )
            if self.selection_threshold is None
            else self._threshold_matrix_macs(native, reference, work[19]),
        }

    def _threshold_matrix_macs(self, native: float, reference: float, tokens: float) -> float:
        """Realised MACs per active token of a thresholded reader (reference :4474-4490).

        Every local slot screens 2 H I; every kept channel (native bytes / 6 H)
        costs 3 H; recovery encodes the skipped local channels; the owner decodes
        R x H.
        """
        if not tokens:
            return 0.0
        p = self.plan
        h, i = p.hidden_size, p.expert_width
        slots = reference / (p.native_read_bytes() // p.top_k)
        kept = native / (6 * h)
        local = 2 * h * i * slots + 3 * h * kept + self.rank * (i * slots - kept)
        return local / tokens + (self.rank * h if self.recovery_owner else 0)
