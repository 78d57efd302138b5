"""Binding of the reader to the fused-MoE blocks of the installed vLLM (0.22), and the
48-layer decode study built on it.

The reference binds vLLM 0.29 through model-class overrides, a `RoutedExperts`
subclass and a patch that adds phase fields to the forward context
(`calibration_free_moe/runtime/experts.py:381-516, 884-1299`).  None of those
extension points exist in vLLM 0.22, where the sparse-MoE block of a Qwen3-MoE
layer owns a `gate` and a `FusedMoE` that routes internally.  The binding here
therefore sits one level up: after the weights are loaded it replaces the
`forward` of every such block by a function that

* computes the router output itself (gate, FP32 softmax, top-k, optional
  renormalisation: what `FusedMoE` does for a softmax router without groups),
* takes the step's phase from the attention metadata of the forward context
  (`num_decode_tokens` where the backend orders decode rows first; otherwise a
  step whose longest query is one token is all decode) into a `PhaseContext`, and
* hands rows, routes and context to `ProgressiveExperts.forward_modular`, whose
  stock callable is the block's original `forward`.

Readers are built from the block's own `w13_weight` (gate rows, then up rows) and
a channel-major copy of `w2_weight`; the sketch comes from the library's
construction kernel and the recovery map from `subspace_bank`, so binding a
48-layer model takes seconds per layer.  On the first step after binding, the
first block checks that the stock block and a dense evaluation of those weights
agree on two rows, so a backend that re-lays the expert weights at load time is
noticed instead of read wrongly.

`decode_study` is the end-to-end measurement on a random-weight model of the
Qwen3-30B-A3B shape: one prefill step, then greedy decode; first with the stock
blocks (logits of every decode step are kept), then with the readers bound and
the tokens forced to the stock run's, which gives decode tokens per second for
both, the mean device time of a sparse-MoE block on the decode steps of either run
(CUDA events around the block) and the full-vocabulary KL(stock || sparse) per step
with the reference's formula (`eval/fidelity.py:34-48`).  It needs a GPU and the installed vLLM; nothing
else in the package imports this module.
"""

from __future__ import annotations

import json
import os
import tempfile
import time
from pathlib import Path
from typing import Any

import torch
from torch import Tensor

from ..reader.bank import subspace_bank
from ..reader.budget import compile_budget
from ..reader.progressive import ProgressiveReader, ReaderWorkspace, channel_major_down
from .experts import PhaseContext, ProgressiveExperts


def decode_rows(metadata: Any, tokens: int) -> int:
    """How many leading rows of a step of `tokens` rows are decode rows.

    `metadata` is the attention metadata of any layer of the step (all layers of a
    step share the batch).  Backends that order decode requests first say how many
    rows they are; for the others a step is all decode when its longest query has
    one token and has no decode rows to separate otherwise.  Without metadata (a
    profiling or warm-up run) no row takes the sparse policy.
    """
    if metadata is None:
        return 0
    count = getattr(metadata, "num_decode_tokens", None)
    if count is not None:
        return min(int(count), tokens)
    longest = getattr(metadata, "max_query_len", None)
    if longest is not None and int(longest) == 1:
        return min(int(getattr(metadata, "num_actual_tokens", tokens)), tokens)
    return 0


def route(logits: Tensor, top_k: int, renormalize: bool) -> tuple[Tensor, Tensor]:
    """Softmax router: FP32 probabilities, the top-k of them, optionally renormalised."""
    weights, ids = torch.softmax(logits.float(), dim=-1).topk(top_k, dim=-1)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights, ids.to(torch.int32)


def dense_block(gate_up: Tensor, down: Tensor, x: Tensor, weights: Tensor, ids: Tensor) -> Tensor:
    """The routed experts of a few rows, evaluated densely in FP32 (binding self-check)."""
    width = gate_up.shape[1] // 2
    out = torch.zeros(x.shape, device=x.device, dtype=torch.float32)
    for row in range(x.shape[0]):
        for slot in range(ids.shape[1]):
            expert = int(ids[row, slot])
            gate, up = (gate_up[expert].float() @ x[row].float()).split(width)
            hidden = torch.nn.functional.silu(gate) * up
            out[row] += float(weights[row, slot]) * (down[expert].float() @ hidden)
    return out


class BoundBlock:
    """What replaces `forward` of one sparse-MoE block."""

    def __init__(self, block: torch.nn.Module, experts: ProgressiveExperts, top_k: int,
                 renormalize: bool) -> None:
        self.block, self.experts = block, experts
        self.top_k, self.renormalize = top_k, renormalize
        self.stock_forward = block.forward
        self.sparse_rows = 0
        self.verify = False
        self.enabled = True   # False: decode rows take the stock block too (the comparison run)
        self.timed: list[tuple[torch.cuda.Event, torch.cuda.Event]] | None = None

    def block_microseconds(self) -> float:
        """Mean device time of this block over the decode steps recorded since `timed = []`."""
        torch.cuda.synchronize()
        spans = [start.elapsed_time(end) for start, end in self.timed or []]
        return 1e3 * sum(spans) / max(len(spans), 1)

    def check_layout(self, x: Tensor) -> None:
        """The stock block and a dense evaluation of the stored weights must agree on a few rows:
        a fused-MoE backend that re-lays w13 / w2 when it loads them would otherwise be read
        wrongly.  Runs inside a model step, where the stock block has its forward context."""
        fused = self.block.experts
        probe = x[:2].contiguous()
        logits, _ = self.block.gate(probe)
        weights, ids = route(logits, self.top_k, self.renormalize)
        want = self.stock_forward(probe).float()
        got = dense_block(fused.w13_weight.data, fused.w2_weight.data, probe, weights, ids)
        scale = want.abs().max().clamp_min(1e-12)
        if float((got - want).abs().max() / scale) > 0.05:
            raise RuntimeError(
                "the stock block does not evaluate w13 (gate rows, then up rows) and w2 as stored; "
                "this fused-MoE backend re-lays the expert weights")

    def __call__(self, hidden_states: Tensor) -> Tensor:
        from vllm.forward_context import get_forward_context, is_forward_context_available

        x = hidden_states.view(-1, hidden_states.shape[-1])
        if self.verify and x.shape[0] and is_forward_context_available():
            self.verify = False
            self.check_layout(x)
        metadata = None
        if is_forward_context_available():
            attention = get_forward_context().attn_metadata
            if isinstance(attention, list):  # micro-batched steps keep their stock path
                attention = None
            if isinstance(attention, dict) and attention:
                metadata = next(iter(attention.values()))
        rows = decode_rows(metadata, x.shape[0])
        if rows == 0:
            return self.stock_forward(hidden_states)
        if self.timed is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.timed.append((start, end))
            start.record()
        if self.enabled:
            logits, _ = self.block.gate(x)
            weights, ids = route(logits, self.top_k, self.renormalize)
            self.sparse_rows += rows
            context = PhaseContext(num_decode_tokens=rows)
            out = self.experts.forward_modular(x, weights, ids, context).view(hidden_states.shape)
        else:
            out = self.stock_forward(hidden_states)
        if self.timed is not None:
            end.record()
        return out


def moe_blocks(model: torch.nn.Module) -> list[tuple[str, torch.nn.Module]]:
    """The sparse-MoE blocks of a loaded model: modules with a `gate` and fused `experts`."""
    found = []
    for name, module in model.named_modules():
        experts = getattr(module, "experts", None)
        if experts is not None and hasattr(module, "gate") and hasattr(experts, "w13_weight"):
            found.append((name, module))
    return found


@torch.no_grad()
def bind(model: torch.nn.Module, *, retention: float, screen_keep: float, rank: int,
         max_tokens: int, selection_score: str = "point") -> list[BoundBlock]:
    """Build one reader per sparse-MoE block of `model` and route its decode rows through it.

    Returns the bound blocks (`unbind` restores the stock forwards).  One workspace
    serves all layers, as in the reference's hook (`runtime/experts.py:1210-1243`).
    """
    bound: list[BoundBlock] = []
    workspace = None
    for index, (name, block) in enumerate(moe_blocks(model)):
        fused = block.experts
        gate_up = fused.w13_weight.data
        down = fused.w2_weight.data
        experts, two_width, hidden = gate_up.shape
        width = two_width // 2
        if down.shape != (experts, hidden, width) or gate_up.dtype != torch.bfloat16:
            raise ValueError(f"{name}: expected unquantised BF16 experts [E, 2I, H] and [E, H, I]")
        top_k = int(fused.top_k)
        renormalize = bool(getattr(fused, "renormalize", True))
        plan = compile_budget(hidden_size=hidden, expert_width=width, top_k=top_k,
                              retention=retention, screen_keep=screen_keep)
        decoder = encoder = None
        if rank:
            u, b, _ = subspace_bank(down, rank)
            decoder, encoder = u.bfloat16(), b.bfloat16()
        if workspace is None:
            workspace = ReaderWorkspace(plan, experts, rank, max_tokens, gate_up.device)
        reader = ProgressiveReader(
            gate_up, channel_major_down(down), encoder, decoder, plan, max_tokens,
            selection_score=selection_score, workspace=workspace, sketch_builder="cuda",
            retain_reference_sketch=False,
        )
        stock = block.forward

        def stock_rows(x: Tensor, _weights: Tensor, _ids: Tensor, forward=stock) -> Tensor:
            return forward(x)

        replacement = BoundBlock(block, ProgressiveExperts(reader, stock_rows), top_k, renormalize)
        replacement.verify = index == 0  # one block stands for the backend's weight layout
        block.forward = replacement
        bound.append(replacement)
    torch.cuda.synchronize()
    return bound


def unbind(bound: list[BoundBlock]) -> None:
    for replacement in bound:
        replacement.block.forward = replacement.stock_forward


def kl_and_top1(reference_logits: Tensor, logits: Tensor) -> tuple[Tensor, Tensor]:
    """Row-wise KL(P_reference || P) in FP32 and argmax agreement (reference eval/fidelity.py:34-48)."""
    reference_logprobs = torch.log_softmax(reference_logits.float(), dim=-1)
    logprobs = torch.log_softmax(logits.float(), dim=-1)
    probabilities = reference_logprobs.exp()
    terms = torch.where(probabilities > 0, probabilities * (reference_logprobs - logprobs),
                        torch.zeros_like(probabilities))
    return terms.sum(dim=-1), reference_logits.argmax(dim=-1) == logits.argmax(dim=-1)


# ---------------------------------------------------------------------------
# the 48-layer decode study
# ---------------------------------------------------------------------------
MODEL_CONFIG = {
    "architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe",
    "hidden_size": 2048, "num_hidden_layers": 48, "num_attention_heads": 32,
    "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 6144,
    "moe_intermediate_size": 768, "num_experts": 128, "num_experts_per_tok": 8,
    "norm_topk_prob": True, "decoder_sparse_step": 1, "mlp_only_layers": [],
    "vocab_size": 151936, "max_position_embeddings": 8192, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "attention_bias": False, "attention_dropout": 0.0,
    "use_sliding_window": False, "sliding_window": None, "bos_token_id": 0, "eos_token_id": 1,
}


class LogitsTap:
    """Wraps `model.compute_logits`: keeps every step's logits, or scores them against kept
    ones and returns the kept ones, so that the sampled tokens repeat the first run's."""

    def __init__(self, model: torch.nn.Module) -> None:
        self.model, self.stock = model, model.compute_logits
        self.kept: list[Tensor] = []
        self.kl: list[Tensor] = []
        self.agree: list[Tensor] = []
        self.compare = False
        self.step = 0
        self.stamps: list[float] = []
        model.compute_logits = self

    def __call__(self, hidden_states: Tensor) -> Tensor | None:
        logits = self.stock(hidden_states)
        if logits is None:
            return logits
        torch.cuda.synchronize()
        self.stamps.append(time.perf_counter())
        if not self.compare:
            self.kept.append(logits.detach().clone())
            return logits
        reference = self.kept[self.step]
        divergence, same = kl_and_top1(reference, logits)
        self.kl.append(divergence)
        self.agree.append(same)
        self.step += 1
        return reference.clone()

    def restart(self, compare: bool) -> None:
        self.compare, self.step, self.stamps = compare, 0, []


def decode_study(*, layers: int = 48, batch: int = 32, prompt_tokens: int = 4096,
                 decode_tokens: int = 256, retention: float = 0.123046875,
                 screen_keep: float = 0.625, rank: int = 64, seed: int = 0,
                 memory_fraction: float = 0.55) -> dict:
    """Stock and sparse greedy decode of a random-weight Qwen3-30B-A3B-shaped model in vLLM."""
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")  # the model lives in this process
    from vllm import LLM, SamplingParams

    directory = Path(tempfile.mkdtemp(prefix="cfm_decode_study_"))
    (directory / "config.json").write_text(json.dumps({**MODEL_CONFIG, "num_hidden_layers": layers}))
    llm = LLM(
        model=str(directory), load_format="dummy", dtype="bfloat16", enforce_eager=True,
        skip_tokenizer_init=True, seed=seed, max_model_len=prompt_tokens + decode_tokens + 16,
        max_num_seqs=batch, max_num_batched_tokens=batch * prompt_tokens,
        gpu_memory_utilization=memory_fraction, enable_prefix_caching=False,
        moe_backend="triton",  # keeps w13 / w2 as loaded; bind() checks that on the first step
    )

    def initialise(model: torch.nn.Module) -> int:
        # Dummy loading leaves weights of magnitude 1e-3; draw the weights the benchmark
        # configurations name instead: N(0, 0.02^2), norm gains one.
        generator = torch.Generator(device="cuda").manual_seed(seed)
        count = 0
        for name, parameter in model.named_parameters():
            if parameter.ndim == 1:
                parameter.data.fill_(1.0)
            else:
                parameter.data.normal_(0.0, 0.02, generator=generator)
            count += parameter.numel()
        return count

    parameters = llm.apply_model(initialise)[0]
    taps = llm.apply_model(LogitsTap)
    tap = taps[0]
    generator = torch.Generator().manual_seed(seed)
    prompts = [
        {"prompt_token_ids": torch.randint(0, MODEL_CONFIG["vocab_size"], (prompt_tokens,),
                                           generator=generator).tolist()}
        for _ in range(batch)
    ]
    sampling = SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True,
                              detokenize=False)

    def run(compare: bool) -> tuple[float, list]:
        tap.restart(compare)
        outputs = llm.generate(prompts, sampling, use_tqdm=False)
        stamps = tap.stamps
        # The first stamp closes the prefill step; the others close decode steps.
        seconds = stamps[-1] - stamps[0]
        return batch * (len(stamps) - 1) / seconds, outputs

    started = time.perf_counter()
    bound = llm.apply_model(lambda model: bind(
        model, retention=retention, screen_keep=screen_keep, rank=rank, max_tokens=batch))[0]
    bind_seconds = time.perf_counter() - started

    def arm(enabled: bool) -> None:
        for replacement in bound:
            replacement.enabled, replacement.timed = enabled, []

    def block_time() -> float:
        return sum(replacement.block_microseconds() for replacement in bound) / len(bound)

    arm(False)
    stock_rate, stock_outputs = run(False)
    stock_block = block_time()
    steps = len(tap.kept)
    arm(True)
    sparse_rate, sparse_outputs = run(True)
    sparse_block = block_time()
    same_tokens = all(
        list(a.outputs[0].token_ids) == list(b.outputs[0].token_ids)
        for a, b in zip(stock_outputs, sparse_outputs)
    )
    divergence = torch.stack(tap.kl[1:]).float()  # step 0 is the prefill step (stock in both runs)
    agreement = torch.stack(tap.agree[1:]).float()
    reports = [replacement.experts.reader.report() for replacement in bound[:1]]
    return {
        "model": f"Qwen3-30B-A3B-shaped, {layers} layers, random weights N(0, 0.02^2), "
                 f"{parameters / 1e9:.1f} B parameters",
        "engine": "vLLM 0.22 in process, eager, one prefill step then greedy decode",
        "batch": batch, "prompt_tokens": prompt_tokens, "decode_steps": steps - 1,
        "stock_decode_tokens_per_s": stock_rate, "sparse_decode_tokens_per_s": sparse_rate,
        "stock_moe_block_us": stock_block, "sparse_moe_block_us": sparse_block,
        "bind_seconds": bind_seconds, "sparse_rows_per_layer": bound[0].sparse_rows,
        "tokens_forced_to_stock": same_tokens,
        "kl_stock_to_sparse_mean": float(divergence.mean()),
        "kl_stock_to_sparse_max": float(divergence.max()),
        "top1_agreement": float(agreement.mean()),
        "prefill_step_kl": float(tap.kl[0].float().mean()),
        "read_fraction_layer0": reports[0]["read_fraction"],
    }


if __name__ == "__main__":
    import argparse

    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--layers", type=int, default=48)
    parser.add_argument("--batch", type=int, default=32)
    parser.add_argument("--prompt-tokens", type=int, default=4096)
    parser.add_argument("--decode-tokens", type=int, default=256)
    parser.add_argument("--memory-fraction", type=float, default=0.55,
                        help="share of the GPU's memory the engine may take (weights and KV cache)")
    arguments = parser.parse_args()
    print(json.dumps(decode_study(layers=arguments.layers, batch=arguments.batch,
                                  prompt_tokens=arguments.prompt_tokens,
                                  decode_tokens=arguments.decode_tokens,
                                  memory_fraction=arguments.memory_fraction)))
