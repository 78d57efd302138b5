"""Benchmark of the sparse MoE decode reader: decode tokens/s on a Qwen3-30B-A3B-shaped layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|triton]
                    [--tokens T | --sweep-tokens T1,T2,...] [--layers L] [--config NAME]
                    [--retention R] [--screen-keep S] [--budgets R1:S1,R2:S2,...]

A step is one call of the reader on one batch of T decode tokens of one MoE
layer.  Steps cycle over L independent layers (own weights, own inputs) so that
consecutive steps touch different memory and the bytes come from HBM, not L2.
Inputs are synthetic (`cfm_b200.synthetic`), drawn on the device.

The JSON line printed by rank 0 reports whole-job tokens/s with inputs resident
(`value`: median of seven samples, each at least 0.3 s of CUDA-graph replays and
at least `--steps` steps, timed with CUDA events), the same through the public
operator with host buffers and copies in the timed region (`e2e`), every
kernel's algorithmic bytes, mean launch time and HBM roofline fraction
(`stage_bytes`, `stage_ms`, `stage_frac`; `roofline` repeats the slowest one),
the whole layer's (`layer_roofline`) and the CPU oracle timed on the host cores
(`cpu_baseline`).  `--sweep-tokens` and `--budgets` print one line per batch size
and budget from one set of layers.  `--impl triton` times the reference's own
Triton reader (installed under baseline/_ref) on the same device with the same
protocol; `--impl reference` times the CPU port of the reference's reader and
adds that Triton measurement as `gpu_comparator` when a device is present.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

import cfm_b200  # noqa: E402,F401
from cfm_b200 import synthetic  # noqa: E402
from cfm_b200.reader.budget import compile_budget  # noqa: E402

METRIC = "sparse-MoE decode tok/s (Qwen3-30B-A3B shape)"
UNIT = "tokens/s"
STAGES = ("cfm_prepare_input", "cfm_route", "cfm_screen", "cfm_select", "cfm_exact",
          "cfm_down", "cfm_encode", "cfm_output")
KERNEL_OF_STAGE = {
    "cfm_prepare_input": "k_prepare", "cfm_route": "k_route", "cfm_screen": "k_screen",
    "cfm_select": "k_select", "cfm_exact": "k_exact", "cfm_down": "k_down",
    "cfm_encode": "k_encode", "cfm_output": "k_output",
}
SAMPLES = 7            # timed samples per number; the median is reported
SAMPLE_SECONDS = 0.3   # least duration of one sample
REFERENCE_INSTALL = ROOT / "baseline" / "_ref"


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def median(values: list[float]) -> float:
    ordered = sorted(values)
    return ordered[len(ordered) // 2]


# ---------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------
def device_layer(shape: synthetic.LayerShape, seed: int, device: torch.device,
                 world: int = 1, rank: int = 0):
    """Random BF16 weights of one layer, drawn on the device.

    Under expert parallelism a rank draws only its E / world experts (own seed);
    router and decoder are replicated (common seed).
    """
    g = torch.Generator(device=device).manual_seed(seed * 64 + rank + 1)
    e, h, i, r = shape.experts // world, shape.hidden, shape.width, shape.rank
    gate_up = torch.empty(e, 2 * i, h, device=device, dtype=torch.bfloat16)
    down = torch.empty(e, i, h, device=device, dtype=torch.bfloat16)  # physical channel-major
    for expert in range(e):  # one expert at a time keeps the FP32 temporaries small
        gate_up[expert] = (torch.randn(2 * i, h, device=device, generator=g) * shape.sigma).bfloat16()
        down[expert] = (torch.randn(i, h, device=device, generator=g) * shape.sigma).bfloat16()
    common = torch.Generator(device=device).manual_seed(seed * 64)
    router = (torch.randn(shape.experts, h, device=device, generator=common) * shape.sigma).bfloat16()
    decoder = torch.linalg.qr(torch.randn(h, r, device=device, generator=common)).Q.bfloat16()
    encoder = torch.stack(
        [torch.linalg.qr(torch.randn(i, r, device=device, generator=g)).Q.T for _ in range(e)]
    ).bfloat16()
    return gate_up, down.transpose(1, 2), router, decoder, encoder, g


def device_batch(shape, router, tokens, generator, device):
    h, k = shape.hidden, shape.top_k
    x = torch.randn(tokens, h, device=device, generator=generator)
    if shape.input_kind == "outliers":
        count = -(-h // 100)
        dims = torch.randperm(h, device=device, generator=generator)[:count]
        x[:, dims] *= 20.0
    elif shape.input_kind == "student_t":
        chi = torch.randn(tokens, h, 3, device=device, generator=generator).square().sum(-1)
        x = x / (chi / 3).sqrt() / 3.0**0.5
    hidden = x.bfloat16()
    logits = hidden.float() @ router.float().T
    if shape.router_bias:
        logits = logits + torch.randn(router.shape[0], device=device, generator=generator)
    weights, ids = torch.softmax(logits, -1, dtype=torch.float32).topk(k, -1)
    if shape.renormalize:
        weights = weights / weights.sum(-1, keepdim=True)
    return hidden, ids.int().contiguous(), weights.float().contiguous()


def algorithmic_bytes(reader, tokens: int) -> dict[str, float]:
    """`distinct_bytes` of a single-GPU reader's last call."""
    return distinct_bytes(reader.plan, reader.native_gu.shape[0], reader.rank, reader.ids,
                          reader.selected, reader.sketch_coordinates, tokens)


def distinct_bytes(p, e: int, r: int, ids, selected, coordinates, tokens: int) -> dict[str, float]:
    """Distinct bytes one call must bring from HBM, from the realised routing and selection.

    `p` is the plan, `e` the number of experts the ids index, `r` the recovery rank;
    `ids` `[T, K]` sorted expert ids (-1 for experts held elsewhere), `selected`
    `[T, N]` the kept-channel mask, `coordinates` `[T, B, KEEP]` the kept rotated
    coordinates.

    Per routed local expert: the code runs of the union of its tokens' kept
    coordinates (kernel layout, I/2 bytes per coordinate), its FP16 scale planes
    and FP32 norms; gate, up and down rows of the union of kept channels; encoder
    rows of the union of skipped channels.  Plus the decoder, the signs and the
    tokens' inputs, outputs and routes.
    """
    h, i, k = p.hidden_size, p.expert_width, p.top_k
    blocks = h // 128
    screened = p.completion_count < p.candidate_count
    ids = ids[:tokens].long()  # [T, K] sorted local ids
    selected = selected[:tokens].reshape(tokens, k, i)
    valid = ids >= 0
    flat = ids.clamp_min(0).reshape(-1)
    kept_union = torch.zeros(e, i, dtype=torch.bool, device=ids.device)
    kept_union.index_put_((flat,), selected.reshape(-1, i) & valid.reshape(-1, 1), accumulate=True)
    skipped_union = torch.zeros_like(kept_union)
    skipped_union.index_put_((flat,), ~selected.reshape(-1, i) & valid.reshape(-1, 1), accumulate=True)
    routed = torch.zeros(e, dtype=torch.bool, device=ids.device)
    routed[flat[valid.reshape(-1)]] = True
    experts = int(routed.sum())
    screen = 0
    if screened:
        coordinates = coordinates[:tokens].long()  # [T, B, KEEP]
        support = torch.zeros(tokens, blocks, 128, dtype=torch.bool, device=ids.device)
        support.scatter_(-1, coordinates, True)
        support = support.reshape(tokens, h)
        coordinate_union = torch.zeros(e, h, dtype=torch.bool, device=ids.device)
        for slot in range(k):  # one slot at a time keeps the temporaries at T x H
            coordinate_union.index_put_(
                (ids[:, slot].clamp_min(0),), support & valid[:, slot, None], accumulate=True)
        screen = int(coordinate_union.sum()) * (i // 2) + experts * (blocks * 2 * (2 * i) + 4 * i)
    kept = int(kept_union.sum())
    exact = kept * 2 * 2 * h
    down = kept * 2 * h
    encode = int(skipped_union.sum()) * 2 * r
    fixed = 2 * h * r + h + tokens * (4 * h + 8 * k)
    return {
        "k_screen": float(screen), "k_exact": float(exact + tokens * 2 * h),
        "k_down": float(down), "k_encode": float(encode), "k_output": float(2 * h * r),
        "total": float(screen + exact + down + encode + fixed),
    }


def packed_batch(batch):
    """The tensors of one step's inputs as views of a single device block.

    The block is attached to the first view as `_packed`; offsets are 256-byte
    aligned, so the views satisfy the reader's alignment contract.
    """
    sizes = [t.numel() * t.element_size() for t in batch]
    offsets, at = [], 0
    for size in sizes:
        offsets.append(at)
        at = (at + size + 255) // 256 * 256
    block = torch.empty(at, dtype=torch.uint8, device=batch[0].device)
    views = []
    for tensor, offset, size in zip(batch, offsets, sizes):
        view = block[offset : offset + size].view(tensor.dtype).view(tensor.shape)
        view.copy_(tensor)
        views.append(view)
    views[0]._packed = block
    return tuple(views)


def expert_parallel_bytes(sharded, tokens: int, world: int) -> dict[str, float]:
    """`algorithmic_bytes` of one rank of an expert-parallel layer with a replicated screen.

    The home side screens and encodes this rank's own tokens over all experts; the
    owner side reads gate, up and down rows of the local experts' kept channels for
    the tokens of all ranks.
    """
    owner, home = sharded.reader, sharded.home
    space = home.workspace
    home_side = distinct_bytes(owner.plan, home.norms.shape[0], home.rank, space.ids,
                               space.selected, space.sketch_coordinates, tokens)
    rows = tokens * world
    kept = torch.zeros(rows, owner.plan.candidate_count + 1, dtype=torch.bool,
                       device=owner.ids.device)
    lists = owner.candidate_ids[-1][:rows].long()
    kept.scatter_(1, torch.where(lists >= 0, lists, owner.plan.candidate_count), True)
    owner_side = distinct_bytes(owner.plan, owner.native_gu.shape[0], 0, owner.ids,
                                kept[:, :-1].contiguous(), owner.sketch_coordinates, rows)
    out = {"k_screen": home_side["k_screen"], "k_encode": home_side["k_encode"],
           "k_output": home_side["k_output"], "k_exact": owner_side["k_exact"],
           "k_down": owner_side["k_down"]}
    out["total"] = (home_side["total"] - home_side["k_exact"] - home_side["k_down"]
                    + owner_side["k_exact"] + owner_side["k_down"])
    return out


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            pass

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        try:
            text, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            text = ""
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in text.strip().splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 7:
                continue
            try:
                clocks.append(float(fields[0]))
                maxima.append(float(fields[1]))
            except ValueError:
                continue
            for name, field in zip(names, fields[3:7]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {
            "sm_mhz": clocks[len(clocks) // 2] if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }


def timed_samples(replay, steps: int, stream, barrier, reduce_max=None) -> tuple[float, int, list]:
    """Median milliseconds per step over SAMPLES samples of CUDA-graph replays.

    `replay(i)` enqueues step i.  A sample is at least `steps` steps and at least
    SAMPLE_SECONDS long (its length comes from one untimed-for-the-record trial of
    `steps` steps); it is bracketed by `barrier()` on both sides and timed with CUDA
    events on the launching stream.  Under several ranks every sample's time is the
    maximum over the ranks (`reduce_max`).
    """
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def run(count: int) -> float:
        barrier()
        begin.record(stream)
        for i in range(count):
            replay(i)
        end.record(stream)
        barrier()
        return begin.elapsed_time(end)

    trial = run(steps)
    if reduce_max is not None:
        trial = reduce_max([trial])[0]
    per_step = max(trial / steps, 1e-3)
    count = max(steps, int(-(-SAMPLE_SECONDS * 1e3 // per_step)))
    samples = [run(count) for _ in range(SAMPLES)]
    if reduce_max is not None:
        samples = reduce_max(samples)
    per_step_samples = [s / count for s in samples]
    return median(per_step_samples), count, per_step_samples


# ---------------------------------------------------------------------------
# CPU arms
# ---------------------------------------------------------------------------
def cpu_arguments(shape, plan, tokens: int):
    from cfm_b200.reader.progressive import channel_major_down
    from cfm_b200.reader.sketch import block_hadamard_signs, build_sketch

    layer, g = synthetic.make_layer(shape, 0)
    hidden, ids, weights = synthetic.make_batch(layer, tokens, g)
    signs = block_hadamard_signs(shape.hidden, "cpu")
    codes, statistics = build_sketch(layer.gate_up, signs)
    down = channel_major_down(layer.down)
    return dict(
        plan=plan, gate_up=layer.gate_up, down=down, codes=codes, statistics=statistics,
        signs=signs, hidden=hidden, ids=ids, weights=weights, encoder=layer.encoder,
        decoder=layer.decoder, norms=down.float().square().sum(1).sqrt(),
    )


def cpu_oracle_rate(shape, plan, tokens: int, seconds: float = 10.0) -> dict:
    """Time the CPU oracle (a port of the reference's PyTorch reader) on the host cores."""
    from oracle import reader_oracle

    arguments = cpu_arguments(shape, plan, tokens)
    reader_oracle.forward(**{**arguments, "hidden": arguments["hidden"][:1],
                             "ids": arguments["ids"][:1], "weights": arguments["weights"][:1]})
    done, elapsed, cores = 0, 0.0, 1
    while elapsed < seconds and done < 64 * tokens:
        start = time.perf_counter()
        cores = reader_oracle.forward(**arguments)["threads"]
        elapsed += time.perf_counter() - start
        done += tokens
    return {
        "value": done / elapsed, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{done} tokens of the {shape.name} layer in batches of {tokens} "
                  f"({elapsed:.1f} s; sketch construction excluded)",
    }


def triton_comparator(args) -> dict:
    """The reference's Triton reader timed on this box by `--impl triton` in a child process."""
    if not torch.cuda.is_available():
        return {"unavailable": "no CUDA device in this process"}
    command = [sys.executable, str(ROOT / "bench.py"), "--impl", "triton", "--config", args.config,
               "--tokens", str(args.tokens), "--layers", str(args.layers), "--steps", "48",
               "--warmup", "12"]
    try:
        done = subprocess.run(command, capture_output=True, text=True, timeout=420)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the Triton reader did not finish within 420 s"}
    for line in reversed(done.stdout.strip().splitlines()):
        if line.startswith("{"):
            result = json.loads(line)
            keep = ("value", "unit", "ms_per_step", "unavailable", "selection_agreement", "options",
                    "failed_variants", "samples_ms_per_step")
            return {key: result[key] for key in keep if key in result}
    tail = (done.stderr or done.stdout).strip().splitlines()[-3:]
    return {"unavailable": "no result line; " + " | ".join(tail)[-400:]}


def run_reference(args, shape, plan) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import reader_oracle

    tokens = min(args.tokens, 64)
    arguments = cpu_arguments(shape, plan, tokens)
    cores = 1
    for _ in range(args.warmup):
        cores = reader_oracle.forward(**arguments)["threads"]
    start = time.perf_counter()
    for _ in range(args.steps):
        reader_oracle.forward(**arguments)
    elapsed = time.perf_counter() - start
    value = tokens * args.steps / elapsed
    sample = f"{tokens} tokens per step of the {shape.name} layer, CPU port of the reference reader"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(shape, plan, tokens, 1, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_gpu_comparator:
        # The reference's own GPU implementation of the same step, same box, for context.
        line["gpu_comparator"] = {"what": "the reference's Triton ProgressiveReader, unmodified, "
                                          "one GPU, CUDA-graph replays", **triton_comparator(args)}
    print(json.dumps(line))


def run_triton(args, shape, plan) -> None:
    """The reference's Triton `ProgressiveReader` on cuda:0, timed like the reader of this repository."""
    base = {"impl": "triton-reference", "metric": METRIC, "unit": UNIT, "n_gpus": 1,
            "config": workload_config(shape, plan, args.tokens, args.layers, 1)}
    if not (REFERENCE_INSTALL / "calibration_free_moe").is_dir():
        print(json.dumps({**base, "unavailable": "baseline/_ref holds no install of the reference"}))
        return
    sys.path.insert(0, str(REFERENCE_INSTALL))
    try:
        from calibration_free_moe.reader.budget import compile_budget as reference_budget
        from calibration_free_moe.reader.progressive import ProgressiveReader as TritonReader
    except Exception as error:  # noqa: BLE001
        print(json.dumps({**base, "unavailable": f"import failed: {error!r}"[:400]}))
        return
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    tokens, layers = args.tokens, args.layers
    reference_plan = reference_budget(
        hidden_size=shape.hidden, expert_width=shape.width, top_k=shape.top_k,
        retention=args.retention if args.retention is not None else shape.retention,
        screen_keep=args.screen_keep if args.screen_keep is not None else shape.screen_keep,
    )
    options = {"selection_score": "point"}
    errors: list = []
    try:
        weights_of_layer, batches = [], []
        for index in range(layers):
            gate_up, down, router, decoder, encoder, g = device_layer(shape, index, device)
            weights_of_layer.append((gate_up, down, encoder, decoder))
            batches.append(device_batch(shape, router, tokens, g, device))
            del router
        first_layer = weights_of_layer[0]
        outs = [torch.empty_like(b[0]) for b in batches]
        stream = torch.cuda.Stream(device)
        readers: list = []

        def step(index: int) -> None:
            readers[index](*batches[index], None, outs[index])

        def build_and_warm() -> None:
            readers.clear()
            for index in range(layers):
                readers.append(TritonReader(*weights_of_layer[index], reference_plan, tokens,
                                            **options))
            torch.cuda.synchronize()  # built on the default stream, used on `stream`
            for index in range(layers):
                step(index)
            stream.synchronize()

        with torch.cuda.stream(stream):
            # The reference's scheduling options do not change its arithmetic
            # (progressive.py:3199-3204).  Its defaults first; if a kernel does not build
            # with the installed Triton, the variants that avoid that kernel, in turn.
            variants = [
                {},
                {"pdl": False},
                {"pdl": False, "grouped_screen_tokens": 1 << 20},
                {"pdl": False, "grouped_screen_tokens": 1 << 20, "grouped_tokens": 1 << 20},
            ]
            for variant in variants:
                options = {"selection_score": "point", **variant}
                try:
                    build_and_warm()
                    break
                except Exception as error:  # noqa: BLE001
                    errors.append({"options": variant,
                                   "error": f"{type(error).__name__}: {error}"[:1200]})
                    if variant is variants[-1]:
                        raise
            graphs = []
            for index in range(layers):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step(index)
                graphs.append(graph)
            for i in range(args.warmup):
                graphs[i % layers].replay()
            step_ms, count, samples = timed_samples(
                lambda i: graphs[i % layers].replay(), args.steps, stream, torch.cuda.synchronize)
        # Agreement of the kept channels with this repository's reader, layer 0, same inputs.
        from cfm_b200.reader.progressive import ProgressiveReader

        ours = ProgressiveReader(*first_layer, plan, tokens, selection_score="point")
        ours(*batches[0])
        readers[0](*batches[0])
        torch.cuda.synchronize()
        theirs = readers[0].selected[:tokens].bool()
        mine = ours.selected[:tokens]
        same = (theirs == mine).all(1)
        agreement = {
            "tokens": tokens, "tokens_with_identical_kept_channels": int(same.sum()),
            "channels_that_differ": int((theirs != mine).sum()) // 2,
            "kept_per_token": plan.final_count,
        }
    except Exception as error:  # noqa: BLE001
        print(json.dumps({**base, "options": options, "failed_variants": errors,
                          "unavailable": f"{type(error).__name__}: {error}"[:600]}))
        return
    print(json.dumps({
        **base, "value": tokens / (step_ms * 1e-3), "ms_per_step": step_ms,
        "steps": count, "warmup": args.warmup, "samples_ms_per_step": [round(s, 5) for s in samples],
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "options": options,
        "failed_variants": errors, "selection_agreement": agreement,
    }))


def workload_config(shape, plan, tokens, layers, gpus) -> dict:
    return {
        "workload": f"{shape.name}-shaped MoE layer, decode batch {tokens}",
        "hidden": shape.hidden, "experts": shape.experts, "expert_width": shape.width,
        "top_k": shape.top_k, "recovery_rank": shape.rank, "kept_channels": plan.final_count,
        "screen_coordinates": plan.screen_coordinates, "selection_score": "point",
        "tokens_per_step": tokens, "layers_cycled": layers,
        "l2": f"steps cycle over {layers} layers with distinct weights, inputs and workspaces",
        "timing": f"median of {SAMPLES} samples, each >= {SAMPLE_SECONDS} s of CUDA-graph replays "
                  "and >= `steps` steps, CUDA events on the launching stream",
        "parallelism": "single GPU" if gpus == 1 else (
            f"expert parallel over {gpus} GPUs: {shape.experts // gpus} experts per rank, "
            f"{tokens} tokens per rank per step; sketch replicated, home-rank screen and "
            "selection, all_gather of hidden rows and router outputs (NCCL), kept-channel "
            "lists and FP32 partial rows stored into the peers' memory by the library's "
            "kernels (NVLink) unless --exchange collective"),
    }


def trace(message: str) -> None:
    """Progress marker on stderr when CFM_BENCH_TRACE is set (for diagnosing multi-rank runs)."""
    if os.environ.get("CFM_BENCH_TRACE"):
        print(f"[rank {os.environ.get('RANK', '0')}] {message}", file=sys.stderr, flush=True)


# ---------------------------------------------------------------------------
# this repository's reader
# ---------------------------------------------------------------------------
def expert_parallel_parity(shape, plan, world: int, rank: int, device) -> dict:
    """Before any timing: the expert-parallel reader against a single-GPU reader on a small layer.

    A layer of the benchmark's shape with 16 experts per rank is sharded like the
    timed one; every rank then gathers all experts, builds a single-GPU reader and
    runs its own tokens through both.  Kept-channel lists must be identical and
    outputs within the tolerance the reference allows between its own paths.
    """
    import torch.distributed as dist

    from cfm_b200.reader.expert_parallel import ExpertParallelReader
    from cfm_b200.reader.progressive import ProgressiveReader

    small = dataclasses.replace(shape, experts=16 * world)
    tokens = 16
    gate_up, down, router, decoder, encoder, g = device_layer(small, 977, device, world, rank)
    sharded = ExpertParallelReader(gate_up, down, encoder, decoder, plan, tokens,
                                   global_experts=small.experts, selection_score="point")
    hidden, ids, weights = device_batch(small, router, tokens, g, device)
    out = sharded(hidden, ids, weights).clone()
    kept = sharded.home.workspace.candidate_ids[:tokens].clone()

    def gathered(local):
        whole = local.new_empty((world * local.shape[0], *local.shape[1:]))
        dist.all_gather_into_tensor(whole, local.contiguous())
        return whole

    all_gate_up = gathered(gate_up)
    all_down = gathered(down.transpose(1, 2)).transpose(1, 2)  # physical [E, I, H]
    all_encoder = gathered(encoder)
    single = ProgressiveReader(all_gate_up, all_down, all_encoder, decoder, plan, tokens,
                               selection_score="point")
    want = single(hidden, ids, weights)
    torch.cuda.synchronize()
    lists_equal = torch.equal(kept, single.candidate_ids[-1][:tokens])
    close = torch.allclose(out.float(), want.float(), rtol=0.016, atol=2e-3)
    worst = float((out.float() - want.float()).abs().max())
    verdict = torch.tensor([int(lists_equal), int(close)], device=device)
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    return {"lists_equal": bool(verdict[0]), "outputs_close": bool(verdict[1]),
            "experts": small.experts, "tokens_per_rank": tokens, "max_abs_difference_rank0": worst}


def expert_parallel_timeline(sharded, batches, stream, repeats: int = 50) -> dict:
    """Median microseconds between the stage boundaries of eager expert-parallel steps.

    Every stage of `ExpertParallelReader` reports when it has been enqueued; a CUDA
    event recorded there on the launching stream closes the interval that stage's
    kernels (or collective) occupy on that stream.  Work on the side stream (the
    recovery encoder) overlaps and has no interval of its own.
    """
    import torch.distributed as dist

    names: list[str] = []
    intervals: dict[str, list[float]] = {}
    layers = len(sharded)
    with torch.cuda.stream(stream):
        for repeat in range(repeats + 5):
            reader = sharded[repeat % layers]
            events = [("start", torch.cuda.Event(enable_timing=True))]
            dist.barrier()
            torch.cuda.synchronize()
            events[0][1].record(stream)

            def trace(name, events=events):
                event = torch.cuda.Event(enable_timing=True)
                event.record(stream)
                events.append((name, event))

            reader.engine.trace = trace
            reader(*batches[repeat % layers])
            reader.engine.trace = None
            stream.synchronize()
            if repeat < 5:
                continue
            for (_, before), (name, after) in zip(events, events[1:]):
                if name not in intervals:
                    names.append(name)
                intervals.setdefault(name, []).append(1e3 * before.elapsed_time(after))
            intervals.setdefault("whole step", []).append(
                1e3 * events[0][1].elapsed_time(events[-1][1]))
    return {name: round(median(intervals[name]), 2) for name in names + ["whole step"]}


def run_ours(args, shape, plans) -> None:
    import ctypes

    from cfm_b200 import _native
    from cfm_b200.reader.progressive import ProgressiveReader
    from cfm_b200.reader.sketch import block_hadamard_signs, build_sketch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    parity = None
    if distributed:
        import torch.distributed as dist

        # The small all_gathers left on NCCL gain nothing from in-switch reduction, and
        # ranks of this benchmark leave without tearing the communicator down.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
        parity = expert_parallel_parity(shape, plans[0][1], world, rank, device)
        if not (parity["lists_equal"] and parity["outputs_close"]):
            if rank == 0:
                print(json.dumps({"error": "expert-parallel parity check failed", **parity}))
            sys.stdout.flush()
            os._exit(3)
        trace("parity checked")
    layers = args.layers
    token_counts = args.sweep_tokens or [args.tokens]
    capacity = max(token_counts)
    weights_of_layer, sketches = [], []
    for index in range(layers):
        gate_up, down, router, decoder, encoder, g = device_layer(shape, index, device, world, rank)
        weights_of_layer.append((gate_up, down, encoder, decoder, router, g))
        # One sketch per layer serves every budget of a sweep.
        sketches.append(build_sketch(gate_up, block_hadamard_signs(shape.hidden, device))
                        if len(plans) > 1 else None)
    stream = torch.cuda.Stream(device)
    for label, plan in plans:
        readers, sharded = [], []
        for index in range(layers):
            gate_up, down, encoder, decoder, _, _ = weights_of_layer[index]
            if distributed:
                from cfm_b200.reader.expert_parallel import ExpertParallelReader

                sharded.append(ExpertParallelReader(
                    gate_up, down, encoder, decoder, plan, capacity, global_experts=shape.experts,
                    selection_score="point", retain_reference_sketch=False, sketch=sketches[index],
                    exchange=args.exchange,
                ))
                readers.append(sharded[-1].reader)
            else:
                readers.append(ProgressiveReader(
                    gate_up, down, encoder, decoder, plan, capacity,
                    selection_score="point", retain_reference_sketch=False,
                    tensor_engine=args.tensor_engine, row_engine=args.row_engine,
                    sketch=sketches[index],
                ))
        trace(f"layers built for {label}")
        for tokens in token_counts:
            batches = []
            for index in range(layers):
                router, g = weights_of_layer[index][4:6]
                batches.append(packed_batch(device_batch(shape, router, tokens, g, device)))
            # Readers and batches were made on the default stream and are used on the
            # benchmark's own (non-blocking) stream from here on: their construction,
            # the zero fill of the workspaces included, has to be complete first.
            torch.cuda.synchronize()
            line = measure(args, shape, plan, tokens, readers, sharded, batches, stream,
                           rank, world, local)
            timeline = (expert_parallel_timeline(sharded, batches, stream)
                        if distributed and args.timeline else None)
            if rank == 0:
                if timeline is not None:
                    line["timeline_us"] = timeline
                if parity is not None:
                    line["parity_checked"] = True
                    line["parity"] = parity
                if len(plans) > 1:
                    line["budget"] = label
                if not args.no_cpu_baseline and world == 1 and len(plans) == 1 \
                        and tokens == token_counts[-1]:
                    line["cpu_baseline"] = cpu_oracle_rate(shape, plan, min(tokens, 64))
                print(json.dumps(line), flush=True)
        del readers, sharded
    if distributed:
        # Tearing down a NCCL communicator while CUDA graphs that captured its
        # collectives are alive blocks on this stack; meet at a barrier and leave
        # without the communicator teardown.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def measure(args, shape, plan, tokens, readers, sharded, batches, stream, rank, world, local):
    """Resident, end-to-end and per-stage timings of one (plan, batch size); the line of rank 0."""
    import ctypes

    from cfm_b200 import _native

    distributed = world > 1
    layers = len(readers)
    device = batches[0][0].device
    outs = [torch.empty_like(b[0]) for b in batches]
    if distributed:
        import torch.distributed as dist

    def step(index: int) -> None:
        hidden, ids, weights = batches[index]
        if distributed:
            outs[index].copy_(sharded[index](hidden, ids, weights))
        else:
            readers[index](hidden, ids, weights, None, outs[index])

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(values: list[float]) -> list[float]:
        box = torch.tensor(values, device=device, dtype=torch.float64)
        dist.all_reduce(box, op=dist.ReduceOp.MAX)
        return box.tolist()

    with torch.cuda.stream(stream):
        for index in range(layers):
            step(index)
        stream.synchronize()
        trace("eager steps done")
        graphs = []
        for index in range(layers):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step(index)
            graphs.append(graph)
        trace("graphs captured")

        # ---- resident-input throughput ---------------------------------
        for i in range(args.warmup):
            graphs[i % layers].replay()
        sampler = ClockSampler(local) if rank == 0 else None
        step_ms, steps_per_sample, samples = timed_samples(
            lambda i: graphs[i % layers].replay(), args.steps, stream, barrier,
            reduce_max if distributed else None)
        clocks = sampler.stop() if sampler else None
        trace("timed region done")

        # ---- end to end: host buffers, copies inside the timed region ---
        # A step's inputs (hidden rows, router ids and weights) sit in one block on both
        # sides, so they cross in one copy.
        host_in = [b[0]._packed.cpu().pin_memory() for b in batches]
        host_out = [torch.empty_like(o, device="cpu").pin_memory() for o in outs]

        def e2e_step(index: int) -> None:
            batches[index][0]._packed.copy_(host_in[index], non_blocking=True)
            graphs[index].replay()
            host_out[index].copy_(outs[index], non_blocking=True)
            stream.synchronize()

        for i in range(args.warmup):
            e2e_step(i % layers)
        e2e_steps = max(args.steps, min(steps_per_sample, 2000))
        e2e_samples = []
        for _ in range(3):
            barrier()
            start = time.perf_counter()
            for i in range(e2e_steps):
                e2e_step(i % layers)
            barrier()
            e2e_samples.append(1e3 * (time.perf_counter() - start) / e2e_steps)
        if distributed:
            e2e_samples = reduce_max(e2e_samples)
        e2e_ms = median(e2e_samples)
        trace("end-to-end region done")

        # ---- per-stage device times (CUDA events on the launching stream) --
        # Every layer's workspace holds the state of its own last call, so one
        # stage can be replayed for all L layers back to back: one graph per stage
        # with L launches, timed as a whole, gives that kernel's mean duration on
        # data that rotates through the layers like the steps above.
        library = _native.load()
        stage_ms = {}
        calls = [] if distributed else [
            readers[i]._call_struct(tokens, *batches[i], None, outs[i], False)
            for i in range(layers)
        ]

        def launch_stage(name: str) -> None:
            for i in range(layers):
                reader = readers[i]
                _native.check(getattr(library, name)(
                    ctypes.byref(reader._layer), reader.workspace.buffer.data_ptr(),
                    reader.workspace.capacity, ctypes.byref(calls[i]),
                    ctypes.c_void_p(stream.cuda_stream)), name)

        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for name in (() if distributed else STAGES):
            launch_stage(name)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                launch_stage(name)
            graph.replay()
            stage_samples = []
            for _ in range(5):
                begin.record(stream)
                for _ in range(10):
                    graph.replay()
                end.record(stream)
                stream.synchronize()
                stage_samples.append(begin.elapsed_time(end) / (10 * layers))
            stage_ms[name] = median(stage_samples)
        if distributed:
            bytes_by_kernel = expert_parallel_bytes(sharded[0], tokens, world)
            report = sharded[0].report()
        else:
            bytes_by_kernel = algorithmic_bytes(readers[0], tokens)
            report = readers[0].report()
        del graphs

    job_bytes = torch.tensor([bytes_by_kernel["total"]], device=device, dtype=torch.float64)
    if distributed:
        dist.all_reduce(job_bytes)  # every rank reads its own experts' bytes
    bytes_by_kernel["total"] = float(job_bytes.item())
    if rank != 0:
        return None
    peak, peak_kind = measured_peaks()
    layer_gbs = bytes_by_kernel["total"] / (step_ms * 1e-3) / 1e9
    kernel_ms = {KERNEL_OF_STAGE[k]: v for k, v in stage_ms.items()}
    stage_frac = {
        kernel: bytes_by_kernel[kernel] / (ms * 1e-3) / 1e9 / peak
        for kernel, ms in kernel_ms.items() if bytes_by_kernel.get(kernel)
    }
    if stage_ms:
        dominant = max(stage_ms, key=stage_ms.get)
        kernel = KERNEL_OF_STAGE[dominant]
        kernel_bytes = bytes_by_kernel.get(kernel, 0.0)
        dominant_ms = stage_ms[dominant]
        roofline_peak = peak
    else:  # expert parallel: the whole layer, all ranks, against N times the peak
        kernel, kernel_bytes, dominant_ms = "whole layer, all ranks", bytes_by_kernel["total"], step_ms
        roofline_peak = peak * world
    achieved = kernel_bytes / (dominant_ms * 1e-3) / 1e9
    h2d = host_in[0].numel() * host_in[0].element_size()
    d2h = host_out[0].numel() * host_out[0].element_size()
    grouped = tokens >= 8 and plan.final_count < plan.candidate_count
    launches = (10 if distributed else len(STAGES)) + int(grouped) * (2 if distributed else 1)
    return {
        "metric": METRIC, "value": tokens * world / (step_ms * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(shape, plan, tokens, layers, world),
        "samples": SAMPLES, "steps_per_sample": steps_per_sample,
        "samples_ms_per_step": [round(s, 5) for s in samples],
        "clocks": clocks,
        "e2e": {"value": tokens * world / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps_per_sample": e2e_steps, "samples_ms_per_step": [round(s, 5) for s in e2e_samples]},
        # Kernels of this library per step (NCCL's kernels are not counted).
        "gpu_launches": launches * args.steps,
        "gpu_launches_per_step": launches,
        "roofline": {
            "bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": roofline_peak,
            "unit": "GB/s", "frac": achieved / roofline_peak,
            # DRAM bytes per launch come from ncu captures; see profiles/ for the kernels
            # and builds they were taken on.
            "traffic": None,
            "algorithmic_bytes_per_launch": kernel_bytes,
            "ms_per_launch": dominant_ms, "peak_source": peak_kind,
        },
        "layer_roofline": {
            "algorithmic_bytes_per_step": bytes_by_kernel["total"], "achieved": layer_gbs,
            "peak": peak * world, "unit": "GB/s", "frac": layer_gbs / (peak * world),
            "frac_of_nominal_8000": layer_gbs / (8000.0 * world),
        },
        "stage_ms": {k: round(v, 5) for k, v in kernel_ms.items()},
        "stage_bytes": {k: v for k, v in bytes_by_kernel.items() if k != "total"},
        "stage_frac": {k: round(v, 4) for k, v in stage_frac.items()},
        "read_cost_bytes_per_token": report["charged_bytes"]
        / max(1.0, report["reference_bytes"] / plan.native_read_bytes()),
        "read_fraction": report["read_fraction"],
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=240)
    parser.add_argument("--warmup", type=int, default=24)
    parser.add_argument("--impl", choices=("ours", "reference", "triton"), default="ours")
    parser.add_argument("--tokens", type=int, default=64)
    parser.add_argument("--sweep-tokens", type=lambda s: [int(v) for v in s.split(",")], default=None,
                        help="comma-separated batch sizes: one line each from one set of layers")
    parser.add_argument("--layers", type=int, default=12)
    parser.add_argument("--config", default="qwen3-30b-a3b", choices=sorted(synthetic.CONFIGS))
    parser.add_argument("--retention", type=float, default=None)
    parser.add_argument("--screen-keep", type=float, default=None)
    parser.add_argument("--budgets", default=None,
                        help="comma-separated retention:screen_keep pairs: one line each")
    parser.add_argument("--quick", action="store_true",
                        help="three samples of 0.1 s instead of seven of 0.3 s (for long sweeps)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-gpu-comparator", action="store_true")
    parser.add_argument("--tensor-engine", default="mma_sync", choices=("mma_sync", "tcgen05"),
                        help="tensor-core path of the expert-major screen")
    parser.add_argument("--timeline", action="store_true",
                        help="expert parallel: also time every stage of eager steps on rank 0")
    parser.add_argument("--exchange", default="auto", choices=("auto", "peer", "collective"),
                        help="expert parallel: kept lists and partial rows over peer memory "
                             "or by NCCL collectives")
    parser.add_argument("--row-engine", default="auto", choices=("auto", "per_token", "expert_major"),
                        help="how batches of eight tokens and more read the native rows")
    args = parser.parse_args()
    if args.quick:
        global SAMPLES, SAMPLE_SECONDS
        SAMPLES, SAMPLE_SECONDS = 3, 0.1
    shape = synthetic.CONFIGS[args.config]

    def plan_for(retention, screen_keep):
        return compile_budget(
            hidden_size=shape.hidden, expert_width=shape.width, top_k=shape.top_k,
            retention=shape.retention if retention is None else retention,
            screen_keep=shape.screen_keep if screen_keep is None else screen_keep,
        )

    if args.budgets:
        plans = []
        for pair in args.budgets.split(","):
            retention, screen_keep = (float(v) for v in pair.split(":"))
            plans.append((f"retention {retention:g}, screen-keep {screen_keep:g}",
                          plan_for(retention, screen_keep)))
    else:
        plans = [("default", plan_for(args.retention, args.screen_keep))]
    if args.impl == "reference":
        if args.steps == 240 and args.warmup == 24:
            args.steps, args.warmup = 5, 3
        run_reference(args, shape, plans[0][1])
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    if args.impl == "triton":
        run_triton(args, shape, plans[0][1])
        return
    run_ours(args, shape, plans)


if __name__ == "__main__":
    main()
