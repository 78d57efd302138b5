"""Benchmark of the sparse MoE decode reader: decode tokens/s on a Qwen3-30B-A3B-shaped layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--tokens T] [--layers L] [--config NAME]

A step is one call of the reader on one batch of T decode tokens of one MoE
layer.  Steps cycle over L independent layers (own weights, own inputs) so that
consecutive steps touch different memory and the bytes come from HBM, not L2.
Inputs are synthetic (`cfm_b200.synthetic`), drawn on the device.

The JSON line printed by rank 0 reports whole-job tokens/s with inputs resident
(`value`), the same through the public operator with host buffers and copies in
the timed region (`e2e`), the dominant kernel's HBM roofline fraction measured
with CUDA events (`roofline`), the whole layer's (`layer_roofline`), and the CPU
oracle timed on the host cores (`cpu_baseline`).
"""

from __future__ import annotations

import argparse
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


# DRAM bytes (read + write) per launch from one `ncu --set full` capture of the default
# workload, two layers cycled; a bench run cannot measure them itself.  Reported for that
# workload only.
NCU_DRAM_BYTES = {
    ("qwen3-30b-a3b", 64): {
        "k_screen": 108.2e6, "k_exact": 344.4e6, "k_down": 160.6e6, "k_encode": 15.8e6,
        "k_select": 3.6e6, "k_output": 8.6e6, "k_prepare": 0.3e6,
    },
}


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
    coordinates = coordinates[:tokens].long()  # [T, B, KEEP]
    support = torch.zeros(tokens, blocks, 128, dtype=torch.bool, device=ids.device)
    support.scatter_(-1, coordinates, True)
    support = support.reshape(tokens, h)
    coordinate_union = torch.zeros(e, h, dtype=torch.bool, device=ids.device)
    coordinate_union.index_put_(
        (flat,), support[:, None, :].expand(tokens, k, h).reshape(-1, h) & valid.reshape(-1, 1),
        accumulate=True,
    )
    experts = int(routed.sum())
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


# ---------------------------------------------------------------------------
# arms
# ---------------------------------------------------------------------------
def cpu_oracle_rate(shape, plan, tokens: int, seconds: float = 10.0) -> dict:
    """Time the CPU oracle (a port of the reference's PyTorch reader) on the host cores."""
    from cfm_b200.reader.progressive import channel_major_down
    from cfm_b200.reader.sketch import block_hadamard_signs, build_sketch
    from oracle import reader_oracle

    layer, g = synthetic.make_layer(shape, 0)
    hidden, ids, weights = synthetic.make_batch(layer, tokens, g)
    signs = block_hadamard_signs(shape.hidden, "cpu")
    codes, statistics = build_sketch(layer.gate_up, signs)
    down = channel_major_down(layer.down)
    norms = down.float().square().sum(1).sqrt()
    arguments = dict(
        plan=plan, gate_up=layer.gate_up, down=down, codes=codes, statistics=statistics,
        signs=signs, hidden=hidden, ids=ids, weights=weights, encoder=layer.encoder,
        decoder=layer.decoder, norms=norms,
    )
    threads = reader_oracle.forward(**{**arguments, "hidden": hidden[:1], "ids": ids[:1],
                                       "weights": weights[:1]})["threads"]
    done, elapsed, cores = 0, 0.0, 1
    while elapsed < seconds and done < 8 * tokens:
        start = time.perf_counter()
        cores = reader_oracle.forward(**arguments)["threads"]
        elapsed += time.perf_counter() - start
        done += tokens
    del threads
    return {
        "value": done / elapsed, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{done} tokens of the {shape.name} layer in batches of {tokens} "
                  f"({elapsed:.1f} s; sketch construction excluded)",
    }


def run_reference(args, shape, plan) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens = min(args.tokens, 64)
    from cfm_b200.reader.progressive import channel_major_down
    from cfm_b200.reader.sketch import block_hadamard_signs, build_sketch
    from oracle import reader_oracle

    layer, g = synthetic.make_layer(shape, 0)
    hidden, ids, weights = synthetic.make_batch(layer, tokens, g)
    signs = block_hadamard_signs(shape.hidden, "cpu")
    codes, statistics = build_sketch(layer.gate_up, signs)
    down = channel_major_down(layer.down)
    arguments = dict(
        plan=plan, gate_up=layer.gate_up, down=down, codes=codes, statistics=statistics,
        signs=signs, hidden=hidden, ids=ids, weights=weights, encoder=layer.encoder,
        decoder=layer.decoder, norms=down.float().square().sum(1).sqrt(),
    )
    cores = 1
    for _ in range(args.warmup):
        cores = reader_oracle.forward(**arguments)["threads"]
    start = time.perf_counter()
    for _ in range(args.steps):
        reader_oracle.forward(**arguments)
    elapsed = time.perf_counter() - start
    value = tokens * args.steps / elapsed
    sample = f"{tokens} tokens per step of the {shape.name} layer, CPU port of the reference reader"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(shape, plan, tokens, 1, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(shape, plan, tokens, layers, gpus) -> dict:
    return {
        "workload": f"{shape.name}-shaped MoE layer, decode batch {tokens}",
        "hidden": shape.hidden, "experts": shape.experts, "expert_width": shape.width,
        "top_k": shape.top_k, "recovery_rank": shape.rank, "kept_channels": plan.final_count,
        "screen_coordinates": plan.screen_coordinates, "selection_score": "point",
        "tokens_per_step": tokens, "layers_cycled": layers,
        "l2": f"steps cycle over {layers} layers with distinct weights, inputs and workspaces",
        "parallelism": "single GPU" if gpus == 1 else (
            f"expert parallel over {gpus} GPUs: {shape.experts // gpus} experts per rank, "
            f"{tokens} tokens per rank per step; sketch replicated, home-rank screen and "
            "selection, all_gather of rows and kept-channel lists, FP32 reduce_scatter "
            "combine (NCCL)"),
    }


def trace(message: str) -> None:
    """Progress marker on stderr when CFM_BENCH_TRACE is set (for diagnosing multi-rank runs)."""
    if os.environ.get("CFM_BENCH_TRACE"):
        print(f"[rank {os.environ.get('RANK', '0')}] {message}", file=sys.stderr, flush=True)


def run_ours(args, shape, plan) -> None:
    import ctypes

    from cfm_b200 import _native
    from cfm_b200.reader.progressive import ProgressiveReader

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    tokens, layers = args.tokens, args.layers
    readers, batches, sharded = [], [], []
    for index in range(layers):
        gate_up, down, router, decoder, encoder, g = device_layer(shape, index, device, world, rank)
        if distributed:
            from cfm_b200.reader.expert_parallel import ExpertParallelReader

            sharded.append(ExpertParallelReader(
                gate_up, down, encoder, decoder, plan, tokens, global_experts=shape.experts,
                selection_score="point", retain_reference_sketch=False,
            ))
            readers.append(sharded[-1].reader)
        else:
            readers.append(ProgressiveReader(
                gate_up, down, encoder, decoder, plan, tokens,
                selection_score="point", retain_reference_sketch=False,
                tensor_engine=args.tensor_engine,
            ))
        batches.append(packed_batch(device_batch(shape, router, tokens, g, device)))
        del router
    outs = [torch.empty_like(b[0]) for b in batches]
    stream = torch.cuda.Stream(device)
    trace("layers built")

    def step(index: int) -> None:
        hidden, ids, weights = batches[index]
        if distributed:
            outs[index].copy_(sharded[index](hidden, ids, weights))
        else:
            readers[index](hidden, ids, weights, None, outs[index])

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

        def barrier() -> None:
            if distributed:
                dist.barrier()
            torch.cuda.synchronize()

        trace("graphs captured")
        # ---- resident-input throughput ---------------------------------
        for i in range(args.warmup):
            graphs[i % layers].replay()
        barrier()
        sampler = ClockSampler(local) if rank == 0 else None
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for i in range(args.steps):
            graphs[i % layers].replay()
        end.record(stream)
        barrier()
        elapsed_ms = begin.elapsed_time(end)
        clocks = sampler.stop() if sampler else None
        trace("timed region done")

        # ---- end to end: host buffers, copies inside the timed region ---
        # A step's inputs (hidden rows, router ids and weights) sit in one block on both
        # sides, so they cross in one copy.
        host_in = [(b[0]._packed.cpu().pin_memory(),) for b in batches]
        host_out = [torch.empty_like(o, device="cpu").pin_memory() for o in outs]

        def e2e_step(index: int) -> None:
            batches[index][0]._packed.copy_(host_in[index][0], non_blocking=True)
            graphs[index].replay()
            host_out[index].copy_(outs[index], non_blocking=True)
            stream.synchronize()

        for i in range(args.warmup):
            e2e_step(i % layers)
        barrier()
        start = time.perf_counter()
        begin.record(stream)
        for i in range(args.steps):
            e2e_step(i % layers)
        end.record(stream)
        barrier()
        e2e_ms = max(begin.elapsed_time(end), 1e3 * (time.perf_counter() - start))
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

        repeats = max(3, min(20, args.steps // layers))
        for name in (() if distributed else STAGES):
            launch_stage(name)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                launch_stage(name)
            graph.replay()
            begin.record(stream)
            for _ in range(repeats):
                graph.replay()
            end.record(stream)
            stream.synchronize()
            stage_ms[name] = begin.elapsed_time(end) / (repeats * layers)
        if distributed:
            bytes_by_kernel = expert_parallel_bytes(sharded[0], tokens, world)
            report = sharded[0].report()
        else:
            bytes_by_kernel = algorithmic_bytes(readers[0], tokens)
            report = readers[0].report()

    times = torch.tensor([elapsed_ms, e2e_ms], device=device, dtype=torch.float64)
    job_bytes = torch.tensor([bytes_by_kernel["total"]], device=device, dtype=torch.float64)
    if distributed:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(job_bytes)  # every rank reads its own experts' bytes
    elapsed_ms, e2e_ms = times.tolist()
    bytes_by_kernel["total"] = float(job_bytes.item())
    if rank == 0:
        peak, peak_kind = measured_peaks()
        total_tokens = tokens * args.steps * world
        step_ms = elapsed_ms / args.steps
        layer_gbs = bytes_by_kernel["total"] / (step_ms * 1e-3) / 1e9
        if stage_ms:
            dominant = max(stage_ms, key=stage_ms.get)
            kernel = KERNEL_OF_STAGE[dominant]
            kernel_bytes = bytes_by_kernel.get(kernel, 0.0)
            kernel_ms = stage_ms[dominant]
        else:  # expert parallel: the whole layer, all ranks, against N times the peak
            kernel, kernel_bytes, kernel_ms = "whole layer, all ranks", bytes_by_kernel["total"], step_ms
        achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
        peak = peak * (1 if stage_ms else world)
        h2d = sum(t.numel() * t.element_size() for t in host_in[0])
        d2h = host_out[0].numel() * host_out[0].element_size()
        line = {
            "metric": METRIC, "value": total_tokens / (elapsed_ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(shape, plan, tokens, layers, world),
            "clocks": clocks,
            "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            # Single GPU: the stages plus the expert grouping.  Expert parallel: six home-side
            # kernels, four owner-side ones and the finish (NCCL's kernels are not counted).
            "gpu_launches": (11 if distributed else len(STAGES) + 1) * args.steps,
            "roofline": {
                "bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_DRAM_BYTES.get((shape.name, tokens), {}).get(kernel)
                if world == 1 else None,
                "algorithmic_bytes_per_launch": kernel_bytes,
                "ms_per_launch": kernel_ms, "peak_source": peak_kind,
            },
            "layer_roofline": {
                "algorithmic_bytes_per_step": bytes_by_kernel["total"], "achieved": layer_gbs,
                "peak": peak if not stage_ms else peak * world, "unit": "GB/s",
                "frac": layer_gbs / (peak if not stage_ms else peak * world),
                "frac_of_nominal_8000": layer_gbs / (8000.0 * world),
            },
            "stage_ms": {KERNEL_OF_STAGE[k]: round(v, 5) for k, v in stage_ms.items()},
            "read_cost_bytes_per_token": report["charged_bytes"]
            / max(1.0, report["reference_bytes"] / plan.native_read_bytes()),
            "read_fraction": report["read_fraction"],
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_oracle_rate(shape, plan, min(tokens, 64))
        print(json.dumps(line))
    if distributed:
        # Tearing down a NCCL communicator while CUDA graphs that captured its
        # collectives are alive blocks on this stack; release the graphs, meet at
        # a barrier, and leave without the communicator teardown.
        del graphs
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=240)
    parser.add_argument("--warmup", type=int, default=24)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--tokens", type=int, default=64)
    parser.add_argument("--layers", type=int, default=12)
    parser.add_argument("--config", default="qwen3-30b-a3b", choices=sorted(synthetic.CONFIGS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--tensor-engine", default="mma_sync", choices=("mma_sync", "tcgen05"),
                        help="tensor-core path of the expert-major screen")
    args = parser.parse_args()
    shape = synthetic.CONFIGS[args.config]
    plan = compile_budget(
        hidden_size=shape.hidden, expert_width=shape.width, top_k=shape.top_k,
        retention=shape.retention, screen_keep=shape.screen_keep,
    )
    if args.impl == "reference":
        if args.steps == 240 and args.warmup == 24:
            args.steps, args.warmup = 5, 3
        run_reference(args, shape, plan)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    run_ours(args, shape, plan)


if __name__ == "__main__":
    main()
