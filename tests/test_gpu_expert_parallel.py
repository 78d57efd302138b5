"""Expert parallelism on two GPUs over NCCL: the sharded reader against the single-GPU reader.

Needs two devices; skipped otherwise.  Ranks are child processes, one per GPU.
"""

import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return int(sock.getsockname()[1])


def _worker(rank, world, port, name, strategy, exchange, results):
    import faulthandler
    import os
    import sys
    from pathlib import Path

    # A rank stuck in a collective would otherwise block the whole test run: after three
    # minutes dump where every thread is and leave.
    faulthandler.dump_traceback_later(180, exit=True)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    root = Path(__file__).resolve().parents[1]
    for entry in (str(root), str(root / "tests"), str(root / "tests" / "golden")):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    import cfm_b200  # noqa: F401
    from cfm_b200.reader.expert_parallel import ExpertParallelReader, linear_expert_map
    from cfm_b200.reader.progressive import ProgressiveReader
    from helpers import prepared

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                            world_size=world, device_id=device)
    try:
        item = prepared(name)
        case = item["case"]
        experts = case.gate_up.shape[0]
        local = experts // world
        span = slice(rank * local, (rank + 1) * local)
        tokens = case.hidden.shape[0] // world
        rows = slice(rank * tokens, (rank + 1) * tokens)

        def channel_major(down):
            return down.transpose(1, 2).contiguous().to(device).transpose(1, 2)

        def statistics(part):
            return part.permute(0, 2, 3, 1).contiguous().to(device).permute(0, 3, 1, 2)

        sharded = ExpertParallelReader(
            case.gate_up[span].to(device), channel_major(item["down"][span]),
            case.encoder[span].to(device) if case.encoder is not None else None,
            case.decoder.to(device) if case.decoder is not None else None,
            case.plan, tokens, global_experts=experts, screen=strategy, exchange=exchange,
            sketch=(item["codes"][span].to(device), statistics(item["statistics"][span])),
            activation=case.activation, selection_score="point",
        )
        assert (sharded.exchange is not None) == (exchange == "peer")
        padding = case.padding[rows].to(device) if case.padding is not None else None
        for _ in range(2 if exchange == "peer" else 1):  # two epochs of the exchange
            out = sharded(case.hidden[rows].to(device), case.ids[rows].to(device),
                          case.weights[rows].to(device), padding)
            torch.cuda.synchronize()
        if sharded.exchange is not None:
            assert sharded.exchange.status() == 0  # no wait ran out
        total = world * tokens
        kept_local = (sharded.reader.ids[:total].cpu() >= 0)
        if strategy == "sharded":
            kept = sharded.reader.selected[:total].cpu()
            scores = sharded.reader.scores[0][rows].cpu()  # summed on the home rank only
        else:
            # The owner's cut-down lists as a mask; the home rank's scores of its own tokens.
            kept = torch.zeros(total, case.plan.candidate_count, dtype=torch.bool)
            for row, ids in enumerate(sharded.reader.candidate_ids[-1][:total].cpu()):
                kept[row, ids[ids >= 0].long()] = True
            scores = sharded.home.workspace.scores[:tokens].cpu()
            home_kept = sharded.home.workspace.candidate_ids[:tokens].cpu()
            report = sharded.report()
            if report["reference_bytes"]:  # a rank whose tokens are all padding reads nothing
                assert 0 < report["read_fraction"] < 1

        # Reference-compatible mode: replicated tokens, all-reduce inside the reader.
        replicated = ProgressiveReader(
            case.gate_up[span].to(device), channel_major(item["down"][span]),
            case.encoder[span].to(device) if case.encoder is not None else None,
            case.decoder.to(device) if case.decoder is not None else None,
            case.plan, case.hidden.shape[0],
            expert_map=linear_expert_map(experts, world, rank),
            sketch=(item["codes"][span].to(device), statistics(item["statistics"][span])),
            activation=case.activation, selection_score="point",
        )
        all_padding = case.padding.to(device) if case.padding is not None else None
        partial = replicated(case.hidden.to(device), case.ids.to(device),
                             case.weights.to(device), all_padding).float()
        dist.all_reduce(partial)
        torch.cuda.synchronize()
        compat_kept = replicated.candidate_ids[-1][: case.hidden.shape[0]].cpu()

        expected = None
        if rank == 0:
            full = ProgressiveReader(
                case.gate_up.to(device), channel_major(item["down"]),
                case.encoder.to(device) if case.encoder is not None else None,
                case.decoder.to(device) if case.decoder is not None else None,
                case.plan, case.hidden.shape[0],
                sketch=(item["codes"].to(device), statistics(item["statistics"])),
                activation=case.activation, selection_score="point",
            )
            reference = full(case.hidden.to(device), case.ids.to(device),
                             case.weights.to(device), all_padding)
            torch.cuda.synchronize()
            expected = (reference.float().cpu(), full.candidate_ids[-1][:total].cpu(),
                        full.scores[0][:total].cpu(), full.selected[:total].cpu())
        if strategy == "replicated" and rank == 0:
            assert torch.equal(home_kept, expected[1][rows])
        results[rank] = (out.float().cpu(), kept, kept_local, scores, partial.cpu(),
                         compat_kept, expected)
    finally:
        dist.destroy_process_group()
        faulthandler.cancel_dump_traceback_later()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("strategy,exchange", [("replicated", "collective"),
                                               ("replicated", "peer"), ("sharded", "collective")])
@pytest.mark.parametrize("name", ["qwen35-e16-t4", "qwen3-e16-t8", "graph-routes"])
def test_sharded_reader_matches_single_gpu(name, strategy, exchange):
    from helpers import prepared

    world = 2
    manager = mp.Manager()
    results = manager.dict()
    for attempt in range(3):  # the probed port can be taken again before rank 0 listens on it
        try:
            mp.spawn(_worker, args=(world, _free_port(), name, strategy, exchange, results),
                     nprocs=world, join=True)
            break
        except Exception as error:
            if "EADDRINUSE" not in str(error) or attempt == 2:
                raise
    case = prepared(name)["case"]
    reference, kept, scores, selected = results[0][6]
    tokens = case.hidden.shape[0] // world
    width = case.plan.expert_width
    active = torch.ones(case.hidden.shape[0], dtype=torch.bool)
    if case.padding is not None:
        active = ~case.padding
    envelope = 2 * torch.finfo(torch.bfloat16).eps * reference.abs().max().item()
    for rank in range(world):
        out, rank_kept, rank_local, home_scores, compat, compat_kept, _ = results[rank]
        rows = slice(rank * tokens, (rank + 1) * tokens)
        # Scores of the home tokens (summed over the ranks, or computed alone on the
        # home rank) equal the single-GPU reader's, bit for bit ...
        assert torch.equal(home_scores[active[rows]], scores[rows][active[rows]])
        # ... and every rank keeps, in its own slots, exactly the single-GPU reader's channels.
        mine = rank_local.repeat_interleave(width, dim=1)
        assert torch.equal(rank_kept[active], (selected & mine)[active])
        assert torch.equal(compat_kept[active], kept[active])
        torch.testing.assert_close(out[active[rows]], reference[rows][active[rows]],
                                   rtol=0, atol=envelope)
        torch.testing.assert_close(compat[active], reference[active], rtol=0, atol=2 * envelope)
        assert not out[~active[rows]].any()
