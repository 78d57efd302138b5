"""Expert-parallel orchestration on CPU: two and four gloo ranks, the oracle as the compute engine.

Checks the host logic of `cfm_b200.reader.expert_parallel` (expert placement,
dispatch, score or selection exchange, combine) for both strategies without a
GPU: every rank holds an equal share of the experts and of the tokens; results must
equal the single-process oracle on the whole layer (selections exactly, outputs
to FP32 re-association).
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import prepared, run_oracle


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return int(sock.getsockname()[1])


class OracleEngine:
    """CPU stand-in for `ShardedScreenEngine`, built on the oracle (test infrastructure)."""

    def __init__(self, oracle, item, rank, world):
        from cfm_b200.reader.expert_parallel import linear_expert_map

        case = item["case"]
        experts = case.gate_up.shape[0]
        local = experts // world
        span = slice(rank * local, (rank + 1) * local)
        self.oracle, self.case = oracle, case
        self.fixed = dict(
            plan=case.plan, gate_up=case.gate_up[span], down=item["down"][span],
            codes=item["codes"][span], statistics=item["statistics"][span], signs=item["signs"],
            encoder=case.encoder[span] if case.encoder is not None else None,
            decoder=case.decoder, activation=case.activation,
            expert_map=linear_expert_map(experts, world, rank), threads=2,
        )
        self.selected = None

    def screen(self, hidden, ids, weights, padding):
        self.inputs = dict(hidden=hidden, ids=ids, weights=weights, padding=padding)
        out = self.oracle.forward(**self.fixed, **self.inputs)
        self.scores = out["scores"].clone()
        self.local_ids = out["sorted_ids"]
        k = self.case.plan.top_k
        self.cuts = torch.zeros(hidden.shape[0], k + 1, dtype=torch.int32)
        return self.scores

    def find_cuts(self, first_row, rows):
        """The cut of each home token from its summed scores: F-th largest key and tie budgets."""
        plan = self.case.plan
        f, k, i = plan.final_count, plan.top_k, plan.expert_width
        for row in range(first_row, first_row + rows):
            keys = self.scores[row].view(torch.int32).long()
            if f == plan.candidate_count:
                continue
            order = torch.argsort(keys, descending=True, stable=True)[:f]
            cut = int(keys[order[-1]])
            kept_ties = (keys[order] == cut).nonzero().flatten()
            tie_slots = order[kept_ties] // i
            self.cuts[row, 0] = cut
            for slot in range(k):
                self.cuts[row, 1 + slot] = int((tie_slots == slot).sum())
        return self.cuts

    def local(self):
        plan = self.case.plan
        k, i, n = plan.top_k, plan.expert_width, plan.candidate_count
        rows = self.scores.shape[0]
        mask = torch.zeros(rows, n, dtype=torch.bool)
        keys = self.scores.view(torch.int32).long().reshape(rows, k, i)
        for row in range(rows):
            for slot in range(k):
                if self.local_ids[row, slot] < 0:
                    continue
                if plan.final_count == n:
                    mask[row, slot * i : (slot + 1) * i] = True
                    continue
                cut, budget = int(self.cuts[row, 0]), int(self.cuts[row, 1 + slot])
                above = keys[row, slot] > cut
                tied = keys[row, slot] == cut
                tied &= tied.cumsum(0) <= budget
                mask[row, slot * i : (slot + 1) * i] = above | tied
        out = self.oracle.forward(**self.fixed, **self.inputs, given_selected=mask)
        self.selected = mask
        rank = self.case.decoder.shape[1] if self.case.decoder is not None else 0
        if rank:
            return torch.cat((out["routed"], out["latent"]), dim=1)
        return out["routed"]

    def finish(self, combined):
        h = self.case.plan.hidden_size
        routed, latent = combined[:, :h], combined[:, h:]
        correction = 0.0
        if latent.shape[1]:
            z = latent.bfloat16().float()
            correction = (self.case.decoder.float() @ z.T).T.bfloat16().float()
        return (routed + correction).bfloat16()


class OracleHomeEngine:
    """CPU stand-in for `ReplicatedScreenEngine`, built on the oracle (test infrastructure)."""

    def __init__(self, oracle, item, rank, world):
        from cfm_b200.reader.expert_parallel import linear_expert_map

        case = item["case"]
        experts = case.gate_up.shape[0]
        local = experts // world
        span = slice(rank * local, (rank + 1) * local)
        self.oracle, self.case = oracle, case
        common = dict(plan=case.plan, signs=item["signs"], activation=case.activation, threads=2)
        # Home side: the sketch and recovery map of every expert (the oracle also takes
        # the native weights, whose results this side does not use).
        self.whole = dict(
            common, gate_up=case.gate_up, down=item["down"], codes=item["codes"],
            statistics=item["statistics"], encoder=case.encoder, decoder=case.decoder,
        )
        # Owner side: native rows of the local experts, no recovery map.
        self.owned = dict(
            common, gate_up=case.gate_up[span], down=item["down"][span], codes=item["codes"][span],
            statistics=item["statistics"][span], encoder=None, decoder=None,
            expert_map=linear_expert_map(experts, world, rank),
        )
        self.selected = None

    def choose(self, hidden, ids, weights, padding):
        out = self.oracle.forward(**self.whole, hidden=hidden, ids=ids, weights=weights,
                                  padding=padding)
        self.latent = out["latent"]
        return out["candidate_ids"]

    def serve(self, hidden, ids, weights, padding, lists):
        mask = torch.zeros(hidden.shape[0], self.case.plan.candidate_count, dtype=torch.bool)
        for row, kept in enumerate(lists):
            mask[row, kept[kept >= 0].long()] = True
        out = self.oracle.forward(**self.owned, hidden=hidden, ids=ids, weights=weights,
                                  padding=padding, given_selected=mask)
        self.local_ids = out["sorted_ids"]
        mine = (self.local_ids >= 0).repeat_interleave(self.case.plan.expert_width, dim=1)
        self.selected = mask & mine
        return out["routed"]

    def finish(self, routed):
        correction = 0.0
        if self.case.decoder is not None:
            z = self.latent.bfloat16().float()
            correction = (self.case.decoder.float() @ z.T).T.bfloat16().float()
        return (routed + correction).bfloat16()


def _worker(rank, world, port, name, strategy, results):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    for entry in (str(root), str(root / "tests"), str(root / "tests" / "golden")):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    import cfm_b200  # noqa: F401
    from cfm_b200.reader.expert_parallel import expert_parallel_forward, replicated_screen_forward
    from oracle import reader_oracle

    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        item = prepared(name)
        case = item["case"]
        tokens = case.hidden.shape[0] // world
        rows = slice(rank * tokens, (rank + 1) * tokens)
        padding = case.padding[rows] if case.padding is not None else None
        if strategy == "sharded":
            engine, forward = OracleEngine(reader_oracle, item, rank, world), expert_parallel_forward
        else:
            engine = OracleHomeEngine(reader_oracle, item, rank, world)
            forward = replicated_screen_forward
        out = forward(engine, case.hidden[rows], case.ids[rows], case.weights[rows], padding)
        results[rank] = (out.float(), engine.selected, engine.local_ids)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize(
    "name, strategy, world",
    [(name, strategy, 2) for name in ("tiny", "qwen35-e16-t4", "graph-routes")
     for strategy in ("replicated", "sharded")]
    + [("qwen35-e16-t4", "replicated", 4), ("qwen35-e16-t4", "sharded", 4)],
)
def test_expert_parallel_ranks_match_single_process(oracle, name, strategy, world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), name, strategy, results), nprocs=world,
             join=True)
    item = prepared(name)
    case = item["case"]
    want = run_oracle(oracle, item)
    tokens = case.hidden.shape[0] // world
    active = torch.ones(case.hidden.shape[0], dtype=torch.bool)
    if case.padding is not None:
        active = ~case.padding
    for rank in range(world):
        out, selected, local_ids = results[rank]
        rows = slice(rank * tokens, (rank + 1) * tokens)
        # Each rank kept, in its own slots, exactly the channels the single-process run kept.
        i = case.plan.expert_width
        mine = (local_ids >= 0).repeat_interleave(i, dim=1)
        assert torch.equal(selected[active], (want["selected"] & mine)[active])
        torch.testing.assert_close(out[active[rows]], want["output"][rows][active[rows]],
                                   rtol=0.016, atol=2e-3)
        assert not out[~active[rows]].any()


def test_linear_expert_map():
    from cfm_b200.reader.expert_parallel import linear_expert_map

    assert linear_expert_map(8, 4, 1).tolist() == [-1, -1, 0, 1, -1, -1, -1, -1]
    with pytest.raises(ValueError):
        linear_expert_map(10, 4, 0)
