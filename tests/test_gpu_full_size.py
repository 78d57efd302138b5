"""The benchmark's full-size layer (128 experts, decode batch 64) on the GPU.

At this size the checks are the properties that do not need a stored answer:
kept lists are the F best scores in ascending candidate order; every token's
result is the same whichever kernel path its batch size selects (one batch of
64, eight batches of 8, single tokens); and a sample of tokens is compared with
the oracle like the small cases are (bit-exact selection, output within 1e-2
relative L2 of the FP32 evaluation).
"""

import sys
from pathlib import Path

import pytest
import torch

from cfm_b200 import synthetic
from cfm_b200.reader.budget import compile_budget
from cfm_b200.reader.progressive import ProgressiveReader
from helpers import relative_l2

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def test_full_size_layer_properties_and_oracle_sample(oracle):
    import bench

    device = torch.device("cuda:0")
    shape = synthetic.CONFIGS["qwen3-30b-a3b"]
    plan = compile_budget(hidden_size=shape.hidden, expert_width=shape.width, top_k=shape.top_k,
                          retention=shape.retention, screen_keep=shape.screen_keep)
    tokens, n, f, i = 64, plan.candidate_count, plan.final_count, plan.expert_width
    gate_up, down, router, decoder, encoder, generator = bench.device_layer(shape, 3, device)
    hidden, ids, weights = bench.device_batch(shape, router, tokens, generator, device)
    reader = ProgressiveReader(gate_up, down, encoder, decoder, plan, tokens,
                               selection_score="point")
    out = reader(hidden, ids, weights).clone()
    torch.cuda.synchronize()
    lists = reader.candidate_ids[-1][:tokens].clone()
    scores = reader.scores[0][:tokens].clone()
    selected = reader.selected[:tokens].clone()

    # Lists: F entries, ascending, in range, and the mask says the same.
    assert int(lists.min()) >= 0 and int(lists.max()) < n
    assert bool((lists[:, 1:] > lists[:, :-1]).all())
    mask = torch.zeros(tokens, n, dtype=torch.bool, device=device)
    mask.scatter_(1, lists.long(), True)
    assert torch.equal(mask, selected) and int(selected.sum()) == tokens * f
    # They are the F best scores: nothing left out beats anything kept.
    worst_kept = torch.where(selected, scores, torch.inf).min(1).values
    best_left = torch.where(selected, -torch.inf, scores).max(1).values
    assert bool((best_left <= worst_kept).all())
    counts = selected.reshape(tokens, plan.top_k, i).sum(-1).int()
    assert torch.equal(reader.counts[:tokens], counts)

    # The same tokens in batches of 8 (expert-major screen) and alone (per-pair screen).
    eight = ProgressiveReader(gate_up, down, encoder, decoder, plan, 8, selection_score="point",
                              sketch=(reader.sketch_codes, reader.sketch_statistics))
    for first in range(0, tokens, 8):
        rows = slice(first, first + 8)
        part = eight(hidden[rows], ids[rows], weights[rows])
        torch.cuda.synchronize()
        assert torch.equal(eight.scores[0][:8], scores[rows])
        assert torch.equal(eight.candidate_ids[-1][:8], lists[rows])
        assert torch.equal(part, out[rows])
    single = ProgressiveReader(gate_up, down, encoder, decoder, plan, 1, selection_score="point",
                               sketch=(reader.sketch_codes, reader.sketch_statistics))
    for token in (0, 21, 63):
        rows = slice(token, token + 1)
        part = single(hidden[rows], ids[rows], weights[rows])
        torch.cuda.synchronize()
        assert torch.equal(single.scores[0][0], scores[token])
        assert torch.equal(single.candidate_ids[-1][0], lists[token])
        assert torch.equal(part[0], out[token])

    # A sample of tokens against the oracle.
    sample = torch.tensor([0, 9, 18, 27, 36, 45, 54, 63])
    arguments = dict(
        plan=plan, gate_up=gate_up.cpu(), down=down.cpu(), codes=reader.sketch_codes.cpu(),
        statistics=reader.sketch_statistics.cpu(), signs=reader.sketch_signs.cpu(),
        hidden=hidden[sample].cpu(), ids=ids[sample].cpu(), weights=weights[sample].cpu(),
        encoder=encoder.cpu(), decoder=decoder.cpu(), norms=reader.norms.cpu(), score="point",
    )
    want = oracle.forward(**arguments)
    assert torch.equal(reader.partial[:tokens][sample].cpu(), want["partial"])
    assert torch.equal(scores[sample].cpu(), want["scores"])
    assert torch.equal(lists[sample].cpu(), want["candidate_ids"])
    torch.testing.assert_close(out[sample].float().cpu(), want["output"], rtol=0.025, atol=0.02)
    exact = oracle.forward(**arguments, fp32=True)
    assert relative_l2(out[sample].cpu(), exact["output"]) < 1e-2
