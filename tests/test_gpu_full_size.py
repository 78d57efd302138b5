"""The benchmark configurations at their full sizes on the GPU.

At these sizes the checks are the properties that do not need a stored answer:
kept lists are the F best scores in ascending candidate order; every token's
selection is the same whichever kernel path its batch size picks (one large
batch, smaller batches, single tokens); outputs of the expert-major row engine
and of the per-token row engine agree within the reference's own tolerance
between its two paths (rtol 0.016, atol 2e-3,
tests/test_progressive_reader.py:875-978 of the reference); and a sample of
tokens is compared with the oracle like the small cases are (projections, scores
and kept ids bit-exact, output within 1e-2 relative L2 of the FP32 evaluation).

Configurations: the Qwen3-30B-A3B-shaped layer (128 experts, batch 64), the
Qwen3.5-35B-A3B-shaped layer (256 experts of width 512, Student-t inputs, biased
router, batch 256) and the wide layer (hidden 4096, width 1536, rank 128) under
its nine retention x screen-keep budgets.
"""

import sys
from pathlib import Path

import pytest
import torch

from cfm_b200 import synthetic
from cfm_b200.reader.budget import compile_budget
from cfm_b200.reader.progressive import ProgressiveReader
from cfm_b200.reader.sketch import block_hadamard_signs, build_sketch
from helpers import relative_l2

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The reference's tolerance between its expert-major and per-token paths.
PATH_RTOL, PATH_ATOL = 0.016, 2e-3


def plan_of(shape, retention=None, screen_keep=None):
    return compile_budget(
        hidden_size=shape.hidden, expert_width=shape.width, top_k=shape.top_k,
        retention=shape.retention if retention is None else retention,
        screen_keep=shape.screen_keep if screen_keep is None else screen_keep,
    )


def check_lists(reader, plan, tokens):
    """Kept lists hold the F best scores in ascending candidate order; counts agree."""
    n, f, i = plan.candidate_count, plan.final_count, plan.expert_width
    device = reader.native_gu.device
    lists = reader.candidate_ids[-1][:tokens].clone()
    scores = reader.scores[0][:tokens].clone()
    selected = reader.selected[:tokens].clone()
    assert int(lists.min()) >= 0 and int(lists.max()) < n
    assert bool((lists[:, 1:] > lists[:, :-1]).all())
    mask = torch.zeros(tokens, n, dtype=torch.bool, device=device)
    mask.scatter_(1, lists.long(), True)
    assert torch.equal(mask, selected) and int(selected.sum()) == tokens * f
    if f < n:  # nothing left out beats anything kept
        worst_kept = torch.where(selected, scores, torch.inf).min(1).values
        best_left = torch.where(selected, -torch.inf, scores).max(1).values
        assert bool((best_left <= worst_kept).all())
    counts = selected.reshape(tokens, plan.top_k, i).sum(-1).int()
    assert torch.equal(reader.counts[:tokens], counts)
    return lists, scores


def check_oracle_sample(oracle, reader, plan, weights_of_layer, batch, out, sample):
    """Projections, scores and kept ids of the sampled tokens bit-equal to the oracle's; output
    within the reference's tolerance and within 1e-2 relative L2 of the FP32 evaluation."""
    gate_up, down, encoder, decoder = weights_of_layer
    hidden, ids, weights = batch
    tokens = hidden.shape[0]
    arguments = dict(
        plan=plan, gate_up=gate_up.cpu(), down=down.cpu(), codes=reader.sketch_codes.cpu(),
        statistics=reader.sketch_statistics.cpu(), signs=reader.sketch_signs.cpu(),
        hidden=hidden[sample].cpu(), ids=ids[sample].cpu(), weights=weights[sample].cpu(),
        encoder=encoder.cpu(), decoder=decoder.cpu(), norms=reader.norms.cpu(), score="point",
    )
    want = oracle.forward(**arguments)
    if plan.final_count < plan.candidate_count:
        assert torch.equal(reader.partial[:tokens][sample].cpu(), want["partial"])
        assert torch.equal(reader.scores[0][:tokens][sample].cpu(), want["scores"])
    assert torch.equal(reader.candidate_ids[-1][:tokens][sample].cpu(), want["candidate_ids"])
    torch.testing.assert_close(out[sample].float().cpu(), want["output"], rtol=0.025, atol=0.02)
    exact = oracle.forward(**arguments, fp32=True)
    assert relative_l2(out[sample].cpu(), exact["output"]) < 1e-2


def test_full_size_layer_properties_and_oracle_sample(oracle):
    import bench

    device = torch.device("cuda:0")
    shape = synthetic.CONFIGS["qwen3-30b-a3b"]
    plan = plan_of(shape)
    tokens = 64
    gate_up, down, router, decoder, encoder, generator = bench.device_layer(shape, 3, device)
    hidden, ids, weights = bench.device_batch(shape, router, tokens, generator, device)
    reader = ProgressiveReader(gate_up, down, encoder, decoder, plan, tokens,
                               selection_score="point")
    out = reader(hidden, ids, weights).clone()
    torch.cuda.synchronize()
    lists, scores = check_lists(reader, plan, tokens)

    # The same tokens in batches of 8 (expert-major kernels too) and alone (per-token kernels).
    sketch = (reader.sketch_codes, reader.sketch_statistics)
    eight = ProgressiveReader(gate_up, down, encoder, decoder, plan, 8, selection_score="point",
                              sketch=sketch)
    for first in range(0, tokens, 8):
        rows = slice(first, first + 8)
        part = eight(hidden[rows], ids[rows], weights[rows])
        torch.cuda.synchronize()
        assert torch.equal(eight.scores[0][:8], scores[rows])
        assert torch.equal(eight.candidate_ids[-1][:8], lists[rows])
        torch.testing.assert_close(part.float(), out[rows].float(), rtol=PATH_RTOL, atol=PATH_ATOL)
    single = ProgressiveReader(gate_up, down, encoder, decoder, plan, 1, selection_score="point",
                               sketch=sketch)
    for token in (0, 21, 63):
        rows = slice(token, token + 1)
        part = single(hidden[rows], ids[rows], weights[rows])
        torch.cuda.synchronize()
        assert torch.equal(single.scores[0][0], scores[token])
        assert torch.equal(single.candidate_ids[-1][0], lists[token])
        torch.testing.assert_close(part[0].float(), out[token].float(), rtol=PATH_RTOL,
                                   atol=PATH_ATOL)

    sample = torch.tensor([0, 9, 18, 27, 36, 45, 54, 63])
    check_oracle_sample(oracle, reader, plan, (gate_up, down, encoder, decoder),
                        (hidden, ids, weights), out, sample)

    # Four tokens per expert on average: the default walks the rows per token.  The
    # expert-major kernels on the same batch keep the same channels and agree on the output.
    grouped = ProgressiveReader(gate_up, down, encoder, decoder, plan, tokens,
                                selection_score="point", sketch=sketch, row_engine="expert_major")
    other = grouped(hidden, ids, weights).clone()
    torch.cuda.synchronize()
    assert torch.equal(grouped.candidate_ids[-1][:tokens], lists)
    assert torch.equal(grouped.latent[:tokens], reader.latent[:tokens])
    torch.testing.assert_close(other.float(), out.float(), rtol=PATH_RTOL, atol=PATH_ATOL)
    check_oracle_sample(oracle, grouped, plan, (gate_up, down, encoder, decoder),
                        (hidden, ids, weights), other, sample)


def test_qwen35_shape_batch_256_and_smaller_batches(oracle):
    """256 experts of width 512, Student-t inputs, router bias: one call of 256 tokens, then
    the same tokens in batches of 64 and 16, both tensor-core screens, and an oracle sample."""
    import bench

    device = torch.device("cuda:0")
    shape = synthetic.CONFIGS["qwen3.5-35b-a3b"]
    plan = plan_of(shape)
    tokens = 256
    gate_up, down, router, decoder, encoder, generator = bench.device_layer(shape, 5, device)
    hidden, ids, weights = bench.device_batch(shape, router, tokens, generator, device)
    reader = ProgressiveReader(gate_up, down, encoder, decoder, plan, tokens,
                               selection_score="point")
    out = reader(hidden, ids, weights).clone()
    torch.cuda.synchronize()
    assert int(reader.workspace.status.abs().sum()) == 0
    lists, scores = check_lists(reader, plan, tokens)
    partial = reader.partial[:tokens].clone()
    # The router bias makes the load uneven: some expert serves many more tokens than the mean.
    load = torch.bincount(ids.reshape(-1).long(), minlength=shape.experts)
    assert int(load.max()) >= 3 * tokens * shape.top_k // shape.experts

    sketch = (reader.sketch_codes, reader.sketch_statistics)
    for batch in (64, 16):
        small = ProgressiveReader(gate_up, down, encoder, decoder, plan, batch,
                                  selection_score="point", sketch=sketch)
        for first in range(0, tokens, batch):
            rows = slice(first, first + batch)
            part = small(hidden[rows], ids[rows], weights[rows])
            torch.cuda.synchronize()
            assert torch.equal(small.scores[0][:batch], scores[rows])
            assert torch.equal(small.candidate_ids[-1][:batch], lists[rows])
            torch.testing.assert_close(part.float(), out[rows].float(), rtol=PATH_RTOL,
                                       atol=PATH_ATOL)
        del small
    tensor = ProgressiveReader(gate_up, down, encoder, decoder, plan, tokens,
                               selection_score="point", sketch=sketch, tensor_engine="tcgen05")
    tensor(hidden, ids, weights)
    torch.cuda.synchronize()
    assert int(tensor.workspace.status.abs().sum()) == 0
    assert torch.equal(tensor.partial[:tokens], partial)
    assert torch.equal(tensor.candidate_ids[-1][:tokens], lists)
    del tensor

    sample = torch.tensor([0, 37, 74, 111, 148, 185, 222, 255])
    check_oracle_sample(oracle, reader, plan, (gate_up, down, encoder, decoder),
                        (hidden, ids, weights), out, sample)


WIDE_BUDGETS = [(r, s) for r in (1 / 16, 1 / 8, 1 / 4) for s in (0.5, 0.625, 1.0)]


def test_wide_layer_budget_sweep(oracle):
    """Hidden 4096, width 1536, rank 128: the nine retention x screen-keep budgets at 32 tokens,
    three of them also at 1 and 256 tokens; an oracle sample for each."""
    import bench

    device = torch.device("cuda:0")
    shape = synthetic.CONFIGS["wide"]
    gate_up, down, router, decoder, encoder, generator = bench.device_layer(shape, 7, device)
    hidden, ids, weights = bench.device_batch(shape, router, 256, generator, device)
    signs = block_hadamard_signs(shape.hidden, device)
    sketch = build_sketch(gate_up, signs)
    layer = (gate_up, down, encoder, decoder)
    large = {WIDE_BUDGETS[0], WIDE_BUDGETS[4], WIDE_BUDGETS[8]}
    for retention, screen_keep in WIDE_BUDGETS:
        plan = plan_of(shape, retention, screen_keep)
        assert plan.final_count == round(retention * plan.candidate_count)
        capacity = 256 if (retention, screen_keep) in large else 32
        reader = ProgressiveReader(*layer, plan, capacity, selection_score="point", sketch=sketch)
        batch = (hidden[:32], ids[:32], weights[:32])
        out = reader(*batch).clone()
        torch.cuda.synchronize()
        lists, scores = check_lists(reader, plan, 32)
        sample = torch.tensor([0, 4, 9, 13, 18, 22, 27, 31])
        check_oracle_sample(oracle, reader, plan, layer, batch, out, sample)
        cost = reader.report()
        price = (plan.selected_weight_bytes() + plan.sketch_read_bytes(False, True)
                 + plan.recovery_read_bytes(shape.rank) + plan.selection_read_bytes(False)
                 + shape.hidden)
        assert cost["charged_bytes"] == 32 * price
        if capacity == 256:
            # Batch 256 (expert-major paths) and batch 1 (per-token paths) keep the same channels.
            whole = reader(hidden, ids, weights).clone()
            torch.cuda.synchronize()
            check_lists(reader, plan, 256)
            assert torch.equal(reader.candidate_ids[-1][:32], lists)
            assert torch.equal(reader.scores[0][:32], scores)
            torch.testing.assert_close(whole[:32].float(), out.float(), rtol=PATH_RTOL,
                                       atol=PATH_ATOL)
            late = torch.tensor([40, 100, 160, 255])
            check_oracle_sample(oracle, reader, plan, layer, (hidden, ids, weights), whole, late)
            tensor = ProgressiveReader(*layer, plan, capacity, selection_score="point",
                                       sketch=sketch, tensor_engine="tcgen05")
            tensor(hidden, ids, weights)
            torch.cuda.synchronize()
            assert int(tensor.workspace.status.abs().sum()) == 0
            assert torch.equal(tensor.partial[:256], reader.partial[:256])
            del tensor
            for token in (0, 17):
                rows = slice(token, token + 1)
                part = reader(hidden[rows], ids[rows], weights[rows])
                torch.cuda.synchronize()
                assert torch.equal(reader.candidate_ids[-1][0], lists[token])
                torch.testing.assert_close(part[0].float(), out[token].float(), rtol=PATH_RTOL,
                                           atol=PATH_ATOL)
        del reader
