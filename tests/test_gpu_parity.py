"""GPU parity: the CUDA reader, called through its C ABI, against the CPU oracle and
the reference's golden vectors on the same seeded inputs.

The oracle is given the reader's own down-column norms (a construction-time
quantity whose FP32 reduction order differs between devices), as the reference's
tests do (tests/test_progressive_reader.py:171).

Bars: kept channel indices, kept rotated coordinates, sketch projections and
scores bit-exact against the oracle (integer dot products and pinned FP32
arithmetic); selections bit-exact against the reference goldens wherever the
reference's own two rotations agree; outputs within the reference's tolerance
(rtol 0.025, atol 0.02) and within 1e-2 relative L2 of the FP32 evaluation.
"""

import pytest
import torch

import cases
from cfm_b200.reader.progressive import ProgressiveReader
from helpers import bf16_from_bits, golden, prepared, relative_l2, run_oracle

pytestmark = pytest.mark.gpu


def make_reader(item, capacity=None, **kwargs):
    case = item["case"]
    device = torch.device("cuda:0")
    sketch = (item["codes"].to(device), _move_statistics(item["statistics"], device))
    return ProgressiveReader(
        case.gate_up.to(device),
        _channel_major(item["down"], device),
        case.encoder.to(device) if case.encoder is not None else None,
        case.decoder.to(device) if case.decoder is not None else None,
        case.plan,
        capacity or case.hidden.shape[0],
        sketch=sketch,
        activation=case.activation,
        selection_score=case.score,
        selection_threshold=case.threshold,
        **kwargs,
    )


def _channel_major(down, device):
    return down.transpose(1, 2).contiguous().to(device).transpose(1, 2)


def _move_statistics(statistics, device):
    return statistics.permute(0, 2, 3, 1).contiguous().to(device).permute(0, 3, 1, 2)


def run_reader(reader, case, **kwargs):
    device = reader.native_gu.device
    padding = case.padding.to(device) if case.padding is not None else None
    out = reader(
        case.hidden.to(device), case.ids.to(device), case.weights.to(device), padding, **kwargs
    )
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("name", cases.NAMES)
def test_reader_matches_oracle_and_golden(oracle, name):
    item = prepared(name)
    case, expected = item["case"], golden(name)
    plan = case.plan
    tokens, n, f = case.hidden.shape[0], plan.candidate_count, plan.final_count
    reader = make_reader(item)
    out = run_reader(reader, case).cpu()
    own = dict(norms=reader.norms.cpu())
    if reader.recovery_geometry is not None:
        own["geometry"] = reader.recovery_geometry.cpu()
    want = run_oracle(oracle, item, **own)
    active = torch.ones(tokens, dtype=torch.bool)
    if case.padding is not None:
        active = ~case.padding
    # Route.
    assert torch.equal(reader.ids[:tokens].cpu()[active], want["sorted_ids"][active])
    assert torch.equal(reader.weights[:tokens].cpu()[active], want["sorted_weights"][active])
    if plan.completion_count < n:
        # Kept coordinates and rotated values, bit-exact.
        assert torch.equal(
            reader.sketch_coordinates[:tokens].cpu()[active], want["coordinates"][active]
        )
        assert torch.equal(reader.sketch_planes[:tokens].cpu()[active], want["planes"][active])
        # Projections and scores, bit-exact.
        assert torch.equal(reader.partial[:tokens].cpu()[active], want["partial"][active])
        assert torch.equal(reader.scores[0][:tokens].cpu()[active], want["scores"][active])
    # Selection, bit-exact against the oracle ...
    assert torch.equal(reader.selected[:tokens].cpu()[active], want["selected"][active])
    assert torch.equal(
        reader.candidate_ids[-1][:tokens].cpu()[active], want["candidate_ids"][active]
    )
    # ... and against the reference golden where its two rotations agree.
    comparable = active & torch.from_numpy(expected["rotation_agrees"])
    assert torch.equal(
        reader.candidate_ids[-1][:tokens].cpu()[comparable],
        torch.from_numpy(expected["selected_ids"])[comparable],
    )
    counts = want["selected"].reshape(tokens, plan.top_k, -1).sum(-1).int()
    if case.threshold is not None:
        assert torch.equal(
            reader.selected[:tokens].cpu().sum(1)[active], want["selected"].sum(1)[active]
        )
    assert torch.equal(reader.counts[:tokens].cpu()[active], counts[active])
    starts = counts.cumsum(-1) - counts
    assert torch.equal(reader.starts[:tokens].cpu()[active], starts[active].int())
    # Output.
    torch.testing.assert_close(out.float()[active], want["output"][active], rtol=0.025, atol=0.02)
    reference_out = bf16_from_bits(expected["output_bits"]).float()
    torch.testing.assert_close(
        out.float()[comparable], reference_out[comparable], rtol=0.025, atol=0.02
    )
    exact = run_oracle(oracle, item, fp32=True, **own)
    assert relative_l2(out[active], exact["output"][active]) < 1e-2
    if case.padding is not None:
        assert not out[case.padding].any()
    if reader.rank:
        torch.testing.assert_close(
            reader.latent[:tokens].cpu()[active], want["latent"][active], rtol=0.015, atol=0.01
        )


def test_results_do_not_depend_on_batch_or_capacity(oracle):
    """Each token's selection is the same alone, in a batch, or in a larger workspace; so is its
    output within one kind of kernels.

    Batches of eight tokens and more read the experts' rows expert-major, smaller ones per
    token: between the two the FP32 sums are associated differently, and the outputs agree
    within the tolerance the reference allows between its own two paths (rtol 0.016, atol
    2e-3, tests/test_progressive_reader.py:875-978 of the reference).  Inside the
    expert-major path a token's sums do not depend on which other tokens share its experts.
    """
    item = prepared("qwen3-e16-t8")
    case = item["case"]
    device = torch.device("cuda:0")
    batch = make_reader(item, capacity=32, row_engine="expert_major")
    full = run_reader(batch, case).clone()
    kept = batch.candidate_ids[-1][:8].clone()
    scores = batch.scores[0][:8].clone()
    # Batches of eight and more with the per-token kernels walk the pairs in expert order:
    # same bits as the single-token calls below.
    ordered = make_reader(item, capacity=32, row_engine="per_token")
    per_token = run_reader(ordered, case).clone()
    assert torch.equal(ordered.candidate_ids[-1][:8], kept)
    torch.testing.assert_close(per_token.float(), full.float(), rtol=0.016, atol=2e-3)
    single = make_reader(item, capacity=1)
    for token in range(8):
        out = single(
            case.hidden[token : token + 1].to(device),
            case.ids[token : token + 1].to(device),
            case.weights[token : token + 1].to(device),
        )
        torch.cuda.synchronize()
        assert torch.equal(single.candidate_ids[-1][0], kept[token])
        assert torch.equal(single.scores[0][0], scores[token])
        torch.testing.assert_close(out[0].float(), full[token].float(), rtol=0.016, atol=2e-3)
        assert torch.equal(out[0], per_token[token])
    # The same tokens twice in one batch of sixteen, the second time in reverse order.
    order = torch.cat([torch.arange(8), torch.arange(7, -1, -1)])
    twice = batch(case.hidden[order].to(device), case.ids[order].to(device),
                  case.weights[order].to(device)).clone()
    torch.cuda.synchronize()
    assert torch.equal(batch.candidate_ids[-1][:16], kept[order.to(device)])
    assert torch.equal(twice, full[order.to(device)])


@pytest.mark.parametrize("name", ["qwen3-e16-t8", "gh-full"])
def test_tcgen05_screen_gives_the_same_bits(name):
    """The tcgen05/TMEM screen against the mma.sync screen and the per-pair screen."""
    item = prepared(name)
    case = item["case"]
    tokens = case.hidden.shape[0]
    device = torch.device("cuda:0")
    # Capacity 8 or more switches the screen to the expert-major kernels.
    legacy = make_reader(item, capacity=max(8, tokens))
    modern = make_reader(item, capacity=max(8, tokens), tensor_engine="tcgen05")
    repeat = -(-8 // tokens)
    hidden = case.hidden.repeat(repeat, 1).to(device)
    ids = case.ids.repeat(repeat, 1).to(device)
    weights = case.weights.repeat(repeat, 1).to(device)
    rows = hidden.shape[0]
    out_legacy = legacy(hidden, ids, weights).clone()
    out_modern = modern(hidden, ids, weights).clone()
    torch.cuda.synchronize()
    assert int(modern.workspace.status[0]) == 0  # no barrier wait ran out
    assert torch.equal(modern.partial[:rows], legacy.partial[:rows])
    assert torch.equal(modern.scores[0][:rows], legacy.scores[0][:rows])
    assert torch.equal(modern.candidate_ids[-1][:rows], legacy.candidate_ids[-1][:rows])
    assert torch.equal(out_modern, out_legacy)
    single = make_reader(item, capacity=1)
    for row in range(tokens):
        single(hidden[row : row + 1], ids[row : row + 1], weights[row : row + 1])
        torch.cuda.synchronize()
        assert torch.equal(single.partial[0], modern.partial[row])


def test_repeated_calls_are_bit_identical():
    item = prepared("qwen35-e16-t4")
    reader = make_reader(item)
    first = run_reader(reader, item["case"]).clone()
    work = reader.read_work.clone()
    for _ in range(3):
        reader.workspace.scores.fill_(float("nan"))
        reader.workspace.partial.fill_(float("nan"))
        again = run_reader(reader, item["case"])
        assert torch.equal(first, again)
    assert torch.equal(reader.read_work, 4 * work)


def test_zero_input_keeps_the_first_candidates():
    item = prepared("zero-input-ties")
    reader = make_reader(item)
    out = run_reader(reader, item["case"])
    f = item["case"].plan.final_count
    expected = torch.arange(f, dtype=torch.int32, device="cuda").expand(2, -1)
    assert torch.equal(reader.candidate_ids[-1][:2], expected)
    assert not out.any()


def test_equal_experts_tie_in_slot_order():
    item = prepared("equal-experts")
    reader = make_reader(item)
    run_reader(reader, item["case"])
    case = item["case"]
    k, i = case.plan.top_k, case.plan.expert_width
    scores = reader.scores[0][:3].reshape(3, k, i)
    assert torch.equal(scores, scores[:, :1].expand(3, k, i))
    top = (
        reader.scores[0][:3].cpu().argsort(dim=1, descending=True, stable=True)
        [:, : case.plan.final_count].sort(dim=1).values
    )
    assert torch.equal(reader.candidate_ids[-1][:3].cpu(), top.int())


def test_int64_ids_bf16_weights_and_prepared_input(oracle):
    item = prepared("gemma-gelu")
    case = item["case"]
    device = torch.device("cuda:0")
    reader = make_reader(item)
    base = run_reader(reader, case).clone()
    kept = reader.candidate_ids[-1][:4].clone()
    hidden = case.hidden.to(device)
    assert reader.prepare_input(hidden)
    out = reader(hidden, case.ids.to(device).long(), case.weights.to(device), input_prepared=True)
    torch.cuda.synchronize()
    assert torch.equal(out, base)
    assert torch.equal(reader.candidate_ids[-1][:4], kept)
    # BF16 router weights change the weights, not the contract.
    out16 = reader(hidden, case.ids.to(device), case.weights.to(device).bfloat16())
    torch.cuda.synchronize()
    assert torch.equal(reader.weights[:4], case_sorted_weights(case).to(device))
    assert torch.isfinite(out16.float()).all()


def case_sorted_weights(case):
    order = case.ids.long().argsort(dim=1, stable=True)
    return case.weights.bfloat16().float().gather(1, order)


def test_read_counters_follow_the_plan():
    item = prepared("qwen3-e16-t8")
    case, plan = item["case"], item["case"].plan
    reader = make_reader(item)
    run_reader(reader, case)
    report = reader.report()
    tokens, rank = 8, reader.rank
    assert report["reference_bytes"] == tokens * plan.native_read_bytes()
    assert report["native_expert_coefficient_bytes"] == tokens * plan.selected_weight_bytes()
    assert report["physical_sketch_bytes"] == tokens * plan.sketch_read_bytes(residual=False)
    assert report["sketch_bytes"] == tokens * plan.sketch_read_bytes(False, sectors=False)
    assert report["recovery_bytes"] == tokens * plan.recovery_read_bytes(rank)
    assert report["selection_parameter_bytes"] == tokens * plan.selection_read_bytes(False)
    assert report["rotation_sign_bytes"] == tokens * plan.hidden_size
    charged = tokens * (
        plan.selected_weight_bytes() + plan.sketch_read_bytes(residual=False)
        + plan.recovery_read_bytes(rank) + plan.selection_read_bytes(False) + plan.hidden_size
    )
    assert report["charged_bytes"] == charged
    assert report["issued_gate_up_bytes"] == tokens * 4 * plan.hidden_size * plan.final_count
    assert report["issued_down_bytes"] == tokens * 2 * plan.hidden_size * plan.final_count
    assert report["issued_recovery_encoder_bytes"] == tokens * 2 * rank * (
        plan.candidate_count - plan.final_count
    )
    assert abs(report["read_fraction"] - 0.1846) < 1e-3


def test_recovery_aware_counters_price_residuals_and_geometry():
    item = prepared("gh-full")
    case, plan = item["case"], item["case"].plan
    reader = make_reader(item)
    assert reader.recovery_geometry is not None and reader.recovery_geometry.shape == (4, 512, 2)
    run_reader(reader, case)
    report = reader.report()
    tokens, rank = 4, reader.rank
    assert report["physical_sketch_bytes"] == tokens * plan.sketch_read_bytes(residual=True)
    assert report["selection_parameter_bytes"] == tokens * plan.selection_read_bytes(True)
    assert report["charged_bytes"] == tokens * (
        plan.selected_weight_bytes() + plan.sketch_read_bytes(residual=True)
        + plan.recovery_read_bytes(rank) + plan.selection_read_bytes(True) + plan.hidden_size
    )
    # The residual variances the score used: variance plane times the kept energy per block.
    stats = item["statistics"][..., 1].float()  # [E, 2I, B]
    energy = reader.norms_input[:tokens].cpu()  # [T, B]
    ids = reader.ids[:tokens].cpu().long()
    expected = torch.einsum("tkrb,tb->tkr", stats[ids], energy)  # [T, K, 2I]
    width = plan.expert_width
    gate = expected[..., :width].reshape(tokens, -1)
    up = expected[..., width:].reshape(tokens, -1)
    torch.testing.assert_close(reader.variances[:tokens, 0].cpu(), gate, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(reader.variances[:tokens, 1].cpu(), up, rtol=1e-5, atol=1e-7)


def test_threshold_can_be_refilled_between_graph_replays_and_is_charged(oracle):
    """Reference tests/test_progressive_reader.py:1178-1304 on this reader."""
    item = prepared("threshold-mid")
    case, plan = item["case"], item["case"].plan
    device = torch.device("cuda:0")
    reader = make_reader(item)
    assert reader.selection_threshold.dtype == torch.float32
    hidden, ids, weights = case.hidden.to(device), case.ids.to(device), case.weights.to(device)
    out = torch.empty_like(hidden)
    reader(hidden, ids, weights, None, out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        reader(hidden, ids, weights, None, out)
    reader.read_work.zero_()
    n, h, rank, tokens = plan.candidate_count, plan.hidden_size, reader.rank, 4
    kept_total = 0
    for threshold, expected_counts in (
        (case.threshold, None), (0.0, [n - 1] * tokens), (torch.finfo(torch.float32).max, [0] * tokens),
    ):
        reader.selection_threshold.fill_(threshold)
        graph.replay()
        torch.cuda.synchronize()
        want = run_oracle(oracle, item, norms=reader.norms.cpu(), threshold=float(threshold))
        assert torch.equal(reader.selected[:tokens].cpu(), want["selected"])
        counts = reader.selected[:tokens].sum(1).tolist()
        if expected_counts is None:
            assert len(set(counts)) > 1 and 0 < sum(counts) < tokens * (n - 1)
        else:
            assert counts == expected_counts
        kept_total += sum(counts)
        torch.testing.assert_close(out.cpu().float(), want["output"], rtol=0.025, atol=0.02)
    calls = 3 * tokens
    report = reader.report()
    assert report["native_expert_coefficient_bytes"] == 6 * h * kept_total
    assert report["recovery_bytes"] == 2 * rank * (calls * (n + h) - kept_total)
    assert report["selection_parameter_bytes"] == calls * (4 * n + 4)
    assert report["physical_selection_parameter_bytes"] == calls * (4 * n + 32)
    assert report["sketch_bytes"] == calls * plan.sketch_read_bytes(False, False)
    assert report["selection_threshold_resident_bytes"] == 4
    k, i = plan.top_k, plan.expert_width
    macs = k * 2 * h * i + 3 * h * kept_total / calls + rank * (n - kept_total / calls + h)
    assert report["matrix_macs_per_token"] == pytest.approx(macs)


def test_layers_with_different_budgets_share_one_workspace(oracle):
    """Per-layer budgets (reference progressive.py:3388-3397): one workspace sized for the largest F."""
    from cfm_b200.reader.budget import compile_budget
    from cfm_b200.reader.progressive import ReaderWorkspace

    item = prepared("qwen35-e16-t4")
    case = item["case"]
    device = torch.device("cuda:0")
    big = case.plan
    small = compile_budget(hidden_size=big.hidden_size, expert_width=big.expert_width,
                           top_k=big.top_k, retention=0.05, screen_keep=0.625)
    assert small.final_count < big.final_count
    shared = ReaderWorkspace(big, 16, 64, 4, device)
    sketch = (item["codes"].to(device), _move_statistics(item["statistics"], device))
    arguments = (case.gate_up.to(device), _channel_major(item["down"], device),
                 case.encoder.to(device), case.decoder.to(device))
    first = ProgressiveReader(*arguments, big, 4, sketch=sketch, workspace=shared,
                              selection_score="point")
    second = ProgressiveReader(*arguments, small, 4, sketch=sketch, workspace=shared,
                               selection_score="point")
    alone = ProgressiveReader(*arguments, small, 4, sketch=sketch, selection_score="point")
    assert second.workspace_bytes == 0 and first.workspace_bytes == shared.bytes
    inputs = (case.hidden.to(device), case.ids.to(device), case.weights.to(device))
    for _ in range(2):  # interleave the layers on the shared buffer
        out_big = first(*inputs).clone()
        out_small = second(*inputs).clone()
        torch.cuda.synchronize()
        expected = alone(*inputs)
        torch.cuda.synchronize()
        assert torch.equal(out_small, expected)
        assert torch.equal(second.candidate_ids[-1][:4], alone.candidate_ids[-1][:4])
        assert second.candidate_ids[-1].shape == (4, small.final_count)
    want = run_oracle(oracle, item, norms=first.norms.cpu())
    torch.testing.assert_close(out_big.cpu().float(), want["output"], rtol=0.025, atol=0.02)
    wrong = compile_budget(hidden_size=big.hidden_size, expert_width=big.expert_width,
                           top_k=big.top_k, retention=0.3, screen_keep=0.625)
    with pytest.raises(ValueError):
        ProgressiveReader(*arguments, wrong, 4, sketch=sketch, workspace=shared,
                          selection_score="point")


def test_engine_side_caller_splits_decode_and_prefill_rows():
    from cfm_b200.runtime.experts import (
        PhaseContext, ProgressiveExperts, dense_routed_experts, reader_work_report,
    )
    from cfm_b200.runtime.ops import register_reader

    item = prepared("qwen35-e16-t4")
    case = item["case"]
    device = torch.device("cuda:0")
    reader = make_reader(item, capacity=2)
    down = _channel_major(item["down"], device)
    dense = dense_routed_experts(case.gate_up.to(device), down)
    experts = ProgressiveExperts(reader, dense, max_policy_rows=2)
    hidden, ids = case.hidden.to(device), case.ids.to(device).long()
    weights = case.weights.to(device)
    # Three decode rows (two reader calls of at most two rows) and one prefill row.
    out = experts.forward_modular(hidden, weights, ids, PhaseContext(num_decode_tokens=3))
    torch.cuda.synchronize()
    direct = make_reader(item, capacity=4)
    expected = direct(hidden, ids, weights)
    torch.cuda.synchronize()
    assert torch.equal(out[:3], expected[:3])
    torch.testing.assert_close(out[3:].float(), dense(hidden[3:], weights[3:], ids[3:]).float())
    report = reader_work_report([reader, direct])
    assert report["reference_bytes"] == 7 * case.plan.native_read_bytes()
    assert abs(report["read_fraction"] - direct.report()["read_fraction"]) < 1e-12
    # The same layer through the opaque torch operator.
    handle = register_reader(direct)
    again = torch.empty_like(hidden)
    torch.ops.cfm_b200.reader_forward(hidden, ids, weights, None, again, handle)
    torch.cuda.synchronize()
    assert torch.equal(again, expected)


@pytest.mark.parametrize("name", ["qwen3-e16-t8", "dense-bypass", "gemma-gelu"])
def test_owner_side_adopts_a_home_selection_bit_for_bit(name):
    """Expert parallelism with a replicated sketch, owner side, on one GPU.

    The whole layer stands in for a rank that owns a quarter of the experts and
    happens to serve every expert of every token: the library then launches
    fewer CTAs than kept channels and down tiles and walks both in strides.
    Adopting the single-GPU reader's kept lists and adding its latent must
    reproduce its output exactly (also for an unscreened plan, F = N).
    """
    import ctypes
    import socket

    import torch.distributed as dist
    from cfm_b200 import _native

    item = prepared(name)
    case = item["case"]
    device = torch.device("cuda:0")
    whole = make_reader(item)
    expected = run_reader(whole, case)
    tokens, experts = case.hidden.shape[0], case.gate_up.shape[0]
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        expert_map = torch.full((4 * experts,), -1, dtype=torch.int32)
        expert_map[:experts] = torch.arange(experts, dtype=torch.int32)
        owner = ProgressiveReader(
            case.gate_up.to(device), _channel_major(item["down"], device), None, None,
            case.plan, tokens, expert_map=expert_map, recovery_owner=True,
            sketch=(item["codes"].to(device), _move_statistics(item["statistics"], device)),
            activation=case.activation, selection_score=case.score,
        )
    finally:
        dist.destroy_process_group()
    hidden, ids, weights = (t.to(device) for t in (case.hidden, case.ids, case.weights))
    routed = torch.empty(tokens, case.plan.hidden_size, device=device, dtype=torch.float32)
    call = owner._call_struct(tokens, hidden, ids, weights, None, routed, False)
    lists = whole.candidate_ids[-1][:tokens].clone()
    call.lists = lists.data_ptr()
    for stage in ("cfm_adopt", "cfm_list_tiles", "cfm_exact", "cfm_down", "cfm_partial_output"):
        owner._stage(stage, call)
    out = torch.empty_like(expected)
    code = whole._library.cfm_finish(
        ctypes.byref(whole._layer), tokens, routed.data_ptr(), whole.latent.data_ptr(),
        out.data_ptr(), ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream))
    _native.check(code, "cfm_finish")
    torch.cuda.synchronize()
    assert torch.equal(owner.candidate_ids[-1][:tokens], lists)  # every slot is local
    assert torch.equal(owner.counts[:tokens], whole.counts[:tokens])
    assert torch.equal(owner.tile_starts[:tokens], whole.tile_starts[:tokens])
    assert torch.equal(out, expected)


def test_contract_violations_raise_before_launch():
    item = prepared("tiny")
    case = item["case"]
    reader = make_reader(item)
    device = torch.device("cuda:0")
    hidden, ids, weights = case.hidden.to(device), case.ids.to(device), case.weights.to(device)
    with pytest.raises(ValueError):
        reader(hidden.float(), ids, weights)
    with pytest.raises(ValueError):
        reader(torch.cat((hidden, hidden)), torch.cat((ids, ids)), torch.cat((weights, weights)))
    with pytest.raises(ValueError):
        reader(hidden, ids[:, :1].contiguous(), weights[:, :1].contiguous())
    with pytest.raises(ValueError):
        reader(hidden, ids, weights, torch.zeros(4, dtype=torch.uint8, device=device))
    with pytest.raises(ValueError):
        ProgressiveReader(
            case.gate_up.to(device), case.down.to(device), None, None, case.plan, 4,
            selection_score="point",
        )  # down is not channel-major


def test_cuda_graph_replay_with_new_inputs(oracle):
    item = prepared("graph-routes")
    case = item["case"]
    device = torch.device("cuda:0")
    reader = make_reader(item)
    hidden, ids = case.hidden.to(device), case.ids.to(device)
    weights, padding = case.weights.to(device), case.padding.to(device)
    out = torch.empty_like(hidden)
    reader(hidden, ids, weights, padding, out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        reader(hidden, ids, weights, padding, out)
    for seed, routes, pad in ((11, [[2, 0], [1, 3]], [False, True]), (29, [[3, 1], [2, 0]], [False, False])):
        fresh = torch.randn(2, 128, generator=torch.Generator().manual_seed(seed)).bfloat16()
        hidden.copy_(fresh)
        ids.copy_(torch.tensor(routes, dtype=torch.int32))
        padding.copy_(torch.tensor(pad))
        graph.replay()
        torch.cuda.synchronize()
        want = oracle.forward(
            plan=case.plan, gate_up=case.gate_up, down=item["down"], codes=item["codes"],
            statistics=item["statistics"], signs=item["signs"], hidden=fresh,
            ids=torch.tensor(routes), weights=case.weights, encoder=case.encoder,
            decoder=case.decoder, padding=torch.tensor(pad), norms=reader.norms.cpu(),
        )
        active = ~torch.tensor(pad)
        assert torch.equal(reader.selected[:2].cpu()[active], want["selected"][active])
        torch.testing.assert_close(out.cpu().float(), want["output"], rtol=0.025, atol=0.02)
