"""Host logic of the vLLM 0.22 binding: which rows of a step are decode rows, the router
restatement, block discovery and the KL formula (reference eval/fidelity.py:34-48)."""

from types import SimpleNamespace

import torch

from cfm_b200.runtime import vllm_binding as binding


def test_decode_rows_from_either_backend_shape():
    assert binding.decode_rows(None, 32) == 0
    # decode-first backends say how many rows are decode rows
    assert binding.decode_rows(SimpleNamespace(num_decode_tokens=5, num_prefills=2), 40) == 5
    assert binding.decode_rows(SimpleNamespace(num_decode_tokens=64), 32) == 32
    # the others: a step whose longest query is one token is all decode
    step = SimpleNamespace(max_query_len=1, num_actual_tokens=30)
    assert binding.decode_rows(step, 32) == 30
    assert binding.decode_rows(SimpleNamespace(max_query_len=4096, num_actual_tokens=4096), 4096) == 0


def test_route_matches_softmax_topk_renormalised():
    generator = torch.Generator().manual_seed(0)
    logits = torch.randn(6, 16, generator=generator)
    weights, ids = binding.route(logits, 4, True)
    assert ids.dtype == torch.int32 and weights.dtype == torch.float32
    probabilities = torch.softmax(logits, dim=-1)
    assert torch.equal(ids.long(), probabilities.topk(4).indices)
    torch.testing.assert_close(weights.sum(-1), torch.ones(6))
    raw, _ = binding.route(logits, 4, False)
    torch.testing.assert_close(raw, probabilities.topk(4).values)


def test_kl_formula():
    generator = torch.Generator().manual_seed(1)
    a, b = torch.randn(3, 50, generator=generator), torch.randn(3, 50, generator=generator)
    divergence, same = binding.kl_and_top1(a, b)
    want = torch.nn.functional.kl_div(
        torch.log_softmax(b, -1), torch.log_softmax(a, -1), log_target=True, reduction="none"
    ).sum(-1)
    torch.testing.assert_close(divergence, want)
    zero, agree = binding.kl_and_top1(a, a)
    assert float(zero.abs().max()) == 0.0 and bool(agree.all())
    assert same.shape == (3,)


def test_moe_blocks_finds_gate_plus_fused_experts():
    class Fused(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w13_weight = torch.nn.Parameter(torch.zeros(2, 4, 2))
            self.w2_weight = torch.nn.Parameter(torch.zeros(2, 2, 2))

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate = torch.nn.Linear(2, 2)
            self.experts = Fused()

    model = torch.nn.Sequential(Block(), torch.nn.Linear(2, 2), Block())
    assert [name for name, _ in binding.moe_blocks(model)] == ["0", "2"]


def test_dense_block_is_the_routed_mlp():
    generator = torch.Generator().manual_seed(2)
    gate_up = torch.randn(3, 8, 6, generator=generator)
    down = torch.randn(3, 6, 4, generator=generator)
    x = torch.randn(2, 6, generator=generator)
    weights = torch.tensor([[0.75, 0.25], [1.0, 0.0]])
    ids = torch.tensor([[0, 2], [1, 0]], dtype=torch.int32)
    got = binding.dense_block(gate_up, down, x, weights, ids)
    gate, up = (gate_up[0] @ x[0]).split(4)
    first = 0.75 * (down[0] @ (torch.nn.functional.silu(gate) * up))
    gate, up = (gate_up[2] @ x[0]).split(4)
    first = first + 0.25 * (down[2] @ (torch.nn.functional.silu(gate) * up))
    torch.testing.assert_close(got[0], first)
