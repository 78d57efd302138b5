"""Host-side pieces of the benchmark: the algorithmic-byte count and the packed input block."""

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from cfm_b200.reader.budget import compile_budget  # noqa: E402


def test_distinct_bytes_of_a_hand_counted_call():
    plan = compile_budget(hidden_size=256, expert_width=64, top_k=2, retention=0.25,
                          screen_keep=0.5)
    h, i, k, rank, experts = 256, 64, 2, 8, 4
    keep, blocks = plan.screen_coordinates, h // 128
    # Two tokens; expert 1 is shared, expert 3 is held elsewhere (-1).
    ids = torch.tensor([[0, 1], [1, -1]], dtype=torch.int32)
    selected = torch.zeros(2, k * i, dtype=torch.bool)
    selected[0, [0, 1, i + 5]] = True          # token 0: channels 0, 1 of expert 0; 5 of expert 1
    selected[1, [5, 6, i + 0]] = True          # token 1: channels 5, 6 of expert 1; slot 1 is remote
    coordinates = torch.arange(keep).expand(2, blocks, keep).contiguous().int()
    got = bench.distinct_bytes(plan, experts, rank, ids, selected, coordinates, 2)
    kept = 2 + 2                                # expert 0: {0, 1}; expert 1: {5, 6}
    skipped = (i - 2) + (i - 1)                 # expert 1 skips every channel but 5 for token 0,
    # and every channel but 5, 6 for token 1: the union of skipped channels is all but 5
    routed = 2
    union_coordinates = routed * blocks * keep  # both tokens keep the same coordinates
    assert got["k_screen"] == union_coordinates * (i // 2) + routed * (blocks * 2 * 2 * i + 4 * i)
    assert got["k_down"] == kept * 2 * h
    assert got["k_exact"] == kept * 4 * h + 2 * 2 * h
    assert got["k_encode"] == skipped * 2 * rank
    fixed = 2 * h * rank + h + 2 * (4 * h + 8 * k)
    assert got["total"] == got["k_screen"] + kept * 6 * h + got["k_encode"] + fixed


def test_packed_batch_views_share_one_block():
    batch = (torch.randn(4, 8).bfloat16(), torch.arange(8, dtype=torch.int32).view(4, 2),
             torch.rand(4, 2))
    views = bench.packed_batch(batch)
    block = views[0]._packed
    assert all(torch.equal(a, b) for a, b in zip(batch, views))
    assert block.dtype == torch.uint8 and block.numel() % 256 == 0
    offsets = [view.data_ptr() - block.data_ptr() for view in views]
    assert offsets == sorted(offsets) and all(offset % 256 == 0 for offset in offsets)
    # One copy of the block refreshes every view.
    fresh = block.clone()
    fresh[: batch[0].numel() * 2] = 0
    block.copy_(fresh)
    assert not views[0].any() and torch.equal(views[1], batch[1])
