"""Sketch construction, packing and rotation on the CPU (reference tests/test_sketch.py,
tests/test_progressive_reader.py:81-99)."""

import hashlib

import pytest
import torch

import cases
from cfm_b200.reader.budget import sketch_code_stride, sketch_storage_bytes
from cfm_b200.reader.sketch import (
    block_hadamard_signs,
    build_sketch,
    mask_rotated_blocks,
    repack_sketch,
    rotate_blocks,
    unpack_sketch,
)
from helpers import golden


def _hadamard(size: int) -> torch.Tensor:
    matrix = torch.ones(1, 1)
    while len(matrix) < size:
        matrix = torch.cat((torch.cat((matrix, matrix), 1), torch.cat((matrix, -matrix), 1)), 0)
    return matrix


def test_packing_scale_and_residual_variance():
    torch.manual_seed(33)
    weights = torch.randn(2, 8, 256).bfloat16()
    codes, statistics = build_sketch(weights)
    original = weights.float().reshape(2, 8, 2, 128)
    member = original.abs() > 0.7 * original.abs().mean(-1, keepdim=True)
    scale = (original.abs() * member).sum(-1) / member.sum(-1)
    trits = torch.where(member, original.sign(), 0).reshape_as(weights)
    assert torch.equal(unpack_sketch(codes, 8, 256).long(), trits.long())
    assert torch.equal(statistics[..., 0], scale.half())
    residual = original - trits.reshape_as(original) * scale[..., None]
    assert torch.equal(statistics[..., 1], residual.square().mean(-1).half())
    assert codes.numel() + statistics.numel() * 2 == 2 * 2 * (128 * 16 + 8 * 4)
    assert statistics.stride() == (4 * 4 * 2, 1, 4 * 4, 2 * 4)


def test_rotation_is_the_signed_sylvester_matrix():
    hidden = 384
    signs = block_hadamard_signs(hidden, "cpu")
    assert set(signs.tolist()) == {-1, 1}
    x = torch.randn(5, hidden, generator=torch.Generator().manual_seed(3)).bfloat16()
    dense = torch.block_diag(*[_hadamard(128)] * 3) / 128**0.5 * signs.float()[None, :]
    torch.testing.assert_close(rotate_blocks(x, signs), x.float() @ dense.T, atol=2e-6, rtol=0)
    torch.testing.assert_close(dense @ dense.T, torch.eye(hidden), atol=1e-6, rtol=0)


def test_mask_keeps_largest_with_ties_to_lower_coordinate():
    x = torch.zeros(1, 128)
    x[0, [5, 9, 70, 100]] = torch.tensor([2.0, -1.0, 1.0, 1.0])
    kept = mask_rotated_blocks(x, 3)
    assert kept.nonzero()[:, 1].tolist() == [5, 9, 70]
    assert torch.equal(mask_rotated_blocks(x, 128), x)
    zero = mask_rotated_blocks(torch.zeros(2, 256), 80)
    assert not zero.any()


@pytest.mark.parametrize("width,hidden", [(160, 384), (512, 256), (768, 256), (528, 128)])
def test_kernel_layout_round_trip(width, hidden):
    g = torch.Generator().manual_seed(7)
    weights = (torch.randn(2, 2 * width, hidden, generator=g) * 0.02).bfloat16()
    codes, _ = build_sketch(weights, block_hadamard_signs(hidden, "cpu"))
    assert codes.shape == (2, sketch_storage_bytes(2 * width, hidden))
    # Padding bytes decode to zero trits and every stored byte is a valid base-3 code.
    assert int(codes.max()) < 243
    words = repack_sketch(codes, 2 * width, hidden).to(torch.int64) & 0xFFFFFFFF
    decoded = torch.stack([((words >> (2 * j)) & 3) - 1 for j in range(16)], -1)
    decoded = decoded.reshape(2, hidden, 2 * width).transpose(1, 2)
    assert torch.equal(decoded.to(torch.int8), unpack_sketch(codes, 2 * width, hidden))
    assert sketch_code_stride(2 * width) % 16 == 0


@pytest.mark.parametrize("name", [n for n in cases.NAMES if n not in ("olmoe-t1",)])
def test_sketch_bytes_match_reference_digests(name):
    """build_sketch reproduces the reference builder byte for byte on every case."""
    case = cases.build(name)
    expected = golden(name)
    signs = block_hadamard_signs(case.plan.hidden_size, "cpu")
    codes, statistics = build_sketch(case.gate_up, signs)
    digest = hashlib.sha256(codes.numpy().tobytes()).digest()
    assert digest == expected["codes_sha256"].tobytes()
    physical = statistics.permute(0, 2, 3, 1).contiguous().view(torch.int16).numpy()
    assert hashlib.sha256(physical.tobytes()).digest() == expected["statistics_sha256"].tobytes()
