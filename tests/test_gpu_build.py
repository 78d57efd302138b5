"""The sketch built by the library's kernel against the reference-identical torch builder.

Both rotate with the same butterfly and apply the same ternary rule; the kernel
adds a block's 128 magnitudes in its own fixed order, torch in its reduction's
order, so a coordinate whose magnitude sits within rounding of 0.7 mean|v| may
come out differently, and a scale may differ in its last FP16 bit.  The test
bounds both (a handful of coordinates among millions), checks that the kernel's
two layouts describe the same trits, and that a reader built on the kernel's
sketch matches the oracle run on that same sketch bit for bit.
"""

import pytest
import torch

from cfm_b200.reader.progressive import ProgressiveReader
from cfm_b200.reader.sketch import (
    block_hadamard_signs, build_sketch, build_sketch_on_device, codes_from_words, repack_sketch,
    repack_sketch_grouped,
)
from helpers import prepared, run_oracle
from test_gpu_parity import _channel_major

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("experts,width,hidden", [(4, 64, 256), (2, 528, 128), (2, 768, 2048)])
def test_kernel_sketch_matches_the_torch_builder(experts, width, hidden):
    device = torch.device("cuda:0")
    generator = torch.Generator().manual_seed(experts * 1000 + width)
    weights = (torch.randn(experts, 2 * width, hidden, generator=generator) * 0.02).bfloat16()
    weights = weights.to(device)
    signs = block_hadamard_signs(hidden, device)
    codes, statistics = build_sketch(weights, signs)
    words, grouped, fast = build_sketch_on_device(weights, signs)
    torch.cuda.synchronize()
    expected = repack_sketch(codes, 2 * width, hidden)
    differing = (words ^ expected).to(torch.int64) & 0xFFFFFFFF
    fields = sum(((differing >> (2 * j)) & 3).ne(0).sum() for j in range(16))
    trits = experts * 2 * width * hidden
    print(f"{int(fields)} of {trits} trits differ from the torch builder")
    assert int(fields) <= max(2, trits // 100_000)
    # The kernel's two layouts hold the same trits.
    own_codes = codes_from_words(words, 2 * width, hidden)
    assert torch.equal(grouped, repack_sketch_grouped(own_codes, 2 * width, hidden))
    assert torch.equal(words, repack_sketch(own_codes, 2 * width, hidden))
    # Scales and residual variances: same FP16 values but for the last bit of a few.
    assert fast.shape == statistics.shape and fast.stride() == statistics.stride()
    torch.testing.assert_close(fast.float(), statistics.float(), rtol=2e-3, atol=1e-7)
    same = (fast == statistics).float().mean()
    assert float(same) > 0.99


def test_reader_on_the_kernel_sketch_matches_the_oracle_on_that_sketch(oracle):
    item = prepared("qwen35-e16-t4")
    case = item["case"]
    device = torch.device("cuda:0")
    reader = ProgressiveReader(
        case.gate_up.to(device), _channel_major(item["down"], device), case.encoder.to(device),
        case.decoder.to(device), case.plan, 8, selection_score="point", sketch_builder="cuda",
    )
    tokens = case.hidden.shape[0]
    out = reader(case.hidden.to(device), case.ids.to(device), case.weights.to(device))
    torch.cuda.synchronize()
    want = run_oracle(oracle, item, codes=reader.sketch_codes.cpu(),
                      statistics=reader.sketch_statistics.cpu(), norms=reader.norms.cpu())
    assert torch.equal(reader.partial[:tokens].cpu(), want["partial"])
    assert torch.equal(reader.scores[0][:tokens].cpu(), want["scores"])
    assert torch.equal(reader.candidate_ids[-1][:tokens].cpu(), want["candidate_ids"])
    torch.testing.assert_close(out.float().cpu(), want["output"], rtol=0.025, atol=0.02)
