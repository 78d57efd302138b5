"""Row splitting and chunking of the engine-side caller (reference runtime/experts.py:334-516)."""

import pytest
import torch

from cfm_b200.runtime.experts import PhaseContext, ProgressiveExperts, reader_rows


class RecordingReader:
    """Stands in for the reader: doubles its rows, records every call."""

    max_tokens = 4

    def __init__(self):
        self.calls = []
        self.prepared = 0

    def __call__(self, x, ids, weights, padding=None, out=None, *, input_prepared=False):
        self.calls.append((x.shape[0], None if padding is None else padding.tolist(), input_prepared))
        result = x * 2
        if out is not None:
            out.copy_(result)
            return out
        return result

    def prepare_input(self, x, padding=None):
        self.prepared += 1
        return True


def stock(x, weights, ids):
    return x * 3


def batch(rows):
    x = torch.arange(rows * 2, dtype=torch.float32).reshape(rows, 2)
    return x, torch.ones(rows, 2), torch.zeros(rows, 2, dtype=torch.int32)


def test_reader_rows_chunks_in_order():
    reader = RecordingReader()
    x, w, ids = batch(10)
    padding = torch.tensor([False] * 9 + [True])
    out = reader_rows(reader, x, ids, w, padding, 4)
    assert torch.equal(out, x * 2)
    assert [c[0] for c in reader.calls] == [4, 4, 2]
    assert reader.calls[-1][1] == [False, True]
    reader.calls.clear()
    reader_rows(reader, x[:3], ids[:3], w[:3], None, 4)
    assert reader.calls == [(3, None, False)]


def test_decode_prefix_goes_sparse_and_the_rest_stock():
    experts = ProgressiveExperts(RecordingReader(), stock, max_policy_rows=4)
    x, w, ids = batch(6)
    out = experts.forward_modular(x, w, ids, PhaseContext(num_decode_tokens=2))
    assert torch.equal(out[:2], x[:2] * 2) and torch.equal(out[2:], x[2:] * 3)
    out = experts.forward_modular(x, w, ids, PhaseContext(num_decode_tokens=0))
    assert torch.equal(out, x * 3)
    out = experts.forward_modular(x, w, ids, PhaseContext(num_decode_tokens=6))
    assert torch.equal(out, x * 2)
    assert [c[0] for c in experts.reader.calls[-2:]] == [4, 2]


def test_generated_prefill_rows_take_the_policy():
    experts = ProgressiveExperts(RecordingReader(), stock, max_policy_rows=4)
    x, w, ids = batch(5)
    split = (torch.tensor([1, 3]), torch.tensor([0, 2, 4]))
    out = experts.forward_modular(x, w, ids, PhaseContext(0, split))
    assert torch.equal(out[[1, 3]], x[[1, 3]] * 2)
    assert torch.equal(out[[0, 2, 4]], x[[0, 2, 4]] * 3)


def test_sparse_prefill_and_early_rotation():
    experts = ProgressiveExperts(RecordingReader(), stock, max_policy_rows=4, sparse_prefill=True)
    x, w, ids = batch(3)
    context = PhaseContext(num_decode_tokens=0, is_padding=torch.tensor([False, False, True]))
    experts.prepare_reader_input(x, context)
    assert experts.reader.prepared == 1 and experts.reader_input_prepared
    out = experts.forward_modular(x, w, ids, context)
    assert torch.equal(out, x * 2)
    assert experts.reader.calls[-1] == (3, [False, False, True], True)
    assert not experts.reader_input_prepared
    with pytest.raises(ValueError):
        ProgressiveExperts(RecordingReader(), stock, max_policy_rows=8)
