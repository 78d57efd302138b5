"""The reader as an opaque torch custom operator.

A compiled model graph must treat the layer as one opaque call (the reference
does the same for its branch operators, runtime/qwen35.py:80-95): the operator
takes the layer's hidden rows and router outputs, writes the output rows in
place, and names its reader by an integer handle, so no Python object crosses
the graph.  The implementation enqueues the CUDA library's kernels on the
current stream; there is no other implementation behind the operator.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ..reader.progressive import ProgressiveReader

_readers: dict[int, ProgressiveReader] = {}


def register_reader(reader: ProgressiveReader) -> int:
    """Make `reader` callable through the operator; returns its handle."""
    handle = len(_readers)
    _readers[handle] = reader
    return handle


@torch.library.custom_op("cfm_b200::reader_forward", mutates_args=("out",), device_types="cuda")
def reader_forward(
    hidden: Tensor, ids: Tensor, weights: Tensor, padding: Tensor | None, out: Tensor, handle: int
) -> None:
    _readers[handle](hidden, ids, weights, padding, out)


@reader_forward.register_fake
def _(hidden, ids, weights, padding, out, handle) -> None:
    return None
