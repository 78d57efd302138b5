"""The screen entry point that brings its own scratch (`cfm_screen_static`).

Some callers of the reader cannot hand it scratch memory and must not trigger a
device allocation: a decode step running inside a serving engine that has
already given all free device memory to its cache pool, or a plugin host that
forbids allocator calls.  For them the library keeps the split screen's scratch
(per-block products and arrival counters) in two arrays of its own image.  This
test calls that entry point through the C ABI, twice in a row on the same
inputs, and requires both results to equal the regular `cfm_screen` output bit
for bit (the bar of the other parity tests); the second call proves that what
the first left in the shared arrays does not leak into the next result, and the
amount of free device memory is the same before and after it.

Collected last on purpose, so a run that stops at the first failure has already
covered every other test.
"""

import ctypes

import pytest
import torch

from cfm_b200 import _native
from helpers import prepared
from test_gpu_parity import make_reader, run_reader

pytestmark = pytest.mark.gpu


def call_static(reader, tokens, out, padding=None, variances=None):
    w = reader.workspace
    io = _native.StaticScreen()
    io.tokens = tokens
    io.ids = w.ids.data_ptr()
    io.quantized = w.quantized.data_ptr()
    io.coordinates = w.coordinates.data_ptr()
    io.exponents = w.exponents.data_ptr()
    io.padding = padding.data_ptr() if padding is not None else None
    io.partial = out.data_ptr()
    if variances is not None:
        io.energies = w.norms.data_ptr()
        io.variances = variances.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    return _native.screen_static()(
        ctypes.byref(reader._layer), ctypes.byref(io), ctypes.c_void_p(stream)
    )


def test_static_scratch_screen_matches_regular_screen_twice():
    item = prepared("qwen35-e16-t4")
    reader = make_reader(item)
    run_reader(reader, item["case"])  # regular path: fills ids, kept values and `partial`
    tokens = item["case"].hidden.shape[0]
    expected = reader.partial[:tokens].clone()
    assert torch.isfinite(expected).all() and expected.abs().sum() > 0
    for repeat in range(2):
        out = torch.full_like(expected, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert call_static(reader, tokens, out) == 0
        torch.cuda.synchronize()
        if repeat:  # the first call on a device may still load the library's device image
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(out, expected)


def test_static_scratch_screen_matches_the_expert_major_screen():
    """Sixteen tokens: the regular screen runs expert-major on the tensor cores, the
    library-scratch screen per (token, expert) pair; same bits."""
    import cases
    from helpers import prepared_case

    item = prepared_case(cases._random("static-t16", 421, 256, 96, 8, 4, 16, 16, 0.125, 0.625))
    reader = make_reader(item)
    run_reader(reader, item["case"])
    expected = reader.partial[:16].clone()
    assert expected.abs().sum() > 0
    out = torch.full_like(expected, float("nan"))
    assert call_static(reader, 16, out) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    assert call_static(reader, 16, out) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(out, expected)


def test_static_scratch_screen_also_gives_the_variances():
    """Recovery-aware score: the variances cfm_screen leaves for the selection come from
    the library-scratch call too when asked for."""
    item = prepared("gh-keep80-gelu")
    reader = make_reader(item)
    run_reader(reader, item["case"])
    tokens = item["case"].hidden.shape[0]
    expected, spread = reader.partial[:tokens].clone(), reader.variances[:tokens].clone()
    assert spread.abs().sum() > 0
    out, variances = torch.full_like(expected, float("nan")), torch.full_like(spread, float("nan"))
    assert call_static(reader, tokens, out, variances=variances) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, expected) and torch.equal(variances, spread)


def test_static_scratch_screen_with_padding_row():
    item = prepared("graph-routes")  # second row is padding
    reader = make_reader(item)
    run_reader(reader, item["case"])
    padding = item["case"].padding.cuda()
    expected = reader.partial[:2].clone()
    out = torch.full_like(expected, float("nan"))
    assert call_static(reader, 2, out, padding) == 0
    torch.cuda.synchronize()
    assert torch.equal(out[0], expected[0])
    assert not out[1].any()  # padded rows are written as zeros


def test_static_scratch_screen_rejects_batches_beyond_its_arrays():
    item = prepared("qwen3-e16-t8")  # 64 pairs x 16 blocks x 1536 rows > 2**20 floats
    reader = make_reader(item)
    run_reader(reader, item["case"])
    out = torch.zeros_like(reader.partial[:8])
    code = call_static(reader, 8, out)
    assert code == _native.E_STATIC_CAPACITY
    message = _native.load().cfm_error_string(code).decode()
    assert "scratch" in message
    assert not out.any()  # nothing was launched
