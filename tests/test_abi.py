"""The C-ABI library: it loads, and exports every entry point the header declares.

No GPU is needed: nothing here launches work.  The only functions called are the
ones that run on the host alone (version, error strings, workspace layout).
"""

import ctypes
import re
from pathlib import Path

import pytest

import cfm_b200  # noqa: F401  (registers the package alias)
from cfm_b200 import _native
from cfm_b200.reader.budget import compile_budget
from cfm_b200.reader.progressive import _dimension_layer

HEADER = Path(__file__).resolve().parents[1] / "include" / "cfm_b200.h"


@pytest.fixture(scope="module")
def library():
    if not _native.LIBRARY.exists():
        _native.build()
    return _native.load()


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"^(?:int|int64_t|const char\*)\s+(cfm_\w+)\s*\(", text, flags=re.M)


def test_header_declares_the_entry_points_the_binding_uses():
    declared = set(declared_functions())
    assert declared, "no declarations found in the header"
    assert set(_native.SYMBOLS) | {"cfm_screen_static"} <= declared


def test_every_declared_entry_point_is_exported(library):
    raw = ctypes.CDLL(str(_native.LIBRARY))
    missing = [name for name in declared_functions() if not hasattr(raw, name)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_versions_agree(library):
    text = HEADER.read_text()
    header_version = int(re.search(r"#define\s+CFM_ABI_VERSION\s+(\d+)", text).group(1))
    assert library.cfm_abi_version() == header_version == _native.ABI_VERSION


def test_error_strings(library):
    library.cfm_error_string.restype = ctypes.c_char_p
    assert library.cfm_error_string(0) == b"success"
    for code in (-1, -2, -3, -4, -5):
        message = library.cfm_error_string(code)
        assert message and message != b"unknown error"


def test_workspace_layout_is_a_host_computation(library):
    plan = compile_budget(hidden_size=2048, expert_width=768, top_k=8,
                          retention=0.123046875, screen_keep=0.625)
    layout = _native.workspace_layout(_dimension_layer(plan, 128, 64), 64)
    offsets = [getattr(layout, name) for name in _native._LAYOUT_ARRAYS]
    assert offsets == sorted(offsets) and len(set(offsets)) == len(offsets)
    assert all(offset % 256 == 0 for offset in offsets)
    assert layout.bytes > offsets[-1]
    # Arrays up to the arrival counters do not depend on the number of kept channels.
    smaller = compile_budget(hidden_size=2048, expert_width=768, top_k=8,
                             retention=0.0615234375, screen_keep=0.625)
    other = _native.workspace_layout(_dimension_layer(smaller, 128, 64), 64)
    assert other.counters == layout.counters and other.bytes < layout.bytes


def test_layout_rejects_bad_dimensions(library):
    plan = compile_budget(hidden_size=2048, expert_width=768, top_k=8,
                          retention=0.123046875, screen_keep=0.625)
    layer = _dimension_layer(plan, 128, 64)
    layout = _native.WorkspaceLayout()
    assert library.cfm_workspace_layout_for(None, 64, ctypes.byref(layout)) == -1
    assert library.cfm_workspace_layout_for(ctypes.byref(layer), 0, ctypes.byref(layout)) == -3
    layer.hidden = 2000  # not a multiple of the rotation block
    assert library.cfm_workspace_layout_for(ctypes.byref(layer), 64, ctypes.byref(layout)) == -2


def test_struct_sizes_match_the_header(library):
    """The ctypes mirrors have the sizes the C structs of the header have on this ABI."""
    pointer = ctypes.sizeof(ctypes.c_void_p)
    assert ctypes.sizeof(_native.Layer) == 14 * 4 + 13 * pointer
    assert ctypes.sizeof(_native.Call) == 6 * 4 + 7 * pointer
    assert ctypes.sizeof(_native.Exchange) == 4 * 4 + _native.MAX_RANKS * pointer
    assert ctypes.sizeof(_native.StaticScreen) == 2 * 4 + 8 * pointer
    text = HEADER.read_text()
    assert int(re.search(r"#define\s+CFM_MAX_RANKS\s+(\d+)", text).group(1)) == _native.MAX_RANKS
    assert (int(re.search(r"#define\s+CFM_PEER_HANDLE_BYTES\s+(\d+)", text).group(1))
            == _native.PEER_HANDLE_BYTES)


def test_exchange_bytes_is_a_host_computation(library):
    plan = compile_budget(hidden_size=2048, expert_width=768, top_k=8,
                          retention=0.123046875, screen_keep=0.625)
    layer = _dimension_layer(plan, 16, 0)
    size = library.cfm_exchange_bytes(ctypes.byref(layer), 8, 64)
    # header, lists i32 [P][T][F], rows f32 [P][T][H]
    assert size == 1024 + 8 * 64 * 756 * 4 + 8 * 64 * 2048 * 4
    assert library.cfm_exchange_bytes(ctypes.byref(layer), 17, 64) == 0  # more ranks than supported


def test_layout_rejects_more_candidates_than_the_selection_takes(library):
    plan = compile_budget(hidden_size=256, expert_width=4096, top_k=8, retention=0.125,
                          screen_keep=0.625)
    with pytest.raises(ValueError):
        _native.workspace_layout(_dimension_layer(plan, 8, 0), 4)  # N = 32768
