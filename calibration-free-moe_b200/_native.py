"""ctypes binding of the CUDA library `libcfm_b200.so` (C ABI in include/cfm_b200.h).

The library is built in-tree by `build()` (nvcc, sm_100a only).  There is no
fallback: `load()` raises if the library is missing, and every stage call raises
on a non-zero return code.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
SOURCES = [PACKAGE / "csrc" / "cfm_reader.cu"]
HEADERS = [PACKAGE / "csrc" / "cfm_device.cuh", PACKAGE / "csrc" / "cfm_grouped.cuh",
           PACKAGE / "csrc" / "cfm_exchange.cuh", PACKAGE / "csrc" / "cfm_select.cuh",
           PACKAGE / "csrc" / "cfm_build.cuh", PACKAGE / "csrc" / "cfm_screen_rows32.cuh",
           PACKAGE.parent / "include" / "cfm_b200.h"]
LIBRARY = PACKAGE / "libcfm_b200.so"
ABI_VERSION = 10

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

# Entry points include/cfm_b200.h declares; `load()` checks each one resolves.
STAGES = (
    "cfm_prepare_input", "cfm_route", "cfm_screen", "cfm_score", "cfm_select", "cfm_exact",
    "cfm_down", "cfm_encode", "cfm_output", "cfm_partial_output", "cfm_adopt", "cfm_list_tiles", "cfm_reader_forward",
)
PEER_SYMBOLS = ("cfm_build_sketch", "cfm_exchange_bytes", "cfm_peer_alloc", "cfm_peer_export", "cfm_peer_import",
                "cfm_peer_release", "cfm_exchange_status", "cfm_finish_rows")
SYMBOLS = (("cfm_abi_version", "cfm_error_string", "cfm_workspace_layout_for", "cfm_finish")
           + STAGES + PEER_SYMBOLS)
MAX_RANKS = 16
PEER_HANDLE_BYTES = 64


class Layer(ctypes.Structure):
    """`struct cfm_layer`."""

    _fields_ = [
        ("hidden", ctypes.c_int32),
        ("width", ctypes.c_int32),
        ("experts", ctypes.c_int32),
        ("top_k", ctypes.c_int32),
        ("final_count", ctypes.c_int32),
        ("keep", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("activation", ctypes.c_int32),
        ("score", ctypes.c_int32),
        ("global_experts", ctypes.c_int32),
        ("recovery_owner", ctypes.c_int32),
        ("tensor_engine", ctypes.c_int32),
        ("row_engine", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("gate_up", ctypes.c_void_p),
        ("down", ctypes.c_void_p),
        ("sketch", ctypes.c_void_p),
        ("sketch_grouped", ctypes.c_void_p),
        ("statistics", ctypes.c_void_p),
        ("norms", ctypes.c_void_p),
        ("geometry", ctypes.c_void_p),
        ("encoder", ctypes.c_void_p),
        ("decoder", ctypes.c_void_p),
        ("signs", ctypes.c_void_p),
        ("expert_map", ctypes.c_void_p),
        ("read_work", ctypes.c_void_p),
        ("selection_threshold", ctypes.c_void_p),
    ]


class Call(ctypes.Structure):
    """`struct cfm_call`."""

    _fields_ = [
        ("tokens", ctypes.c_int32),
        ("ids_are_int64", ctypes.c_int32),
        ("weights_are_bf16", ctypes.c_int32),
        ("input_prepared", ctypes.c_int32),
        ("scores_ready", ctypes.c_int32),
        ("row_offset", ctypes.c_int32),
        ("hidden", ctypes.c_void_p),
        ("ids", ctypes.c_void_p),
        ("weights", ctypes.c_void_p),
        ("padding", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("lists", ctypes.c_void_p),
        ("exchange", ctypes.c_void_p),
    ]


class Exchange(ctypes.Structure):
    """`struct cfm_exchange`."""

    _fields_ = [
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("blocks", ctypes.c_void_p * MAX_RANKS),
    ]


_LAYOUT_ARRAYS = (
    "ids", "weights", "norms", "planes", "coordinates", "quantized", "exponents", "parts",
    "counters", "partial", "scores", "selected", "completed", "candidate_ids", "counts",
    "starts", "tile_starts", "activations", "exact", "down_parts", "encoder_parts", "latent",
    "status", "limbs", "group_offsets", "group_pairs", "cuts", "variances", "unscales", "zero_limbs",
    "tile_list", "tile_count",
)


class WorkspaceLayout(ctypes.Structure):
    """`struct cfm_workspace_layout`."""

    _fields_ = (
        [("bytes", ctypes.c_int64)]
        + [(name, ctypes.c_int64) for name in _LAYOUT_ARRAYS]
        + [
            ("parts_tokens", ctypes.c_int32),
            ("down_tiles", ctypes.c_int32),
            ("encoder_tiles", ctypes.c_int32),
            ("reserved", ctypes.c_int32),
        ]
    )


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA library for sm_100a into the package directory."""
    newest = max(p.stat().st_mtime for p in SOURCES + HEADERS)
    if not force and LIBRARY.exists() and LIBRARY.stat().st_mtime >= newest:
        return LIBRARY
    command = [nvcc(), *NVCC_FLAGS, f"-I{PACKAGE.parent / 'include'}", f"-I{PACKAGE / 'csrc'}"]
    if verbose:
        command += ["-Xptxas", "-v"]
    command += ["-o", str(LIBRARY), *map(str, SOURCES)]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"nvcc failed:\n{done.stdout}\n{done.stderr}")
    if verbose:
        print(done.stderr)
    return LIBRARY


_library: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load the built library and bind its entry points.  Raises if it is absent."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY.exists():
        raise RuntimeError(
            f"{LIBRARY} is missing: the CUDA library has not been built "
            "(run `python -c 'import __graft_entry__ as g; g.build()'` at the repository "
            "root). This package has no CPU or PyTorch fallback."
        )
    library = ctypes.CDLL(os.fspath(LIBRARY))
    for symbol in SYMBOLS:
        if not hasattr(library, symbol):
            raise RuntimeError(f"{LIBRARY} does not export {symbol}")
    library.cfm_abi_version.restype = ctypes.c_int
    if library.cfm_abi_version() != ABI_VERSION:
        raise RuntimeError("libcfm_b200.so was built from another ABI version; rebuild it")
    library.cfm_error_string.restype = ctypes.c_char_p
    library.cfm_error_string.argtypes = [ctypes.c_int]
    library.cfm_workspace_layout_for.restype = ctypes.c_int
    library.cfm_workspace_layout_for.argtypes = [
        ctypes.POINTER(Layer), ctypes.c_int32, ctypes.POINTER(WorkspaceLayout),
    ]
    for stage in STAGES:
        function = getattr(library, stage)
        function.restype = ctypes.c_int
        function.argtypes = [
            ctypes.POINTER(Layer), ctypes.c_void_p, ctypes.c_int32, ctypes.POINTER(Call),
            ctypes.c_void_p,
        ]
    library.cfm_finish.restype = ctypes.c_int
    library.cfm_finish.argtypes = [
        ctypes.POINTER(Layer), ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_void_p,
    ]
    library.cfm_build_sketch.restype = ctypes.c_int
    library.cfm_build_sketch.argtypes = [
        ctypes.POINTER(Layer), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_void_p, ctypes.c_void_p,
    ]
    library.cfm_exchange_bytes.restype = ctypes.c_int64
    library.cfm_exchange_bytes.argtypes = [ctypes.POINTER(Layer), ctypes.c_int32, ctypes.c_int32]
    library.cfm_peer_alloc.restype = ctypes.c_int
    library.cfm_peer_alloc.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]
    library.cfm_peer_export.restype = ctypes.c_int
    library.cfm_peer_export.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    library.cfm_peer_import.restype = ctypes.c_int
    library.cfm_peer_import.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
    library.cfm_peer_release.restype = ctypes.c_int
    library.cfm_peer_release.argtypes = [ctypes.c_void_p, ctypes.c_int32]
    library.cfm_exchange_status.restype = ctypes.c_int
    library.cfm_exchange_status.argtypes = [ctypes.POINTER(Exchange),
                                            ctypes.POINTER(ctypes.c_int32)]
    library.cfm_finish_rows.restype = ctypes.c_int
    library.cfm_finish_rows.argtypes = [
        ctypes.POINTER(Layer), ctypes.POINTER(Exchange), ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_void_p,
    ]
    _library = library
    return library


def check(code: int, what: str) -> None:
    """Raise for a non-zero return code of the library."""
    if code:
        message = load().cfm_error_string(code).decode()
        raise RuntimeError(f"{what} failed: {message} (code {code})")


def workspace_layout(layer: Layer, capacity: int) -> WorkspaceLayout:
    layout = WorkspaceLayout()
    code = load().cfm_workspace_layout_for(ctypes.byref(layer), capacity, ctypes.byref(layout))
    if code:
        raise ValueError(load().cfm_error_string(code).decode())
    return layout


class StaticScreen(ctypes.Structure):
    """`struct cfm_static_screen`."""

    _fields_ = [
        ("tokens", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("ids", ctypes.c_void_p),
        ("quantized", ctypes.c_void_p),
        ("coordinates", ctypes.c_void_p),
        ("exponents", ctypes.c_void_p),
        ("padding", ctypes.c_void_p),
        ("partial", ctypes.c_void_p),
        ("energies", ctypes.c_void_p),
        ("variances", ctypes.c_void_p),
    ]


E_STATIC_CAPACITY = -5
STATIC_PARTS_FLOATS = 1 << 20
STATIC_MAX_PAIRS = 1024


def screen_static():
    """The `cfm_screen_static` entry point, bound on first use."""
    function = load().cfm_screen_static
    function.restype = ctypes.c_int
    function.argtypes = [ctypes.POINTER(Layer), ctypes.POINTER(StaticScreen), ctypes.c_void_p]
    return function
