"""Ternary sketch of the gate/up expert rows: rotation, construction, packing.

Host-side construction code (torch tensor ops, CPU or CUDA tensors); the decode
hot path reads the sketch through the CUDA kernels only.  Interface and values
follow the reference's `calibration_free_moe/reader/sketch.py`
(`block_hadamard_signs` :22, `rotate_blocks` :38, `mask_rotated_blocks` :53,
`require_sketch_acquisition` :71, `build_sketch` :84, `unpack_sketch` :209).

`rotate_blocks`, `mask_rotated_blocks` and `require_sketch_acquisition` restate the
reference's functions of the same names: the butterfly's stage order, the tie rule
of the mask (equal magnitudes keep the lower coordinate) and the acquisition tag
are the contract with banks and sketches built by the reference, so they leave
no freedom beyond naming.

Two storage layouts exist here:

* the reference layout, five trits per byte in coordinate-major 32-byte tiles,
  which is what `build_sketch` returns and `ProgressiveReader(sketch=...)`
  accepts; and
* the kernel layout made by `repack_sketch`, two bits per trit, sixteen rows
  per 32-bit word, `[E, H, 2 I / 16]` words coordinate-major, which is what the
  screening kernel streams from HBM.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from .budget import ROTATION_BLOCK, SECTOR, sketch_code_stride, sketch_storage_bytes

# Tag a fitted (nonzero) recovery bank must carry to be used with this sketch.
ACQUISITION = "ternary-hadamard-sketch-v1"
# Byte holding five zero trits: (0+1) * (1 + 3 + 9 + 27 + 81).
ZERO_BYTE = 121
# TWN threshold factor: a rotated coordinate is kept when |v| > 0.7 * mean|v|.
TWN_FACTOR = 0.7
# Rows (channels of one plane) per 32-bit word of the kernel layout.
WORD_ROWS = 16


def block_hadamard_signs(hidden: int, device: torch.device | str) -> Tensor:
    """Model-wide +-1 int8 signs of the rotation, drawn on the CPU with seed 0.

    Reference reader/sketch.py:22.  The draw happens on the CPU generator and is
    then moved, so every device sees the same signs.
    """
    if hidden % ROTATION_BLOCK:
        raise ValueError("Hadamard sketch requires hidden width divisible by 128")
    generator = torch.Generator().manual_seed(0)
    bits = torch.randint(0, 2, (hidden,), generator=generator)
    return (bits * 2 - 1).to(device=device, dtype=torch.int8)


def rotate_blocks(x: Tensor, signs: Tensor | None) -> Tensor:
    """FP32 blockdiag(H128)/sqrt(128) . diag(signs) applied to the last axis.

    Reference reader/sketch.py:38.  The butterfly order is part of the contract:
    seven stages with half-widths 1, 2, ..., 64, each replacing a (left, right)
    pair of width-w runs by (left + right, left - right), then one multiply by
    1/sqrt(128).  Only additions and subtractions precede that multiply, so the
    result is bit-reproducible on any IEEE device.
    """
    if signs is None:
        return x.float()
    blocks = signs.numel() // ROTATION_BLOCK
    v = x.float().reshape(-1, blocks, ROTATION_BLOCK)
    v = v * signs.float().reshape(1, blocks, ROTATION_BLOCK)
    half = 1
    while half < ROTATION_BLOCK:
        runs = v.reshape(-1, blocks, ROTATION_BLOCK // (2 * half), 2, half)
        left, right = runs[..., 0, :], runs[..., 1, :]
        v = torch.stack((left + right, left - right), dim=-2)
        v = v.reshape(-1, blocks, ROTATION_BLOCK)
        half *= 2
    return (v * (1 / math.sqrt(ROTATION_BLOCK))).reshape(x.shape)


def mask_rotated_blocks(x: Tensor, keep: int = ROTATION_BLOCK) -> Tensor:
    """Zero all but the `keep` largest |v| of every 128-block (reference :53).

    Ties at the cut are resolved towards the lower coordinate.
    """
    if keep == ROTATION_BLOCK:
        return x
    v = x.reshape(*x.shape[:-1], -1, ROTATION_BLOCK)
    with torch.no_grad():
        size = v.abs()
        cut = size.sort(dim=-1, descending=True).values[..., keep - 1 : keep]
        above = size > cut
        equal = size == cut
        room = keep - above.sum(dim=-1, keepdim=True)
        member = above | (equal & (equal.cumsum(dim=-1) <= room))
    return torch.where(member, v, 0.0).reshape_as(x)


def require_sketch_acquisition(bank: dict[str, object]) -> None:
    """Reject a nonzero recovery bank fitted for another acquisition rule (reference :71)."""
    decoder, encoder = bank["decoder"], bank["encoder"]
    if not isinstance(decoder, Tensor) or not isinstance(encoder, Tensor):
        raise TypeError("Recovery bank parameters must be tensors")
    nonzero = bool(torch.count_nonzero(decoder)) or bool(torch.count_nonzero(encoder))
    if nonzero:
        plan = bank.get("plan")
        if not isinstance(plan, dict) or plan.get("acquisition") != ACQUISITION:
            raise ValueError(
                f"Nonzero recovery bank requires {ACQUISITION} acquisition"
            )


def _code_offsets(rows: int, hidden: int, device: torch.device) -> Tensor:
    """Byte offset of (rotated coordinate h, code byte j) inside one expert's codes.

    j = 2 * (channel // 5) + plane.  Bytes below `body` (the whole 32-byte tiles
    of the stride) lie coordinate-major at h * body + j; the 16-byte remainder,
    when the stride has one, lies after all bodies, with the remainders of
    blocks 2m and 2m + 1 interleaved per coordinate in one 32-byte sector.
    Returns int64 [hidden, stride].
    """
    stride = sketch_code_stride(rows)
    blocks = hidden // ROTATION_BLOCK
    body, tail = stride // SECTOR * SECTOR, stride % SECTOR
    h = torch.arange(hidden, device=device, dtype=torch.int64)[:, None]
    j = torch.arange(stride, device=device, dtype=torch.int64)[None, :]
    offsets = h * body + j
    if tail:
        block, lane = h // ROTATION_BLOCK, h % ROTATION_BLOCK
        sector = (block // 2) * ROTATION_BLOCK + lane
        in_tail = blocks * ROTATION_BLOCK * body + sector * SECTOR
        in_tail = in_tail + (block % 2) * tail + (j - body)
        offsets = torch.where(j < body, offsets, in_tail)
    return offsets


def build_sketch(weights: Tensor, signs: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """Build the sketch of native gate/up rows `[E, 2 I, H]` (reference :84).

    Per expert, row and rotated 128-block: a coordinate keeps its sign when
    |v| > 0.7 * mean|v| (ternary weight network rule); the block scale is the
    mean magnitude of the kept coordinates (over max(count, 1)); the residual
    variance is mean((v - sign * scale)^2).  Returns

    * codes  uint8 `[E, sketch_storage_bytes(2 I, H)]`, reference layout: per
      coordinate, byte 2g + p packs trits+1 of channels 5g..5g+4 of plane p
      (0 gate, 1 up) with weights 1, 3, 9, 27, 81; unused positions are 121;
    * statistics float16, logical `[E, 2 I, B, 2]` (scale, residual variance)
      over physical `[E, B, 2, 2 I]`.

    One expert at a time, so the FP32 copy stays transient.
    """
    experts, rows, hidden = weights.shape
    if hidden % ROTATION_BLOCK or rows % 2:
        raise ValueError(
            "Ternary sketch requires 128-coordinate blocks and paired gate/up rows"
        )
    device = weights.device
    blocks, width = hidden // ROTATION_BLOCK, rows // 2
    stride = sketch_code_stride(rows)
    groups = (width + 4) // 5
    codes = torch.full(
        (experts, sketch_storage_bytes(rows, hidden)),
        ZERO_BYTE,
        device=device,
        dtype=torch.uint8,
    )
    physical = torch.empty((experts, blocks, 2, rows), device=device, dtype=torch.float16)
    statistics = physical.permute(0, 3, 1, 2)
    offsets = _code_offsets(rows, hidden, device)[:, : 2 * groups].reshape(-1)
    place = torch.tensor([1, 3, 9, 27, 81], device=device, dtype=torch.int16)
    for expert in range(experts):
        v = weights[expert].float().reshape(rows, blocks, ROTATION_BLOCK)
        if signs is not None:
            v = rotate_blocks(v, signs)
        size = v.abs()
        member = size > TWN_FACTOR * size.mean(dim=-1, keepdim=True)
        scale = (size * member).sum(-1) / member.sum(-1).clamp_min(1)
        ternary = torch.where(member, v.sign(), 0)
        residual = (v - ternary * scale.unsqueeze(-1)).square().mean(-1)
        # digits[h, plane, channel] in {0, 1, 2}, padded to whole groups of five.
        digits = (ternary.to(torch.int16) + 1).reshape(2, width, hidden).permute(2, 0, 1)
        if groups * 5 != width:
            digits = torch.nn.functional.pad(digits, (0, groups * 5 - width), value=1)
        packed = (digits.reshape(hidden, 2, groups, 5) * place).sum(-1)
        # byte order per coordinate: (group 0 gate, group 0 up, group 1 gate, ...)
        packed = packed.permute(0, 2, 1).reshape(-1).to(torch.uint8)
        codes[expert, offsets] = packed
        statistics[expert] = torch.stack((scale, residual), dim=-1).to(torch.float16)
    return codes, statistics


def unpack_sketch(codes: Tensor, rows: int, hidden: int) -> Tensor:
    """Decode reference-layout codes into int8 trits `[..., rows, hidden]` (reference :209)."""
    width = rows // 2
    offsets = _code_offsets(rows, hidden, codes.device)
    row = torch.arange(rows, device=codes.device, dtype=torch.int64)
    channel, plane = row % width, row // width
    byte = 2 * (channel // 5) + plane
    digit = 3 ** (channel % 5)
    gathered = codes[..., offsets[:, byte]].to(torch.int32)  # [..., hidden, rows]
    trits = (gathered // digit) % 3 - 1
    return trits.transpose(-1, -2).to(torch.int8)


def kernel_words(rows: int) -> int:
    """32-bit words per rotated coordinate in the kernel layout."""
    return rows // WORD_ROWS


def repack_sketch(codes: Tensor, rows: int, hidden: int) -> Tensor:
    """Re-lay reference codes as the 2-bit kernel layout, int32 `[E, H, rows/16]`.

    Word w of coordinate h holds rows 16 w .. 16 w + 15 (gate rows first, then
    up rows); bits [2 j, 2 j + 1] hold trit + 1 of row 16 w + j.  Each
    coordinate's words are one contiguous run, so a kept coordinate is one
    coalesced read of rows / 4 bytes.  One expert at a time.
    """
    if rows % (2 * WORD_ROWS):
        raise ValueError("Kernel sketch layout needs expert width divisible by 16")
    experts = codes.shape[0]
    words = kernel_words(rows)
    out = torch.empty((experts, hidden, words), device=codes.device, dtype=torch.int32)
    shifts = (2 * torch.arange(WORD_ROWS, device=codes.device, dtype=torch.int64))
    for expert in range(experts):
        digits = unpack_sketch(codes[expert], rows, hidden).to(torch.int64) + 1
        grouped = digits.transpose(0, 1).reshape(hidden, words, WORD_ROWS)
        word = (grouped << shifts).sum(-1)  # < 2**32, held in int64
        out[expert] = torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)
    return out


# Bit position of coordinate c (0..15) inside a word of the grouped layout: four
# masked shifts of the word then give the byte-permute selectors of coordinates
# 0-3, 4-7, 8-11 and 12-15.
GROUPED_BIT = tuple(
    4 * c if c < 4 else 4 * (c - 4) + 2 if c < 8 else 16 + 4 * (c - 8) if c < 12 else 18 + 4 * (c - 12)
    for c in range(16)
)


def repack_sketch_grouped(codes: Tensor, rows: int, hidden: int) -> Tensor:
    """Re-lay reference codes row-major for the expert-major screen, int32 `[E, B, rows, 8]`.

    Word w of (block b, row r) holds coordinates 16 w .. 16 w + 15 of that block,
    trit + 1 in two bits at the positions of `GROUPED_BIT`.  A row's 128
    coordinates of one block are 32 contiguous bytes and consecutive rows follow
    each other, so a warp reading 16 rows reads 512 contiguous bytes.
    """
    experts = codes.shape[0]
    blocks = hidden // ROTATION_BLOCK
    out = torch.empty((experts, blocks, rows, 8), device=codes.device, dtype=torch.int32)
    shifts = torch.tensor(GROUPED_BIT, device=codes.device, dtype=torch.int64)
    for expert in range(experts):
        digits = unpack_sketch(codes[expert], rows, hidden).to(torch.int64) + 1  # [rows, H]
        grouped = digits.reshape(rows, blocks, 8, 16).permute(1, 0, 2, 3)
        word = (grouped << shifts).sum(-1)
        out[expert] = torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)
    return out


def build_sketch_on_device(weights: Tensor, signs: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    """The sketch of CUDA gate/up rows `[E, 2 I, H]`, built by the library's kernel.

    Returns `(words, grouped_words, statistics)`: the two kernel layouts
    (`repack_sketch` and `repack_sketch_grouped` of the reference-layout codes) and
    the FP16 statistics (logical `[E, 2 I, B, 2]` over physical `[E, B, 2, 2 I]`),
    without the reference-layout codes in between: one pass over the weights, a
    few milliseconds per layer instead of seconds.  Rotation and rule are those of
    `build_sketch`; the block sums are added in another order, so single
    coordinates within rounding of the threshold may differ from it
    (`codes_from_words` gives the reference-layout codes of the result).
    """
    import ctypes

    from .. import _native

    experts, rows, hidden = weights.shape
    if (not weights.is_cuda or weights.dtype != torch.bfloat16 or not weights.is_contiguous()
            or hidden % ROTATION_BLOCK or rows % (2 * WORD_ROWS)):
        raise ValueError("Expected contiguous CUDA BF16 gate/up rows [E, 2I, H], H % 128 == 0, I % 16 == 0")
    device = weights.device
    blocks = hidden // ROTATION_BLOCK
    words = torch.empty((experts, hidden, rows // WORD_ROWS), device=device, dtype=torch.int32)
    grouped = torch.empty((experts, blocks, rows, 8), device=device, dtype=torch.int32)
    physical = torch.empty((experts, blocks, 2, rows), device=device, dtype=torch.float16)
    layer = _native.Layer()
    layer.hidden, layer.width, layer.experts = hidden, rows // 2, experts
    signs = signs.to(device=device, dtype=torch.int8).contiguous()
    with torch.cuda.device(device):
        code = _native.load().cfm_build_sketch(
            ctypes.byref(layer), weights.data_ptr(), signs.data_ptr(), words.data_ptr(),
            grouped.data_ptr(), physical.data_ptr(),
            ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream),
        )
    _native.check(code, "cfm_build_sketch")
    return words, grouped, physical.permute(0, 3, 1, 2)


def codes_from_words(words: Tensor, rows: int, hidden: int) -> Tensor:
    """Reference-layout codes (as `build_sketch` returns them) of a coordinate-major sketch.

    `words` int32 `[E, H, rows / 16]`.  One expert at a time.
    """
    experts = words.shape[0]
    width = rows // 2
    groups = (width + 4) // 5
    device = words.device
    codes = torch.full((experts, sketch_storage_bytes(rows, hidden)), ZERO_BYTE, device=device,
                       dtype=torch.uint8)
    offsets = _code_offsets(rows, hidden, device)[:, : 2 * groups].reshape(-1)
    place = torch.tensor([1, 3, 9, 27, 81], device=device, dtype=torch.int16)
    shifts = 2 * torch.arange(WORD_ROWS, device=device, dtype=torch.int64)
    for expert in range(experts):
        unsigned = words[expert].to(torch.int64) & 0xFFFFFFFF
        digits = ((unsigned.unsqueeze(-1) >> shifts) & 3).reshape(hidden, rows).to(torch.int16)
        digits = digits.reshape(hidden, 2, width)
        if groups * 5 != width:
            digits = torch.nn.functional.pad(digits, (0, groups * 5 - width), value=1)
        packed = (digits.reshape(hidden, 2, groups, 5) * place).sum(-1)
        codes[expert, offsets] = packed.permute(0, 2, 1).reshape(-1).to(torch.uint8)
    return codes
