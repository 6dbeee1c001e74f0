"""Reader of GGUF version 3 files, the container the reference's hybrid path loads quantized tensors from
(crates/stark-engine/src/engine/hybrid/weights.rs:2770-2866): magic ``GGUF``, version 3, tensor and
metadata counts, typed key/value metadata, then per tensor its name, rank (1..4), dimensions (fastest
first in the file; reversed here, as the reference does, so that ``shape[0]`` is the slowest), ggml
type and data offset; tensor data starts at the next multiple of ``general.alignment`` (default 32).
The same checks as the reference: version, alignment a power of two <= 4096, unknown types, empty
dimensions, sizes that overflow 64 bits, unaligned / truncated / overlapping / duplicate tensors; every
admitted block type is sized, whether or not this engine can multiply with it.

Tensors of the types this engine multiplies with go straight to the device:
``tensor.qmatrix()`` -> ``stark_b200.ops.QMatrix`` for Q8_0 (8) and Q4_K (12), two-dimensional or
``[experts, rows, columns]`` expert banks.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np


class GGUFError(ValueError):
    pass


F32, F16, Q8_0, Q4_K, BF16 = 0, 1, 8, 12, 30
# bytes per block, values per block for every ggml type the reference admits from a GGUF header
# (block_layout, weights.rs:2565-2584): a file may hold tensors this engine cannot multiply (Q6_K output
# heads beside Q4_K layers, for example); they are sized and span-checked like the rest and only
# qmatrix() / array() refuse them.
_BLOCKS = {F32: (4, 1), F16: (2, 1), BF16: (2, 1), Q8_0: (34, 32), 10: (84, 256), 11: (110, 256),
           Q4_K: (144, 256), 13: (176, 256), 14: (210, 256), 16: (66, 256), 17: (74, 256), 18: (98, 256),
           23: (136, 256)}
_ADMITTED = set(_BLOCKS)  # weights.rs:2811
_U64 = 1 << 64
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass
class GGUFTensor:
    name: str
    kind: int
    shape: tuple          # slowest dimension first
    data: np.ndarray      # uint8 view of the encoded bytes (memory-mapped)

    def qmatrix(self):
        from . import ops
        if self.kind not in (Q8_0, Q4_K) or len(self.shape) not in (2, 3):
            raise GGUFError(f"{self.name}: only 2-D or 3-D Q8_0 / Q4_K tensors become device matrices")
        experts = self.shape[0] if len(self.shape) == 3 else 1
        rows, columns = self.shape[-2], self.shape[-1]
        return ops.QMatrix.from_gguf(self.data.reshape(experts * rows, -1), self.kind, rows, columns, experts=experts)

    def array(self) -> np.ndarray:
        """Unquantized tensors as numpy (F32 as float32; F16 / BF16 as their 16-bit patterns)."""
        if self.kind == F32:
            return self.data.view(np.float32).reshape(self.shape)
        if self.kind in (F16, BF16):
            return self.data.view(np.uint16).reshape(self.shape)
        raise GGUFError(f"{self.name}: quantized tensor, use qmatrix()")


class _Reader:
    def __init__(self, buf: np.ndarray):
        self.buf, self.pos = buf, 0

    def take(self, n: int) -> bytes:
        if self.pos + n > self.buf.size:
            raise GGUFError("truncated GGUF header")
        out = self.buf[self.pos:self.pos + n].tobytes()
        self.pos += n
        return out

    def scalar(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.scalar("<Q")
        if n > 1 << 20:
            raise GGUFError("unreasonable GGUF string length")
        return self.take(n).decode("utf-8")

    def value(self, kind: int, depth: int = 0):
        if kind in _SCALARS:
            return self.scalar(_SCALARS[kind])
        if kind == 8:
            return self.string()
        if kind == 9 and depth == 0:
            elem, count = self.scalar("<I"), self.scalar("<Q")
            if count > 1 << 24:
                raise GGUFError("unreasonable GGUF array length")
            return [self.value(elem, 1) for _ in range(count)]
        raise GGUFError("unknown GGUF metadata type")


def element_count(dims) -> int:
    """Product of the dimensions with the reference's refusals (`product`, weights.rs:2556-2563)."""
    total = 1
    for d in dims:
        if d == 0:
            raise GGUFError("empty tensor dimension")
        total *= int(d)
        if total >= _U64:
            raise GGUFError("tensor size overflow")
    return total


def encoded_size(kind: int, count: int) -> int:
    if kind not in _BLOCKS:
        raise GGUFError("unsupported weight block format")
    nbytes, values = _BLOCKS[kind]
    if count % values:
        raise GGUFError("weight dimension is not block aligned")
    size = count // values * nbytes
    if size >= _U64:
        raise GGUFError("encoded weight size overflow")
    return size


def read_gguf(path) -> tuple[dict, dict]:
    """Returns ``(tensors by name, metadata)``; tensor bytes stay memory-mapped."""
    path = Path(path)
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    r = _Reader(buf)
    if r.take(4) != b"GGUF" or r.scalar("<I") != 3:
        raise GGUFError("GGUF version three is required")
    tensor_count, metadata_count = r.scalar("<Q"), r.scalar("<Q")
    if tensor_count > 1 << 20 or metadata_count > 1 << 20:
        raise GGUFError("unreasonable GGUF counts")
    metadata = {}
    for _ in range(metadata_count):
        name, kind = r.string(), r.scalar("<I")
        value = r.value(kind)
        if not name or name in metadata:
            raise GGUFError("duplicate GGUF metadata")
        metadata[name] = value
    alignment = metadata.get("general.alignment", 32)
    if not isinstance(alignment, int) or alignment <= 0 or alignment & (alignment - 1) or alignment > 4096:
        raise GGUFError("invalid GGUF alignment")
    infos = {}
    for _ in range(tensor_count):
        name, rank = r.string(), r.scalar("<I")
        if not name or not 1 <= rank <= 4:
            raise GGUFError("invalid GGUF tensor identity or rank")
        dims = [r.scalar("<Q") for _ in range(rank)]
        kind, offset = r.scalar("<I"), r.scalar("<Q")
        if kind not in _ADMITTED:
            raise GGUFError("unsupported GGUF tensor type")
        size = encoded_size(kind, element_count(dims))
        encoded_size(kind, dims[0])  # the fastest dimension holds whole blocks
        if offset % alignment:
            raise GGUFError("unaligned GGUF tensor")
        if name in infos:
            raise GGUFError("duplicate GGUF tensor")
        infos[name] = (kind, tuple(reversed(dims)), offset, size)
    start = (r.pos + alignment - 1) & ~(alignment - 1)
    if start > buf.size:
        raise GGUFError("truncated GGUF header")
    spans = sorted((start + off, start + off + size) for _, _, off, size in infos.values())
    end = start
    for lo, hi in spans:
        if lo >= _U64 or hi >= _U64:
            raise GGUFError("GGUF offset overflow")
        if hi > buf.size:
            raise GGUFError("truncated GGUF tensor")
        if lo < end:
            raise GGUFError("overlapping GGUF tensors")
        end = hi
    tensors = {name: GGUFTensor(name, kind, shape, buf[start + off:start + off + size])
               for name, (kind, shape, off, size) in infos.items()}
    return tensors, metadata
