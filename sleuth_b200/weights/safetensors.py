"""Reading and writing ``.safetensors`` files, and a checkpoint made of one or several of them.

File layout (sleuth/formats/safetensors.py:3-12): an unsigned 64-bit little-endian header length,
a UTF-8 JSON header ``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``
and the raw little-endian row-major bytes; offsets count from the start of the data section.

The reader maps the file and hands out tensors that view the mapping directly (no copy on the
host); the loader copies each one to the device while the mapping is open. A header that is too
long, a file that is too short, overlapping or out-of-range offsets, an unknown dtype or a byte count
that disagrees with the shape are refused (the checks of sleuth/formats/safetensors.py:87-107, plus
the overlap check).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path

import torch

DTYPE_OF = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
NAME_OF = {v: k for k, v in DTYPE_OF.items()}
HEADER_LIMIT = 100 << 20


class SafetensorsError(ValueError):
    pass


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def write_safetensors(tensors: dict[str, torch.Tensor], path, metadata: dict[str, str] | None = None) -> None:
    """Write ``tensors`` in the order given. The file appears under its name only when complete."""
    path = Path(path)
    header, offset, blobs = {}, 0, []
    for name, t in tensors.items():
        if t.dtype not in NAME_OF:
            raise TypeError(f"{name}: dtype {t.dtype} cannot be stored in safetensors")
        t = t.detach().cpu().contiguous()
        n = t.numel() * t.element_size()
        header[name] = {"dtype": NAME_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
        blobs.append(t)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    tmp = path.with_name(path.name + ".partial")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for t in blobs:
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)


class SafetensorsFile:
    """One mapped file. ``entries[name] = (dtype, shape, begin, end)`` with absolute byte offsets."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: {size} bytes is too small for a safetensors file")
        self._fh = open(self.path, "rb")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n > HEADER_LIMIT or 8 + n > size:
            self._fh.close()
            raise SafetensorsError(f"{self.path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            self._fh.close()
            raise SafetensorsError(f"{self.path}: the header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", None) or {}
        start = 8 + n
        self.entries: dict[str, tuple] = {}
        spans = []
        for name, info in header.items():
            code = info.get("dtype")
            if code not in DTYPE_OF:
                self._fh.close()
                raise SafetensorsError(f"{self.path}: tensor {name} has unsupported dtype {code!r}")
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(v) for v in info["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if b < 0 or e < b or e - b != count * _itemsize(DTYPE_OF[code]) or start + e > size:
                self._fh.close()
                raise SafetensorsError(f"{self.path}: tensor {name} {list(shape)} {code} has inconsistent "
                                       f"offsets [{b}, {e}) in a data section of {size - start} bytes")
            self.entries[name] = (DTYPE_OF[code], shape, start + b, start + e)
            if e > b:
                spans.append((b, e, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                self._fh.close()
                raise SafetensorsError(f"{self.path}: tensors {n0} and {n1} overlap")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > start else None

    def names(self) -> list[str]:
        return list(self.entries)

    def describe(self, name: str) -> tuple[torch.dtype, tuple]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as a read-only view of the mapping; valid until ``close``."""
        dtype, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # torch warns that the buffer is read-only; it is only read
            flat = torch.frombuffer(self._mm, dtype=torch.uint8, count=e - b, offset=b)
        return flat.view(dtype).reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass   # a view is still alive; the mapping goes when it does
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Every tensor of one file, copied out."""
    with SafetensorsFile(path) as f:
        return {k: f.tensor(k).clone() for k in f.names()}


class Checkpoint:
    """The tensors of a model folder by name: ``model.safetensors``, or the shards listed in
    ``model.safetensors.index.json``, or every ``*.safetensors`` in the folder
    (sleuth/formats/hf.py:54-67)."""

    def __init__(self, folder):
        folder = Path(folder)
        index = folder / "model.safetensors.index.json"
        weight_map = None
        if index.exists():
            weight_map = json.loads(index.read_text())["weight_map"]
            files = sorted(set(weight_map.values()))
        else:
            files = sorted(p.name for p in folder.glob("*.safetensors"))
        if not files:
            raise SafetensorsError(f"{folder}: no .safetensors file")
        self.files = {name: SafetensorsFile(folder / name) for name in files}
        self.where: dict[str, SafetensorsFile] = {}
        for fname, f in self.files.items():
            for k in f.names():
                if weight_map is None or weight_map.get(k) == fname:
                    self.where[k] = f

    def names(self) -> list[str]:
        return list(self.where)

    def describe(self, name: str):
        return self.where[name].describe(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
