"""Reading and writing safetensors files by tensor name.

The file format: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype": "BF16"|"F32"|..., "shape": [...], "data_offsets": [begin, end]}}`
(offsets relative to the byte after the header), then the raw little-endian data.
The reference reads every `*.safetensors` of a folder into one dict through the
safetensors package (engine/models/_loader.py:64-76); this reader memory-maps the
files and hands out tensors one name at a time, so a large model is never held
twice in host memory.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Iterable

import torch

_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(RuntimeError):
    pass


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._file = open(self.path, "rb")
        head = self._file.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        (header_len,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{self.path}: header length {header_len} exceeds file size {size}")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from e
        header.pop("__metadata__", None)
        self.entries: dict[str, dict] = header
        self._data_start = 8 + header_len
        self._mmap = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        for name, entry in self.entries.items():
            begin, end = entry["data_offsets"]
            if entry["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name} has unknown dtype {entry['dtype']}")
            numel = 1
            for s in entry["shape"]:
                numel *= s
            itemsize = torch.empty((), dtype=_DTYPES[entry["dtype"]]).element_size()
            if end - begin != numel * itemsize or self._data_start + end > size:
                raise SafetensorsError(f"{self.path}: tensor {name} has inconsistent offsets")

    def keys(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that views the mapped file (read-only; copy before writing)."""
        entry = self.entries[name]
        begin, end = entry["data_offsets"]
        dtype = _DTYPES[entry["dtype"]]
        shape = tuple(entry["shape"])
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._mmap)[self._data_start + begin : self._data_start + end]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(view, dtype=dtype)
        return flat.reshape(shape)

    def close(self) -> None:
        try:
            self._mmap.close()
        except (BufferError, ValueError):
            pass  # tensors still view the map; it goes when they do
        self._file.close()


class SafetensorsFolder:
    """All `*.safetensors` files of a model folder as one name -> tensor table."""

    def __init__(self, folder: str | Path) -> None:
        self.folder = Path(folder)
        if not self.folder.is_dir():
            raise FileNotFoundError(f"Model folder does not exist: {self.folder}")
        paths = sorted(self.folder.glob("*.safetensors"))
        if not paths:
            raise SafetensorsError(f"No safetensors files found at {self.folder}.")
        self.files = [SafetensorsFile(p) for p in paths]
        self._where: dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.keys():
                if name in self._where:
                    raise SafetensorsError(
                        f"tensor {name} appears in both {self._where[name].path.name} and {f.path.name}"
                    )
                self._where[name] = f

    def keys(self) -> list[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def save_safetensors(path: str | Path, tensors: Iterable[tuple[str, torch.Tensor]]) -> None:
    """Writes tensors (host, any of the known dtypes) in the given order."""
    items = [(name, t.detach().cpu().contiguous()) for name, t in tensors]
    header: dict[str, dict] = {}
    offset = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
