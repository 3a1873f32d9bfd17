"""Reader and writer for the safetensors container (one JSON header, raw tensors).

File layout: an unsigned 64-bit little-endian header length ``n``, ``n`` bytes of
JSON mapping each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the first byte after the header), then the data. The reference's
precedent for reading a model folder of ``config.json`` plus ``*.safetensors`` is
python/instinct/backends/base.py:124-156.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

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
_NAMES = {dtype: name for name, dtype in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read on demand."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._file = open(self.path, "rb")
        try:
            size = self.path.stat().st_size
            if size < 8:
                raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
            (header_len,) = struct.unpack("<Q", self._file.read(8))
            if header_len > size - 8:
                raise SafetensorsError(f"{self.path}: header length exceeds the file")
            try:
                header = json.loads(self._file.read(header_len))
            except (json.JSONDecodeError, UnicodeDecodeError) as exc:
                raise SafetensorsError(f"{self.path}: header is not JSON: {exc}") from exc
            if not isinstance(header, dict):
                raise SafetensorsError(f"{self.path}: header is not a JSON object")
            self._data_start = 8 + header_len
            self.metadata = header.pop("__metadata__", {}) or {}
            self.tensors: dict[str, TensorInfo] = {}
            for name, entry in header.items():
                if not isinstance(entry, dict):
                    raise SafetensorsError(f"{self.path}: the entry of tensor '{name}' is not an object")
                dtype = _DTYPES.get(entry.get("dtype"))
                if dtype is None:
                    raise SafetensorsError(
                        f"{self.path}: tensor '{name}' has unsupported dtype {entry.get('dtype')!r}"
                    )
                try:
                    shape = tuple(int(s) for s in entry["shape"])
                    begin, end = (int(v) for v in entry["data_offsets"])
                except (KeyError, TypeError, ValueError) as exc:
                    raise SafetensorsError(f"{self.path}: tensor '{name}' has no usable shape and data_offsets") from exc
                if any(s < 0 for s in shape):
                    raise SafetensorsError(f"{self.path}: tensor '{name}' has a negative size")
                count = 1
                for s in shape:
                    count *= s
                if end - begin != count * dtype.itemsize or begin < 0:
                    raise SafetensorsError(f"{self.path}: tensor '{name}' has a bad byte range")
                if self._data_start + end > size:
                    raise SafetensorsError(f"{self.path}: tensor '{name}' runs past the file")
                self.tensors[name] = TensorInfo(name, dtype, shape, begin, end)
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        except Exception:
            self._file.close()
            raise

    def read(self, name: str) -> torch.Tensor:
        """A private copy of one tensor, on the CPU, in its stored dtype."""
        info = self.tensors[name]
        count = 1
        for s in info.shape:
            count *= s
        if count == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        raw = self._map[self._data_start + info.begin : self._data_start + info.end]
        flat = torch.frombuffer(bytearray(raw), dtype=info.dtype, count=count)
        return flat.reshape(info.shape)

    def close(self) -> None:
        if getattr(self, "_map", None) is not None:
            self._map.close()
            self._map = None
        self._file.close()

    def __enter__(self) -> "SafetensorsFile":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()


def write_safetensors(
    path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None
) -> None:
    """Write ``tensors`` in name order, back to back; the data section starts 8-byte aligned."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has unsupported dtype {tensor.dtype}")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(blob)))
        out.write(blob)
        for name in order:
            tensor = tensors[name].detach().cpu().contiguous()
            if tensor.numel():
                out.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
