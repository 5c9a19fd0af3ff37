"""Reading and writing the safetensors container, by tensor name.

File layout: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`,
then the raw little-endian payload.  This replaces the reference's exporter and
byte-offset manifest (tools/dump_weights.py:31-66, src/include/qwen_loader.h:27-59):
tensors are found by name in the checkpoint itself.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` returns a CPU view of the payload."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._fh = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON ({exc})") from None
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + header_len
        payload = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}': {info!r}") from None
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * _itemsize(dtype) or begin < 0 or end > payload:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({info['dtype']}, shape {list(shape)}) has offsets "
                    f"[{begin}, {end}) that do not match its size or the payload of {payload} bytes (truncated file?)")
            self.entries[name] = (dtype, shape, begin, end)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._data_start + begin)
        return flat.view(shape)

    def close(self) -> None:
        # Views handed out keep the mapping alive; only the descriptor is closed here.
        self._fh.close()


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Writes CPU tensors under their names; dtypes are kept as given."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        ordered.append(t)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for t in ordered:
            if t.numel():
                fh.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
