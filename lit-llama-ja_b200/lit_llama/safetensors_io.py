"""Reader and writer for the safetensors container, standard library + torch only.

Layout of a file: an 8-byte little-endian length n, n bytes of JSON mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header; the
optional ``"__metadata__"`` entry is skipped), then the tensors' bytes.  The reader maps the file and
hands out tensors one by one, so that a checkpoint streams disk -> host -> HBM without a second copy of
the whole file in memory (the streaming idea of ``checkpoint_stream.py``, for this container).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """``with SafetensorsFile(path) as f: f.shape(name); f.get(name)``.  ``get`` returns a CPU tensor that owns its memory."""

    def __init__(self, path):
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        head = self._fh.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if n > size - 8:
            raise ValueError(f"{self.path}: header length {n} exceeds the file")
        self.entries: Dict[str, dict] = {k: v for k, v in json.loads(self._fh.read(n)).items() if k != "__metadata__"}
        self._base = 8 + n
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, e in self.entries.items():
            lo, hi = e["data_offsets"]
            if e["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {e['dtype']}")
            count = 1
            for d in e["shape"]:
                count *= d
            if hi - lo != count * torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size() or self._base + hi > size:
                raise ValueError(f"{self.path}: tensor {name!r} does not fit its byte range")

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {k: tuple(v["shape"]) for k, v in self.entries.items()}

    def get(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        lo, hi = e["data_offsets"]
        dtype = _DTYPES[e["dtype"]]
        if hi == lo:
            return torch.empty(e["shape"], dtype=dtype)
        raw = bytearray(self._map[self._base + lo:self._base + hi])      # little-endian on disk = host order on x86 / arm64
        return torch.frombuffer(raw, dtype=dtype).reshape(e["shape"])


def save_safetensors(tensors: Dict[str, torch.Tensor], path) -> None:
    """Write ``tensors`` (any device) in the container's layout, data in the order given."""
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    js = json.dumps(header, separators=(",", ":")).encode()
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)
