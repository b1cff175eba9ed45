"""Reading and writing the safetensors container, without the safetensors package.

The format: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [lo, hi]}, "__metadata__": {...}}`` and the
raw little-endian tensor bytes.  The reference reads the same files through
``safetensors.safe_open`` (src/qwen25vl_lite/model.py:312-348); reading them here keeps
the loader free of optional packages and lets it map the file once and hand out views.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch

_TO_TORCH = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


class SafetensorsFile:
    """One mapped file; ``tensor(name)`` returns a CPU tensor that views the mapping."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise ValueError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise ValueError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        header = json.loads(self._fh.read(hlen).decode("utf-8"))
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._entries: Dict[str, dict] = header
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        for name, meta in header.items():
            lo, hi = meta["data_offsets"]
            if meta["dtype"] not in _TO_TORCH:
                raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
            if not (0 <= lo <= hi and self._base + hi <= size):
                raise ValueError(f"{path}: tensor {name!r} lies outside the file")

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _TO_TORCH[self._entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        meta = self._entries[name]
        lo, hi = meta["data_offsets"]
        dtype = _TO_TORCH[meta["dtype"]]
        count = 1
        for s in meta["shape"]:
            count *= int(s)
        if count == 0:
            return torch.empty(tuple(meta["shape"]), dtype=dtype)
        if (hi - lo) != count * torch.empty((), dtype=dtype).element_size():
            raise ValueError(f"{self.path}: tensor {name!r} has {hi - lo} bytes for shape {meta['shape']}")
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # the mapping is read-only; the views are only read from
            flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + lo)
        return flat.reshape(tuple(meta["shape"]))


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The shards an index names, else ``model.safetensors`` (model.py:312-327)."""
    index_path = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index_path):
        with open(index_path, "r", encoding="utf-8") as fh:
            shards = sorted(set(json.load(fh)["weight_map"].values()))
    elif os.path.isfile(os.path.join(model_dir, "model.safetensors")):
        shards = ["model.safetensors"]
    else:
        raise FileNotFoundError(
            f"no safetensors weights under {model_dir!r}: expected model.safetensors or model.safetensors.index.json")
    return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None) -> None:
    """Writes ``(name, tensor)`` pairs in the order given.  The tensors are taken one at a
    time, so a generator keeps the peak at one tensor."""
    pairs = []
    header: Dict[str, dict] = {}
    offset = 0
    tmp_path = path + ".data.tmp"
    with open(tmp_path, "wb") as data:
        for name, t in tensors:
            t = t.detach().to("cpu").contiguous()
            if t.dtype not in _FROM_TORCH:
                raise ValueError(f"cannot store dtype {t.dtype} ({name})")
            raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
            header[name] = {"dtype": _FROM_TORCH[t.dtype], "shape": list(t.shape),
                            "data_offsets": [offset, offset + len(raw)]}
            data.write(raw)
            offset += len(raw)
            pairs.append(name)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as out, open(tmp_path, "rb") as data:
        out.write(struct.pack("<Q", len(blob)))
        out.write(blob)
        while True:
            chunk = data.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    os.remove(tmp_path)
