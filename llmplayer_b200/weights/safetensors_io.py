"""Reading and writing the safetensors container.

Layout of a file: an unsigned 64-bit little-endian header length, a JSON header
mapping each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header), then the raw little-endian data.
The reference reads GGUF through a memory map (model/ModelLoader.java:79-124);
this reader maps the file the same way and hands out tensors by name.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch

from ..errors import WeightError

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "F64": (torch.float64, 8),
    "U8": (torch.uint8, 1),
    "I8": (torch.int8, 1),
    "I16": (torch.int16, 2),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """One mapped safetensors file; tensors are views of the map until cloned."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._fh = open(path, "rb")
        except OSError as exc:
            raise WeightError(f"cannot open {path}: {exc}") from None
        if size < 8:
            raise WeightError(f"{path}: truncated file ({size} bytes, no header length)")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise WeightError(f"{path}: header length {hlen} does not fit the file of {size} bytes")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightError(f"{path}: header is not JSON ({exc})") from None
        if not isinstance(header, dict):
            raise WeightError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        data_size = size - self._base
        for name, info in header.items():
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise WeightError(f"{path}: malformed header entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise WeightError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
            count = 1
            for s in shape:
                count *= s
            if begin < 0 or end < begin or end > data_size:
                raise WeightError(
                    f"{path}: tensor {name!r} spans bytes [{begin}, {end}) outside the data of {data_size} bytes "
                    "(truncated file?)")
            if end - begin != count * _DTYPES[dtype][1]:
                raise WeightError(
                    f"{path}: tensor {name!r} of shape {list(shape)} and dtype {dtype} needs "
                    f"{count * _DTYPES[dtype][1]} bytes, header gives {end - begin}")
            self._entries[name] = (dtype, shape, begin, end)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def keys(self) -> Iterable[str]:
        return self._entries.keys()

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        dtype, shape, _, _ = self._entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A copy of the named tensor in its stored dtype, on the host."""
        dtype, shape, begin, end = self._entries[name]
        tdtype = _DTYPES[dtype][0]
        if end == begin:
            return torch.empty(shape, dtype=tdtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin, offset=self._base + begin)
        flat = torch.from_numpy(raw.copy())
        del raw
        return flat.view(tdtype).reshape(shape)

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass
            self._map = None
        self._fh.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, tensor in tensors.items():
        t = tensor.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * ((8 - len(head) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(head)))
        fh.write(head)
        for raw in blobs:
            fh.write(raw)
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> Dict[str, SafetensorsFile]:
    """Open ``model.safetensors``, or the shards an index file names.

    Returns a map from tensor name to the file that holds it.
    """
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    owners: Dict[str, SafetensorsFile] = {}
    if os.path.exists(single):
        handle = SafetensorsFile(single)
        for name in handle.keys():
            owners[name] = handle
        return owners
    if os.path.exists(index):
        try:
            with open(index, "r", encoding="utf-8") as fh:
                weight_map = json.load(fh)["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as exc:
            raise WeightError(f"{index}: malformed index ({exc})") from None
        handles: Dict[str, SafetensorsFile] = {}
        for shard in sorted(set(weight_map.values())):
            handles[shard] = SafetensorsFile(os.path.join(model_dir, shard))
        for shard, handle in handles.items():
            for name in handle.keys():
                if name in owners:
                    raise WeightError(f"tensor {name!r} appears in more than one shard of {model_dir}")
                owners[name] = handle
        return owners
    raise WeightError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir!r}")
