"""Reading and writing the safetensors container, without any library for it.

Format (as read by spymaster2h/spyinfer src/utils/safetensors_reader.cpp:69-99): an
unsigned 64-bit little-endian header length, a JSON header ``{name: {"dtype", "shape",
"data_offsets": [begin, end]}}`` (``__metadata__`` is skipped), then the raw data.  A model
folder holds ``model.safetensors``, or shards listed in ``model.safetensors.index.json``
under ``weight_map`` (:15-43).  Unlike the reference, the end offset is checked against
shape and dtype, and a truncated file is an error that names the tensor.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One file, memory-mapped (private, copy-on-write: the file is never written);
    ``tensor(name)`` is a CPU view into the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file's {size} bytes (truncated file?)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        header.pop("__metadata__", None)
        self.entries: Dict[str, dict] = header
        self._data_start = 8 + n
        self._size = size
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None
        problems = []
        for name, e in header.items():
            dt = e.get("dtype")
            if dt not in _DTYPES:
                problems.append(f"{name}: dtype {dt!r} is not supported (supported: {', '.join(_DTYPES)})")
                continue
            numel = 1
            for d in e["shape"]:
                numel *= int(d)
            begin, end = e["data_offsets"]
            if end - begin != numel * _DTYPES[dt][1]:
                problems.append(f"{name}: data_offsets span {end - begin} bytes, shape {e['shape']} of {dt} needs {numel * _DTYPES[dt][1]}")
            elif self._data_start + end > size:
                problems.append(f"{name}: data ends at byte {self._data_start + end}, the file has {size} (truncated file?)")
        if problems:
            raise SafetensorsError(f"{path}: " + "; ".join(problems))

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(int(d) for d in self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dtype = _DTYPES[e["dtype"]][0]
        begin, end = e["data_offsets"]
        shape = self.shape(name)
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        return torch.frombuffer(buf, dtype=dtype).reshape(shape)

    def close(self):
        # tensors handed out may still view the map; let the garbage collector release it
        self._f.close()


def shard_paths(model_dir: str) -> List[str]:
    """The files of a model folder: the shards an index names (sorted, unique), else ``model.safetensors``."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            weight_map = json.load(f).get("weight_map", {})
        return [os.path.join(model_dir, p) for p in sorted(set(weight_map.values()))]
    single = os.path.join(model_dir, "model.safetensors")
    if not os.path.isfile(single):
        raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")
    return [single]


def write_safetensors(path: str, layout: List[Tuple[str, torch.dtype, Tuple[int, ...]]],
                      tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writes a file whose header is fixed by ``layout`` (name, dtype, shape, in file order)
    and whose data comes from ``tensors``, an iterable that yields the same names in the same
    order, so that a model larger than host memory can be streamed."""
    header, offset = {}, 0
    for name, dtype, shape in layout:
        if dtype not in _NAMES:
            raise SafetensorsError(f"{name}: cannot store dtype {dtype}")
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(d) for d in shape], "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        expected = iter(layout)
        for name, t in tensors:
            want = next(expected, None)
            if want is None or want[0] != name or tuple(t.shape) != tuple(want[2]) or t.dtype != want[1]:
                raise SafetensorsError(f"write_safetensors: got {name} {tuple(t.shape)} {t.dtype}, the layout expects {want}")
            t = t.detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
        if next(expected, None) is not None:
            raise SafetensorsError("write_safetensors: fewer tensors than the layout names")
