"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header (name -> dtype, shape, data_offsets), then the raw little-endian tensor bytes.

Tensors are read through a memory map, so a file is paged in as its tensors are copied to the
device and is never held twice on the host.  The reference does not read weight files: it takes a
``state_dict`` from a downloaded library model (src/utils/load_model.py:10-18).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Iterator

import numpy as np
import torch

# safetensors dtype tag -> (numpy dtype that has the same bytes, torch dtype to view them as)
_READ = {
    "F64": (np.float64, torch.float64), "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16), "BF16": (np.uint16, torch.bfloat16),
    "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8), "BOOL": (np.bool_, torch.bool),
}
_WRITE = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
    torch.uint8: "U8", torch.bool: "BOOL",
}


class SafetensorsFile:
    """One open .safetensors file: names, shapes and lazily mapped tensors."""

    def __init__(self, path: str) -> None:
        self.path = path
        self._handle = open(path, "rb")
        size = os.fstat(self._handle.fileno()).st_size
        head = self._handle.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its header length)")
        (header_len,) = struct.unpack("<Q", head)
        if header_len <= 0 or 8 + header_len > size:
            raise ValueError(f"{path}: not a safetensors file (header length {header_len})")
        header = json.loads(self._handle.read(header_len).decode("utf-8"))
        header.pop("__metadata__", None)
        self._data_start = 8 + header_len
        self._entries: dict[str, dict] = header
        for name, entry in header.items():
            if entry["dtype"] not in _READ:
                raise ValueError(f"{path}: tensor '{name}' has unsupported dtype {entry['dtype']}")
            begin, end = entry["data_offsets"]
            if not 0 <= begin <= end <= size - self._data_start:
                raise ValueError(f"{path}: tensor '{name}' lies outside the file")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self._entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _READ[self._entries[name]["dtype"]][1]

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as a read-only view of the mapped file (copy it before changing it)."""
        entry = self._entries[name]
        np_dtype, torch_dtype = _READ[entry["dtype"]]
        begin, end = entry["data_offsets"]
        shape = tuple(entry["shape"])
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if (end - begin) != count * np.dtype(np_dtype).itemsize:
            raise ValueError(f"{self.path}: tensor '{name}' has {end - begin} bytes, "
                             f"its shape {shape} needs {count * np.dtype(np_dtype).itemsize}")
        array = np.frombuffer(self._map, dtype=np_dtype, count=count,
                              offset=self._data_start + begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the map is read-only, by intent
            tensor = torch.from_numpy(array) if count else torch.empty(0)
        if torch_dtype == torch.bfloat16:
            tensor = tensor.view(torch.bfloat16)
        return tensor.reshape(shape)

    def close(self) -> None:
        # tensors handed out keep the map alive; only the handle is closed here
        self._handle.close()


def save_tensors(path: str, tensors: dict[str, torch.Tensor]) -> None:
    """Write tensors in the given order, each aligned to 8 bytes."""
    header: dict[str, dict] = {}
    offset = 0
    blobs: list[bytes | memoryview] = []
    for name, tensor in tensors.items():
        if tensor.dtype not in _WRITE:
            raise ValueError(f"tensor '{name}': dtype {tensor.dtype} cannot be stored")
        t = tensor.detach().to("cpu").contiguous()
        raw = t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()
        data = raw.tobytes()
        header[name] = {"dtype": _WRITE[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + len(data)]}
        blobs.append(data)
        offset += len(data)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for data in blobs:
            handle.write(data)
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> Iterator[SafetensorsFile]:
    """model.safetensors, or the shards that model.safetensors.index.json names."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        yield SafetensorsFile(single)
        return
    if os.path.isfile(index):
        with open(index) as handle:
            shards = sorted(set(json.load(handle)["weight_map"].values()))
        for shard in shards:
            yield SafetensorsFile(os.path.join(model_dir, shard))
        return
    raise FileNotFoundError(f"{model_dir}: neither model.safetensors nor "
                            f"model.safetensors.index.json found")
