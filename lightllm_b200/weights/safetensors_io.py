"""Reading and writing the safetensors container: ``[u64 LE header length][JSON header][data]``.

Format as the reference parses it (src/model/model_loader.cpp:48-122): the JSON maps a
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` relative to the
first byte after the header; ``__metadata__`` is skipped.  Unlike the reference's
helpers, which assume BF16 on disk whatever the header says
(src/engine/engine_server.cpp:291-310), tensors are converted by the header's dtype.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# header name -> (numpy dtype used to view the bytes, torch dtype of the result)
_DTYPES = {
    "F64": (np.float64, torch.float64),
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_TORCH_TO_NAME = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
    torch.uint8: "U8", torch.bool: "BOOL",
}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str                 # header spelling: F32, BF16, ...
    shape: Tuple[int, ...]
    begin: int                 # byte offsets inside the data section
    end: int
    file: str

    @property
    def is_float(self) -> bool:
        return self.dtype in ("F64", "F32", "F16", "BF16")

    @property
    def is_32bit_float(self) -> bool:
        return self.dtype in ("F32", "F64")


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are read on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: invalid safetensors header (file of {size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: invalid safetensors header length {hlen}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: invalid safetensors header: {e}") from None
        self._data_offset = 8 + hlen
        self._data_size = size - self._data_offset
        self.metadata = header.pop("__metadata__", None) or {}
        self.tensors: Dict[str, TensorInfo] = {}
        for name, rec in header.items():
            dtype = rec.get("dtype")
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: unknown safetensors dtype {dtype!r} for tensor {name!r}")
            shape = tuple(int(s) for s in rec["shape"])
            begin, end = (int(x) for x in rec["data_offsets"])
            nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(_DTYPES[dtype][0]).itemsize
            if end - begin != nbytes or begin < 0 or end > self._data_size:
                raise SafetensorsError(
                    f"{path}: byte size mismatch for {name!r}: offsets [{begin},{end}) vs {nbytes} bytes "
                    f"for {dtype}{list(shape)}")
            self.tensors[name] = TensorInfo(name, dtype, shape, begin, end, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.tensors)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU torch tensor of its stored dtype (a private copy)."""
        info = self.tensors.get(name)
        if info is None:
            raise SafetensorsError(f"tensor not found: {name}")
        np_dtype, torch_dtype = _DTYPES[info.dtype]
        count = int(np.prod(info.shape, dtype=np.int64))
        arr = np.frombuffer(self._mm, dtype=np_dtype, count=count, offset=self._data_offset + info.begin)
        arr = np.array(arr, copy=True).reshape(info.shape)
        t = torch.from_numpy(arr)
        if info.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


class Checkpoint:
    """All tensors of a model folder: ``model.safetensors`` (src/engine/engine_server.cpp:402),
    or the shards that ``model.safetensors.index.json`` names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self.files: List[SafetensorsFile] = []
        if os.path.isfile(single):
            self.files.append(SafetensorsFile(single))
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            for shard in sorted(set(weight_map.values())):
                self.files.append(SafetensorsFile(os.path.join(model_dir, shard)))
        else:
            raise SafetensorsError(f"cannot open {single}: no model.safetensors (or index) in the model folder")
        self.tensors: Dict[str, TensorInfo] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name, info in f.tensors.items():
                self.tensors[name] = info
                self._owner[name] = f

    def read(self, name: str) -> torch.Tensor:
        if name not in self._owner:
            raise SafetensorsError(f"tensor not found: {name}")
        return self._owner[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    """Write CPU tensors to one safetensors file, names sorted, data 8-byte aligned header."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of tensor {name!r}")
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.uint16).numpy().tobytes() if hasattr(torch, "uint16") else t.view(torch.int16).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)
