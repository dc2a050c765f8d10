"""Reading and writing the safetensors container (own code, no dependency).

Layout: 8 bytes little-endian header length, a JSON header mapping tensor name
to {dtype, shape, data_offsets}, then the raw little-endian data.  The reference
reads tensors by name from its own container (GGUF) one at a time
(zllm src/backend/candle/quantized_llama_fork.rs:755-791); here the file is
memory-mapped and every tensor is a view until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Dict, Tuple

import torch

from ..errors import ModelError

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsFile:
    """A memory-mapped safetensors file: ``keys()``, ``meta(name)``, ``tensor(name)``."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as e:
            raise ModelError(f"cannot open model file {self.path}: {e}") from e
        head = self._fh.read(8)
        if len(head) != 8:
            raise ModelError(f"invalid safetensors file {self.path}: shorter than its length field")
        (hlen,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if hlen <= 0 or 8 + hlen > size:
            raise ModelError(f"invalid safetensors file {self.path}: header length {hlen} exceeds the file")
        try:
            self.header = json.loads(self._fh.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise ModelError(f"invalid safetensors file {self.path}: header is not JSON ({e})") from e
        self.header.pop("__metadata__", None)
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        for name, m in self.header.items():
            lo, hi = m["data_offsets"]
            if m["dtype"] not in DTYPES:
                raise ModelError(f"{self.path}: tensor {name!r} has unsupported dtype {m['dtype']}")
            n = 1
            for s in m["shape"]:
                n *= s
            want = n * torch.empty((), dtype=DTYPES[m["dtype"]]).element_size()
            if hi - lo != want or self._base + hi > size:
                raise ModelError(f"{self.path}: tensor {name!r} has {hi - lo} bytes, its shape needs {want}")

    def keys(self):
        return list(self.header.keys())

    def meta(self, name) -> Tuple[torch.dtype, Tuple[int, ...]]:
        m = self.header[name]
        return DTYPES[m["dtype"]], tuple(m["shape"])

    def tensor(self, name) -> torch.Tensor:
        m = self.header[name]
        lo, hi = m["data_offsets"]
        dtype = DTYPES[m["dtype"]]
        if hi == lo:
            return torch.empty(m["shape"], dtype=dtype)
        n = (hi - lo) // torch.empty((), dtype=dtype).element_size()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the map is read-only; the views are only ever copied from
            t = torch.frombuffer(self._mm, dtype=dtype, count=n, offset=self._base + lo)
        return t.reshape(m["shape"])

    def close(self):
        # views made by ``tensor`` keep the map alive; dropping our references is enough
        self._mm = None
        self._fh.close()


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None):
    """Write tensors (CPU, contiguous) under their names, in the given order."""
    header = {}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in NAMES:
            raise ModelError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    if metadata:
        header["__metadata__"] = metadata
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for t in blobs:
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_model_files(model_dir) -> Dict[str, SafetensorsFile]:
    """tensor name -> the file that holds it: ``model.safetensors`` or the shards named by
    ``model.safetensors.index.json``."""
    model_dir = Path(model_dir)
    single = model_dir / "model.safetensors"
    index = model_dir / "model.safetensors.index.json"
    where: Dict[str, SafetensorsFile] = {}
    if single.exists():
        f = SafetensorsFile(single)
        for k in f.keys():
            where[k] = f
        return where
    if index.exists():
        try:
            wm = json.loads(index.read_text())["weight_map"]
        except (OSError, KeyError, json.JSONDecodeError) as e:
            raise ModelError(f"invalid {index}: {e}") from e
        files: Dict[str, SafetensorsFile] = {}
        for name, fname in wm.items():
            if fname not in files:
                files[fname] = SafetensorsFile(model_dir / fname)
            if name not in files[fname].header:
                raise ModelError(f"{index} places {name!r} in {fname}, which does not hold it")
            where[name] = files[fname]
        return where
    raise ModelError(f"cannot open model folder {model_dir}: neither model.safetensors nor "
                     "model.safetensors.index.json is there")
