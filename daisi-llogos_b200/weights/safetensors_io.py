"""Reading and writing the safetensors container.

File layout: an 8-byte little-endian header length, a JSON header mapping each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian data.  The
reference reads its own container the same way: header and tensor infos first,
data as memory-mapped spans looked up by name (Model/MmapModelLoader.cs:17-34,
:184-196).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

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
    """One memory-mapped .safetensors file; tensors are views of the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self._data0 = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt = _DTYPES.get(e.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {e.get('dtype')!r}")
            shape = tuple(int(s) for s in e["shape"])
            b, en = (int(x) for x in e["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if en - b != n * torch.empty(0, dtype=dt).element_size() or self._data0 + en > size:
                raise SafetensorsError(f"{path}: tensor '{name}' has inconsistent offsets [{b}, {en})")
            self.entries[name] = (dt, shape, b, en)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in the mapping."""
        dt, shape, b, en = self.entries[name]
        n = 1
        for s in shape:
            n *= s
        if n == 0:
            return torch.empty(shape, dtype=dt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            t = torch.frombuffer(self._mm, dtype=dt, count=n, offset=self._data0 + b)
        return t.view(shape)

    def close(self) -> None:
        """Closes the file.  The mapping itself lives as long as tensors view it (they hold a
        reference to it) and is unmapped when the last of them is gone."""
        self._f.close()


class ModelFiles:
    """All tensors of a model folder: ``model.safetensors`` or the shards its index names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            for name, fname in weight_map.items():
                if fname not in self._files:
                    self._files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
                if name not in self._files[fname].entries:
                    raise SafetensorsError(f"{index}: '{name}' is not in {fname}")
                self._where[name] = fname
        elif os.path.isfile(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def names(self):
        return self._where.keys()

    def info(self, name: str):
        return self._files[self._where[name]].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write CPU tensors to one file without gaps: wider element types first, then by name,
    so that every tensor starts on a multiple of its element size; the header is padded
    to a multiple of 64 bytes."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors, key=lambda n: (-tensors[n].element_size(), n))
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-(8 + len(blob))) % 64)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
