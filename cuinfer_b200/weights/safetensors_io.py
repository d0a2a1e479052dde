"""Reader and writer for the safetensors container, written against the format itself.

Layout (as the reference's reader walks it, csrc/model/checkpoint.cpp:77-126): an 8-byte
little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}`` with an
optional ``__metadata__`` entry, then the tensor bytes.  A model folder holds either one
``model.safetensors`` or a ``model.safetensors.index.json`` whose ``weight_map`` names the
shard of every tensor (csrc/model/checkpoint.cpp:42-58).  Files are memory-mapped read-only;
a tensor is materialised only when it is asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping

import torch


class WeightError(RuntimeError):
    """A checkpoint that cannot be read or does not fit the model; the message lists why."""


_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int          # byte offsets inside the data section
    end: int
    file_index: int


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file."""

    def __init__(self, path: str) -> None:
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as exc:
            raise WeightError(f"cannot open {path}: {exc.strerror or exc}") from exc
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise WeightError(f"invalid safetensors file {path}: shorter than its 8-byte length field")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len == 0 or header_len > _MAX_HEADER or 8 + header_len > size:
            raise WeightError(f"invalid safetensors header size {header_len} in {path} (file has {size} bytes)")
        def no_duplicates(pairs):
            # a name that occurs twice in the header is an error (csrc/model/checkpoint.cpp:121-124), not "the last wins"
            out = {}
            for key, value in pairs:
                if key in out:
                    raise WeightError(f"duplicate tensor '{key}' in the header of {path}")
                out[key] = value
            return out

        try:
            header = json.loads(self._fh.read(header_len).decode("utf-8"), object_pairs_hook=no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightError(f"invalid safetensors header in {path}: {exc}") from exc
        if not isinstance(header, dict):
            raise WeightError(f"invalid safetensors header in {path}: not an object")
        self.data_start = 8 + header_len
        data_size = size - self.data_start
        self.entries: Dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name = meta["dtype"]
                shape = tuple(int(s) for s in meta["shape"])
                begin, end = (int(o) for o in meta["data_offsets"])
            except (KeyError, TypeError, ValueError) as exc:
                raise WeightError(f"invalid safetensors entry for '{name}' in {path}: {exc}") from exc
            if dtype_name not in _DTYPES:
                raise WeightError(f"unsupported safetensors dtype {dtype_name} for '{name}' in {path}")
            dtype, width = _DTYPES[dtype_name]
            if any(s < 0 for s in shape):
                raise WeightError(f"invalid shape {list(shape)} for '{name}' in {path}")
            count = 1
            for s in shape:
                count *= s
            if not (0 <= begin <= end <= data_size) or end - begin != count * width:
                raise WeightError(
                    f"invalid data_offsets [{begin}, {end}) for '{name}' in {path}: "
                    f"shape {list(shape)} of {dtype_name} needs {count * width} bytes of {data_size}"
                )
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, 0)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns a copy of the bytes of ``name``."""
        e = self.entries[name]
        lo, hi = self.data_start + e.begin, self.data_start + e.end
        if hi == lo:
            return torch.empty(e.shape, dtype=e.dtype)
        raw = bytearray(self._map[lo:hi])
        return torch.frombuffer(raw, dtype=e.dtype).reshape(e.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()


class Checkpoint:
    """All tensors of a model folder by name, over one file or an index of shards."""

    def __init__(self, model_dir: str) -> None:
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        self._files: list[SafetensorsFile] = []
        self._where: Dict[str, int] = {}
        try:
            if os.path.exists(index_path):
                try:
                    with open(index_path, "r", encoding="utf-8") as fh:
                        weight_map = json.load(fh)["weight_map"]
                except (OSError, KeyError, json.JSONDecodeError, TypeError) as exc:
                    raise WeightError(f"invalid safetensors index {index_path}: {exc}") from exc
                shard_ids: Dict[str, int] = {}
                for name, shard in weight_map.items():
                    if shard not in shard_ids:
                        shard_ids[shard] = len(self._files)
                        self._files.append(SafetensorsFile(os.path.join(model_dir, shard)))
                    fid = shard_ids[shard]
                    if name not in self._files[fid].entries:
                        raise WeightError(f"index maps '{name}' to {shard}, which does not hold it")
                    self._where[name] = fid
            else:
                f = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
                self._files.append(f)
                for name in f.entries:
                    self._where[name] = 0
        except WeightError as exc:
            self.close()
            raise WeightError(f"failed to load checkpoint {model_dir}: {exc}") from exc

    def names(self) -> list[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def entry(self, name: str) -> TensorEntry:
        return self._files[self._where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self) -> None:
        for f in self._files:
            f.close()
        self._files = []


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file, names sorted."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot store dtype {t.dtype} for '{name}'")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
