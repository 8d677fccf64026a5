"""Reader and writer for the safetensors container, by tensor name.

File layout: 8 bytes little-endian header length, a JSON header mapping each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian data. A folder
holds either ``model.safetensors`` or ``model.safetensors.index.json`` with a
``weight_map`` from tensor name to shard file, as the reference's by-name
mechanism expects (python/vosti_kernels/checkpoint.py:15-29).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One shard, memory-mapped; tensors are views of the mapping."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as handle:
            head = handle.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{self.path}: truncated (no header length)")
            (length,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if length <= 0 or 8 + length > size:
                raise SafetensorsError(f"{self.path}: header length {length} exceeds file size {size}")
            try:
                header = json.loads(handle.read(length))
            except (json.JSONDecodeError, UnicodeDecodeError) as error:
                raise SafetensorsError(f"{self.path}: header is not JSON: {error}") from error
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY)
        self._base = 8 + length
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dtype, shape = info["dtype"], tuple(int(s) for s in info["shape"])
                begin, end = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as error:
                raise SafetensorsError(f"{self.path}: bad entry for '{name}': {error}") from error
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {dtype}")
            count = 1
            for s in shape:
                count *= s
            width = torch.empty(0, dtype=_DTYPES[dtype]).element_size()
            if end - begin != count * width or self._base + end > size or begin < 0:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has data range "
                                       f"[{begin},{end}) inconsistent with shape {shape} {dtype}")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=_DTYPES[dtype])
        flat = torch.frombuffer(self._map, dtype=_DTYPES[dtype], count=(end - begin)
                                // torch.empty(0, dtype=_DTYPES[dtype]).element_size(),
                                offset=self._base + begin)
        return flat.view(shape)


def write_safetensors(path: str | Path, tensors: Dict[str, torch.Tensor],
                      metadata: Dict[str, str] | None = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    ordered = sorted(tensors)
    for name in ordered:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has unsupported dtype {t.dtype}")
        size = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in ordered:
            t = tensors[name].detach().cpu().contiguous()
            handle.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_model_shards(model_dir: str | Path) -> Dict[str, SafetensorsFile]:
    """Map every tensor name of a model folder to the shard that holds it."""
    root = Path(model_dir)
    index, single = root / "model.safetensors.index.json", root / "model.safetensors"
    by_name: Dict[str, SafetensorsFile] = {}
    if index.is_file():
        payload = json.loads(index.read_text())
        mapping = payload.get("weight_map") if isinstance(payload, dict) else None
        if not isinstance(mapping, dict) or not mapping:
            raise SafetensorsError(f"{index}: invalid weight_map")
        shards: Dict[str, SafetensorsFile] = {}
        for name, shard in mapping.items():
            path = (root / shard).resolve()
            if path.parent != root.resolve() or not path.is_file():
                raise SafetensorsError(f"{index}: shard '{shard}' is missing or outside the folder")
            if shard not in shards:
                shards[shard] = SafetensorsFile(path)
            if name not in shards[shard].entries:
                raise SafetensorsError(f"{index}: tensor '{name}' is not in shard '{shard}'")
            by_name[name] = shards[shard]
        return by_name
    if single.is_file():
        shard = SafetensorsFile(single)
        return {name: shard for name in shard.names()}
    raise SafetensorsError(f"{root} holds neither model.safetensors nor model.safetensors.index.json")
