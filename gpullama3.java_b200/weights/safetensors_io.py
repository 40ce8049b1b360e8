"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header ``{name: {dtype, shape, data_offsets}}`` and the raw little-endian tensor bytes.  (The
reference reads GGUF, core/model/GGUF.java:84-144 of the reference project, with the same
shape: header, tensor table, one mapped data region, tensors as slices of it.)"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch


class WeightError(ValueError):
    """A weight file is missing, malformed, or does not hold what the model needs."""


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One mapped ``.safetensors`` file; ``tensor(name)`` returns a CPU tensor that views the map."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        if not self.path.is_file():
            raise WeightError(f"weight file {self.path} does not exist")
        size = self.path.stat().st_size
        if size < 8:
            raise WeightError(f"{self.path}: too short to be a safetensors file ({size} bytes)")
        self._file = open(self.path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise WeightError(f"{self.path}: header length {header_len} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{self.path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise WeightError(f"{self.path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + header_len
        data_len = size - self._data_start
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(o) for o in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise WeightError(f"{self.path}: bad header entry for {name!r}: {info!r}") from e
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            if begin < 0 or end > data_len or end - begin != nbytes:
                raise WeightError(f"{self.path}: tensor {name!r} claims bytes [{begin}, {end}) for shape {shape} "
                                  f"{info['dtype']} ({nbytes} bytes) in a data region of {data_len} bytes")
            self.entries[name] = (dtype, shape, begin, end)
        # a private copy-on-write map: torch can view it as writable memory, the file never changes
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        t = torch.frombuffer(self._map, dtype=dtype, count=(end - begin) // torch.empty((), dtype=dtype).element_size(),
                             offset=self._data_start + begin)
        return t.view(shape)

    def close(self) -> None:
        # tensors handed out keep the map alive through the buffer protocol; only the handle closes
        self._file.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors to one safetensors file (names sorted, data 8-byte aligned header)."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot store dtype {t.dtype} of {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")


def open_model_files(model_dir: str | Path) -> dict[str, SafetensorsFile]:
    """The weight files of a model folder, by the tensor names they hold: ``model.safetensors``, or
    the shards named by ``model.safetensors.index.json``."""
    model_dir = Path(model_dir)
    index = model_dir / "model.safetensors.index.json"
    single = model_dir / "model.safetensors"
    by_name: dict[str, SafetensorsFile] = {}
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            raise WeightError(f"{index}: not a shard index (needs a 'weight_map' object)") from e
        files: dict[str, SafetensorsFile] = {}
        for name, fname in weight_map.items():
            if fname not in files:
                files[fname] = SafetensorsFile(model_dir / fname)
            if name not in files[fname].entries:
                raise WeightError(f"{index}: says {name!r} is in {fname}, which does not hold it")
            by_name[name] = files[fname]
        for fname, f in files.items():
            for name in f.names():
                by_name.setdefault(name, f)
    elif single.is_file():
        f = SafetensorsFile(single)
        for name in f.names():
            by_name[name] = f
    else:
        raise WeightError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir}")
    return by_name
