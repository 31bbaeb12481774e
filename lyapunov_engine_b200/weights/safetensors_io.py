"""Reading and writing safetensors files without any library.

The format: 8 bytes little-endian length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}``,
then the tensors' bytes, offsets relative to the end of the header.  Files are
memory-mapped; a tensor is a view into the map until it is copied to the
device.

The reference reads checkpoints with ``safetensors.torch.load_file``
(python/lyapunov_engine/models/weight_loader.py:5,49-57).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, shape, begin, end, file

    @property
    def is_32bit(self) -> bool:
        return self.dtype in (torch.float32, torch.int32)


class SafetensorsFile:
    """One memory-mapped file and the table of its tensors."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: truncated (header of {n} bytes in a file of {size})")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not JSON: {e}") from e
        self._data_start = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            code = info.get("dtype")
            if code not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {code!r}")
            dtype, width = _DTYPES[code]
            shape = tuple(int(x) for x in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            count = 1
            for x in shape:
                count *= x
            if end - begin != count * width:
                raise SafetensorsError(f"{path}: tensor {name!r}: {end - begin} bytes for shape {shape} of {code}")
            if self._data_start + end > size:
                raise SafetensorsError(f"{path}: truncated (tensor {name!r} ends at byte "
                                       f"{self._data_start + end}, the file has {size})")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, self)

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only view of the tensor's bytes in the map (CPU)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=e.end - e.begin, offset=self._data_start + e.begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the map is read-only; nothing writes through the view
            return torch.from_numpy(raw).view(e.dtype).view(e.shape)

    def close(self):
        # Views handed out keep the map alive; closing is left to the collector.
        self._f.close()


def open_folder(folder: str) -> dict[str, TensorEntry]:
    """Every tensor of every ``*.safetensors`` file in the folder, by name.  A
    name present in two files is an error (the reference lets the later file
    win, python/lyapunov_engine/models/weight_loader.py:54-57)."""
    if not os.path.isdir(folder):
        raise SafetensorsError(f"{folder}: not a folder")
    files = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"{folder}: no .safetensors file in the model folder")
    table: dict[str, TensorEntry] = {}
    for name in files:
        st = SafetensorsFile(os.path.join(folder, name))
        for key, entry in st.entries.items():
            if key in table:
                raise SafetensorsError(f"tensor {key!r} is in both {table[key].file.path} and {st.path}")
            table[key] = entry
    return table


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    """Writes tensors (CPU, contiguous) in name order."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
