"""The safetensors container: u64 little-endian header length, a JSON header
`{name: {dtype, shape, data_offsets}}`, then the data area
(the reference's reader: src/safetensors.c:147-179, checks at :507-526).

Own reader and writer, so that a model folder can be read and written without
any other package.  Tensors come back as torch CPU tensors in the dtype they
are stored in.
"""
import json
import mmap
import os
import struct

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# name in the file -> (torch dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """A read-only memory map of one file; `tensor(name)` copies nothing until
    the caller moves or converts it."""

    def __init__(self, path):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise SafetensorsError(f"{path}: no such file") from None
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than its 8-byte header length")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None)
        self._data0 = 8 + hlen
        data_len = size - self._data0
        self.entries = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], [int(s) for s in info["shape"]], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: entry '{name}' lacks dtype, shape or data_offsets") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has dtype {dt}; handled: {sorted(_DTYPES)}")
            numel = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension")
                numel *= s
            if not (0 <= b <= e <= data_len) or e - b != numel * _DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' data_offsets [{b},{e}) do not fit shape {shape} of {dt} "
                    f"in a data area of {data_len} bytes")
            self.entries[name] = (dt, tuple(shape), b, e)

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype(self, name):
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name):
        dt, shape, b, e = self.entries[name]
        tdt = _DTYPES[dt][0]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._data0 + b)
        # a copy: the result must not dangle once the map is closed
        t = torch.from_numpy(raw.copy())
        return t.view(tdt).reshape(shape)

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path, tensors, metadata=None):
    """Write `{name: torch tensor}` in name order, data 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of '{name}'")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
