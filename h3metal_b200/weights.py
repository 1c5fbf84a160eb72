"""The .h3m weight container, reading and writing, for the int8 linear path.

Same file format as the reference's h3metal/weights.py (layout :1-18, Writer :51-128, read_header :131-138,
WeightFile :141-202), so files produced by the reference's converters can be read here and vice versa:

    b"H3MW", u32 version (1), u64 header length, UTF-8 JSON header, zero padding up to 8 MiB, tensor data

Every tensor starts on a 256-byte boundary and does not cross a multiple of the chunk size (1 GiB) unless it is
marked host-only. The JSON header maps names to entries: a plain tensor is {"offset", "nbytes", "shape", "dtype"};
a linear layer is {"kind": "linear", "fmt", "N", "K", "G", "w": {...}, "sw": {...}, "bias": {...}}; "meta" carries
the model configuration and "chunk" the chunk size.

What differs from the reference is where the bytes go: the reference maps the file and hands the mapping to the GPU
without copying (Apple's unified memory); a B200 has its own memory, so `WeightFile` maps the file on the host and
uploads a tensor to HBM the first time it is asked for (and keeps it). 180 GB of HBM hold any of the models whole,
so there is no streaming, prefetch or eviction here; those calls of the reference are accepted and do nothing.
"""

from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np

from .gpu import Gpu, Tensor
from .ops import QWeight

MAGIC = b"H3MW"
VERSION = 1
DATA_START = 8 << 20
CHUNK = 1 << 30
ALIGN = 256

_NP = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16, "i8": np.int8, "u8": np.uint8, "i32": np.int32,
       "u16": np.uint16}
_CODE_DTYPE = {"q8": "i8", "h8": "i8", "f16": "f16", "bf16": "bf16"}


def _align(x: int) -> int:
    return -(-x // ALIGN) * ALIGN


class Writer:
    """Appends tensors to a new .h3m file one at a time; close() writes the header and renames the file into place."""

    def __init__(self, path: str, meta: dict):
        self.path, self.meta = path, meta
        self._partial = path + ".partial"
        self._file = open(self._partial, "wb")
        self._file.truncate(DATA_START)
        self._end = DATA_START          # first free byte after everything written so far
        self._holes = []                # [start, stop) skipped in front of a chunk boundary, reusable by small tensors
        self.entries = {}

    def _allocate(self, nbytes: int, host_only: bool) -> int:
        if not host_only:
            if nbytes > CHUNK:
                raise ValueError(f"tensor of {nbytes} bytes exceeds the {CHUNK}-byte chunk")
            for hole in self._holes:
                start = _align(hole[0])
                if start + nbytes <= hole[1]:
                    hole[0] = start + nbytes
                    return start
        start = _align(self._end)
        if not host_only and start // CHUNK != (start + nbytes - 1) // CHUNK:
            boundary = (start // CHUNK + 1) * CHUNK
            self._holes.append([start, boundary])
            start = boundary
        self._end = start + nbytes
        return start

    def _put(self, data: np.ndarray, host_only: bool = False) -> dict:
        raw = np.ascontiguousarray(data).reshape(-1).view(np.uint8)
        start = self._allocate(raw.nbytes, host_only)
        self._file.seek(start)
        self._file.write(memoryview(raw))
        return {"offset": start, "nbytes": int(raw.nbytes)}

    def tensor(self, name: str, data: np.ndarray, dtype: str, host_only: bool = False):
        if name in self.entries:
            raise KeyError(f"duplicate tensor {name}")
        entry = self._put(data, host_only)
        entry.update(shape=list(data.shape), dtype=dtype)
        if host_only:
            entry["host_only"] = True
        self.entries[name] = entry

    def linear(self, name: str, fmt: str, N: int, K: int, w: np.ndarray, sw: np.ndarray | None,
               bias: np.ndarray | None = None, G: int = 128, extra: dict | None = None):
        entry = {"kind": "linear", "fmt": fmt, "N": N, "K": K, "G": G, "w": self._put(w)}
        if sw is not None:
            entry["sw"] = self._put(np.asarray(sw, dtype=np.float32))
        if bias is not None:
            entry["bias"] = self._put(np.asarray(bias, dtype=np.float32))
        entry.update(extra or {})
        self.entries[name] = entry

    def close(self):
        header = json.dumps({"meta": self.meta, "chunk": CHUNK, "tensors": self.entries}, separators=(",", ":")).encode()
        if 16 + len(header) > DATA_START:
            raise ValueError("header does not fit the reserved region")
        self._file.seek(0)
        self._file.write(MAGIC + struct.pack("<IQ", VERSION, len(header)) + header)
        self._file.truncate(-(-self._end // 16384) * 16384)
        self._file.close()
        os.replace(self._partial, self.path)


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        if f.read(4) != MAGIC:
            raise ValueError(f"{path} is not an h3metal weight file")
        version, length = struct.unpack("<IQ", f.read(12))
        if version != VERSION:
            raise ValueError(f"{path}: unsupported weight file version {version}")
        return json.loads(f.read(length))


class WeightFile:
    """An .h3m file: tensors and int8 linear layers as views of device memory, uploaded on first use."""

    def __init__(self, gpu: Gpu, path: str):
        self.gpu, self.path = gpu, path
        hdr = read_header(path)
        self.meta, self.entries = hdr["meta"], hdr["tensors"]
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        self._resident = {}   # (offset, nbytes) -> Tensor

    def __contains__(self, name):
        return name in self.entries

    def _host(self, offset: int, nbytes: int) -> np.ndarray:
        return np.frombuffer(self._map, dtype=np.uint8, count=nbytes, offset=offset)

    def _device(self, part: dict, shape, dtype: str) -> Tensor:
        key = (part["offset"], part["nbytes"])
        t = self._resident.get(key)
        if t is None:
            t = self.gpu.upload(self._host(*key).view(_NP[dtype]).reshape(shape), dtype)
            self._resident[key] = t
        return t

    def tensor(self, name: str) -> Tensor:
        e = self.entries[name]
        if e.get("host_only"):
            raise ValueError(f"{name} is stored for the CPU only")
        return self._device(e, tuple(e["shape"]), e["dtype"])

    def host(self, name: str) -> np.ndarray:
        """The tensor as a read-only NumPy view of the mapped file."""
        e = self.entries[name]
        return self._host(e["offset"], e["nbytes"]).view(_NP[e["dtype"]]).reshape(e["shape"])

    def linear(self, name: str) -> QWeight:
        e = self.entries[name]
        fmt, N, K = e["fmt"], e["N"], e["K"]
        if fmt not in _CODE_DTYPE:
            raise NotImplementedError(f"{name}: weight format {fmt!r} is outside the int8 linear path")
        w = self._device(e["w"], (N, K), _CODE_DTYPE[fmt])
        sw = self._device(e["sw"], (e["sw"]["nbytes"] // 4,), "f32") if "sw" in e else None
        bias = self._device(e["bias"], (N,), "f32") if "bias" in e else None
        return QWeight(fmt, w, sw, N, K, e.get("G", 128), bias)

    # The reference manages which file pages are resident (its GPU reads the mapping itself). Here every tensor that
    # was asked for lives in HBM, so these are accepted for compatibility and have nothing to do.
    def prefetch(self, names=None):
        pass

    def release(self, names):
        pass

    def touch(self, names):
        pass

    def nbytes(self, names) -> int:
        total = 0
        for name in names:
            e = self.entries[name]
            total += e["nbytes"] if "offset" in e else sum(e[k]["nbytes"] for k in ("w", "sw", "bias") if k in e)
        return total

    def close(self):
        self._resident.clear()
        self._map.close()
        self._file.close()
