"""Reading and writing the safetensors container, with no third-party reader.

Format (as src/inspect/safetensors_header.cpp:21-63 states it): an 8-byte
little-endian header length, a JSON header ``{name: {dtype, shape,
data_offsets}}`` (``__metadata__`` skipped), then the raw little-endian tensor
bytes.  A zero or oversized header length and ``end < begin`` are refused.
The file set of a model folder follows src/core/weights.cpp:208-249: the index
``model.safetensors.index.json`` if every shard it names exists, else
``model.safetensors``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import numpy as np


class SafetensorsError(ValueError):
    pass


# dtype tag -> (numpy storage dtype, bytes per element)
_DTYPES = {
    "F64": (np.float64, 8), "F32": (np.float32, 4), "F16": (np.float16, 2),
    "BF16": (np.uint16, 2),  # numpy has no bfloat16: kept as raw 16-bit words
    "I64": (np.int64, 8), "I32": (np.int32, 4), "I16": (np.int16, 2), "I8": (np.int8, 1),
    "U8": (np.uint8, 1), "BOOL": (np.bool_, 1),
}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorEntry:
    """One tensor of a safetensors file: where its bytes are and what they mean."""

    name: str
    dtype: str            # the safetensors tag: "BF16", "F32", ...
    shape: Tuple[int, ...]
    file: str
    begin: int            # absolute byte offsets in ``file``
    end: int


def read_header(path: str) -> List[TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"safetensors: '{path}' is shorter than its 8-byte header length")
        (n,) = struct.unpack("<Q", head)
        if n == 0 or n > _MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"safetensors: '{path}' has an invalid header length {n}")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"safetensors: '{path}' header is not valid JSON: {e}")
    if not isinstance(header, dict):
        raise SafetensorsError(f"safetensors: '{path}' header is not a JSON object")
    base = 8 + n
    out: List[TensorEntry] = []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype = info["dtype"]
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"safetensors: '{path}' has a malformed entry for '{name}'")
        if dtype not in _DTYPES:
            raise SafetensorsError(f"safetensors: '{path}' tensor '{name}' has unsupported dtype '{dtype}'")
        if end < begin or base + end > size:
            raise SafetensorsError(f"safetensors: '{path}' tensor '{name}' has invalid data offsets [{begin}, {end})")
        count = 1
        for s in shape:
            count *= s
        if count * _DTYPES[dtype][1] != end - begin:
            raise SafetensorsError(
                f"safetensors: '{path}' tensor '{name}' of shape {list(shape)} and dtype {dtype} "
                f"does not fill its {end - begin} bytes")
        out.append(TensorEntry(name, dtype, shape, path, base + begin, base + end))
    return out


def model_files(model_dir: str) -> List[str]:
    """The safetensors files of a model folder (src/core/weights.cpp:208-249)."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            j = json.load(f)
        wm = j.get("weight_map") if isinstance(j, dict) else None
        if not isinstance(wm, dict):
            raise SafetensorsError(f"weights: '{index}' has no 'weight_map' object")
        shards = sorted({os.path.join(model_dir, v) for v in wm.values()})
        if shards and all(os.path.isfile(s) for s in shards):
            return shards
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    raise SafetensorsError(f"weights: no model.safetensors[.index.json] in '{model_dir}'")


class SafetensorsFile:
    """Memory-mapped view of one file; ``array(entry)`` is a zero-copy numpy view."""

    def __init__(self, path: str):
        self.path = path
        self.entries = read_header(path)
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def array(self, e: TensorEntry) -> np.ndarray:
        np_dtype, _ = _DTYPES[e.dtype]
        a = np.frombuffer(self._mm, dtype=np_dtype, count=(e.end - e.begin) // _DTYPES[e.dtype][1],
                          offset=e.begin)
        return a.reshape(e.shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass  # views still alive; the mapping goes with them
        self._f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, str, Tuple[int, ...], bytes]]) -> None:
    """Write ``(name, dtype tag, shape, raw little-endian bytes)`` items as one file.

    Items are consumed one at a time so a large model never sits in memory twice;
    the header is built first from the sizes, which needs the items twice, so
    pass a list or a re-iterable.
    """
    items = list(tensors)
    header: Dict[str, dict] = {}
    off = 0
    for name, dtype, shape, data in items:
        if dtype not in _DTYPES:
            raise SafetensorsError(f"safetensors: cannot write dtype '{dtype}'")
        n = len(data)
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + n]}
        off += n
    header["__metadata__"] = {"format": "pt"}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, _, _, data in items:
            f.write(data)
    os.replace(tmp, path)


def write_safetensors_streaming(path: str, entries, produce) -> None:
    """Write a file whose tensors are made one at a time: ``entries`` is a list of
    ``(name, dtype tag, shape)`` and ``produce(i)`` returns the raw little-endian
    bytes (any buffer) of entry ``i``.  The header is computed from the shapes, so
    a multi-gigabyte model never sits in memory."""
    header: Dict[str, dict] = {}
    off = 0
    sizes = []
    for name, dtype, shape in entries:
        if dtype not in _DTYPES:
            raise SafetensorsError(f"safetensors: cannot write dtype '{dtype}'")
        n = _DTYPES[dtype][1]
        for s_ in shape:
            n *= int(s_)
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + n]}
        sizes.append(n)
        off += n
    header["__metadata__"] = {"format": "pt"}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for i, n in enumerate(sizes):
            data = memoryview(produce(i)).cast("B")
            if data.nbytes != n:
                raise SafetensorsError(f"safetensors: tensor {entries[i][0]} produced {data.nbytes} bytes, expected {n}")
            f.write(data)
    os.replace(tmp, path)
