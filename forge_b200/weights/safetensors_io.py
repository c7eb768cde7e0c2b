"""Reading and writing safetensors files without any library: an 8-byte little-endian header length,
a JSON header {name: {dtype, shape, data_offsets}}, then raw little-endian tensor bytes.

Tensors come back as torch tensors of the dtype they are stored in (BF16 stays bfloat16, F32 stays
float32, I32 stays int32): nothing is narrowed or widened on the way in.
"""
import json
import mmap
import os
import struct
import warnings

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; ``tensor(name)`` copies one tensor out."""

    def __init__(self, path):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated file ({size} bytes, no header length)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: truncated file (header says {n} bytes, file has {size})")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        self.metadata = header.pop("__metadata__", {})
        self.entries = header
        self._base = 8 + n
        self._size = size
        for name, info in header.items():
            b, e = info["data_offsets"]
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            numel = 1
            for s in info["shape"]:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[info["dtype"]]).element_size()
            if e - b != want or self._base + e > size:
                raise SafetensorsError(f"{path}: truncated or inconsistent data for tensor {name} "
                                       f"(offsets {b}:{e}, expected {want} bytes, file has {size - self._base})")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return tuple(self.entries[name]["shape"])

    def dtype(self, name):
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name):
        info = self.entries[name]
        b, e = info["data_offsets"]
        dt = _DTYPES[info["dtype"]]
        if e == b:
            return torch.empty(tuple(info["shape"]), dtype=dt)
        buf = memoryview(self._mm)[self._base + b:self._base + e]
        # frombuffer shares the (read-only) mapping; clone so the file can be closed
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(buf, dtype=dt).reshape(tuple(info["shape"])).clone()

    def close(self):
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._f.close()


def write_safetensors(path, tensors, metadata=None):
    """Writes {name: CPU torch tensor} in the order given."""
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


def open_model_files(model_dir):
    """{tensor name: SafetensorsFile} for ``model.safetensors`` or the shards of ``model.safetensors.index.json``."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    files = {}
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        return {n: f for n in f.names()}, [f]
    if os.path.isfile(index):
        with open(index) as fh:
            weight_map = json.load(fh)["weight_map"]
        opened = {}
        for name, shard in weight_map.items():
            if shard not in opened:
                opened[shard] = SafetensorsFile(os.path.join(model_dir, shard))
            if name not in opened[shard].entries:
                raise SafetensorsError(f"{index}: {name} is not in shard {shard}")
            files[name] = opened[shard]
        return files, list(opened.values())
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
