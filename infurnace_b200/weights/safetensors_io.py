"""Reading and writing safetensors files without a library.

The format: 8 bytes little-endian header length n, n bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``, then
the tensors' bytes; offsets count from the end of the header.  A reader maps the file
and hands out zero-copy views, so a tensor's bytes go from the page cache to the device
without a second host copy.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

from ..errors import WeightError

# safetensors dtype tag -> (bytes per element, torch dtype name)
DTYPES = {
    "F64": (8, "float64"), "F32": (4, "float32"), "F16": (2, "float16"), "BF16": (2, "bfloat16"),
    "I64": (8, "int64"), "I32": (4, "int32"), "I16": (2, "int16"), "I8": (1, "int8"),
    "U8": (1, "uint8"), "BOOL": (1, "bool"),
}
_TAG_OF = {v[1]: k for k, v in DTYPES.items()}


class SafetensorsFile:
    """One mapped ``.safetensors`` file: ``entries`` maps name -> (dtype tag, shape)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > (100 << 20):
            raise WeightError(f"{path}: header length {n} is not plausible for a file of {size} bytes")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self.entries: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
        self._ranges: Dict[str, Tuple[int, int]] = {}
        for name, info in header.items():
            tag, shape = info["dtype"], tuple(int(s) for s in info["shape"])
            begin, end = info["data_offsets"]
            if tag not in DTYPES:
                raise WeightError(f"{path}: tensor {name} has unknown dtype {tag}")
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * DTYPES[tag][0] or begin < 0 or self._base + end > size:
                raise WeightError(f"{path}: tensor {name} has data offsets that do not match its shape")
            self.entries[name] = (tag, shape)
            self._ranges[name] = (begin, end)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str):
        """A CPU torch tensor viewing the file's bytes (read-only: copy before writing)."""
        import torch
        tag, shape = self.entries[name]
        begin, end = self._ranges[name]
        dtype = getattr(torch, DTYPES[tag][1])
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes to the view
            flat = torch.frombuffer(self._mm, dtype=dtype, count=(end - begin) // DTYPES[tag][0],
                                    offset=self._base + begin)
        return flat.view(shape)

    def close(self):
        # views handed out keep the mapping alive through the buffer protocol
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass
        self._f.close()


def list_weight_files(model_dir: str) -> List[str]:
    """The safetensors files of a model folder: those its index names, else every
    ``*.safetensors`` file in it."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_dir, n) for n in names]
    files = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not files:
        raise WeightError(f"no .safetensors file in {model_dir}")
    return [os.path.join(model_dir, n) for n in files]


def write_safetensors(path: str, tensors: Iterable[Tuple[str, "object"]], metadata: Mapping[str, str] = None) -> None:
    """Write (name, CPU torch tensor) pairs.  ``tensors`` is consumed twice (pass a list)
    or may hold callables that produce the tensor, so that a large model is written
    one tensor at a time."""
    import torch
    items = list(tensors)
    header, offset = {}, 0
    metas = []
    for name, t in items:
        if callable(t):
            shape, dtype = t.shape, t.dtype       # a producer object with shape/dtype attributes
        else:
            shape, dtype = tuple(t.shape), t.dtype
        tag = _TAG_OF[str(dtype).replace("torch.", "")]
        count = 1
        for s in shape:
            count *= s
        nbytes = count * DTYPES[tag][0]
        header[name] = {"dtype": tag, "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        metas.append(nbytes)
        offset += nbytes
    if metadata:
        header["__metadata__"] = dict(metadata)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for (name, t), nbytes in zip(items, metas):
            if callable(t):
                t = t()
            t = t.detach().contiguous().cpu()
            raw = t.view(torch.uint8) if t.numel() else t
            data = raw.numpy().tobytes() if t.numel() else b""
            if len(data) != nbytes:
                raise WeightError(f"tensor {name} produced {len(data)} bytes, expected {nbytes}")
            f.write(data)
    os.replace(tmp, path)
