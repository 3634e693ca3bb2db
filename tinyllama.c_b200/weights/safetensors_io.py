"""Reading and writing safetensors files.

The reference maps a GGUF file and binds zero-copy tensor views into it
(core.c:1349-1395, 546-592).  The same idea for safetensors: an 8-byte little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, then raw
little-endian data; the file is memory-mapped and every tensor is a view into the map.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Tuple

import torch

_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
           "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: str) -> Tuple[Dict[str, dict], int]:
    """(header entries without __metadata__, offset of the data section)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (n,) = struct.unpack("<Q", raw)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
    header.pop("__metadata__", None)
    data_len = size - 8 - n
    for name, ent in header.items():
        try:
            b, e = ent["data_offsets"]
            dt, shape = ent["dtype"], ent["shape"]
        except (KeyError, TypeError, ValueError) as ex:
            raise SafetensorsError(f"{path}: malformed entry for '{name}'") from ex
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
        count = 1
        for s in shape:
            count *= s
        if not (0 <= b <= e <= data_len) or e - b != count * torch.empty(0, dtype=_DTYPES[dt]).element_size():
            raise SafetensorsError(f"{path}: tensor '{name}' data range [{b}, {e}) does not match its shape "
                                   f"{shape} / the file's {data_len} data bytes")      # core.c:1338-1344
    return header, 8 + n


def load_file(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one file as read-only views into a memory map (CPU tensors)."""
    header, base = read_header(path)
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    out = {}
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")       # torch warns that the buffer is not writable; nothing writes to it
        for name, ent in header.items():
            dt = _DTYPES[ent["dtype"]]
            b, e = ent["data_offsets"]
            if e == b:
                t = torch.empty(ent["shape"], dtype=dt)
            else:
                t = torch.frombuffer(mm, dtype=dt, count=(e - b) // torch.empty(0, dtype=dt).element_size(),
                                     offset=base + b).reshape(ent["shape"])
            out[name] = t
    return out


def load_model_dir(model_dir: str) -> Dict[str, torch.Tensor]:
    """model.safetensors, or the shards named by model.safetensors.index.json."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return load_file(single)
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        out: Dict[str, torch.Tensor] = {}
        for shard in sorted(set(weight_map.values())):
            tensors = load_file(os.path.join(model_dir, shard))
            for name, t in tensors.items():
                if name in out:
                    raise SafetensorsError(f"{model_dir}: tensor '{name}' appears in two shards")
                out[name] = t
        return out
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def save_file(tensors: Dict[str, torch.Tensor], path: str) -> None:
    header, off, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
