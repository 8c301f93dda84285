"""Reader and writer for the safetensors container.

Layout: ``uint64 header_len`` (little endian), a JSON header, then raw tensor
bytes whose offsets are relative to the end of the header.  The reader checks
what the reference's reader checks (src/Inference/llama_import.jl:288-343):
length prefix, header is one JSON object without duplicate keys, known dtypes,
byte span equal to shape times element size, ranges that tile the payload
without overlap, gap or trailing bytes.  A sharded folder is followed through
``model.safetensors.index.json`` (:432-476).

Tensors come back as ``torch`` CPU tensors in their stored dtype
(BF16 / F16 / F32 / I32 / I64); nothing is converted here.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Mapping

import numpy as np
import torch

from ..config.registry import parse_strict_json
from ..errors import invalid

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_TORCH_TO_NAME = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100_000_000


def _check_int(v, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise invalid(f"safetensors: {what} must be a non-negative integer, got {v!r}")
    return v


def read_safetensors_file(path: str) -> Dict[str, torch.Tensor]:
    if not os.path.isfile(path):
        raise invalid(f"safetensors: no such file: {path}")
    size = os.path.getsize(path)
    if size < 8:
        raise invalid(f"safetensors: {path}: truncated length prefix")
    with open(path, "rb") as f:
        (hdr_len,) = struct.unpack("<Q", f.read(8))
        if not (2 <= hdr_len <= min(_MAX_HEADER, size - 8)):
            raise invalid(f"safetensors: {path}: invalid or truncated header length {hdr_len}")
        text = f.read(hdr_len).decode("utf-8", errors="strict")
        if not text.startswith("{"):
            raise invalid(f"safetensors: {path}: header must start with '{{'")
        header = parse_strict_json(text, f"safetensors header of {path}")
        data_size = size - 8 - hdr_len
        entries = []
        for name, meta in header.items():
            if name == "__metadata__":
                if not (isinstance(meta, dict) and all(isinstance(v, str) for v in meta.values())):
                    raise invalid(f"safetensors: {path}: __metadata__ must map strings to strings")
                continue
            if not (isinstance(meta, dict) and all(k in meta for k in ("dtype", "shape", "data_offsets"))):
                raise invalid(f"safetensors: {path}: entry {name!r} lacks dtype/shape/data_offsets")
            dt = meta["dtype"]
            if dt not in _DTYPES:
                raise invalid(f"safetensors: {path}: tensor {name!r} has unsupported dtype {dt!r}")
            if not isinstance(meta["shape"], list):
                raise invalid(f"safetensors: {path}: tensor {name!r} shape must be an array")
            shape = tuple(_check_int(d, f"{name} shape") for d in meta["shape"])
            offs = meta["data_offsets"]
            if not (isinstance(offs, list) and len(offs) == 2):
                raise invalid(f"safetensors: {path}: tensor {name!r} data_offsets must hold two integers")
            b0, b1 = (_check_int(b, f"{name} offset") for b in offs)
            if not (0 <= b0 <= b1 <= data_size):
                raise invalid(f"safetensors: {path}: tensor {name!r} invalid data range [{b0}, {b1})")
            n = 1
            for d in shape:
                n *= d       # Python integers do not wrap
            if n * _DTYPES[dt][1] != b1 - b0:
                raise invalid(f"safetensors: {path}: tensor {name!r} byte span disagrees with shape and dtype")
            entries.append((b0, b1, name, shape, dt))
        entries.sort()
        cursor = 0
        for b0, b1, name, _, _ in entries:
            if b0 != cursor:
                raise invalid(f"safetensors: {path}: overlapping or unindexed bytes at tensor {name!r}")
            cursor = b1
        if cursor != data_size:
            raise invalid(f"safetensors: {path}: unindexed trailing payload bytes")
        out: Dict[str, torch.Tensor] = {}
        if data_size == 0:
            for _, _, name, shape, dt in entries:
                out[name] = torch.empty(shape, dtype=_DTYPES[dt][0])
            return out
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        base = 8 + hdr_len
        for b0, b1, name, shape, dt in entries:
            tdt = _DTYPES[dt][0]
            if b1 == b0:
                out[name] = torch.empty(shape, dtype=tdt)
                continue
            raw = np.frombuffer(mm, dtype=np.uint8, count=b1 - b0, offset=base + b0)
            # copy out of the mapping: the tensors outlive the file handle
            t = torch.from_numpy(raw.copy()).view(tdt).reshape(shape)
            out[name] = t
        del raw
        try:
            mm.close()
        except BufferError:
            pass
        return out


def read_model_tensors(model_dir: str) -> Dict[str, torch.Tensor]:
    """All tensors of a model folder: ``model.safetensors`` or its shard index."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return read_safetensors_file(single)
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            idx = parse_strict_json(f.read(), index)
        wm = idx.get("weight_map")
        if not isinstance(wm, dict) or not wm:
            raise invalid(f"{index}: 'weight_map' must be a non-empty object")
        out: Dict[str, torch.Tensor] = {}
        for shard in sorted(set(wm.values())):
            if not isinstance(shard, str) or os.path.basename(shard) != shard:
                raise invalid(f"{index}: shard name {shard!r} must be a plain file name")
            tensors = read_safetensors_file(os.path.join(model_dir, shard))
            for name, t in tensors.items():
                if wm.get(name) != shard:
                    raise invalid(f"{index}: tensor {name!r} found in {shard!r} but not indexed there")
                out[name] = t
        missing = [n for n in wm if n not in out]
        if missing:
            raise invalid(f"{index}: indexed tensors missing from their shards: {missing[:8]}")
        return out
    raise invalid(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def write_safetensors_file(path: str, tensors: Mapping[str, torch.Tensor],
                           metadata: Mapping[str, str] | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    cursor = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_NAME:
            raise invalid(f"safetensors: cannot store dtype {t.dtype} (tensor {name!r})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [cursor, cursor + nbytes]}
        blobs.append(t)
        cursor += nbytes
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(text) % 8) % 8
    text += b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for t in blobs:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
