"""Reader for ``.safetensors`` checkpoints: an 8-byte little-endian header length, a JSON header
``name -> {dtype, shape, data_offsets}``, then the raw little-endian data.  The file is memory-mapped and each tensor
is copied out once; no third-party reader is involved (the reference goes through ``safetensors.torch``,
lite_llama/models/weights.py:40-76)."""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}


def read_safetensors(path: str | Path) -> dict[str, torch.Tensor]:
    """All tensors of one file as CPU tensors that own their memory."""
    path = Path(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file")
        (hlen,) = struct.unpack("<Q", head)
        size = path.stat().st_size
        if hlen > size - 8:
            raise ValueError(f"{path}: header length {hlen} exceeds the file")
        header = json.loads(f.read(hlen))
        base = 8 + hlen
        with mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as mm:
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                dtype = _DTYPES.get(meta["dtype"])
                if dtype is None:
                    raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
                lo, hi = meta["data_offsets"]
                shape = tuple(meta["shape"])
                count = 1
                for d in shape:
                    count *= d
                if hi - lo != count * torch.empty((), dtype=dtype).element_size() or base + hi > size:
                    raise ValueError(f"{path}: tensor {name} does not fit its byte range")
                if count == 0:
                    out[name] = torch.empty(shape, dtype=dtype)
                    continue
                buf = bytearray(mm[base + lo:base + hi])
                out[name] = torch.frombuffer(buf, dtype=dtype).reshape(shape)
    return out


def read_checkpoint(model_dir: str | Path) -> dict[str, torch.Tensor]:
    """Every ``*.safetensors`` file of a directory merged into one name -> tensor map."""
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file under {model_dir}")
    out: dict[str, torch.Tensor] = {}
    for f in files:
        out.update(read_safetensors(f))
    return out


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor]) -> None:
    """The inverse of :func:`read_safetensors` (tests and tools write small checkpoints with it)."""
    names = {v: k for k, v in _DTYPES.items()}
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
