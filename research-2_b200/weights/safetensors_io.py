"""Reading and writing the safetensors container.

The format is an 8-byte little-endian header length, a JSON header (name -> dtype, shape,
data_offsets relative to the end of the header) and the raw little-endian tensor bytes
(the reference reads the same header: kelpie-models/kelpie_models/sdk/hf.py:132-150). Tensors
are returned in the dtype the file stores: nothing is converted here.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F64": torch.float64,
    "I32": torch.int32,
    "I64": torch.int64,
    "U8": torch.uint8,
}
_NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: str | Path) -> tuple[dict, int]:
    """(header dict without __metadata__, offset of the data section)."""
    path = Path(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", raw)
        size = path.stat().st_size
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n))
        except json.JSONDecodeError as err:
            raise SafetensorsError(f"{path}: header is not valid JSON ({err})") from None
    header.pop("__metadata__", None)
    return header, 8 + n


def read_file(path: str | Path) -> dict[str, torch.Tensor]:
    """Every tensor of one file by name. The tensors are copies (the mapping is closed)."""
    path = Path(path)
    header, base = read_header(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY) as mm:
        for name, info in header.items():
            dtype = DTYPES.get(info["dtype"])
            if dtype is None:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {info['dtype']!r}")
            begin, end = info["data_offsets"]
            shape = tuple(info["shape"])
            count = 1
            for s in shape:
                count *= s
            itemsize = torch.empty((), dtype=dtype).element_size()
            if end - begin != count * itemsize or base + end > len(mm):
                raise SafetensorsError(
                    f"{path}: tensor {name!r} with shape {shape} and dtype {info['dtype']} "
                    f"does not match its {end - begin} bytes"
                )
            if count == 0:
                out[name] = torch.empty(shape, dtype=dtype)
                continue
            flat = torch.frombuffer(mm, dtype=dtype, count=count, offset=base + begin)
            out[name] = flat.clone().reshape(shape)
            del flat
    return out


def read_folder(model_dir: str | Path) -> dict[str, torch.Tensor]:
    """All `*.safetensors` files of a folder, in sorted order, as one dict
    (kelpie-models/kelpie_models/sdk/hf.py:27-50)."""
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise SafetensorsError(f"{model_dir}: no .safetensors file in the model folder")
    out: dict[str, torch.Tensor] = {}
    for file in files:
        out.update(read_file(file))
    return out


def write_file(path: str | Path, tensors: dict[str, torch.Tensor]) -> None:
    header: dict = {}
    blobs: list[bytes] = []
    offset = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        data = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(data)]}
        blobs.append(data)
        offset += len(data)
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for blob in blobs:
            f.write(blob)
