"""``DTEN`` binary tensor payload: the wire format of the reference's tensor-parallel transports.

Layout (little endian): ``magic 0x4454454E ("DTEN") | version 1 | dtype ordinal | ndims | dims... | u64 byte count | raw
data``; the reference only ships F32 payloads (core/.../model/tensorparallel/transport/BinaryTensorPayloadCodec.java:14-81).
The dtype ordinal is the position in the reference's ``DType`` enum (tensor/.../DType.java:3-33). Kept so that tools
written against the reference's rank / collective servers can exchange tensors with this code base; the GPU path never
serialises tensors (ranks share NVLink peer memory).
"""
from __future__ import annotations

import struct

import torch

MAGIC = 0x4454454E
VERSION = 1
_ORDINALS = ["BOOL", "U8", "I8", "I16", "U16", "F16", "BF16", "I32", "U32", "F32", "F64", "I64", "U64", "Q4"]
_TORCH = {"BOOL": torch.bool, "U8": torch.uint8, "I8": torch.int8, "I16": torch.int16, "F16": torch.float16, "BF16": torch.bfloat16,
          "I32": torch.int32, "F32": torch.float32, "F64": torch.float64, "I64": torch.int64}
_NAMES = {v: k for k, v in _TORCH.items()}


def encode(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    name = _NAMES.get(t.dtype)
    if name is None:
        raise ValueError(f"unsupported dtype {t.dtype}")
    raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
    head = struct.pack("<IIII", MAGIC, VERSION, _ORDINALS.index(name), t.dim())
    dims = struct.pack("<" + "I" * t.dim(), *t.shape) if t.dim() else b""
    return head + dims + struct.pack("<Q", len(raw)) + raw


def decode(buf: bytes) -> torch.Tensor:
    if len(buf) < 16:
        raise ValueError("DTEN payload too short")
    magic, version, ordinal, nd = struct.unpack_from("<IIII", buf, 0)
    if magic != MAGIC:
        raise ValueError(f"bad DTEN magic 0x{magic:08X}")
    if version != VERSION:
        raise ValueError(f"unsupported DTEN version {version}")
    if ordinal >= len(_ORDINALS) or _ORDINALS[ordinal] not in _TORCH:
        raise ValueError(f"unsupported DTEN dtype ordinal {ordinal}")
    off = 16
    dims = struct.unpack_from("<" + "I" * nd, buf, off) if nd else ()
    off += 4 * nd
    (nbytes,) = struct.unpack_from("<Q", buf, off)
    off += 8
    if off + nbytes > len(buf):
        raise ValueError("DTEN payload truncated")
    dt = _TORCH[_ORDINALS[ordinal]]
    numel = 1
    for d in dims:
        numel *= d
    if numel * torch.empty((), dtype=dt).element_size() != nbytes:
        raise ValueError("DTEN byte count does not match the shape")
    if numel == 0:
        return torch.empty(dims, dtype=dt)
    return torch.frombuffer(bytearray(buf[off : off + nbytes]), dtype=dt).reshape(dims).clone()
