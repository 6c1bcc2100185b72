"""Safetensors reader/writer that understands the non-standard ``"Q4"`` dtype and ``.qb`` scale sidecars.

File layout: ``u64 LE header_len | JSON header | data``; the header maps a tensor name to
``{dtype, shape, data_offsets}`` plus an optional ``__metadata__`` entry. A ``"Q4"`` entry records the *logical*
shape and carries ``numel / 2`` payload bytes; its scales live in ``<name>.qb`` (``F32``, ``[..., cols/32]``)
(reference: safetensors/src/main/java/io/teknek/deliverance/safetensors/DefaultWeightLoader.java:198-240,
SafeTensorWriter.java:100-160, Weights.java:133-136). Multi-file checkpoints use
``model.safetensors.index.json`` with ``{metadata, weight_map}``.

Files are mapped with ``mmap`` and tensors are zero-copy views until they are moved to a device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Iterable, Mapping

import torch

from .jq4 import BLOCK

_DTYPES: dict[str, tuple[torch.dtype, int]] = {
    "BOOL": (torch.bool, 1),
    "U8": (torch.uint8, 1),
    "I8": (torch.int8, 1),
    "I16": (torch.int16, 2),
    "U16": (torch.uint16, 2),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "U32": (torch.uint32, 4),
    "F32": (torch.float32, 4),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "U64": (torch.uint64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}

INDEX_FILE = "model.safetensors.index.json"
SINGLE_FILE = "model.safetensors"


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


@dataclass
class Q4Tensor:
    """A JQ4 weight: packed nibbles ``[..., cols/2]`` uint8 + scales ``[..., cols/32]`` f32 and its logical shape."""

    packed: torch.Tensor
    scales: torch.Tensor
    shape: tuple[int, ...]

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        from .jq4 import q4_dequantize

        return q4_dequantize(self.packed, self.scales, dtype).reshape(self.shape)

    def to(self, device) -> "Q4Tensor":
        return Q4Tensor(self.packed.to(device), self.scales.to(device), self.shape)


def _view(raw, dtype) -> torch.Tensor:
    """Zero-copy tensor over a read-only mapping. Loaded weights are never written in place (every consumer converts or copies
    them to the device), so torch's warning about non-writable buffers is silenced here."""
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)
        return torch.frombuffer(raw, dtype=dtype)


class SafeTensorFile:
    """One mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise ValueError(f"{path}: too small to be a safetensors file")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if 8 + hlen > size:
            raise ValueError(f"{path}: header length {hlen} exceeds file size {size}")
        header = json.loads(self._mm[8 : 8 + hlen].decode("utf-8"))
        self.metadata: dict = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        self.infos: dict[str, TensorInfo] = {}
        for name, ent in header.items():
            b, e = ent["data_offsets"]
            self.infos[name] = TensorInfo(name, ent["dtype"], tuple(int(s) for s in ent["shape"]), int(b), int(e))
        self._buf = memoryview(self._mm)

    def names(self) -> list[str]:
        return list(self.infos)

    def raw(self, name: str) -> memoryview:
        info = self.infos[name]
        return self._buf[self._data_start + info.begin : self._data_start + info.end]

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy view of a dense entry (or of the packed bytes of a ``Q4`` entry)."""
        info = self.infos[name]
        raw = self.raw(name)
        if info.dtype == "Q4":
            numel = 1
            for s in info.shape:
                numel *= s
            if len(raw) != numel // 2:
                raise ValueError(f"{name}: Q4 payload has {len(raw)} bytes, expected {numel // 2}")
            t = _view(raw, torch.uint8) if len(raw) else torch.empty(0, dtype=torch.uint8)
            return t.reshape(*info.shape[:-1], info.shape[-1] // 2)
        dt, size = _DTYPES[info.dtype]
        numel = 1
        for s in info.shape:
            numel *= s
        if len(raw) != numel * size:
            raise ValueError(f"{name}: payload has {len(raw)} bytes, expected {numel * size}")
        if numel == 0:
            return torch.empty(info.shape, dtype=dt)
        return _view(raw, dt).reshape(info.shape)

    def close(self) -> None:
        try:
            self._buf.release()
            self._mm.close()
        except (BufferError, ValueError):
            pass  # live tensor views keep the mapping alive; the OS reclaims it with the process
        self._fh.close()


def _payload(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.numel() == 0:
        return b""
    return t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.uint8 else t.numpy().tobytes()


def canonical_shape(shape: Iterable[int]) -> list[int]:
    """1-D tensors are rewritten as ``[1, N]`` (reference SafeTensorWriter.java:150-155)."""
    shape = [int(s) for s in shape]
    return [1, shape[0]] if len(shape) == 1 else shape


def write_safetensors(
    path: str,
    tensors: Mapping[str, "torch.Tensor | Q4Tensor"],
    metadata: Mapping[str, str] | None = None,
    canonicalize_1d: bool = False,
) -> None:
    """Write one file. A :class:`Q4Tensor` value produces the ``Q4`` entry followed by its ``.qb`` sidecar."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    payloads: list[bytes] = []
    offset = 0

    def add(name: str, dtype: str, shape, data: bytes):
        nonlocal offset
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + len(data)]}
        payloads.append(data)
        offset += len(data)

    for name, t in tensors.items():
        if isinstance(t, Q4Tensor):
            shape = canonical_shape(t.shape) if canonicalize_1d else list(t.shape)
            add(name, "Q4", shape, _payload(t.packed))
            qshape = list(shape)
            qshape[-1] = qshape[-1] // BLOCK
            add(name + ".qb", "F32", qshape, _payload(t.scales.to(torch.float32)))
        else:
            if t.dtype not in _NAMES:
                raise ValueError(f"{name}: unsupported dtype {t.dtype}")
            shape = canonical_shape(t.shape) if canonicalize_1d else list(t.shape)
            add(name, _NAMES[t.dtype], shape, _payload(t))
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for p in payloads:
            f.write(p)
    os.replace(tmp, path)


def write_sharded(
    out_dir: str,
    tensors: Mapping[str, "torch.Tensor | Q4Tensor"],
    max_shard_bytes: int = 5 << 30,
    metadata: Mapping[str, str] | None = None,
    canonicalize_1d: bool = False,
) -> list[str]:
    """Shards named ``model-%05d.safetensors`` plus the index json (reference ModelQuantizer.java:35-37,151-154)."""
    os.makedirs(out_dir, exist_ok=True)
    shards: list[dict] = [{}]
    size = 0
    for name, t in tensors.items():
        n = (t.packed.numel() + t.scales.numel() * 4) if isinstance(t, Q4Tensor) else t.numel() * t.element_size()
        if shards[-1] and size + n > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][name] = t
        size += n
    files = []
    weight_map: dict[str, str] = {}
    total = 0
    for i, sh in enumerate(shards):
        fname = "model-%05d.safetensors" % (i + 1)
        write_safetensors(os.path.join(out_dir, fname), sh, metadata, canonicalize_1d)
        files.append(fname)
        for name, t in sh.items():
            weight_map[name] = fname
            if isinstance(t, Q4Tensor):
                weight_map[name + ".qb"] = fname
                total += t.packed.numel() + t.scales.numel() * 4
            else:
                total += t.numel() * t.element_size()
    with open(os.path.join(out_dir, INDEX_FILE), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    return files
