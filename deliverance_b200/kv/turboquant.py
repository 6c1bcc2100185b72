"""MSE "TurboQuant" codec for KV snapshots and compressed host / disk copies of prefix pages.

Pipeline per row (reference: core/.../tensor/MseTurboQuantCodec.java:12-22,84-160): take the row norm, normalise, rotate with a
fixed random sign flip followed by a Walsh-Hadamard transform (after which coordinates are close to Gaussian with variance
1/d), quantise every coordinate with a Lloyd-Max scalar codebook for that distribution (1..8 bits), pack the codes, keep the
norm in fp32. Decoding looks the centroids up, undoes the rotation and rescales. On the GPU the live KV pages are shared by
reference count and never compressed; this codec serves exported snapshots (``snapshot_pages`` / ``restore_pages``) where
the reference's 94 MB -> 11.9 MB figure applies (core/prefix_cache_turboquant.md:33-37).
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass

import torch


def block_compress(raw: bytes, codec: str) -> bytes:
    """``LZ4``: the LZ4 block format (the extension's host codec, csrc/lz4_block.cpp); ``DEFLATE``: zlib level 1."""
    if codec == "DEFLATE":
        return zlib.compress(raw, 1)
    from ..ops import require_ext

    return require_ext().lz4_compress(raw)


def block_decompress(data: bytes, n_out: int, codec: str) -> bytes:
    if codec == "DEFLATE":
        return zlib.decompress(data)
    from ..ops import require_ext

    return require_ext().lz4_decompress(data, n_out)


def _hadamard(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised fast Walsh-Hadamard transform over the last dimension (a power of two)."""
    d = x.shape[-1]
    h = 1
    y = x.clone()
    while h < d:
        y = y.reshape(*y.shape[:-1], d // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], dim=-2).reshape(*x.shape[:-1], d)
        h *= 2
    return y


def lloyd_max_gaussian(bits: int, iters: int = 60) -> torch.Tensor:
    """Centroids of the Lloyd-Max quantiser of a unit Gaussian (2^bits levels)."""
    n = 1 << bits
    g = torch.Generator().manual_seed(1234)
    samples = torch.randn(200_000, generator=g).sort().values
    c = torch.quantile(samples, (torch.arange(n, dtype=torch.float32) + 0.5) / n)
    for _ in range(iters):
        edges = (c[1:] + c[:-1]) / 2
        idx = torch.bucketize(samples, edges)
        sums = torch.zeros(n).index_add_(0, idx, samples)
        cnt = torch.zeros(n).index_add_(0, idx, torch.ones_like(samples)).clamp_min(1)
        c = sums / cnt
    return c


@dataclass
class Encoded:
    codes: torch.Tensor  # uint8 packed
    norms: torch.Tensor  # fp32 [rows]
    shape: tuple
    bits: int


class MseTurboQuantCodec:
    def __init__(self, dim: int, bits: int = 3, seed: int = 7):
        if not 1 <= bits <= 8:
            raise ValueError("bits must be 1..8")
        self.dim = dim
        self.pdim = 1 << max(0, math.ceil(math.log2(dim)))
        self.bits = bits
        g = torch.Generator().manual_seed(seed)
        self.signs = (torch.randint(0, 2, (self.pdim,), generator=g) * 2 - 1).float()
        self.centroids = lloyd_max_gaussian(bits)
        self.edges = (self.centroids[1:] + self.centroids[:-1]) / 2

    def _device_tables(self, device):
        tables = self.__dict__.setdefault("_tables", {})
        key = str(torch.device(device))
        if key not in tables:
            tables[key] = (self.signs.to(device), self.edges.to(device), self.centroids.to(device))
        return tables[key]

    def encode(self, x: torch.Tensor) -> Encoded:
        if x.is_cuda and 32 <= self.pdim <= 1024 and x.dtype in (torch.float32, torch.bfloat16):
            # one kernel per tensor on the device that holds the pages (csrc/aux.cu::tq_encode_kernel); only codes and norms cross PCIe
            from ..ops import require_ext

            signs, edges, _ = self._device_tables(x.device)
            codes, norms = require_ext().tq_encode(x.reshape(-1, self.dim).contiguous(), signs, edges, self.bits)
            return Encoded(codes.reshape(-1).cpu(), norms.cpu(), tuple(x.shape), self.bits)
        rows = x.reshape(-1, self.dim).float().cpu()
        norms = rows.norm(dim=1)
        unit = rows / norms.clamp_min(1e-20).unsqueeze(1)
        if self.pdim != self.dim:
            unit = torch.nn.functional.pad(unit, (0, self.pdim - self.dim))
        rot = _hadamard(unit * self.signs) / math.sqrt(self.pdim)  # orthonormal
        z = rot * math.sqrt(self.pdim)  # ~ N(0, 1) per coordinate
        codes = torch.bucketize(z, self.edges).to(torch.uint8)
        return Encoded(self._pack(codes), norms, tuple(x.shape), self.bits)

    def decode(self, e: Encoded, dtype=torch.float32, device=None) -> torch.Tensor:
        if device is not None and torch.device(device).type == "cuda" and 32 <= self.pdim <= 1024 and dtype in (torch.float32, torch.bfloat16):
            from ..ops import require_ext

            signs, _, centroids = self._device_tables(torch.device(device))
            out = require_ext().tq_decode(e.codes.reshape(e.norms.numel(), -1).to(device), e.norms.to(device), signs, centroids, self.dim, self.bits,
                                          dtype == torch.bfloat16)
            return out.reshape(e.shape)
        rows = e.norms.numel()
        codes = self._unpack(e.codes, rows * self.pdim).reshape(rows, self.pdim).long()
        z = self.centroids[codes] / math.sqrt(self.pdim)
        unit = _hadamard(z) / math.sqrt(self.pdim) * self.signs
        out = unit[:, : self.dim] * e.norms.unsqueeze(1)
        return out.reshape(e.shape).to(dtype)

    def _pack(self, codes: torch.Tensor) -> torch.Tensor:
        flat = codes.reshape(-1).to(torch.int64)
        nbits = flat.numel() * self.bits
        bitpos = torch.arange(self.bits).unsqueeze(0)
        bits = ((flat.unsqueeze(1) >> bitpos) & 1).reshape(-1).to(torch.uint8)
        pad = (-nbits) % 8
        if pad:
            bits = torch.cat([bits, torch.zeros(pad, dtype=torch.uint8)])
        b = bits.reshape(-1, 8).to(torch.int64)
        return (b << torch.arange(8)).sum(dim=1).to(torch.uint8)

    def _unpack(self, packed: torch.Tensor, n: int) -> torch.Tensor:
        bits = ((packed.to(torch.int64).unsqueeze(1) >> torch.arange(8)) & 1).reshape(-1)[: n * self.bits]
        return (bits.reshape(n, self.bits) << torch.arange(self.bits)).sum(dim=1)

    def compressed_bytes(self, e: Encoded) -> int:
        return e.codes.numel() + e.norms.numel() * 4


def snapshot_pages(kv, pages: list[int], n_tokens: int, compression: str = "NONE", bits: int = 3) -> dict:
    """Host copy of the K/V rows of ``pages`` for every attention layer (``NONE`` | ``LZ4`` | ``DEFLATE`` | ``MSE_TURBOQUANT``)."""
    out = {"compression": compression, "n_tokens": n_tokens, "layers": {}}
    codec = None
    for i, k in enumerate(kv.k):
        if k is None:
            continue
        kk, vv = kv.gather_rows(i, pages, n_tokens)
        if compression == "MSE_TURBOQUANT":
            codec = codec or MseTurboQuantCodec(kk.shape[-1], bits)
            out["layers"][i] = (codec.encode(kk), codec.encode(vv))
        elif compression in ("LZ4", "DEFLATE"):
            raw = lambda t: (block_compress(t.cpu().contiguous().view(torch.uint8).numpy().tobytes(), compression), tuple(t.shape), t.dtype)  # noqa: E731
            out["layers"][i] = (raw(kk), raw(vv))
        else:
            out["layers"][i] = (kk.cpu().clone(), vv.cpu().clone())
    out["codec"] = codec
    return out


def restore_pages(kv, snap: dict, pages: list[int]) -> None:
    """Write a snapshot back into ``pages`` (allocated by the caller)."""
    n = snap["n_tokens"]
    ps = kv.page_size
    for i, (ek, ev) in snap["layers"].items():
        if snap["compression"] == "MSE_TURBOQUANT":
            dt = kv.k[i].dtype if kv.k[i].dtype in (torch.float32, torch.bfloat16) else torch.float32
            kk, vv = snap["codec"].decode(ek, dt, kv.device), snap["codec"].decode(ev, dt, kv.device)
        elif snap["compression"] in ("LZ4", "DEFLATE"):
            def un(e):
                n_out = int(torch.tensor(e[1]).prod().item()) * torch.empty(0, dtype=e[2]).element_size()
                return torch.frombuffer(bytearray(block_decompress(e[0], n_out, snap["compression"])), dtype=torch.uint8).view(e[2]).reshape(e[1])

            kk, vv = un(ek), un(ev)
        else:
            kk, vv = ek, ev
        for p_i, page in enumerate(pages[: (n + ps - 1) // ps]):
            a, b = p_i * ps, min(n, (p_i + 1) * ps)
            kv.k[i][page, :, : b - a] = kk[:, a:b].to(kv.k[i].dtype).to(kv.device)
            kv.v[i][page, :, : b - a] = vv[:, a:b].to(kv.v[i].dtype).to(kv.device)
