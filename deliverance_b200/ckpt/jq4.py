"""JQ4 packed 4-bit weight format and the block-32 int8 (Q8/"I8") activation format.

Format facts (reference: tensor/src/main/java/io/teknek/deliverance/tensor/impl/Q4ByteBufferTensor.java:55-109,
safetensors/src/main/java/io/teknek/deliverance/safetensors/ModelQuantizer.java:491-531,
native/src/main/c/simd/vector_simd.c:1122-1143):

* a block is 32 consecutive elements in row-major flat order;
* ``scale = v_max / -8`` where ``v_max`` is the *signed* value of the first element with the largest magnitude,
  ``inv = 1/scale`` (0 when scale is 0);
* ``q = min(15, trunc(v * inv + 8.5))``;
* byte ``j`` (0..15) of a block holds ``q[j] | q[j + 16] << 4`` ("split-half" packing), 16 bytes per block;
* dequantised value = ``(nibble - 8) * scale``;
* the scales live in a float32 sidecar tensor of shape ``[..., cols / 32]``.

Everything here is vectorised torch on the host so that it is bit-exact with the scalar definition above and can
also run on a CUDA device (the device quantiser kernel in ``ops`` is tested against this file).
"""
from __future__ import annotations

import torch

BLOCK = 32
HALF = 16


def q4_quantize(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``w`` (any float dtype, last dim % 32 == 0) to (packed uint8 ``[..., cols/2]``, scales f32 ``[..., cols/32]``)."""
    if w.shape[-1] % BLOCK != 0:
        raise ValueError(f"JQ4 needs the last dimension to be a multiple of {BLOCK}, got {tuple(w.shape)}")
    lead = w.shape[:-1]
    cols = w.shape[-1]
    blocks = w.to(torch.float32).reshape(-1, BLOCK)
    absv = blocks.abs()
    # first element with the largest magnitude (strict '>' in the scalar loop keeps the first one)
    idx = torch.argmax(absv, dim=1, keepdim=True)
    # torch.argmax returns the first maximal index on CPU and CUDA for ties
    vmax = torch.gather(blocks, 1, idx).squeeze(1)
    # The scalar loop starts from Float.MIN_VALUE: an all-zero block keeps max = MIN_VALUE and scale = -0.0
    all_zero = absv.amax(dim=1) == 0
    scale = vmax / -8.0
    scale = torch.where(all_zero, torch.full_like(scale, -0.0), scale)
    inv = torch.where(scale != 0, 1.0 / scale, torch.zeros_like(scale))
    f = blocks * inv.unsqueeze(1) + 8.5
    f = torch.nan_to_num(f, nan=0.0, posinf=127.0, neginf=-128.0)
    q = torch.clamp(torch.trunc(f), max=15).to(torch.int32) & 0xFF
    q = torch.clamp(q, max=15)  # a negative trunc wraps through (byte); values never go below 0 here
    lo = q[:, :HALF]
    hi = q[:, HALF:]
    packed = (lo | (hi << 4)).to(torch.uint8)
    return packed.reshape(*lead, cols // 2), scale.reshape(*lead, cols // BLOCK)


def q4_dequantize(packed: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse of :func:`q4_quantize`: ``(nibble - 8) * scale`` in fp32, then cast to ``dtype``."""
    lead = packed.shape[:-1]
    cols = packed.shape[-1] * 2
    b = packed.reshape(-1, HALF).to(torch.int32)
    lo = (b & 0xF) - 8
    hi = ((b >> 4) & 0xF) - 8
    vals = torch.cat([lo, hi], dim=1).to(torch.float32) * scales.reshape(-1, 1).to(torch.float32)
    return vals.reshape(*lead, cols).to(dtype)


def q8_quantize(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Block-32 int8 quantisation: ``scale = max|v| / 127``, ``q = round(v * 127 / max)``
    (reference: tensor/src/main/java/io/teknek/deliverance/tensor/impl/Q8ByteBufferTensor.java:57-79)."""
    if x.shape[-1] % BLOCK != 0:
        raise ValueError("Q8 needs the last dimension to be a multiple of 32")
    lead = x.shape[:-1]
    cols = x.shape[-1]
    blocks = x.to(torch.float32).reshape(-1, BLOCK)
    amax = blocks.abs().amax(dim=1)
    scale = amax / 127.0
    inv = torch.where(scale != 0, 1.0 / scale, torch.zeros_like(scale))
    q = torch.round(blocks * inv.unsqueeze(1)).clamp(-127, 127).to(torch.int8)
    return q.reshape(*lead, cols), scale.reshape(*lead, cols // BLOCK)


def q8_dequantize(q: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    lead = q.shape[:-1]
    cols = q.shape[-1]
    vals = q.reshape(-1, BLOCK).to(torch.float32) * scales.reshape(-1, 1)
    return vals.reshape(*lead, cols).to(dtype)


def q4_scalar_reference(values: list[float]) -> tuple[bytes, float]:
    """Plain-Python restatement of one block, used by the tests as an independent oracle."""
    import struct

    def f32(v: float) -> float:
        return struct.unpack("<f", struct.pack("<f", v))[0]

    assert len(values) == BLOCK
    vmax, amax = 1.401298464324817e-45, 1.401298464324817e-45
    for v in values:
        a = -v if v < 0 else v
        if a > amax:
            vmax, amax = v, a
    scale = f32(vmax / -8.0)
    inv = f32(1.0 / scale) if scale != 0.0 else 0.0
    out = bytearray(HALF)
    for j in range(HALF):
        q0 = min(15, int(f32(f32(values[j] * inv) + 8.5)))
        q1 = min(15, int(f32(f32(values[j + HALF] * inv) + 8.5)))
        out[j] = (q0 | (q1 << 4)) & 0xFF
    return bytes(out), scale
