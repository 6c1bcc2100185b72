"""Op surface of the framework.

Every function dispatches on the device of its inputs: CUDA tensors run the hand-written sm_100a kernels of the in-tree
extension (and raise if that extension is missing — there is no silent eager fallback on a GPU box); CPU tensors run the
plain PyTorch statements in :mod:`.ref` (fp32 oracle, CPU tests, the TinyLlama-shape fp32 plumbing configuration).

The surface mirrors the reference's ``TensorOperations`` SPI (tensor/.../operations/TensorOperations.java:12-283):
GEMM with shared-input batches (fused qkv / gate|up weights), accumulate/scale (folded into norm + residual kernels),
quantize, activation-multiply, gather-rows-add (embedding), paged decode attention.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import ref
from .build import load_extension
from ..ckpt.safetensors_io import Q4Tensor

_ext = None
_ext_checked = False
# number of kernels of this extension launched so far (each op adds what it launches; benchmarks read the difference)
LAUNCHES = [0]


def _count(n: int = 1) -> None:
    LAUNCHES[0] += n


def ext():
    """The compiled extension, or ``None`` when it has not been built."""
    global _ext, _ext_checked
    if not _ext_checked:
        _ext = load_extension()
        _ext_checked = True
        if _ext is not None and os.environ.get("DLV_GEMM_PDL", "1") == "0":
            _ext.gemm_pdl(False)
        persist = os.environ.get("DLV_GEMM_PERSIST", "0")
        if _ext is not None and persist in ("1", "race"):
            _ext.gemm_persist(True, False, persist != "race")
        if _ext is not None and os.environ.get("DLV_DECODE_MERGE", "launch") == "kernel":
            _MERGE_IN_KERNEL[0] = True
            _ext.decode_merge_in_kernel(True)
        if _ext is not None and os.environ.get("DLV_GEMV_MAX_ROWS", "") in ("16", "0"):  # comparisons: 9..16 rows on the GEMV too, or none
            set_gemv_max_rows(int(os.environ["DLV_GEMV_MAX_ROWS"]))
        if _ext is not None and os.environ.get("DLV_BOUNDS_CHECK", "0") == "1":
            _ext.set_bounds_check(True)
    return _ext


def set_gemm_pdl(on: bool) -> None:
    """Programmatic dependent launch of the GEMM kernels (their prologue and weight prefetch overlap the previous kernel's tail)."""
    require_ext().gemm_pdl(bool(on))


def require_ext():
    e = ext()
    if e is None:
        raise RuntimeError(
            "deliverance_b200 CUDA extension is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(or `python -m deliverance_b200.ops.build`) before using CUDA tensors")
    return e


def _cuda(t: torch.Tensor) -> bool:
    return t.device.type == "cuda"


def check_status(device: Optional[int] = None) -> None:
    """Raise if a kernel on ``device`` recorded a wait that ran out (bounded mbarrier / flag waits)."""
    e = ext()
    if e is None or not torch.cuda.is_available():
        return
    dev = torch.cuda.current_device() if device is None else device
    code = e.take_status(dev)
    if code:
        names = {1: "an mbarrier wait ran out of time", 2: "a peer-flag wait ran out of time", 3: "bad kernel arguments"}
        raise RuntimeError(f"deliverance_b200 kernel status {code}: {names.get(code, 'unknown')}")


def set_bounds_check(on: bool = True) -> None:
    """Guard areas around every output the extension's kernels write (4 KB of a byte pattern on both sides); ``check_guards``
    verifies them. Also switched on by ``DLV_BOUNDS_CHECK=1`` in the environment. A debugging mode: outputs cost an extra fill."""
    e = ext()
    if e is not None:
        e.set_bounds_check(bool(on))


def check_guards() -> None:
    """Raise if a kernel wrote outside one of the outputs allocated since the last call (bounds checking must be on)."""
    e = ext()
    if e is None or not torch.cuda.is_available():
        return
    bad = e.check_guards()
    if bad:
        raise RuntimeError("deliverance_b200: a kernel wrote outside " + "; ".join(bad))


# ---------------------------------------------------------------------------------------------------------- linear
Q4_STAGE_BYTES = 10240


def _q4_swizzle_index(device) -> torch.Tensor:
    r = torch.arange(128, device=device)
    c = torch.arange(4, device=device)
    return c.unsqueeze(0) ^ ((r >> 1) & 3).unsqueeze(1)  # [row, chunk position] -> logical 32-element block


def prepack_q4(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Tile-pack a JQ4 weight for the tensor-core GEMM: ``[N, K/2]`` nibbles + ``[N, K/32]`` scales ->
    ``[ceil(N/128), ceil(K/128), 10240]`` bytes. One 10240-byte stage is a 128-row x 128-k tile: 8192 bytes of packed
    nibbles (row ``r`` at ``r*64``; its four 16-byte blocks stored at chunk ``block ^ ((r >> 1) & 3)``, which makes the
    shared-memory reads of the dequantising warps conflict-free) followed by 2048 bytes of fp32 scales ``[row][4]``.
    Padding rows / k carry zero scales. A stage is one contiguous DRAM burst and one bulk copy in the kernel."""
    N, half = packed.shape
    K = half * 2
    NT, KB = (N + 127) // 128, (K + 127) // 128
    dev = packed.device
    pk = torch.zeros(NT * 128, KB * 64, dtype=torch.uint8, device=dev)
    pk[:N, :half] = packed
    sc = torch.zeros(NT * 128, KB * 4, dtype=torch.float32, device=dev)
    sc[:N, : K // 32] = scales[:, : K // 32]
    raw = pk.view(NT, 128, KB, 4, 16).permute(0, 2, 1, 3, 4)  # nt, kb, row, block, 16 B
    idx = _q4_swizzle_index(dev).view(1, 1, 128, 4, 1).expand(NT, KB, 128, 4, 16)
    raw = torch.gather(raw, 3, idx).reshape(NT, KB, 8192)
    scb = sc.view(NT, 128, KB, 4).permute(0, 2, 1, 3).contiguous().view(torch.uint8).reshape(NT, KB, 2048)
    return torch.cat([raw, scb], dim=2).contiguous()


def unpack_q4(tiles: torch.Tensor, N: int, K: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`prepack_q4`: returns (packed ``[N, K/2]``, scales ``[N, K/32]``)."""
    NT, KB, _ = tiles.shape
    dev = tiles.device
    raw = tiles[:, :, :8192].reshape(NT, KB, 128, 4, 16)
    idx = _q4_swizzle_index(dev).view(1, 1, 128, 4, 1).expand(NT, KB, 128, 4, 16)
    raw = torch.gather(raw, 3, idx)  # the xor swizzle is its own inverse
    packed = raw.permute(0, 2, 1, 3, 4).reshape(NT * 128, KB * 64)[:N, : K // 2].contiguous()
    sc = tiles[:, :, 8192:].contiguous().view(torch.float32).reshape(NT, KB, 128, 4).permute(0, 2, 1, 3).reshape(NT * 128, KB * 4)
    return packed, sc[:N, : K // 32].contiguous()


class LinearWeight:
    """A ``[N, K]`` projection weight, dense (bf16 on CUDA, fp32 on CPU) or JQ4. JQ4 weights keep the checkpoint layout
    (packed + scales) on the CPU and the tile-packed layout of :func:`prepack_q4` on CUDA devices."""

    def __init__(self, w: "torch.Tensor | Q4Tensor", bias: Optional[torch.Tensor] = None):
        self.bias = bias
        self._handle = None
        self.tiles = None
        if isinstance(w, Q4Tensor):
            self.q4 = True
            self.packed = w.packed.reshape(-1, w.packed.shape[-1]).contiguous()
            self.scales = w.scales.reshape(-1, w.scales.shape[-1]).contiguous().to(torch.float32)
            self.N, self.K = int(self.packed.shape[0]), int(self.packed.shape[1]) * 2
            self.w = None
        else:
            self.q4 = False
            self.w = w.contiguous()
            self.N, self.K = int(w.shape[0]), int(w.shape[1])
            self.packed = self.scales = None

    @property
    def device(self) -> torch.device:
        if self.q4:
            return (self.tiles if self.tiles is not None else self.packed).device
        return self.w.device

    def to(self, device, dtype: Optional[torch.dtype] = None) -> "LinearWeight":
        device = torch.device(device)
        bias = None if self.bias is None else self.bias.to(device=device, dtype=torch.float32)
        if self.q4:
            out = LinearWeight.__new__(LinearWeight)
            out.q4, out.N, out.K, out.w, out._handle, out.bias = True, self.N, self.K, None, None, bias
            packed, scales = self.checkpoint_layout()
            if device.type == "cuda":
                out.tiles = prepack_q4(packed.to(device), scales.to(device))
                out.packed = out.scales = None
            else:
                out.tiles = None
                out.packed, out.scales = packed.to(device), scales.to(device)
            return out
        return LinearWeight(self.w.to(device=device, dtype=dtype or self.w.dtype), bias)

    def checkpoint_layout(self) -> tuple[torch.Tensor, torch.Tensor]:
        """(packed ``[N, K/2]``, scales ``[N, K/32]``) whatever the resident layout is."""
        if self.tiles is not None:
            return unpack_q4(self.tiles, self.N, self.K)
        return self.packed, self.scales

    def dense(self, dtype=torch.float32) -> torch.Tensor:
        if self.q4:
            from ..ckpt.jq4 import q4_dequantize

            p, s = self.checkpoint_layout()
            return q4_dequantize(p, s, dtype)
        return self.w.to(dtype)

    def handle(self):
        if self._handle is None:
            e = require_ext()
            if self.q4:
                if self.tiles is None:
                    raise RuntimeError("JQ4 weight is not on a CUDA device")
                self._handle = e.GemmWeight(self.tiles, True, self.N, self.K)
            else:
                if self.w.dtype != torch.bfloat16:
                    self.w = self.w.to(torch.bfloat16)
                self._handle = e.GemmWeight(self.w, False, self.N, self.K)
            if self.bias is not None and self.bias.dtype != torch.float32:
                self.bias = self.bias.float()
        return self._handle

    def nbytes(self) -> int:
        if self.q4:
            return self.tiles.numel() if self.tiles is not None else self.packed.numel() + self.scales.numel() * 4
        return self.w.numel() * self.w.element_size()


def linear(x: torch.Tensor, w: LinearWeight, out_f32: bool = False, impl: int = 0, force_splits: int = 0,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [T, K] @ W[N, K]^T (+ bias)``."""
    if _cuda(x):
        _count()
        return w.handle().run(x, out, w.bias, out_f32, impl, force_splits)
    if w.q4:
        y = ref.linear_q4(x, w.packed, w.scales, w.bias)
    else:
        y = ref.linear_dense(x, w.w, w.bias)
    return y.float() if out_f32 else y


_ACT_KINDS = {"silu": 1, "swish": 1, "gelu_pytorch_tanh": 2, "gelu_new": 2, "gelu_tanh": 2, "gelu_fast": 2}


def fused_act_kind(act: str) -> int:
    """Code of an activation the GEMM epilogue can apply (0: none)."""
    return _ACT_KINDS.get((act or "silu").lower(), 0)


def interleave_gate_up(gate, up, block: int = 64):
    """Row order for :func:`linear_act`: blocks of ``block`` gate rows, each followed by the up rows of the same outputs, so that
    one 128-row weight tile of the GEMM holds both halves of 64 outputs. Works on dense tensors and on JQ4 tensors (rows of the
    packed nibbles and of the scales move together)."""
    from ..ckpt.safetensors_io import Q4Tensor

    def mix(a, b):
        n = a.shape[0]
        if n % block != 0 or b.shape != a.shape:
            raise ValueError(f"gate / up rows ({n}) must be equal and a multiple of {block}")
        return torch.stack([a.reshape(n // block, block, -1), b.reshape(n // block, block, -1)], dim=1).reshape(2 * n, -1).contiguous()

    if isinstance(gate, Q4Tensor) and isinstance(up, Q4Tensor):
        packed, scales = mix(gate.packed, up.packed), mix(gate.scales, up.scales)
        return Q4Tensor(packed, scales, (packed.shape[0], packed.shape[1] * 2))
    if isinstance(gate, Q4Tensor) or isinstance(up, Q4Tensor):
        gate = gate.dequantize(torch.float32) if isinstance(gate, Q4Tensor) else gate
        up = up.dequantize(torch.float32) if isinstance(up, Q4Tensor) else up
    return mix(gate, up.to(gate.dtype))


def linear_gated(x: torch.Tensor, w: LinearWeight, act: str) -> torch.Tensor:
    """``act(x @ Wg^T) * (x @ Wu^T)`` for a weight that holds the gate rows followed by the up rows (plain order). One kernel for
    1..8 rows of a JQ4 weight on CUDA (the small-batch GEMV's epilogue), projection + activation kernel otherwise."""
    if _cuda(x) and w.q4 and x.shape[0] <= GEMV_MAX_ROWS:
        kind = fused_act_kind(act)
        if kind:
            out = w.handle().run_gemv_act(x, kind)
            if out is not None:
                _count()
                return out
    return act_mul(linear(x, w), act)


def linear_act(x: torch.Tensor, w: LinearWeight, act: str, block: int = 64) -> torch.Tensor:
    """``act(x @ Wg^T) * (x @ Wu^T)`` in one GEMM whose epilogue applies the gated activation; ``w`` holds the gate and up rows in
    the order of :func:`interleave_gate_up`. Returns ``[T, N / 2]``."""
    if _cuda(x):
        kind = fused_act_kind(act)
        if kind == 0:
            raise ValueError(f"activation '{act}' is not available in the GEMM epilogue")
        _count()
        return w.handle().run_act(x, kind)
    y = ref.linear_q4(x, w.packed, w.scales, None) if w.q4 else ref.linear_dense(x, w.w, None)
    T, n2 = y.shape
    y = y.reshape(T, n2 // (2 * block), 2, block)
    g, u = y[:, :, 0, :].reshape(T, n2 // 2), y[:, :, 1, :].reshape(T, n2 // 2)
    return (ref.act_fn(act)(g.float()) * u.float()).to(x.dtype)


# ---------------------------------------------------------------------------------------------------------- norms etc.
def rmsnorm(x, w, eps, offset=0.0):
    if _cuda(x):
        _count()
        return require_ext().rmsnorm(x, w, eps, offset)
    return ref.rmsnorm(x, w, eps, offset)


def add_rmsnorm(x, residual, w, eps, offset=0.0, res_mult=1.0):
    """``residual += x * res_mult`` in place; returns ``rmsnorm(residual)``."""
    if _cuda(x):
        _count()
        return require_ext().add_rmsnorm(x, residual, w, eps, offset, res_mult)
    return ref.add_rmsnorm(x, residual, w, eps, offset, res_mult)


def layernorm(x, w, b, eps):
    if _cuda(x):
        _count()
        return require_ext().layernorm(x, w, b, eps)
    return ref.layernorm(x, w, b, eps)


def act_mul(gate_up, act):
    if _cuda(gate_up):
        _count()
        return require_ext().act_mul(gate_up, act)
    return ref.act_mul(gate_up, act)


def activation(x, act):
    if _cuda(x):
        _count()
        return require_ext().activation(x.contiguous(), act)
    return ref.act_fn(act)(x.float()).to(x.dtype)


def embedding(table, ids, scale=1.0, pos_table=None, pos=None, type_table=None, types=None, dtype=None):
    if _cuda(table):
        _count()
        return require_ext().embedding(table, ids.to(torch.int32), scale, pos_table, None if pos is None else pos.to(torch.int32),
                                       type_table, None if types is None else types.to(torch.int32))
    out = ref.embedding(table, ids, scale, torch.float32)
    if pos_table is not None:
        out = out + pos_table[pos.long()].float()
    if type_table is not None:
        out = out + (type_table[types.long()].float() if types is not None else type_table[0].float())
    return out.to(dtype or table.dtype)


def _check_full_rotary(cos, D: int) -> None:
    """The kernels rotate the pairs (d, d + D/2); a table that covers only part of the head (partial rotary embedding, where the
    pairs lie inside the rotated sub-range) would silently mean something else, so it is refused. No supported family needs it."""
    if cos is not None and cos.shape[1] * 2 != D:
        raise NotImplementedError(f"rotary table covers {cos.shape[1] * 2} of {D} head dims: partial rotary embedding is not supported by the CUDA kernels")


def rope_kv(qkv, positions, slots, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, H, KV, D, eps, norm_offset=0.0):
    """Per-head q/k RMSNorm (optional) + RoPE (optional) + paged cache write. Returns q ``[T, H*D]`` (a view on CUDA)."""
    if _cuda(qkv):
        _check_full_rotary(cos, D)
        _count()
        require_ext().rope_kv(qkv, positions.to(torch.int32), slots, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, H, KV, D, eps,
                              norm_offset)
        return qkv[:, : H * D]
    q = ref.qk_prepare_and_cache(qkv, positions.long(), slots.long(), H, KV, D, q_norm_w, k_norm_w, eps, norm_offset, cos, sin,
                                 k_cache, v_cache)
    return q.reshape(qkv.shape[0], H * D)


def linear_rope_kv(x, w: LinearWeight, positions, slots, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, H, KV, D, eps, norm_offset=0.0):
    """q|k|v projection + per-head q/k RMSNorm + RoPE + paged cache write as ONE kernel on CUDA (the GEMM epilogue does the head
    work: a 128-row weight tile is one head, so ``D`` must be 128); the oracle path composes the separate operators. Returns q
    ``[T, H*D]``."""
    if _cuda(x):
        if D != 128:
            raise ValueError("the fused q/k/v epilogue needs head_dim 128")
        _check_full_rotary(cos, D)
        if x.shape[0] <= GEMV_MAX_ROWS and w.q4 and w.handle().gemv_ok(x.shape[0], x.stride(0)):
            # a handful of rows: the small-batch GEMV plus the stand-alone rotary kernel beat the tcgen05 tile's fixed cost
            return rope_kv(linear(x, w), positions, slots, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, H, KV, D, eps, norm_offset)
        _count()
        return w.handle().run_qkv(x, positions.to(torch.int32), slots, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, H, KV, eps, norm_offset, w.bias)
    return rope_kv(linear(x, w), positions, slots, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, H, KV, D, eps, norm_offset)


def decode_splits(num_seqs: int, kv_heads: int, max_ctx: int, sms: int = 148) -> int:
    """Split-KV factor: enough CTAs for two waves, at least four 32-key tiles per split."""
    ctas = max(1, num_seqs * kv_heads)
    want = max(1, (2 * sms + ctas - 1) // ctas)
    tiles = max(1, (max_ctx + 31) // 32)
    return int(max(1, min(want, tiles // 4 if tiles >= 8 else 1, 64)))


GEMV_MAX_ROWS = 8  # JQ4 projections of at most this many token rows run on the mma.sync GEMV (16 is possible and measured slower than tcgen05)


def set_gemv_max_rows(n: int) -> None:
    """Most token rows of a JQ4 projection that go to the mma.sync GEMV (0, 8 or 16)."""
    global GEMV_MAX_ROWS
    GEMV_MAX_ROWS = int(n)
    if _ext is not None:
        _ext.gemv_max_rows(int(n))


_MERGE_IN_KERNEL = [False]


def set_decode_merge_in_kernel(on: bool) -> None:
    """Split-KV decode attention on the tensor-core kernel: merge the splits in a second launch (default) or inside the kernel, by
    the CTA that finishes last for a sequence and KV head (``DLV_DECODE_MERGE=kernel``). The second launch is the faster one
    on B200: Qwen3-4B shape, context 2048, 5.89 ms per step at batch 64 against 6.17 ms, 515 tokens/s at batch 1 against 499;
    the merge is a chain of dependent loads, which 2048 small CTAs overlap and the tail of a streaming CTA does not."""
    _MERGE_IN_KERNEL[0] = bool(on)
    if ext() is not None:
        ext().decode_merge_in_kernel(bool(on))


def decode_attention(q, k_cache, v_cache, block_tables, ctx_lens, H, scale, softcap=0.0, window=0, splits=1, impl=0):
    """One query row per sequence against the paged cache. q ``[B, H*D]`` -> ``[B, H*D]``. ``impl`` 0 = tensor-core kernel
    (GQA group as MMA rows) when the shape allows, 1 = CUDA-core kernel."""
    if _cuda(q):
        merged = impl == 0 and _MERGE_IN_KERNEL[0] and H // k_cache.shape[1] <= 16  # the last-arriving CTA merges the splits
        _count(1 if splits <= 1 or merged else 2)
        return require_ext().decode_attention(q, k_cache, v_cache, block_tables, ctx_lens, H, scale, softcap, window, splits, impl)
    B = q.shape[0]
    D = k_cache.shape[-1]
    qs = torch.arange(B)
    o = ref.paged_attention(q.reshape(B, H, D), k_cache, v_cache, block_tables, qs, torch.ones(B, dtype=torch.long), ctx_lens,
                            scale, softcap, window, True)
    return o.reshape(B, H * D)


def prefill_tiles(q_lens: list[int], tile: int = 64) -> tuple[list[int], list[int]]:
    seqs, q0s = [], []
    for i, n in enumerate(q_lens):
        for s in range(0, n, tile):
            seqs.append(i)
            q0s.append(s)
    return seqs, q0s


PREFILL_ATTN = [os.environ.get("DLV_PREFILL_ATTN", "auto")]  # "auto": the tcgen05 / TMA kernel where it applies; "mma": the mma.sync kernel; "tc"


def _prefill_tc_ok(q, k_cache) -> bool:
    """Shapes the tcgen05 prefill kernel takes: head_dim 64 / 128 / 256, pages of 32 / 64 / 128 tokens, 16-byte aligned query rows."""
    return (k_cache.shape[-1] in (64, 128, 256) and k_cache.shape[2] in (32, 64, 128) and q.stride(0) % 8 == 0 and q.stride(1) == 1
            and q.data_ptr() % 16 == 0 and q.dtype == torch.bfloat16)


def prefill_attention(q, k_cache, v_cache, block_tables, q_start, q_len, ctx_lens, H, scale, softcap=0.0, window=0, causal=True,
                      tile_seq=None, tile_q0=None, impl=None, q_len_host=None, tiles_for=None):
    """Ragged query rows against the paged cache (K/V of the new tokens are already in the cache). ``impl``: ``"tc"`` = the tcgen05 /
    TMA kernel (256-row query tiles, 128 for head_dim 256), ``"mma"`` = the mma.sync kernel (64-row tiles, ``tile_seq`` / ``tile_q0``);
    default from ``DLV_PREFILL_ATTN`` (``auto``: the tcgen05 kernel for the shapes it takes). ``tiles_for(rows)`` returns the device
    tile arrays for a tile height (``ForwardBatch.tiles``); without it they are built from ``q_len_host`` or a read-back of ``q_len``."""
    if _cuda(q):
        mode = impl or PREFILL_ATTN[0]
        if mode == "tc" or (mode == "auto" and _prefill_tc_ok(q, k_cache)):
            ext = require_ext()
            rows = ext.prefill_tc_tile_rows(int(k_cache.shape[-1]))
            if tiles_for is not None:
                ts_d, t0_d = tiles_for(rows)
            else:
                lens = q_len_host if q_len_host is not None else [int(v) for v in q_len.tolist()]
                ts, t0 = prefill_tiles(list(lens), rows)
                ts_d = torch.tensor(ts, dtype=torch.int32, device=q.device)
                t0_d = torch.tensor(t0, dtype=torch.int32, device=q.device)
            _count()
            return ext.prefill_attention_tc(q, k_cache, v_cache, block_tables, q_start, q_len, ctx_lens, ts_d, t0_d, H, scale, softcap, window, causal)
        if tile_seq is None:
            if tiles_for is not None:
                tile_seq, tile_q0 = tiles_for(64)
            else:
                ts, t0 = prefill_tiles([int(v) for v in q_len.tolist()])
                tile_seq = torch.tensor(ts, dtype=torch.int32, device=q.device)
                tile_q0 = torch.tensor(t0, dtype=torch.int32, device=q.device)
        _count()
        return require_ext().prefill_attention(q, k_cache, v_cache, block_tables, q_start, q_len, ctx_lens, tile_seq, tile_q0, H, scale,
                                               softcap, window, causal)
    T = q.shape[0]
    D = k_cache.shape[-1]
    o = ref.paged_attention(q.reshape(T, H, D), k_cache, v_cache, block_tables, q_start, q_len, ctx_lens, scale, softcap, window, causal)
    return o.reshape(T, H * D)


def argmax(logits, mask=None, softcap=0.0, inv_scale=1.0):
    """First-maximum argmax over allowed tokens; returns (index int64 [B], post-processed value [B])."""
    if _cuda(logits):
        _count()
        idx, val = require_ext().argmax(logits, mask, softcap, inv_scale)
        return idx, val
    lf = logits_post(logits.clone().float(), mask, softcap, inv_scale)
    val, idx = torch.max(lf, dim=-1)  # torch CPU max returns the first maximal index
    return idx, val


def logits_post(logits, mask=None, softcap=0.0, inv_scale=1.0):
    """In place: ``softcap(logits * inv_scale)``, disallowed tokens -> -inf. ``mask`` is an int32 allow-bitmask."""
    if _cuda(logits):
        _count()
        require_ext().logits_post(logits, mask, softcap, inv_scale)
        return logits
    if inv_scale != 1.0:
        logits.mul_(inv_scale)
    if softcap and softcap > 0:
        logits.copy_(torch.tanh(logits / softcap) * softcap)
    if mask is not None:
        V = logits.shape[-1]
        bits = unpack_mask(mask, V)
        logits.masked_fill_(~bits, float("-inf"))
    return logits


def unpack_mask(mask: torch.Tensor, V: int) -> torch.Tensor:
    """int32 bitmask ``[B, ceil(V/32)]`` -> bool ``[B, V]``."""
    m = mask.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(32, device=mask.device, dtype=torch.int64)
    bits = ((m.unsqueeze(-1) >> shifts) & 1).bool().reshape(mask.shape[0], -1)
    return bits[:, :V]


def q4_quantize(w: torch.Tensor):
    if _cuda(w):
        _count()
        p, s = require_ext().q4_quantize(w.contiguous())
        return p, s
    from ..ckpt.jq4 import q4_quantize as host

    return host(w)


# ---------------------------------------------------------------------------------------------------------- grouped (MoE)
class GroupedLinearWeight:
    """The projection weights of a rank's local experts stacked for the grouped tcgen05 GEMM (CUDA only): JQ4 experts are
    concatenated tile row by tile row (each expert padded to whole 128-row tiles), dense experts row by row. One launch
    covers every expert that has rows; the work list comes from ``moe_items`` on the device, so nothing syncs with the host."""

    def __init__(self, weights: list):
        w0 = weights[0]
        if any(w.N != w0.N or w.K != w0.K or w.q4 != w0.q4 for w in weights):
            raise ValueError("experts of one layer must share shape and quantisation")
        self.E, self.N, self.K, self.q4 = len(weights), w0.N, w0.K, w0.q4
        e = require_ext()
        if self.q4:
            self.data = torch.cat([w.tiles for w in weights], 0).contiguous()
            self.handle = e.GemmWeight(self.data, True, self.E * ((self.N + 127) // 128) * 128, self.K)
        else:
            self.data = torch.cat([w.w for w in weights], 0).contiguous()
            self.handle = e.GemmWeight(self.data, False, self.E * self.N, self.K)

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def run(self, xs: torch.Tensor, items: torch.Tensor, bn: int, splits: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _count()
        return self.handle.run_grouped(xs, items, self.N, bn, splits, out)

    def run_gemv_act(self, xs: torch.Tensor, items: torch.Tensor, act: str, perm: Optional[torch.Tensor] = None, k: int = 1) -> Optional[torch.Tensor]:
        """Decode-size work items (at most 8 rows each): gate|up projection with ``act(gate) * up`` in the epilogue of the mma.sync
        grouped GEMV; the experts' rows are in plain order (gate rows, then up rows). ``None`` when the shape or the activation is
        outside that kernel (the caller then runs projection and activation as two steps). With ``perm`` (the grouping permutation,
        ``[tokens * k]``) ``xs`` is the ungathered ``[tokens, K]`` activation: grouped row r reads token ``perm[r] // k``."""
        kind = fused_act_kind(act)
        if kind == 0 or not self.q4:
            return None
        out = self.handle.run_grouped_gemv_act(xs, items, self.N, kind, perm, k)
        if out is None:
            return None
        _count()
        return out

    def run_act(self, xs: torch.Tensor, items: torch.Tensor, bn: int, splits: int, act: str) -> torch.Tensor:
        """Grouped gate|up projection with ``act(gate) * up`` in the epilogue; the experts' rows must be in the order of
        :func:`interleave_gate_up`. Returns ``[rows, N / 2]``."""
        _count()
        return self.handle.run_grouped_act(xs, items, self.N, bn, splits, fused_act_kind(act))


_GEMV_MIN_EXPERTS = int(os.environ.get("DLV_MOE_GEMV_MIN_EXPERTS", "1"))


def moe_token_tile(rows: int, local_experts: int, q4: bool = True) -> int:
    """Token tile (UMMA N) of the grouped GEMM for ``rows`` routed rows spread over ``local_experts`` experts."""
    avg = rows / max(1, local_experts)
    # Grouped GEMV (4 or 8 rows per work item, mma.sync) for a handful of rows per expert: a tcgen05 tile costs several microseconds
    # of set-up per (expert, 128 weight rows) whatever the row count. DLV_MOE_GEMV_MIN_EXPERTS restricts it to ranks with at least
    # that many local experts (comparisons).
    # (bf16 experts still have the CUDA-core GEMV only: worth it just for very many experts, as measured with that kernel)
    need = _GEMV_MIN_EXPERTS if q4 else max(96, _GEMV_MIN_EXPERTS)
    if local_experts >= need and avg <= 3:
        return 4
    if local_experts >= need and avg <= 6:
        return 8
    for bn in (16, 32, 64, 128):
        if avg <= bn * 0.75:
            return bn
    return 256
