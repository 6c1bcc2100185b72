"""Decoder-only model graph shared by llama, mistral, qwen2, qwen3, gemma2, gemma3, mixtral, qwen3_moe and granitemoehybrid.

One graph, configured by :class:`~deliverance_b200.config.ModelConfig` flags, over the ragged-batch op surface in
:mod:`deliverance_b200.ops`. Per layer (reference: core/.../generator/TransformerBlock.java:161-200):
pre-attention norm -> fused qkv projection -> per-head q/k norm + RoPE + paged KV write -> paged attention -> o_proj
[-> tensor-parallel all-reduce] [-> gemma2 post-attention norm] -> residual -> pre-FF norm -> gate|up -> act*mul ->
down [-> all-reduce] [-> post-FF norm] -> residual. Residual adds are folded into the following norm kernel.

Tensor names per family follow the loader contract of the reference (LlamaModel.java:45-183, Qwen2Model.java:79-81,
Qwen3Model.java:60-125, Qwen3MoeModel.java:67-123, MixtralModel.java:79-96, Gemma2Model.java:56-172,
GraniteMoeHybridModel.java:118-181). Tensor-parallel shards: q/k/v/gate/up by output rows, o/down by input columns,
everything else replicated (DefaultTransformerWeightPolicyResolver.java:10-26).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .. import ops
from ..ckpt.loader import ShardSpec, WeightLoader, shard_dense, shard_q4
from ..ckpt.safetensors_io import Q4Tensor
from ..config import ModelConfig
from ..ops import LinearWeight, ref
from ..parallel.context import SINGLE, TensorParallelContext, TensorParallelPlanner
from .batch import ForwardBatch


@dataclass
class LoraSlot:
    """Runtime LoRA delta for one projection: ``out += (x @ A^T) @ (scale * B)^T``."""

    a: torch.Tensor  # [r, in]
    b_scaled: torch.Tensor  # [out, r]


@dataclass
class LayerWeights:
    kind: str = "attention"  # "attention" | "sliding" | "mamba"
    input_norm: Optional[torch.Tensor] = None
    qkv: Optional[LinearWeight] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    o: Optional[LinearWeight] = None
    post_attn_norm: Optional[torch.Tensor] = None  # gemma2 only
    pre_ff_norm: Optional[torch.Tensor] = None
    post_ff_norm: Optional[torch.Tensor] = None  # gemma2 only
    gate_up: Optional[LinearWeight] = None
    down: Optional[LinearWeight] = None
    # MoE
    router: Optional[LinearWeight] = None
    experts_gate_up: list = field(default_factory=list)  # per local expert (CPU); stacked in *_grouped on CUDA
    experts_down: list = field(default_factory=list)
    experts_gate_up_grouped: Optional[object] = None
    experts_down_grouped: Optional[object] = None
    expert0: int = 0  # first expert held by this rank (expert parallelism)
    n_local_experts: int = 0  # 0 = all
    shared_gate_up: Optional[LinearWeight] = None  # granite shared MLP
    shared_down: Optional[LinearWeight] = None
    # mamba2
    mamba: Optional[dict] = None
    lora: dict = field(default_factory=dict)  # projection name -> LoraSlot
    fused_act: bool = False  # gate_up holds interleaved rows and the GEMM epilogue applies the gated activation
    fused_act_experts: bool = False  # the same for the routed experts' gate|up weights


def _cat_weights(parts: list) -> "torch.Tensor | Q4Tensor":
    """Concatenate projection weights along output rows (all dense or all JQ4)."""
    if all(isinstance(p, Q4Tensor) for p in parts):
        packed = torch.cat([p.packed for p in parts], dim=0)
        scales = torch.cat([p.scales for p in parts], dim=0)
        return Q4Tensor(packed, scales, (packed.shape[0], packed.shape[1] * 2))
    dense = [p.dequantize(torch.float32) if isinstance(p, Q4Tensor) else p for p in parts]
    dt = dense[0].dtype
    return torch.cat([d.to(dt) for d in dense], dim=0)


class DecoderModel:
    """Weights + forward for one rank."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None,
                 tp: TensorParallelContext = SINGLE):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.tp = tp
        TensorParallelPlanner.validate(cfg, tp.size)
        if self.device.type == "cuda" and cfg.num_heads and cfg.head_dim not in (64, 128, 256):
            raise ValueError(f"head_dim {cfg.head_dim} is not supported by the CUDA attention kernels (64, 128, 256)")
        self.n_heads = cfg.num_heads // tp.size
        self.n_kv = max(1, cfg.num_kv_heads // tp.size)  # with more ranks than KV heads, size / kv_heads ranks replicate one head
        self.layers: list[LayerWeights] = []
        self.embed: Optional[torch.Tensor] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[LinearWeight] = None
        self.cos = self.sin = None
        self.cos_local = self.sin_local = None  # rotary tables of sliding-window layers when their base differs (gemma3)
        self.layer_hook: Optional[Callable[[int, str, torch.Tensor], None]] = None  # debug / trace hook
        self.profiler = None
        self.active_lora: Optional[str] = None
        self.shard_head = True  # split the output head over the vocabulary under tensor parallelism
        # opt-in (DLV_FUSED_ACT=1): act(gate) * up inside the gate|up GEMM epilogue instead of a separate kernel
        self.fused_act = os.environ.get("DLV_FUSED_ACT", "0") == "1"
        # head_dim 128 on CUDA: q/k norm + rotary embedding + KV write inside the q|k|v GEMM epilogue (one launch and one round trip of
        # the q|k|v tensor less per layer; measured 1 % of the decode step at 64 sequences, 3 % at 8). DLV_FUSED_ROPE=0 turns it off,
        # DLV_FUSED_ROPE=1 forces it on the CPU oracle path (tests of the composition).
        want = os.environ.get("DLV_FUSED_ROPE", "auto")
        self.fused_rope = (want == "1" or (want != "0" and torch.device(device).type == "cuda")) and cfg.head_dim == 128 and cfg.use_rope
        self.vocab_shard: Optional[tuple] = None
        self._moe_impl = None
        # opt-in (DLV_TP_SEQ_PARALLEL=1): sequence-parallel prefill under tensor parallelism for batches of at least this many rows
        self.sp_min_rows: Optional[int] = 256 * tp.size if (tp.enabled and os.environ.get("DLV_TP_SEQ_PARALLEL", "0") == "1") else None
        self._sp = None  # (M, rows per rank, first own row, own rows) while such a forward runs
        self._sp_ordered = False

    # ------------------------------------------------------------------------------------------------ loading
    def _dev(self, t: torch.Tensor, dtype=None) -> torch.Tensor:
        return t.to(device=self.device, dtype=dtype or self.dtype).contiguous()

    def _lin(self, w, bias=None) -> LinearWeight:
        lw = LinearWeight(w if isinstance(w, Q4Tensor) else w.to(self.dtype), None if bias is None else bias.float())
        return lw.to(self.device, self.dtype)

    def load(self, loader: WeightLoader, head_quant: Optional[str] = None, prefix: str = "model.") -> "DecoderModel":
        cfg, tp = self.cfg, self.tp
        row = lambda groups=1: ShardSpec("row", tp.rank, tp.size, groups) if tp.enabled else None  # noqa: E731
        col = ShardSpec("col", tp.rank, tp.size) if tp.enabled else None

        def get(name, shard=None):
            return loader.load(name, shard)

        def vec(name):
            t = loader.load(name)
            return self._dev(t.reshape(-1) if not isinstance(t, Q4Tensor) else t.dequantize().reshape(-1))

        if not loader.has(prefix + "embed_tokens.weight"):
            # text tower of a multimodal checkpoint (gemma3): the language model's tensors carry a wrapper prefix
            for alt in ("language_model.model.", "model.language_model."):
                if loader.has(alt + "embed_tokens.weight"):
                    prefix = alt
                    break
        emb = loader.load(prefix + "embed_tokens.weight")
        emb_dense = emb.dequantize(torch.float32) if isinstance(emb, Q4Tensor) else emb
        self.embed = self._dev(emb_dense)
        for i in range(cfg.num_layers):
            p = f"{prefix}layers.{i}."
            lw = LayerWeights(kind=cfg.layer_type(i))
            lw.input_norm = vec(p + "input_layernorm.weight")
            if lw.kind == "mamba":
                lw.mamba = self._load_mamba(loader, p + "mamba.")
            else:
                kv_row = row()
                if tp.enabled and cfg.num_kv_heads % tp.size != 0:
                    kv_row = ShardSpec("row", tp.rank // (tp.size // cfg.num_kv_heads), cfg.num_kv_heads)
                shard_of = {"q": row(), "k": kv_row, "v": kv_row}
                parts = [get(p + f"self_attn.{n}_proj.weight", shard_of[n]) for n in ("q", "k", "v")]
                bias = None
                if cfg.qkv_bias and loader.has(p + "self_attn.q_proj.bias"):
                    bias = torch.cat([loader.load(p + f"self_attn.{n}_proj.bias", shard_of[n]).float().reshape(-1) for n in ("q", "k", "v")])
                lw.qkv = self._lin(_cat_weights(parts), bias)
                if cfg.qk_norm:
                    lw.q_norm = vec(p + "self_attn.q_norm.weight")
                    lw.k_norm = vec(p + "self_attn.k_norm.weight")
                lw.o = self._lin(get(p + "self_attn.o_proj.weight", col))
            if cfg.post_norms:
                lw.post_attn_norm = vec(p + "post_attention_layernorm.weight")
                lw.pre_ff_norm = vec(p + "pre_feedforward_layernorm.weight")
                lw.post_ff_norm = vec(p + "post_feedforward_layernorm.weight")
            else:
                lw.pre_ff_norm = vec(p + "post_attention_layernorm.weight")
            self._load_ff(loader, lw, i, p, get, row, col)
            self.layers.append(lw)
        self.final_norm = vec(prefix + "norm.weight")
        # output head: lm_head.weight, else tied to the embedding table; optional load-time JQ4 quantisation
        if not cfg.tie_word_embeddings and loader.has("lm_head.weight"):
            head = loader.load("lm_head.weight")
        else:
            head = emb
        # Under tensor parallelism each rank holds a contiguous slice of the vocabulary rows of the head: it projects 1 / size of
        # the logits, greedy decoding exchanges one (value, index) pair per row, sampling gathers the slices.
        self.vocab_shard = None
        if tp.enabled and self.shard_head and cfg.vocab_size % tp.size == 0:
            vs = cfg.vocab_size // tp.size
            self.vocab_shard = (tp.rank * vs, (tp.rank + 1) * vs)
            spec = ShardSpec("row", tp.rank, tp.size)
            tied_dense = head is emb and not isinstance(head, Q4Tensor)
            head = shard_q4(head, spec) if isinstance(head, Q4Tensor) else shard_dense(head, spec)
        else:
            tied_dense = head is emb and not isinstance(head, Q4Tensor)
        if head_quant and head_quant.upper() == "Q4" and not isinstance(head, Q4Tensor):
            from ..ckpt.jq4 import q4_quantize

            hp, hs = q4_quantize(head.float())
            head = Q4Tensor(hp, hs, tuple(head.shape))
        if isinstance(head, Q4Tensor) or not tied_dense or self.device.type != "cuda":
            self.lm_head = self._lin(head)
        elif self.vocab_shard is not None:
            self.lm_head = LinearWeight(self.embed[self.vocab_shard[0] : self.vocab_shard[1]])  # a row slice of the embedding table
        else:
            self.lm_head = LinearWeight(self.embed)  # share storage with the embedding table
        if cfg.use_rope:
            cos, sin = ref.rope_tables(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_factor)
            self.cos, self.sin = cos.to(self.device), sin.to(self.device)
            if cfg.rope_local_theta > 0:
                cos, sin = ref.rope_tables(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_local_theta, 1.0)
                self.cos_local, self.sin_local = cos.to(self.device), sin.to(self.device)
        return self

    def _load_ff(self, loader, lw, i, p, get, row, col):
        cfg = self.cfg
        mt = cfg.model_type
        E = cfg.num_experts
        ep = self.tp.enabled and E > 0 and E % self.tp.size == 0  # expert parallelism: this rank holds E / size whole experts
        e0, ne = ((self.tp.rank * (E // self.tp.size), E // self.tp.size) if ep else (0, E))
        sparse = mt == "mixtral" or (mt == "qwen3_moe" and cfg.is_sparse_layer(i)) or (mt == "granitemoehybrid" and E > 0)
        if sparse:
            lw.expert0, lw.n_local_experts = e0, ne
        if mt == "mixtral":
            lw.router = self._lin(loader.load(p + "block_sparse_moe.gate.weight"))
            for e in range(e0, e0 + ne):
                ep_ = p + f"block_sparse_moe.experts.{e}."
                lw.experts_gate_up.append(self._lin(self._gate_up_rows(lw, get(ep_ + "w1.weight"), get(ep_ + "w3.weight"))))
                lw.experts_down.append(self._lin(get(ep_ + "w2.weight")))
        elif mt == "qwen3_moe" and cfg.is_sparse_layer(i):
            lw.router = self._lin(loader.load(p + "mlp.gate.weight"))
            for e in range(e0, e0 + ne):
                ep_ = p + f"mlp.experts.{e}."
                lw.experts_gate_up.append(self._lin(self._gate_up_rows(lw, get(ep_ + "gate_proj.weight"), get(ep_ + "up_proj.weight"))))
                lw.experts_down.append(self._lin(get(ep_ + "down_proj.weight")))
        elif mt == "granitemoehybrid":
            lw.shared_gate_up = self._lin(get(p + "shared_mlp.input_linear.weight"))
            lw.shared_down = self._lin(get(p + "shared_mlp.output_linear.weight"))
            if E > 0:
                lw.router = self._lin(loader.load(p + "block_sparse_moe.router.layer.weight"))
                win = get(p + "block_sparse_moe.input_linear.weight")  # [E, 2I, hidden]
                wout = get(p + "block_sparse_moe.output_linear.weight")  # [E, hidden, I]
                for e in range(e0, e0 + ne):
                    lw.experts_gate_up.append(self._lin(_slice_expert(win, e)))
                    lw.experts_down.append(self._lin(_slice_expert(wout, e)))
        else:
            parts = [get(p + "mlp.gate_proj.weight", row()), get(p + "mlp.up_proj.weight", row())]
            if self.fused_act and parts[0].shape[0] % 64 == 0 and ops.fused_act_kind(cfg.hidden_act):
                # gate and up rows interleaved per 64 outputs: the GEMM epilogue applies act(gate) * up (ops.linear_act)
                lw.gate_up = self._lin(ops.interleave_gate_up(parts[0], parts[1]))
                lw.fused_act = True
            else:
                lw.gate_up = self._lin(_cat_weights(parts))
            lw.down = self._lin(get(p + "mlp.down_proj.weight", col))
        if lw.experts_gate_up and self.device.type == "cuda":
            lw.experts_gate_up_grouped = ops.GroupedLinearWeight(lw.experts_gate_up)
            lw.experts_down_grouped = ops.GroupedLinearWeight(lw.experts_down)
            lw.experts_gate_up, lw.experts_down = [], []

    def _gate_up_rows(self, lw, gate, up):
        """Rows of one expert's gate|up projection: concatenated, or (opt-in) interleaved per 64 outputs for the GEMM epilogue
        activation; the layer remembers which (all experts of a layer share the choice)."""
        # (ranks that hold very many experts may route decode batches to the CUDA-core grouped GEMV, which has no such epilogue)
        if self.fused_act and gate.shape[0] % 64 == 0 and ops.fused_act_kind(self.cfg.hidden_act) and (lw.n_local_experts or 0) < 96:
            lw.fused_act_experts = True
            return ops.interleave_gate_up(gate, up)
        return _cat_weights([gate, up])

    def _load_mamba(self, loader, p) -> dict:
        f32 = lambda n: self._dev(loader.load_dense(p + n), torch.float32)  # noqa: E731
        m = {
            "in_proj": self._lin(loader.load(p + "in_proj.weight")),
            "out_proj": self._lin(loader.load(p + "out_proj.weight")),
            "conv_w": f32("conv1d.weight"),
            "conv_b": f32("conv1d.bias") if loader.has(p + "conv1d.bias") else None,
            "dt_bias": f32("dt_bias").reshape(-1),
            "A_log": f32("A_log").reshape(-1),
            "D": f32("D").reshape(-1),
            "norm_w": f32("norm.weight").reshape(-1),
        }
        return m

    # ------------------------------------------------------------------------------------------------ LoRA hot swap
    def set_lora(self, adapter=None, prefix: str = "model.") -> None:
        """Activate (or with ``None`` clear) a run-time LoRA adapter: every targeted projection gets ``(x A^T)(sB)^T`` added
        to its output, the base weights (JQ4 included) stay untouched. Fused projections stack the A matrices of their parts
        and place the B matrices block-diagonally so one pair of skinny GEMMs serves q|k|v (or gate|up). The adapter id joins
        the prefix-cache salt, so cached prefixes of another adapter are never reused
        (reference: core/.../generator/LoraDeltaApplier.java:43-63, safetensors/.../ResolvedLoraAdapter.java:22-45)."""
        if adapter is not None and self.tp.enabled:
            raise ValueError("run-time LoRA is not supported under tensor parallelism")
        for i, lw in enumerate(self.layers):
            lw.lora = {}
            if adapter is None or lw.kind == "mamba":
                continue
            p = f"{prefix}layers.{i}."
            groups = {"qkv": [p + f"self_attn.{n}_proj.weight" for n in ("q", "k", "v")], "o": [p + "self_attn.o_proj.weight"],
                      "gate_up": [p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], "down": [p + "mlp.down_proj.weight"]}
            for slot, names in groups.items():
                if slot == "gate_up" and lw.fused_act and any(adapter.has(n) for n in names):
                    raise ValueError("run-time LoRA on gate_proj / up_proj is not available with the fused activation epilogue (DLV_FUSED_ACT)")
                w = getattr(lw, slot)
                if w is None or not any(adapter.has(n) for n in names):
                    continue
                out_total, r = w.N, adapter.config.r
                rows = self._lora_part_rows(slot, out_total)
                a_parts, b_full = [], torch.zeros(out_total, r * len(names))
                off = 0
                for j, n in enumerate(names):
                    if adapter.has(n):
                        A, Bs = adapter.resolved(n)
                        if Bs.shape[0] != rows[j]:
                            raise ValueError(f"{n}: adapter B has {Bs.shape[0]} rows, the projection has {rows[j]}")
                        a_parts.append(A)
                        b_full[off : off + rows[j], j * r : (j + 1) * r] = Bs
                    else:
                        a_parts.append(torch.zeros(r, w.K))
                    off += rows[j]
                lw.lora[slot] = LoraSlot(self._dev(torch.cat(a_parts, 0)), self._dev(b_full))
        self.active_lora = None if adapter is None else adapter.id

    def _lora_part_rows(self, slot: str, out_total: int) -> list:
        cfg = self.cfg
        if slot == "qkv":
            return [cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim]
        if slot == "gate_up":
            return [out_total // 2, out_total // 2]
        return [out_total]

    # ------------------------------------------------------------------------------------------------ forward
    def _trace(self, layer: int, stage: str, t: torch.Tensor) -> None:
        if self.layer_hook is not None:
            self.layer_hook(layer, stage, t)

    def _stage(self, name: str):
        return self.profiler.stage(name) if self.profiler is not None else _NULL

    def embed_tokens(self, batch: ForwardBatch) -> torch.Tensor:
        return ops.embedding(self.embed, batch.token_ids, self.cfg.embedding_multiplier, dtype=self.dtype)

    def _lora(self, lw: LayerWeights, name: str, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        slot = lw.lora.get(name)
        if slot is None:
            return y
        from ..ckpt.lora import apply_lora_delta

        return apply_lora_delta(x, y, slot.a, slot.b_scaled)

    def attention(self, i: int, lw: LayerWeights, x: torch.Tensor, batch: ForwardBatch, kv, norm_after=None):
        """Self-attention block output. With ``norm_after = (residual, post_w, norm_w)`` returns ``(y, fused)``: when ``fused`` the
        tensor-parallel sum, the residual add and the norm that follow were done behind the output projection and ``y`` is already
        ``rmsnorm(residual)``; otherwise ``y`` is the block output as without the argument."""
        cfg = self.cfg
        k_cache, v_cache = kv.layer(i)
        local_rope = lw.kind == "sliding" and self.cos_local is not None
        cos, sin = (self.cos_local, self.sin_local) if local_rope else (self.cos, self.sin)
        if self.fused_rope and "qkv" not in lw.lora and self._sp is None:
            # norm + rotary + cache write in the projection's epilogue (one launch instead of two, q is written once); a
            # sequence-parallel forward gathers its input inside the projection and keeps the two-kernel form
            with self._stage("causalselfattention.qkv_projection"):
                q = ops.linear_rope_kv(x, lw.qkv, batch.positions, batch.slots, lw.q_norm, lw.k_norm, cos, sin, k_cache, v_cache,
                                       self.n_heads, self.n_kv, cfg.head_dim, cfg.norm_eps, cfg.norm_weight_offset)
        else:
            with self._stage("causalselfattention.qkv_projection"):
                qkv = self._col_parallel(x, lw.qkv)
                if lw.lora:
                    qkv = self._lora(lw, "qkv", x, qkv)
            with self._stage("causalselfattention.rope"):
                q = ops.rope_kv(qkv, batch.positions, batch.slots, lw.q_norm, lw.k_norm, cos, sin, k_cache, v_cache,
                                self.n_heads, self.n_kv, cfg.head_dim, cfg.norm_eps, cfg.norm_weight_offset)
        window = cfg.window(i)
        with self._stage("causalselfattention.score_value"):
            if batch.is_decode:
                a = ops.decode_attention(q, k_cache, v_cache, batch.block_tables, batch.ctx_len, self.n_heads, cfg.scale,
                                         cfg.attn_softcap, window, batch.decode_splits)
            else:
                a = ops.prefill_attention(q, k_cache, v_cache, batch.block_tables, batch.q_start, batch.q_len, batch.ctx_len,
                                          self.n_heads, cfg.scale, cfg.attn_softcap, window, True, batch.tile_seq, batch.tile_q0, tiles_for=batch.tiles)
        with self._stage("causalselfattention.output_projection"):
            if norm_after is not None and not lw.lora:
                x = self._row_parallel_norm(a, lw.o, norm_after)
                if x is not None:
                    return x, True
            o = self._row_parallel(a, lw.o, f"layer.{i}.self_attn.o_proj")
            if lw.lora:
                o = self._lora(lw, "o", a, o)
        return (o, False) if norm_after is not None else o

    # ---- sequence parallelism for prefill-size batches under tensor parallelism (opt-in) ----
    # Between a row-parallel and the next column-parallel projection every rank keeps only the token rows it owns: the sum over
    # ranks becomes a reduce-scatter, residual add and norms run on 1 / size of the rows, and the column-parallel projection
    # gathers its input (peer-memory kernels of parallel/fused.py on GPUs, plain collectives otherwise).
    def _sp_plan(self, batch: ForwardBatch):
        """``(M, rows_per_rank, first, count)`` when this forward runs sequence parallel, else ``None``."""
        if not self.tp.enabled or batch.is_decode or self.sp_min_rows is None or type(self) is not DecoderModel:
            return None
        M = int(batch.token_ids.shape[0])
        if M < self.sp_min_rows or self.cfg.model_type == "granitemoehybrid":
            return None
        if any(lw.kind == "mamba" or lw.lora or lw.fused_act for lw in self.layers):
            return None
        if any(lw.router is not None for lw in self.layers):
            # mixture-of-experts layers run sequence parallel only with expert parallelism over peer memory (token rows travel to the
            # experts' owners and back: parallel/fused.py::ExpertAllToAll)
            ne = next(lw.n_local_experts for lw in self.layers if lw.router is not None)
            if (self.tp.fused is None or batch.token_ids.device.type != "cuda" or not ne or ne == self.cfg.num_experts or ne > 128
                    or self.cfg.model_type == "granitemoehybrid" or torch.cuda.is_current_stream_capturing()):
                return None
        from ..parallel.fused import row_cut

        rpr, first, count = row_cut(M, self.tp.size, self.tp.rank)
        return M, rpr, first, count

    def _gather_rows(self, x_own: torch.Tensor) -> torch.Tensor:
        M, rpr, _, _ = self._sp
        if x_own.shape[0] < rpr:
            x_own = torch.cat([x_own, x_own.new_zeros(rpr - x_own.shape[0], x_own.shape[1])], dim=0)
        return torch.cat(self.tp.collectives.all_gather(x_own.contiguous()), dim=0)[:M]

    def _col_parallel(self, x: torch.Tensor, w: LinearWeight) -> torch.Tensor:
        """Column-parallel projection; in a sequence-parallel forward ``x`` holds this rank's rows and the result all rows."""
        if self._sp is None:
            return ops.linear(x, w)
        if self.tp.fused is not None and x.device.type == "cuda":
            # the first gather of a forward orders the ranks itself; later ones follow a reduce-scatter, which does
            ordered, self._sp_ordered = self._sp_ordered, True
            return self.tp.fused.all_gather_linear(x, self._sp[0], w, ordered=ordered)
        return ops.linear(self._gather_rows(x), w)

    def _row_parallel_norm(self, x: torch.Tensor, w: LinearWeight, norm_after):
        """Row-parallel projection + tensor-parallel sum + residual add + norm behind it, when the peer-memory path takes it
        (decode-size batches on GPUs); ``None`` otherwise."""
        if self._sp is not None or not self.tp.enabled or self.tp.fused is None or x.device.type != "cuda":
            return None
        fn = getattr(self.tp.fused, "linear_reduce_norm", None)
        if fn is None:
            return None
        residual, post_w, norm_w = norm_after
        return fn(x, w, residual, norm_w, post_w, self.cfg.norm_eps, self.cfg.norm_weight_offset, self.cfg.residual_multiplier)

    def _row_parallel(self, x: torch.Tensor, w: LinearWeight, key: str) -> torch.Tensor:
        """Row-parallel projection followed by the tensor-parallel sum (sequence parallel: only this rank's rows of it)."""
        if self._sp is not None:
            _, _, first, count = self._sp
            if self.tp.fused is not None and x.device.type == "cuda":
                return self.tp.fused.linear_reduce_scatter(x, w, key)
            return self.tp.all_reduce(key, ops.linear(x, w))[first:first + count].contiguous()
        if self.tp.enabled and self.tp.fused is not None and x.device.type == "cuda":
            return self.tp.fused.linear_all_reduce(x, w, key)
        y = ops.linear(x, w)
        if self.tp.enabled:
            with self._stage("causalselfattention.all_reduce" if "attn" in key else "mlpblock.all_reduce"):
                y = self.tp.all_reduce(key, y)
        return y

    def feed_forward(self, i: int, lw: LayerWeights, x: torch.Tensor, norm_after=None):
        """Feed-forward block output; ``norm_after`` as in :meth:`attention` (dense blocks only)."""
        cfg = self.cfg
        if lw.router is not None and cfg.model_type != "granitemoehybrid":
            if self._sp is not None:
                from .moe import moe_forward_sharded

                with self._stage("moe.forward"):
                    a2a = self.tp.fused.expert_a2a(lw.n_local_experts, cfg.hidden_size, cfg.experts_per_token)
                    y = moe_forward_sharded(self, i, lw, x, a2a, self._sp[0])
            else:
                y = self.moe(i, lw, x)
            return (y, False) if norm_after is not None else y
        if cfg.model_type == "granitemoehybrid":
            with self._stage("mlpblock.shared"):
                h = ops.act_mul(ops.linear(x, lw.shared_gate_up), cfg.hidden_act)
                y = ops.linear(h, lw.shared_down)
            if lw.router is not None:
                y = y + self.moe(i, lw, x)
            return (y, False) if norm_after is not None else y
        if lw.fused_act:
            with self._stage("mlpblock.gate_up_projection"):
                h = ops.linear_act(x, lw.gate_up, cfg.hidden_act)
        elif self._sp is None and not lw.lora and x.shape[0] <= ops.GEMV_MAX_ROWS:
            with self._stage("mlpblock.gate_up_projection"):  # a handful of rows: projection and gated activation in one launch
                h = ops.linear_gated(x, lw.gate_up, cfg.hidden_act)
        else:
            with self._stage("mlpblock.gate_up_projection"):
                gu = self._col_parallel(x, lw.gate_up)
                if lw.lora:
                    gu = self._lora(lw, "gate_up", x, gu)
            with self._stage("mlpblock.activation_multiply"):
                h = ops.act_mul(gu, cfg.hidden_act)
        with self._stage("mlpblock.down_projection"):
            if norm_after is not None and not lw.lora:
                x2 = self._row_parallel_norm(h, lw.down, norm_after)
                if x2 is not None:
                    return x2, True
            d = self._row_parallel(h, lw.down, f"layer.{i}.mlp.down_proj")
            if lw.lora:
                d = self._lora(lw, "down", h, d)
        return (d, False) if norm_after is not None else d

    def moe(self, i: int, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        from .moe import moe_forward

        with self._stage("moe.forward"):
            return moe_forward(self, i, lw, x)

    def mamba(self, i: int, lw: LayerWeights, x: torch.Tensor, batch: ForwardBatch, kv) -> torch.Tensor:
        from .mamba import mamba_forward

        with self._stage("mamba.forward"):
            return mamba_forward(self, i, lw, x, batch, kv)

    def forward_hidden(self, batch: ForwardBatch, kv) -> torch.Tensor:
        """Run every layer; returns the final-normed hidden states ``[T, hidden]``."""
        cfg = self.cfg
        residual = self.embed_tokens(batch)
        self._trace(-1, "embed", residual)
        self._sp, self._sp_ordered = self._sp_plan(batch), False
        if self._sp is not None:
            residual = residual[self._sp[2]:self._sp[2] + self._sp[3]].contiguous()  # the residual stream stays row-sharded
        try:
            x = self._layers_forward(batch, kv, residual)
            if self._sp is not None:
                x = self._gather_rows(x)
        finally:
            self._sp = None
        return x

    def _layers_forward(self, batch: ForwardBatch, kv, residual: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        eps, off, rm = cfg.norm_eps, cfg.norm_weight_offset, cfg.residual_multiplier
        x = ops.rmsnorm(residual, self.layers[0].input_norm, eps, off)
        for i, lw in enumerate(self.layers):
            # Under fused tensor parallelism a decode-size row-parallel projection hands the sum over the ranks, the residual add and the
            # norm behind it to one row-wise kernel (``fused`` below); every other case runs the steps one by one.
            split = self.tp.enabled and self.tp.fused is not None and self.layer_hook is None and type(self) is DecoderModel
            if lw.kind == "mamba":
                a, fused = self.mamba(i, lw, x, batch, kv), False
            elif split:
                a, fused = self.attention(i, lw, x, batch, kv, (residual, lw.post_attn_norm, lw.pre_ff_norm))
            else:
                a, fused = self.attention(i, lw, x, batch, kv), False
            if fused:
                x = a
            else:
                if lw.post_attn_norm is not None:
                    a = ops.rmsnorm(a, lw.post_attn_norm, eps, off)
                self._trace(i, "attn", a)
                x = ops.add_rmsnorm(a, residual, lw.pre_ff_norm, eps, off, rm)
            nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.final_norm
            f, fused = self.feed_forward(i, lw, x, (residual, lw.post_ff_norm, nxt)) if split else (self.feed_forward(i, lw, x), False)
            if fused:
                x = f
            else:
                if lw.post_ff_norm is not None:
                    f = ops.rmsnorm(f, lw.post_ff_norm, eps, off)
                self._trace(i, "ff", f)
                x = ops.add_rmsnorm(f, residual, nxt, eps, off, rm)
            self._trace(i, "out", residual)
        return x

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """fp32 logits (before logit scaling / softcap, which the sampler applies): the full vocabulary, or this rank's slice
        of it when the head is sharded (``vocab_shard``; see :meth:`greedy_tokens` / :meth:`full_logits`)."""
        with self._stage("sampler.output_projection"):
            return ops.linear(hidden_rows, self.lm_head, out_f32=True)

    def greedy_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        """First-maximum argmax over the whole vocabulary from (possibly sharded) logits; int64 ``[B]`` on the logits' device."""
        idx, val = ops.argmax(logits)
        if self.vocab_shard is None:
            return idx
        pair = torch.stack([val.float(), idx.float()], dim=1).contiguous()  # vocabulary slices are < 2^24 wide: exact in fp32
        parts = torch.stack(self.tp.collectives.all_gather(pair), dim=0)  # [size, B, 2]
        best = torch.argmax(parts[:, :, 0], dim=0)  # first maximum = lowest rank = lowest global index on ties
        local = parts[best, torch.arange(parts.shape[1], device=parts.device), 1].to(torch.int64)
        return local + best.to(torch.int64) * (self.vocab_shard[1] - self.vocab_shard[0])

    def full_logits(self, logits: torch.Tensor) -> torch.Tensor:
        if self.vocab_shard is None:
            return logits
        return torch.cat(self.tp.collectives.all_gather(logits.contiguous()), dim=1)

    def forward(self, batch: ForwardBatch, kv, all_rows: bool = False) -> torch.Tensor:
        h = self.forward_hidden(batch, kv)
        if not all_rows and batch.logits_rows is not None and not batch.is_decode:
            h = h.index_select(0, batch.logits_rows)
        return self.logits(h.contiguous())

    # ------------------------------------------------------------------------------------------------ misc
    def kv_layout(self) -> dict:
        cfg = self.cfg
        return {"layers": cfg.num_layers, "kv_heads": self.n_kv, "head_dim": cfg.head_dim,
                "layer_kinds": [cfg.layer_type(i) for i in range(cfg.num_layers)]}

    def weight_bytes(self) -> int:
        n = self.embed.numel() * self.embed.element_size()
        for lw in self.layers:
            for w in (lw.qkv, lw.o, lw.gate_up, lw.down, lw.router, lw.shared_gate_up, lw.shared_down):
                if w is not None:
                    n += w.nbytes()
            for w in lw.experts_gate_up + lw.experts_down:
                n += w.nbytes()
            for w in (lw.experts_gate_up_grouped, lw.experts_down_grouped):
                if w is not None:
                    n += w.nbytes()
        if self.lm_head is not None and (self.lm_head.q4 or self.lm_head.w is not self.embed):
            n += self.lm_head.nbytes()
        return n


def _slice_expert(w, e: int):
    if isinstance(w, Q4Tensor):
        return Q4Tensor(w.packed[e], w.scales[e], tuple(w.shape[1:]))
    return w[e]


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL = _Null()
