"""Public entry points: ``AutoModelForCausalLM``, ``AutoModelForEmbeddings``, ``AutoModelForSequenceClassification``.

The builder mirrors the reference's ``AutoModelForCausaLm.Builder`` options that make sense on GPUs
(core/.../model/AutoModelForCausaLm.java:106-760): working dtype, KV-cache settings, tensor parallel rank/size and
collectives, output-head quantisation, max batch size, quantise-on-demand, LoRA adapter (merge at load), guided-decoding
settings, JSON ``AutoModelConfig``. ``model_type`` dispatch follows ``readConfig`` / ``newModel`` (:522-583). The text-level
``generate(session, prompt, params, on_event)`` keeps the reference's response fields (text, text with special tokens,
reasoning, finish reason, token counts, timings, tool calls) and its stop order.
"""
from __future__ import annotations

import json
import logging
import os
import uuid
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .ckpt.loader import WeightLoader
from .ckpt.lora import LoraAdapter, MergingWeightLoader
from .ckpt.quantizer import quantize_on_demand
from .config import ModelConfig, load_config
from .engine.engine import Engine, EngineConfig, Request
from .guided.index import DEFAULT_SETTINGS, SketchesSettings
from .guided.processor import LogitsProcessorFactory
from .kv.paged import KvCacheSettings
from .models.bert import BertModel
from .models.gpt2 import Gpt2Model
from .models.transformer import DecoderModel
from .parallel.context import SINGLE, TensorParallelContext
from .params import FinishReason, GeneratorParameters, Response
from .prompt.chat import PromptBuilder, PromptContext
from .prompt.parsers import (Gemma4ToolCallParser, StopStringDetector, ToolCallParser, parse_gemma4_response,
                             parser_for_model, prompt_ends_inside_reasoning, split_reasoning)
from .tokenizer.auto import AutoTokenizer, IncrementalDetokenizer, SpecialTextView


_log = logging.getLogger("deliverance_b200.generation")


@dataclass
class AutoModelConfig:
    """JSON-serialisable builder options (reference: core/.../model/AutoModelConfig.java:21-103)."""

    model: str = ""
    device: str = "auto"
    dtype: str = "auto"
    output_head_quantization: Optional[str] = None
    max_batch_size: int = 8192
    max_seqs: int = 128
    quantize_on_demand: bool = False
    lora_adapter: Optional[str] = None
    cuda_graphs: bool = True
    kv_block_size: int = 32
    kv_max_prefix_tokens: int = 512
    kv_max_entries: int = 10_000
    kv_policy: str = "START_AND_END"
    kv_pages: Optional[int] = None
    profile_stages: bool = False

    decode_interleave: int = 0  # EngineConfig.decode_interleave
    kv_checkpoints: int = 4
    kv_anchors: tuple = (32, 64, 128)
    kv_compression: str = "NONE"
    kv_turboquant_bits: int = 4
    ignored: tuple = ()  # reference keys that have no meaning on this runtime (kept for diagnostics)

    # reference key -> field (core/.../model/AutoModelConfig.java:24-37,66-75); benchmark configs under benchmarks/configs/*.json load unchanged
    _REF_KEYS = {"outputHeadQuantization": "output_head_quantization", "maxBatchSize": "max_batch_size"}
    _REF_KV_KEYS = {"maxEntries": "kv_max_entries", "blockSize": "kv_block_size", "maxPrefixTokensPerPrompt": "kv_max_prefix_tokens",
                    "prefixCheckpointPolicy": "kv_policy", "prefixCompression": "kv_compression", "prefixTurboQuantBits": "kv_turboquant_bits",
                    "maxPrefixCheckpointsPerPrompt": "kv_checkpoints", "contextRowsPerPageTarget": "kv_block_size"}
    # CPU-runtime knobs of the reference: working dtypes (activations are bf16 here), WebGPU offload switches, the tensor runtime
    _REF_IGNORED = ("workingMemoryType", "workingQuantType", "gpuPrefill", "gpuDecode", "gpuDecodeAttention", "packedPrefill", "download",
                    "tensorRuntimeMode", "tensorPlanTrace")

    @staticmethod
    def from_json(path_or_text: str) -> "AutoModelConfig":
        """Accepts this package's snake_case keys and the reference's JSON layout (camelCase, nested ``kvBufferCache`` and
        ``quantizeOnDemand`` objects)."""
        text = open(path_or_text).read() if os.path.exists(path_or_text) else path_or_text
        d = json.loads(text)
        known = {f for f in AutoModelConfig.__dataclass_fields__} - {"ignored"}
        out = {k: v for k, v in d.items() if k in known}
        ignored = [k for k in d if k in AutoModelConfig._REF_IGNORED]
        for k, f in AutoModelConfig._REF_KEYS.items():
            if k in d:
                out[f] = d[k]
        kvb = d.get("kvBufferCache") or {}
        for k, f in AutoModelConfig._REF_KV_KEYS.items():
            if k in kvb and kvb[k] is not None:
                out[f] = kvb[k]
        if kvb.get("prefixCheckpointAnchors"):
            out["kv_anchors"] = tuple(int(a) for a in kvb["prefixCheckpointAnchors"])
        if d.get("quantizeOnDemand"):
            out["quantize_on_demand"] = True
        unknown = [k for k in d if k not in known and k not in AutoModelConfig._REF_KEYS and k not in AutoModelConfig._REF_IGNORED
                   and k not in ("kvBufferCache", "quantizeOnDemand")]
        if unknown:
            raise ValueError(f"unknown configuration keys: {', '.join(sorted(unknown))}")
        cfg = AutoModelConfig(**out)
        cfg.ignored = tuple(ignored)
        return cfg


def _device(name: str) -> torch.device:
    if name == "auto":
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return torch.device(name)


def build_model(cfg: ModelConfig, device, dtype, tp: TensorParallelContext):
    if cfg.model_type == "gpt2":
        return Gpt2Model(cfg, device, dtype, tp)
    if cfg.model_type == "bert":
        return BertModel(cfg, device, dtype)
    if cfg.model_type == "gemma4_text":
        from .models.gemma4 import Gemma4Model

        return Gemma4Model(cfg, device, dtype, tp)
    return DecoderModel(cfg, device, dtype, tp)


class CausalLanguageModel:
    """Text-level facade over one engine (reference: core/.../model/DefaultCausalLanguageModel.java:28-148)."""

    def __init__(self, model, engine: Engine, tokenizer, name: str, sketches: SketchesSettings = DEFAULT_SETTINGS):
        self.model = model
        self.engine = engine
        self.tokenizer = tokenizer
        self.name = name
        self.cfg: ModelConfig = model.cfg
        self.tool_parser: ToolCallParser = parser_for_model(name)
        eos = set(self.cfg.eos_token_ids)
        if tokenizer.eos_token_id is not None:
            eos.add(tokenizer.eos_token_id)
        self.eos_ids = eos
        engine.eos_ids = frozenset(eos)
        engine.special_ids = frozenset(tokenizer.special_ids)
        engine.sampler.decode_token = lambda i: tokenizer.decode([i])
        self.guides = LogitsProcessorFactory(tokenizer, eos, self.cfg.vocab_size, sketches)
        self.generation_hook: Optional[Callable] = None
        self.adapters: dict = {}

    # -- prompts ---------------------------------------------------------------------------------------------------
    def prompt_builder(self) -> PromptBuilder:
        return PromptBuilder(self.tokenizer.chat_template, self.tokenizer.bos_token, self.tokenizer.eos_token)

    def encode_prompt(self, text: str) -> list[int]:
        ids = self.tokenizer.encode(text)
        bos = self.cfg.bos_token_id if self.cfg.bos_token_id is not None else self.tokenizer.bos_token_id
        if bos is not None:
            while ids and ids[0] == bos:  # strip leading BOS, then add exactly one when the family uses it
                ids = ids[1:]
            if self.cfg.add_bos and self.tokenizer.add_bos_token is not False and self.cfg.model_type not in ("qwen2", "qwen3", "qwen3_moe"):
                ids = [bos] + ids
        return ids

    # -- LoRA hot swap ---------------------------------------------------------------------------------------------
    def register_lora(self, adapter_dir: str, adapter_id: Optional[str] = None) -> str:
        """Load an adapter directory and keep it ready for :meth:`activate_lora`; returns its id."""
        ad = LoraAdapter(adapter_dir, adapter_id)
        self.adapters[ad.id] = ad
        return ad.id

    def activate_lora(self, adapter_id: Optional[str]) -> None:
        """Switch the run-time adapter (``None`` = base model). Allowed only between requests: all sequences of a batch share
        one adapter. Captured decode graphs are dropped because the set of launched kernels changes."""
        if self.engine.has_work():
            raise RuntimeError("cannot switch the LoRA adapter while requests are in flight")
        if adapter_id is not None and adapter_id not in self.adapters:
            raise KeyError(f"unknown LoRA adapter '{adapter_id}' (registered: {sorted(self.adapters)})")
        self.model.set_lora(None if adapter_id is None else self.adapters[adapter_id])
        self.engine._graphs.clear()

    # -- generation ------------------------------------------------------------------------------------------------
    def submit(self, prompt, params: Optional[GeneratorParameters] = None, on_event=None, session: Optional[str] = None) -> "Generation":
        params = params or GeneratorParameters()
        has_tools = bool(getattr(prompt, "has_tools", False))
        if isinstance(prompt, PromptContext):
            prompt = prompt.prompt
        ids = self.encode_prompt(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        gen = Generation(self, params, on_event, session or str(uuid.uuid4()), has_tools)
        gen.starts_in_reasoning = isinstance(prompt, str) and prompt_ends_inside_reasoning(prompt)
        guide = self.guides.create(params)
        stopper = StopStringDetector(gen.detok_special, params.stop_words, params.include_stop_str_in_output,
                                     self.tool_parser if has_tools else None)
        gen.stopper = stopper
        gen.request = self.engine.add_request(ids, params, gen._on_token, guide, stopper)
        return gen

    def generate(self, prompt, params: Optional[GeneratorParameters] = None, on_event=None, session: Optional[str] = None) -> Response:
        gen = self.submit(prompt, params, on_event, session)
        self.engine.run([gen.request])
        return gen.finish()

    def generate_many(self, prompts: list, params: Optional[GeneratorParameters] = None) -> list[Response]:
        import copy

        gens = [self.submit(p, copy.deepcopy(params) if params else None) for p in prompts]
        self.engine.run([g.request for g in gens])
        return [g.finish() for g in gens]

    def close(self) -> None:
        pass


class Generation:
    """One in-flight request: incremental detokenisation, event emission, final :class:`Response` assembly."""

    def __init__(self, clm: CausalLanguageModel, params, on_event, session, has_tools):
        self.clm = clm
        self.params = params
        self.on_event = on_event
        self.session = session
        self.has_tools = has_tools
        self.starts_in_reasoning = False  # the prompt ended inside <think> (set by submit)
        self.detok_plain = IncrementalDetokenizer(clm.tokenizer, skip_special=True)
        self.detok_special = SpecialTextView(clm.tokenizer, self.detok_plain)
        self.request: Optional[Request] = None
        self.stopper: Optional[StopStringDetector] = None

    def _on_token(self, token: int, request: Request) -> None:
        import time

        self.detok_special.push(token)
        piece = self.detok_plain.push(token)
        if self.on_event is not None and piece:
            self.on_event(token, piece, self.detok_special.text, (time.perf_counter() - request.t_submit) * 1e3)

    def finish(self) -> Response:
        r = self.request.response()
        text, text_sp = self.detok_plain.text, self.detok_special.text
        if self.stopper is not None and self.stopper.truncate_at is not None:
            cut = text_sp[: self.stopper.truncate_at]
            text_sp = cut
            # the plain text is the special-token text minus specials: cut it at the same stop string
            for s in self.params.stop_words:
                i = text.find(s)
                if i >= 0:
                    text = text[: i + (len(s) if self.params.include_stop_str_in_output else 0)]
                    break
        r.text_with_special_tokens = text_sp
        if _log.isEnabledFor(logging.INFO):
            # per-request lines in the reference's wording (core/.../model/GenerationEngine.java:131-132, 259-266)
            n, dt = r.generated_tokens, max(r.total_ms - r.ttft_ms, 1e-6)
            _log.info("time_to_first_token=%.1f ms prefix_length=%d", r.ttft_ms, r.prefix_hit_tokens)
            _log.info("generation_complete prompt_tokens=%d generated_tokens=%d total_ms=%.1f tokens_per_second=%.2f decode_tokens_per_second=%.2f finish=%s",
                      r.prompt_tokens, n, r.total_ms, n / max(r.total_ms, 1e-6) * 1e3, max(n - 1, 0) / dt * 1e3, r.finish_reason.name)
        if isinstance(self.clm.tool_parser, Gemma4ToolCallParser):  # gemma-4 marks its thought channel with special tokens
            content, reasoning = parse_gemma4_response(text_sp, text)
        else:
            content, reasoning = split_reasoning(text, self.starts_in_reasoning)
        r.reasoning = reasoning
        r.text = content
        if self.has_tools:
            calls = self.clm.tool_parser.extract(text_sp)
            if calls:
                r.tool_calls = calls
                r.finish_reason = FinishReason.TOOL_CALL
                r.text = self.clm.tool_parser.strip(content)
        return r


class AutoModelForCausalLM:
    class Builder:
        def __init__(self, model_dir: str):
            self.model_dir = model_dir
            self.conf = AutoModelConfig(model=model_dir)
            self.tp = SINGLE
            self.kv = KvCacheSettings()
            self.sketches = DEFAULT_SETTINGS
            self.name: Optional[str] = None
            self.layer_hook = None

        def with_device(self, device: str):
            self.conf.device = device
            return self

        def with_working_memory_type(self, dtype: str):
            self.conf.dtype = dtype
            return self

        def with_kv_cache_settings(self, kv: KvCacheSettings):
            self.kv = kv
            return self

        def with_tensor_parallel(self, rank: int, size: int, collectives=None):
            self.tp = TensorParallelContext(rank, size, collectives)
            return self

        def with_tensor_parallel_context(self, tp: TensorParallelContext):
            self.tp = tp
            return self

        def with_output_head_quantization(self, q: Optional[str]):
            self.conf.output_head_quantization = q
            return self

        def with_max_batch_size(self, n: int):
            self.conf.max_batch_size = n
            return self

        def with_quantize_on_demand(self, on: bool = True):
            self.conf.quantize_on_demand = on
            return self

        def with_lora_adapter(self, adapter_dir: str):
            self.conf.lora_adapter = adapter_dir
            return self

        def with_sketches_settings(self, s: SketchesSettings):
            self.sketches = s
            return self

        def with_config(self, conf: AutoModelConfig):
            model = self.conf.model
            self.conf = conf
            self.conf.model = conf.model or model
            self.model_dir = self.conf.model
            self.kv = KvCacheSettings(block_size=conf.kv_block_size, max_prefix_tokens=conf.kv_max_prefix_tokens,
                                      max_entries=conf.kv_max_entries, policy=conf.kv_policy, checkpoints=conf.kv_checkpoints, anchors=tuple(conf.kv_anchors),
                                      compression=conf.kv_compression, enabled=conf.kv_max_entries > 0 and conf.kv_max_prefix_tokens > 0)
            return self

        def with_name(self, name: str):
            self.name = name
            return self

        def with_tensor_parallel_collectives(self, collectives):
            """Collectives of an already configured rank / size (reference: withTensorParallelCollectives)."""
            self.tp = TensorParallelContext(self.tp.rank, self.tp.size, collectives)
            return self

        def with_download(self, on: bool = True, home: Optional[str] = None):
            """Treat the model argument as ``owner/name`` and fetch it into the local model cache when it is not there yet
            (reference: withDownload + ModelFetcher; needs network access, a directory that exists is used as it is)."""
            self._download, self._download_home = on, home
            return self

        def _accept(self, key: str, value):
            """Builder switches of the reference's CPU / WebGPU runtime that select code paths this runtime does not have
            (there is one CUDA path): accepted so that ported code keeps working, recorded for diagnostics."""
            self.conf.ignored = tuple(self.conf.ignored) + (f"{key}={value}",)
            return self

        def with_working_quant_type(self, dtype):  # activations stay bf16; int8 block activations are a CPU-kernel input format
            return self._accept("workingQuantType", dtype)

        def with_tensor_provider(self, provider):
            return self._accept("tensorProvider", getattr(provider, "__name__", provider))

        def with_parallel_settings(self, settings):  # gossip membership: ranks are fixed at launch on one node
            return self._accept("parallelSettings", settings)

        def with_gpu_prefill(self, on: bool = True):
            return self._accept("gpuPrefill", on)

        def with_gpu_decode(self, on: bool = True):
            return self._accept("gpuDecode", on)

        def with_gpu_decode_attention(self, on: bool = True):
            return self._accept("gpuDecodeAttention", on)

        def with_packed_prefill(self, on: bool = True):
            return self._accept("packedPrefill", on)

        def with_tensor_runtime_mode(self, mode):
            return self._accept("tensorRuntimeMode", mode)

        def with_tensor_plan_trace(self, on: bool = True):
            """The reference prints its tensor plan per generation; the counterpart here is the stage profiler's report."""
            return self.with_profile_stages(on) if on else self

        def with_layer_debug_hook(self, hook):
            self.layer_hook = hook
            return self

        def with_profile_stages(self, on: bool = True):
            self.conf.profile_stages = on
            return self

        def build_local_transformer_model(self):
            """Weights + model graph only (no engine, no tokenizer)."""
            conf = self.conf
            model_dir = self.model_dir
            if getattr(self, "_download", False) and not os.path.isdir(model_dir):
                from .ckpt.fetch import ModelFetcher

                kw = {"home": self._download_home} if self._download_home else {}
                model_dir = ModelFetcher.from_id(model_dir, **kw).maybe_download()
            if conf.quantize_on_demand:
                cache_root = os.path.expanduser(os.environ.get("DELIVERANCE_HOME", "~/.deliverance"))
                target = os.path.join(cache_root, os.path.basename(os.path.normpath(model_dir)) + "-JQ4")
                model_dir = quantize_on_demand(model_dir, target)
            cfg = load_config(model_dir)
            dev = _device(conf.device)
            dtype = {"auto": None, "bf16": torch.bfloat16, "BF16": torch.bfloat16, "f32": torch.float32, "F32": torch.float32,
                     "f16": torch.float16}.get(conf.dtype, None)
            if conf.lora_adapter:
                loader = MergingWeightLoader(model_dir, LoraAdapter(conf.lora_adapter))
            else:
                loader = WeightLoader(model_dir)
            model = build_model(cfg, dev, dtype, self.tp)
            if isinstance(model, BertModel):
                model.load(loader)
            else:
                model.load(loader, head_quant=conf.output_head_quantization)
                model.layer_hook = self.layer_hook
                if conf.profile_stages or os.environ.get("DELIVERANCE_PROFILE_STAGES"):
                    from .utils.profiler import InferenceProfiler

                    model.profiler = InferenceProfiler(dev)
            return model, model_dir

        def build(self) -> CausalLanguageModel:
            model, model_dir = self.build_local_transformer_model()
            if isinstance(model, BertModel):
                raise ValueError("bert checkpoints load through AutoModelForEmbeddings / AutoModelForSequenceClassification")
            conf = self.conf
            econf = EngineConfig(max_batch_tokens=conf.max_batch_size, max_seqs=conf.max_seqs, num_pages=conf.kv_pages,
                                 cuda_graphs=conf.cuda_graphs and not (conf.profile_stages or bool(os.environ.get("DELIVERANCE_PROFILE_STAGES"))),
                                 kv=self.kv, decode_interleave=conf.decode_interleave)
            engine = Engine(model, econf)
            tok = AutoTokenizer.from_pretrained(model_dir)
            return CausalLanguageModel(model, engine, tok, self.name or os.path.basename(os.path.normpath(model_dir)), self.sketches)

    @staticmethod
    def new_builder(model_dir: str) -> "AutoModelForCausalLM.Builder":
        return AutoModelForCausalLM.Builder(model_dir)

    @staticmethod
    def from_pretrained(model_dir: str, **kw) -> CausalLanguageModel:
        b = AutoModelForCausalLM.Builder(model_dir)
        for k, v in kw.items():
            if hasattr(b.conf, k):
                setattr(b.conf, k, v)
            else:
                raise TypeError(f"unknown option {k}")
        return b.build()
