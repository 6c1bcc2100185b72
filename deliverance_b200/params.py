"""Request parameters and results (field names follow the reference so that callers can switch over).

``GeneratorParameters``: core/.../generator/GeneratorParameters.java:12-30. ``Response``: core/.../generator/Response.java:10-23.
``FinishReason`` wire names: core/.../generator/FinishReason.java:4-23.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Callable, Optional


class FinishReason(enum.Enum):
    MAX_TOKENS = "length"
    STOP_TOKEN = "stop"
    STOP_STRING = "stop"
    TOOL_CALL = "tool_calls"
    GUIDED_COMPLETE = "stop"
    ERROR = "error"
    CANCELLED = "cancelled"

    @property
    def wire(self) -> str:
        return self.value


@dataclass
class GeneratorParameters:
    temperature: float = 0.0
    ntokens: Optional[int] = None  # absolute position limit (prompt + generation); default = context length
    seed: int = 42
    cache_salt: str = ""
    stop_words: list[str] = field(default_factory=list)
    include_stop_str_in_output: bool = False
    guided_choice: Optional[list[str]] = None
    guided_regex: Optional[str] = None
    guided_json: Optional[Any] = None
    max_tokens: Optional[int] = None
    logprobs: bool = False
    top_logprobs: int = 0
    xtc_threshold: Optional[float] = None
    xtc_probability: Optional[float] = None
    top_k: Optional[float] = None
    top_p: Optional[float] = None
    uniform_top_p: Optional[float] = None
    lora_adapter: Optional[str] = None

    def validate(self) -> None:
        modes = sum(x is not None for x in (self.guided_choice, self.guided_regex, self.guided_json))
        if modes > 1:
            raise ValueError("only one of guided_choice, guided_regex, guided_json may be set")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.uniform_top_p is not None and self.temperature == 0:
            raise ValueError("uniform_top_p requires temperature > 0")
        if self.top_k is not None and self.xtc_threshold:
            raise ValueError("top_k cannot be combined with xtc")
        if self.uniform_top_p is not None and self.top_p is None:
            raise ValueError("uniform_top_p requires top_p")
        # value ranges of AbstractGeneratorSampler.sampleTopKTopP (core/.../model/AbstractGeneratorSampler.java:267-279)
        if self.top_p is not None and not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.uniform_top_p is not None and not 0.0 < self.uniform_top_p <= 1.0:
            raise ValueError("uniform_top_p must be in (0, 1]")
        if self.top_k is not None and self.top_k <= 0:
            raise ValueError("top_k must be > 0")


@dataclass
class TokenLogProb:
    token_id: int
    token: str
    logprob: float
    top: list["TokenLogProb"] = field(default_factory=list)


@dataclass
class ToolCall:
    id: str
    name: str
    arguments: Any
    type: str = "function"


@dataclass
class Response:
    text: str = ""
    text_with_special_tokens: str = ""
    reasoning: Optional[str] = None
    finish_reason: FinishReason = FinishReason.MAX_TOKENS
    prompt_tokens: int = 0
    generated_tokens: int = 0
    sampler_returns: list[TokenLogProb] = field(default_factory=list)
    ttft_ms: float = 0.0
    avg_ms_per_token: float = 0.0
    total_ms: float = 0.0
    tool_calls: list[ToolCall] = field(default_factory=list)
    token_ids: list[int] = field(default_factory=list)
    prefix_hit_tokens: int = 0

    @property
    def tokens_per_second(self) -> float:
        """Generated tokens after the first / (total - TTFT) (core/InferenceBenchmark.md:92-98)."""
        dt = self.total_ms - self.ttft_ms
        return (self.generated_tokens - 1) * 1000.0 / dt if dt > 0 and self.generated_tokens > 1 else 0.0


# event callback: (token_id, token_text, text_with_special, ms_since_start)
GenerateEvent = Callable[[int, str, str, float], None]
