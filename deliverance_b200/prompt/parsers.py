"""Tool-call extraction, end-of-turn detection and reasoning (``<think>``) splitting.

Reference behaviour: ``ToolCallParser{extract, shouldEndTurn}`` (core/.../toolcallparser/ToolCallParser.java:17-38);
Qwen — JSON after ``<tools>`` or inside ``<tool_call>...</tool_call>``, brace-matched ``{name, arguments}``, ids assigned
from 101 (QwenToolCallParser.java:14-71); Llama — JSON ``{type, function, parameters}`` in the reply, ``<|eot_id|>`` ends
the turn (LlamaToolCallParser.java:27-75); parser chosen by model-name prefix (AutoModelForCausaLm.java:80-90).
``ReasoningTextSplitter`` streams ``<think>...</think>`` into a separate channel and holds back partial tags
(core/.../model/ReasoningTextSplitter.java:26-100).
"""
from __future__ import annotations

import json
from typing import Optional

from ..params import ToolCall


def _match_braces(text: str, start: int) -> Optional[str]:
    """The balanced ``{...}`` object starting at ``start`` (string-aware), or ``None``."""
    depth, in_str, esc = 0, False, False
    for i in range(start, len(text)):
        c = text[i]
        if in_str:
            if esc:
                esc = False
            elif c == "\\":
                esc = True
            elif c == '"':
                in_str = False
            continue
        if c == '"':
            in_str = True
        elif c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                return text[start : i + 1]
    return None


def _json_objects(text: str) -> list[dict]:
    out, i = [], 0
    while True:
        j = text.find("{", i)
        if j < 0:
            return out
        obj = _match_braces(text, j)
        if obj is None:
            return out
        try:
            v = json.loads(obj)
            if isinstance(v, dict):
                out.append(v)
            i = j + len(obj)
        except ValueError:
            i = j + 1


class ToolCallParser:
    def extract(self, text: str) -> list[ToolCall]:
        return []

    def should_end_turn(self, text_with_special: str) -> bool:
        return False

    def strip(self, text: str) -> str:
        """Response text with the tool-call markup removed."""
        return text


class DefaultToolCallParser(ToolCallParser):
    pass


class QwenToolCallParser(ToolCallParser):
    FIRST_ID = 101

    def extract(self, text: str) -> list[ToolCall]:
        calls: list[ToolCall] = []
        regions = []
        pos = 0
        while True:
            a = text.find("<tool_call>", pos)
            if a < 0:
                break
            b = text.find("</tool_call>", a)
            regions.append(text[a + len("<tool_call>") : b if b >= 0 else len(text)])
            if b < 0:
                break
            pos = b + len("</tool_call>")
        if not regions and "<tools>" in text:
            regions.append(text[text.find("<tools>") + len("<tools>") :])
        for reg in regions:
            for obj in _json_objects(reg):
                if "name" in obj:
                    calls.append(ToolCall(str(self.FIRST_ID + len(calls)), str(obj["name"]), obj.get("arguments", obj.get("parameters", {}))))
        return calls

    def strip(self, text: str) -> str:
        for tag in ("<tool_call>", "<tools>"):
            i = text.find(tag)
            if i >= 0:
                text = text[:i]
        return text.rstrip()


class LlamaToolCallParser(ToolCallParser):
    def extract(self, text: str) -> list[ToolCall]:
        marker = "<|end_header_id|>"
        if marker in text:
            text = text[text.rfind(marker) + len(marker) :]
        calls = []
        for obj in _json_objects(text):
            name = obj.get("function") if isinstance(obj.get("function"), str) else obj.get("name")
            if name and ("parameters" in obj or "arguments" in obj):
                calls.append(ToolCall(f"call_{len(calls)}", str(name), obj.get("parameters", obj.get("arguments", {}))))
        return calls

    def should_end_turn(self, text_with_special: str) -> bool:
        return text_with_special.endswith("<|eot_id|>")

    def strip(self, text: str) -> str:
        return "" if self.extract(text) else text


class MixtralToolCallParser(ToolCallParser):
    """Placeholder like the reference's stub: Mixtral replies are never parsed into calls."""


class Gemma4ToolCallParser(ToolCallParser):
    """``<|tool_call>call:NAME{args}<tool_call|>`` regions. ``args`` is either JSON or the template's relaxed form with bare
    keys and ``<|"|>`` as the string quote (reference: core/.../toolcallparser/Gemma4ToolCallParser.java and its test vectors
    in Gemma4ToolCallParserTest.java). Ids count from 101; a closed region ends the turn."""

    OPEN, CLOSE, QUOTE = "<|tool_call>", "<tool_call|>", '<|"|>'
    FIRST_ID = 101

    def extract(self, text: str) -> list[ToolCall]:
        calls: list[ToolCall] = []
        pos = 0
        while True:
            a = text.find(self.OPEN, pos)
            if a < 0:
                break
            b = text.find(self.CLOSE, a)
            body = text[a + len(self.OPEN) : b if b >= 0 else len(text)].strip()
            pos = (b + len(self.CLOSE)) if b >= 0 else len(text)
            if not body.startswith("call:"):
                continue
            brace = body.find("{")
            if brace < 0:
                continue
            name = body[5:brace].strip()
            raw = _match_braces(body, brace)
            if not name or raw is None:
                continue
            try:
                args = json.loads(self._to_json(raw))
            except ValueError:
                continue
            if isinstance(args, dict):
                calls.append(ToolCall(str(self.FIRST_ID + len(calls)), name, args))
        return calls

    def _to_json(self, raw: str) -> str:
        """Relaxed argument syntax -> JSON: ``<|"|>`` becomes a quote, bare object keys get quoted (outside strings only)."""
        out, i, in_str = [], 0, False
        while i < len(raw):
            if raw.startswith(self.QUOTE, i):
                out.append('"')
                in_str = not in_str
                i += len(self.QUOTE)
                continue
            c = raw[i]
            if in_str:
                if c == '"':  # a literal quote inside a <|"|>-delimited string
                    out.append('\\"')
                elif c == "\\" and i + 1 < len(raw):
                    out.append(raw[i : i + 2])
                    i += 1
                else:
                    out.append(c)
                i += 1
                continue
            if c == '"':  # ordinary JSON string: copy verbatim
                j = i + 1
                while j < len(raw) and raw[j] != '"':
                    j += 2 if raw[j] == "\\" else 1
                out.append(raw[i : j + 1])
                i = j + 1
                continue
            if c.isalpha() or c == "_":
                j = i
                while j < len(raw) and (raw[j].isalnum() or raw[j] in "_.-"):
                    j += 1
                word = raw[i:j]
                k = j
                while k < len(raw) and raw[k].isspace():
                    k += 1
                if k < len(raw) and raw[k] == ":" and word not in ("true", "false", "null"):
                    out.append(json.dumps(word))
                else:
                    out.append(word)
                i = j
                continue
            out.append(c)
            i += 1
        return "".join(out)

    def should_end_turn(self, text_with_special: str) -> bool:
        return self.CLOSE in text_with_special


def parser_for_model(name: str) -> ToolCallParser:
    n = (name or "").lower()
    base = n.split("/")[-1]
    if base.startswith("qwen"):
        return QwenToolCallParser()
    if base.startswith(("llama", "meta-llama")) or "llama-3" in base:
        return LlamaToolCallParser()
    if base.startswith("mixtral"):
        return MixtralToolCallParser()
    if base.startswith(("gemma-4", "gemma4")):
        return Gemma4ToolCallParser()
    return DefaultToolCallParser()


class ReasoningTextSplitter:
    """Streaming splitter: text between ``<think>`` and ``</think>`` goes to the reasoning channel."""

    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self, start_in_reasoning: bool = False):
        self.in_reasoning = start_in_reasoning
        self.buf = ""
        self.content = ""
        self.reasoning = ""

    def accept(self, piece: str) -> tuple[str, str]:
        """Feed a text fragment; returns (content delta, reasoning delta)."""
        self.buf += piece
        c_out, r_out = "", ""
        while self.buf:
            tag = self.CLOSE if self.in_reasoning else self.OPEN
            i = self.buf.find(tag)
            if i >= 0:
                seg = self.buf[:i]
                if self.in_reasoning:
                    r_out += seg
                else:
                    c_out += seg
                self.buf = self.buf[i + len(tag) :]
                self.in_reasoning = not self.in_reasoning
                continue
            # hold back a suffix that could be the start of the tag
            keep = 0
            for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-k:]):
                    keep = k
                    break
            seg = self.buf[: len(self.buf) - keep]
            if self.in_reasoning:
                r_out += seg
            else:
                c_out += seg
            self.buf = self.buf[len(self.buf) - keep :]
            break
        self.content += c_out
        self.reasoning += r_out
        return c_out, r_out

    def flush(self) -> tuple[str, str]:
        seg, self.buf = self.buf, ""
        if self.in_reasoning:
            self.reasoning += seg
            return "", seg
        self.content += seg
        return seg, ""


class Gemma4ChannelSplitter(ReasoningTextSplitter):
    """Streaming splitter for gemma-4 channel markers: ``<|channel>thought\n ... <channel|>`` is the reasoning channel."""

    OPEN, CLOSE = "<|channel>thought\n", "<channel|>"


_GEMMA4_MARKERS = ("<|channel>", "<channel|>", "<|turn>", "<turn|>", "<|think|>")


def parse_gemma4_response(text_with_special: str, fallback: str = "") -> tuple[str, Optional[str]]:
    """(content, reasoning) of a complete gemma-4 reply: the first closed thought channel is the reasoning, what is left
    with the channel / turn markers removed is the content; without a closed thought channel the cleaned fallback text is the
    content (reference: core/.../model/gemma4/Gemma4ResponseParser.java:10-52 and Gemma4ResponseParserTest.java)."""

    def clean(t: str) -> str:
        for m in _GEMMA4_MARKERS:
            t = t.replace(m, "")
        return t.strip()

    start_tag, end_tag = Gemma4ChannelSplitter.OPEN, Gemma4ChannelSplitter.CLOSE
    a = text_with_special.find(start_tag) if text_with_special else -1
    b = text_with_special.find(end_tag, a + len(start_tag)) if a >= 0 else -1
    if b < 0:
        return clean(fallback or ""), None
    reasoning = text_with_special[a + len(start_tag) : b].strip()
    content = clean(text_with_special[:a] + text_with_special[b + len(end_tag) :]) or clean(fallback or "")
    return content, (reasoning or None)


def prompt_ends_inside_reasoning(prompt: str) -> bool:
    """True when the rendered prompt already opened ``<think>`` and did not close it (thinking templates end the generation
    prompt with ``<think>\n``): the generated text then starts in the reasoning channel
    (reference: core/.../model/ReasoningTextSplitter.java ``promptEndsInsideReasoning``)."""
    a = prompt.rfind(ReasoningTextSplitter.OPEN)
    return a >= 0 and prompt.find(ReasoningTextSplitter.CLOSE, a) < 0


def split_reasoning(text: str, start_in_reasoning: bool = False) -> tuple[str, Optional[str]]:
    s = ReasoningTextSplitter(start_in_reasoning)
    s.accept(text)
    s.flush()
    return s.content.lstrip("\n") if s.reasoning else s.content, (s.reasoning.strip() or None)


class StopStringDetector:
    """Engine-side stopper: stop strings over the accumulated text with special tokens, tool-parser end of turn."""

    def __init__(self, detok, stop_words: list[str], include_stop: bool, tool_parser: Optional[ToolCallParser] = None):
        self.detok = detok
        self.stop_words = [s for s in (stop_words or []) if s]
        self.include_stop = include_stop
        self.tool_parser = tool_parser
        self.truncate_at: Optional[int] = None

    def check(self, request):
        from ..params import FinishReason

        text = self.detok.text
        for s in self.stop_words:
            i = text.find(s)
            if i >= 0:
                self.truncate_at = i + (len(s) if self.include_stop else 0)
                return FinishReason.STOP_STRING
        if self.tool_parser is not None and self.tool_parser.should_end_turn(text):
            return FinishReason.STOP_TOKEN
        return None
