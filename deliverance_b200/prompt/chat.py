"""Prompt construction: HF ``chat_template`` rendering with Jinja2 and a message builder.

Template variables follow the reference's ``PromptSupport`` (core/.../safetensors/prompt/PromptSupport.java:163-306):
``messages`` (``{role, content, tool_calls?, tool_call_id?}``), ``add_generation_prompt``, ``bos_token``, ``eos_token``,
``tools`` (only when non-empty) and any ``chat_template_kwargs`` (for instance ``enable_thinking``). A request may override
the template. The reference carries a hand-written ChatML renderer for Qwen3 templates that use ``messages[::-1]`` because
its Java Jinja engine cannot slice; Jinja2 handles that natively, and the same ChatML renderer is kept here only as the
fallback for models without any template.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class Function:
    name: str
    description: str = ""
    parameters: dict = field(default_factory=dict)


@dataclass
class Tool:
    function: Function
    type: str = "function"

    def to_dict(self) -> dict:
        return {"type": self.type, "function": {"name": self.function.name, "description": self.function.description,
                                                "parameters": self.function.parameters}}


@dataclass
class PromptContext:
    prompt: str
    has_tools: bool = False


def _jinja_env():
    import jinja2
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(msg):
        raise jinja2.exceptions.TemplateError(msg)

    def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
        return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

    def strftime_now(fmt):
        import datetime

        return datetime.datetime.now().strftime(fmt)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
    env.filters["tojson"] = tojson
    env.globals["raise_exception"] = raise_exception
    env.globals["strftime_now"] = strftime_now
    return env


def render_chatml(messages: list[dict], tools: list[dict], add_generation_prompt: bool, enable_thinking: Optional[bool]) -> str:
    """ChatML: ``<|im_start|>role\\n...<|im_end|>\\n`` with ``<tools>`` block and ``<tool_call>`` / ``<tool_response>`` wrapping."""
    out = []
    msgs = list(messages)
    if tools:
        sys_text = msgs[0]["content"] + "\n\n" if msgs and msgs[0]["role"] == "system" else ""
        if msgs and msgs[0]["role"] == "system":
            msgs = msgs[1:]
        out.append("<|im_start|>system\n" + sys_text + "# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                   "You are provided with function signatures within <tools></tools> XML tags:\n<tools>")
        for t in tools:
            out.append("\n" + json.dumps(t, ensure_ascii=False))
        out.append("\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
                   "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n"
                   "</tool_call><|im_end|>\n")
    for m in msgs:
        role, content = m["role"], m.get("content") or ""
        if role == "tool":
            out.append(f"<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n")
            continue
        body = content
        for tc in m.get("tool_calls") or []:
            fn = tc.get("function", tc)
            args = fn.get("arguments")
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except ValueError:
                    pass
            body += ("\n" if body else "") + "<tool_call>\n" + json.dumps({"name": fn.get("name"), "arguments": args}, ensure_ascii=False) + "\n</tool_call>"
        out.append(f"<|im_start|>{role}\n{body}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
        if enable_thinking is False:
            out.append("<think>\n\n</think>\n\n")
    return "".join(out)


class PromptBuilder:
    """Collects messages / tools and renders them with the model's (or an overriding) chat template."""

    def __init__(self, chat_template: Optional[str] = None, bos_token: Optional[str] = None, eos_token: Optional[str] = None):
        self.template = chat_template
        self.bos_token = bos_token or ""
        self.eos_token = eos_token or ""
        self.messages: list[dict] = []
        self.tools: list[dict] = []
        self.kwargs: dict[str, Any] = {}
        self.add_generation_prompt = True

    def add_system(self, text: str) -> "PromptBuilder":
        self.messages.append({"role": "system", "content": text})
        return self

    def add_user(self, text: str) -> "PromptBuilder":
        self.messages.append({"role": "user", "content": text})
        return self

    def add_assistant(self, text: str, tool_calls: Optional[list[dict]] = None) -> "PromptBuilder":
        m: dict = {"role": "assistant", "content": text}
        if tool_calls:
            m["tool_calls"] = tool_calls
        self.messages.append(m)
        return self

    def add_tool_result(self, tool_call_id: Optional[str], content: str, name: Optional[str] = None) -> "PromptBuilder":
        m = {"role": "tool", "content": content}
        if tool_call_id is not None:
            m["tool_call_id"] = tool_call_id
        if name:
            m["name"] = name
        self.messages.append(m)
        return self

    def add_tools(self, tools) -> "PromptBuilder":
        for t in tools or []:
            self.tools.append(t.to_dict() if isinstance(t, Tool) else dict(t))
        return self

    def with_template(self, template: Optional[str]) -> "PromptBuilder":
        if template:
            self.template = template
        return self

    def with_kwargs(self, kwargs: Optional[dict]) -> "PromptBuilder":
        self.kwargs.update(kwargs or {})
        return self

    def continue_final_message(self, on: bool = True) -> "PromptBuilder":
        """Render so that the model continues the last message instead of starting a new turn (a prefilled assistant reply):
        no generation prompt, and the rendered text is cut right after the last message's content."""
        self._continue_final = on
        return self

    def _select_template(self) -> Optional[str]:
        """A tokenizer may carry several named templates (a dict, or a list of ``{"name", "template"}``): ``tool_use`` is taken
        when tools are present and it exists, otherwise ``default``; a ``template_name`` kwarg picks one by name."""
        t = self.template
        if isinstance(t, list):
            t = {e["name"]: e["template"] for e in t if isinstance(e, dict) and "name" in e and "template" in e}
        if isinstance(t, dict):
            name = self.kwargs.get("template_name")
            if name is not None:
                if name not in t:
                    raise ValueError(f"chat template '{name}' not found (available: {', '.join(sorted(t))})")
                return t[name]
            if self.tools and "tool_use" in t:
                return t["tool_use"]
            if "default" in t:
                return t["default"]
            raise ValueError(f"no default chat template among: {', '.join(sorted(t))}")
        return t

    def build(self) -> PromptContext:
        if not self.messages:
            raise ValueError("a prompt needs at least one message")
        cont = getattr(self, "_continue_final", False)
        gen = self.add_generation_prompt and not cont
        template = self._select_template()
        if template:
            variables = {"messages": self.messages, "add_generation_prompt": gen, "bos_token": self.bos_token, "eos_token": self.eos_token}
            if self.tools:
                variables["tools"] = self.tools
            variables.update({k: v for k, v in self.kwargs.items() if k != "template_name"})
            text = _jinja_env().from_string(template).render(**variables)
        else:
            text = render_chatml(self.messages, self.tools, gen, self.kwargs.get("enable_thinking"))
        if cont:
            final = self.messages[-1].get("content") or ""
            if isinstance(final, list):  # text parts: the last text part is what gets continued
                final = next((p.get("text", "") for p in reversed(final) if isinstance(p, dict) and p.get("type", "text") == "text"), "")
            final = final.strip()
            i = text.rfind(final) if final else -1
            if i < 0:
                raise ValueError("continue_final_message: the final message does not appear in the rendered chat (does the template "
                                 "rewrite message contents?)")
            # keep the message's own trailing whitespace when the template kept it, drop what the template adds after it
            end = i + len(final)
            raw = self.messages[-1].get("content") if isinstance(self.messages[-1].get("content"), str) else final
            tail = raw[len(raw.rstrip()):]
            text = text[:end] + (tail if text[end:end + len(tail)] == tail else "")
        return PromptContext(text, bool(self.tools))
