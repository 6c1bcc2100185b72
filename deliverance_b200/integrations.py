"""Framework-style chat-model adapter: one ``ChatModel`` interface over the HTTP API or over an in-process model.

The reference ships this as Spring AI modules: a ``ChatModel`` over HTTP (blocking + streaming, tool calls with the
framework's tool-execution loop, guided-decoding options; spring-ai-deliverance/.../DeliveranceChatModel.java,
DeliveranceChatOptions.java, DeliveranceApi.java) and the same interface embedded in the application's process
(spring-ai-deliverance-embedded/.../EmbeddedDeliveranceChatModel.java, EmbeddedDeliveranceOptionsMapper.java). The Python
shape of that contract:

    model = HttpChatModel("http://127.0.0.1:8080")              # or EmbeddedChatModel(AutoModelForCausalLM.from_pretrained(dir))
    reply = model.call([{"role": "user", "content": "2+2?"}], ChatOptions(temperature=0.0, max_tokens=32))
    for delta in model.stream(messages, options): ...
    reply = model.call(messages, ChatOptions(tools=[ToolCallback("add", "adds", schema, fn)]))   # tools are executed, results fed back

``ChatOptions`` merge like the reference's (per-call options over the model's defaults); unknown extras go to the request as
they are (HTTP) or are rejected (embedded).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator, Optional


@dataclass
class ToolCallback:
    name: str
    description: str
    parameters: dict
    fn: Callable[..., Any]

    def spec(self) -> dict:
        return {"type": "function", "function": {"name": self.name, "description": self.description, "parameters": self.parameters}}

    def invoke(self, arguments: Any) -> str:
        args = json.loads(arguments) if isinstance(arguments, str) and arguments.strip() else (arguments or {})
        out = self.fn(**args) if isinstance(args, dict) else self.fn(args)
        return out if isinstance(out, str) else json.dumps(out)


@dataclass
class ChatOptions:
    model: Optional[str] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[float] = None
    uniform_top_p: Optional[float] = None
    xtc_threshold: Optional[float] = None
    xtc_probability: Optional[float] = None
    max_tokens: Optional[int] = None
    seed: Optional[int] = None
    stop: Optional[list] = None
    guided_json: Optional[dict] = None
    guided_regex: Optional[str] = None
    guided_choice: Optional[list] = None
    chat_template_kwargs: Optional[dict] = None
    tools: list = field(default_factory=list)  # ToolCallback entries
    max_tool_rounds: int = 8
    extra: dict = field(default_factory=dict)

    def merged(self, over: Optional["ChatOptions"]) -> "ChatOptions":
        """Per-call options win over these defaults field by field; tools and extras are combined."""
        if over is None:
            return self
        out = dataclasses.replace(self)
        for f in dataclasses.fields(self):
            v = getattr(over, f.name)
            if f.name == "tools":
                names = {t.name for t in over.tools}
                out.tools = [t for t in self.tools if t.name not in names] + list(over.tools)
            elif f.name == "extra":
                out.extra = {**self.extra, **over.extra}
            elif f.name == "max_tool_rounds":
                out.max_tool_rounds = over.max_tool_rounds
            elif v is not None:
                setattr(out, f.name, v)
        return out

    def request_fields(self) -> dict:
        skip = {"tools", "max_tool_rounds", "extra"}
        body = {f.name: getattr(self, f.name) for f in dataclasses.fields(self) if f.name not in skip and getattr(self, f.name) is not None}
        if self.tools:
            body["tools"] = [t.spec() for t in self.tools]
        body.update(self.extra)
        return body


@dataclass
class ChatReply:
    content: str = ""
    reasoning: Optional[str] = None
    tool_calls: list = field(default_factory=list)  # OpenAI-shaped dicts of the LAST model turn that asked for tools
    finish_reason: str = "stop"
    usage: dict = field(default_factory=dict)
    messages: list = field(default_factory=list)  # the conversation including tool traffic


class ChatModel:
    """Subclasses implement ``_complete`` (one model turn) and ``_stream`` (one streamed turn)."""

    def __init__(self, defaults: Optional[ChatOptions] = None):
        self.defaults = defaults or ChatOptions()

    def _complete(self, messages: list, opts: ChatOptions) -> ChatReply:  # pragma: no cover - interface
        raise NotImplementedError

    def _stream(self, messages: list, opts: ChatOptions) -> Iterator[tuple]:  # pragma: no cover - interface
        raise NotImplementedError

    def call(self, messages: list, options: Optional[ChatOptions] = None) -> ChatReply:
        """Blocking call. While the model asks for tools that have callbacks, they are executed and their results appended as
        ``tool`` messages, up to ``max_tool_rounds`` model turns; a call to an unknown tool is returned to the caller."""
        opts = self.defaults.merged(options)
        convo = [dict(m) for m in messages]
        by_name = {t.name: t for t in opts.tools}
        reply = ChatReply()
        for _ in range(max(1, opts.max_tool_rounds)):
            reply = self._complete(convo, opts)
            if not reply.tool_calls or not all(tc["function"]["name"] in by_name for tc in reply.tool_calls):
                break
            convo.append({"role": "assistant", "content": reply.content, "tool_calls": reply.tool_calls})
            for tc in reply.tool_calls:
                try:
                    result = by_name[tc["function"]["name"]].invoke(tc["function"].get("arguments"))
                except Exception as e:  # noqa: BLE001 - the model sees the failure and may correct itself
                    result = f"tool {tc['function']['name']} failed: {e}"
                convo.append({"role": "tool", "tool_call_id": tc.get("id"), "name": tc["function"]["name"], "content": result})
        reply.messages = convo + ([{"role": "assistant", "content": reply.content}] if not reply.tool_calls else [])
        return reply

    def stream(self, messages: list, options: Optional[ChatOptions] = None) -> Iterator[tuple]:
        """Yields ("content" | "reasoning" | "tool_calls" | "finish", value) for one model turn (no tool execution)."""
        return self._stream([dict(m) for m in messages], self.defaults.merged(options))


class HttpChatModel(ChatModel):
    def __init__(self, base_url: str = "http://127.0.0.1:8080", defaults: Optional[ChatOptions] = None, client=None, **client_kw):
        super().__init__(defaults)
        if client is None:
            from .client import DeliveranceClient

            client = DeliveranceClient(base_url, **client_kw)
        self.client = client

    def _complete(self, messages, opts):
        j = self.client.chat(messages, **opts.request_fields())
        if "error" in j:
            raise RuntimeError(j["error"].get("message", "server error"))
        ch = j["choices"][0]
        m = ch["message"]
        return ChatReply(m.get("content") or "", m.get("reasoning_content") or m.get("reasoning"), list(m.get("tool_calls") or []),
                         ch.get("finish_reason") or "stop", j.get("usage") or {})

    def _stream(self, messages, opts):
        return self.client.stream_chat(messages, **opts.request_fields())


class EmbeddedChatModel(ChatModel):
    """The same interface over a model loaded in this process (``deliverance_b200.api.CausalLanguageModel``)."""

    def __init__(self, clm, defaults: Optional[ChatOptions] = None):
        super().__init__(defaults)
        self.clm = clm

    def _prepare(self, messages, opts):
        from .params import GeneratorParameters

        if opts.extra:
            raise ValueError(f"options without an embedded equivalent: {', '.join(opts.extra)}")
        pb = self.clm.prompt_builder().with_kwargs(opts.chat_template_kwargs)
        for m in messages:
            role, content = m["role"], m.get("content") or ""
            if role in ("system", "developer"):
                pb.add_system(content)
            elif role == "user":
                pb.add_user(content)
            elif role == "assistant":
                pb.add_assistant(content, m.get("tool_calls"))
            elif role in ("tool", "function"):
                pb.add_tool_result(m.get("tool_call_id"), content, m.get("name"))
            else:
                raise ValueError(f"unsupported message role '{role}'")
        pb.add_tools([t.spec() for t in opts.tools])
        p = GeneratorParameters()
        for name in ("temperature", "top_p", "top_k", "uniform_top_p", "xtc_threshold", "xtc_probability", "max_tokens", "seed", "guided_json",
                     "guided_regex", "guided_choice"):
            v = getattr(opts, name)
            if v is not None:
                setattr(p, name, v)
        if opts.stop:
            p.stop_words = list(opts.stop)
        p.validate()
        return pb.build(), p

    @staticmethod
    def _tool_calls(r) -> list:
        return [{"id": tc.id, "type": "function", "function": {"name": tc.name, "arguments": tc.arguments if isinstance(tc.arguments, str)
                                                                else json.dumps(tc.arguments)}} for tc in (r.tool_calls or [])]

    def _complete(self, messages, opts):
        ctx, p = self._prepare(messages, opts)
        r = self.clm.generate(ctx, p)
        return ChatReply(r.text, r.reasoning, self._tool_calls(r), r.finish_reason.wire,
                         {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.generated_tokens, "total_tokens": r.prompt_tokens + r.generated_tokens})

    def _stream(self, messages, opts):
        import queue
        import threading

        ctx, p = self._prepare(messages, opts)
        q: "queue.Queue" = queue.Queue()

        def run():
            try:
                r = self.clm.generate(ctx, p, on_event=lambda tok, piece, text, ms: q.put(("content", piece)))
                if r.tool_calls:
                    q.put(("tool_calls", self._tool_calls(r)))
                q.put(("finish", r.finish_reason.wire))
            except Exception as e:  # noqa: BLE001
                q.put(("error", e))
            q.put(None)

        threading.Thread(target=run, daemon=True).start()
        while True:
            item = q.get()
            if item is None:
                return
            if item[0] == "error":
                raise item[1]
            yield item
