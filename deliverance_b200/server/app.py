"""OpenAI-style HTTP API.

Endpoints and payloads follow the reference's Spring controllers (web/src/main/java/net/deliverance/http/):
``POST /chat/completions`` (ChatCompletionController.java:234-443, request mapping ChatCompletionService.java:17-128),
``POST /v1/completions`` + ``/completions`` (:99-232), ``POST /embeddings`` (EmbeddingController.java:38-53),
``GET /models`` (ModelController.java:26-46), ``GET /tp/status`` (TensorParallelDiagnosticsController.java:22-40).
Streaming is SSE with ``X-Deliverance-Session``, comment heartbeats every second that also detect a closed client and cancel
the generation, ``content`` / reasoning deltas (field ``reasoning_content`` in openai mode, ``reasoning`` in vllm mode),
tool-call deltas after generation with content buffered while tools are present, a final chunk with ``finish_reason`` and
``data: [DONE]``. Optional HTTP Basic / JWT (HS256) auth on ``/chat``, ``/embeddings``, ``/models``
(auth/SecurityConfig.java:30-71). ``guided_choice`` is accepted here as well (the reference maps only regex / json).
"""
from __future__ import annotations

import asyncio
import base64
import hashlib
import hmac
import json
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

from fastapi import Request  # module level: handler annotations are resolved from the module namespace

from ..params import FinishReason, GeneratorParameters, Response
from ..prompt.parsers import ReasoningTextSplitter, prompt_ends_inside_reasoning
from .runner import EngineRunner


@dataclass
class ServerSettings:
    reasoning_field: str = "openai"  # openai -> reasoning_content, vllm -> reasoning
    basic_user: Optional[str] = None
    basic_password: Optional[str] = None
    jwt_secret: Optional[str] = None
    heartbeat_s: float = 1.0
    request_timeout_s: float = 600.0
    pre_generate: Optional[Callable[[dict, GeneratorParameters], Optional[str]]] = None  # may rewrite or reject (return error text)
    # Under load every streamed token costs the interpreter an event-loop wake-up, a JSON chunk and a socket write, and with
    # a hundred streams that work competes with the engine thread. Above `coalesce_above` concurrent requests a stream sends
    # one chunk per `coalesce_tokens` tokens (or every `coalesce_ms`); the first token always goes out at once.
    # Back-pressure: with more than this many requests in the server (running, waiting for admission or not yet picked up by the
    # engine thread) a new one is refused with 429 and a Retry-After header instead of queueing without bound (0: no limit).
    max_queue: int = 0
    coalesce_above: int = 16
    coalesce_tokens: int = 4
    coalesce_ms: float = 50.0

    @property
    def reasoning_key(self) -> str:
        return "reasoning" if self.reasoning_field == "vllm" else "reasoning_content"


@dataclass
class ModelRegistry:
    generation: dict = field(default_factory=dict)  # name -> EngineRunner
    embedding: dict = field(default_factory=dict)  # name -> EmbeddingModel
    tp_status: Callable[[], dict] = lambda: {"enabled": False, "size": 1, "rank": 0}
    membership: Optional[object] = None  # parallel.gossip.TensorParallelMembership when the deployment is gossip-managed

    def find(self, name: Optional[str]) -> EngineRunner:
        if not self.generation:
            raise KeyError("no generation model is loaded")
        if name in self.generation:
            return self.generation[name]
        if name is None or name == "":
            return next(iter(self.generation.values()))
        raise KeyError(f"model '{name}' is not loaded (available: {', '.join(self.generation)})")


def map_chat_request(body: dict, runner: EngineRunner):
    """Request JSON -> (PromptContext, GeneratorParameters)."""
    clm = runner.clm
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ValueError("'messages' must be a non-empty list")
    if body.get("chat_template_kwargs") is not None and not isinstance(body["chat_template_kwargs"], dict):
        raise ValueError("'chat_template_kwargs' must be an object")
    b = clm.prompt_builder().with_template(body.get("chat_template")).with_kwargs(body.get("chat_template_kwargs"))
    for m in msgs:
        if not isinstance(m, dict):
            raise ValueError("every entry of 'messages' must be an object with 'role' and 'content'")
        role = m.get("role")
        content = m.get("content")
        if isinstance(content, list):  # text parts
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type", "text") == "text")
        content = "" if content is None else content if isinstance(content, str) else json.dumps(content)
        if role == "system":
            b.add_system(content)
        elif role == "user":
            b.add_user(content)
        elif role == "assistant":
            b.add_assistant(content, m.get("tool_calls"))
        elif role == "developer":  # newer name of the system role
            b.add_system(content)
        elif role in ("tool", "function"):  # "function": result message of the legacy functions API
            b.add_tool_result(m.get("tool_call_id"), content, m.get("name"))
        else:
            raise ValueError(f"unsupported message role '{role}'")
    b.add_tools(select_tools(body))
    if body.get("add_generation_prompt") is False:
        b.add_generation_prompt = False
    if body.get("continue_final_message"):  # the model continues the last (assistant) message instead of opening a new turn
        b.continue_final_message()
    return b.build(), map_params(body)


def select_tools(body: dict):
    """The tool list the template sees: ``tools`` (or the legacy ``functions`` list wrapped into tool entries), filtered by
    ``tool_choice`` / legacy ``function_call``: "none" hides the tools, a named function keeps only that one, "auto" / "required"
    keep all. The reference's request schema carries these fields (web/deliverance_specification.yaml,
    CreateChatCompletionRequest) without acting on them; they are honoured here so OpenAI clients behave as they expect."""
    tools = body.get("tools")
    if tools is not None and (not isinstance(tools, list) or not all(isinstance(t, dict) for t in tools)):
        raise ValueError("'tools' must be a list of tool objects")
    if not tools and body.get("functions"):
        tools = [{"type": "function", "function": f} for f in body["functions"] if isinstance(f, dict)]
    if not tools:
        return None
    choice = body.get("tool_choice")
    if choice is None:
        choice = body.get("function_call")
    if choice == "none":
        return None
    name = None
    if isinstance(choice, dict):
        name = (choice.get("function") or {}).get("name") or choice.get("name")
    if name:
        picked = [t for t in tools if (t.get("function") or t).get("name") == name]
        if not picked:
            raise ValueError(f"tool_choice names unknown function '{name}'")
        return picked
    return tools


def map_params(body: dict) -> GeneratorParameters:
    p = GeneratorParameters()
    if body.get("temperature") is not None:
        p.temperature = float(body["temperature"])
    for src, dst in (("top_p", "top_p"), ("top_k", "top_k"), ("uniform_top_p", "uniform_top_p"), ("xtc_threshold", "xtc_threshold"),
                     ("xtc_probability", "xtc_probability")):
        if body.get(src) is not None:
            setattr(p, dst, float(body[src]))
    if body.get("n") not in (None, 1):
        raise ValueError("only n = 1 is supported")
    if body.get("max_tokens") is not None:
        p.max_tokens = int(body["max_tokens"])
        if p.max_tokens <= 0:
            raise ValueError("max_tokens must be > 0")
    if body.get("ntokens") is not None:
        p.ntokens = int(body["ntokens"])
    if body.get("seed") is not None:
        p.seed = int(body["seed"])
    stop = body.get("stop")
    if isinstance(stop, str):
        p.stop_words = [stop]
    elif isinstance(stop, list):
        p.stop_words = [str(s) for s in stop]
    p.include_stop_str_in_output = bool(body.get("include_stop_str_in_output", False))
    p.logprobs = bool(body.get("logprobs", False))
    p.top_logprobs = int(body.get("top_logprobs") or 0)
    if not 0 <= p.top_logprobs <= 20:
        raise ValueError("top_logprobs must be between 0 and 20")
    p.guided_regex = body.get("guided_regex")
    if p.guided_regex is not None and not isinstance(p.guided_regex, str):
        raise ValueError("'guided_regex' must be a string")
    p.guided_json = body.get("guided_json")
    rf = body.get("response_format")
    if isinstance(rf, dict) and p.guided_json is None and p.guided_regex is None:
        if rf.get("type") == "json_schema":
            js = rf.get("json_schema") or {}
            p.guided_json = js.get("schema", js)
    p.guided_choice = body.get("guided_choice")
    p.cache_salt = str(body.get("cache_salt") or "")
    p.validate()
    return p


def _finish(r: Response) -> str:
    return r.finish_reason.wire if r.finish_reason not in (FinishReason.ERROR, FinishReason.CANCELLED) else "stop"


def _tool_calls_json(r: Response) -> list[dict]:
    return [{"id": c.id, "type": c.type, "function": {"name": c.name, "arguments": c.arguments if isinstance(c.arguments, str) else json.dumps(c.arguments)}}
            for c in r.tool_calls]


def _logprobs_json(r: Response) -> Optional[dict]:
    if not r.sampler_returns:
        return None
    return {"content": [{"token": lp.token, "logprob": lp.logprob, "bytes": list(lp.token.encode("utf-8")),
                         "top_logprobs": [{"token": t.token, "logprob": t.logprob, "bytes": list(t.token.encode("utf-8"))} for t in lp.top]}
                        for lp in r.sampler_returns]}


def _usage(r: Response) -> dict:
    return {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.generated_tokens, "total_tokens": r.prompt_tokens + r.generated_tokens}


def verify_jwt_hs256(token: str, secret: str) -> bool:
    try:
        h, p, s = token.split(".")
        sig = base64.urlsafe_b64decode(s + "=" * (-len(s) % 4))
        good = hmac.new(secret.encode(), f"{h}.{p}".encode(), hashlib.sha256).digest()
        if not hmac.compare_digest(sig, good):
            return False
        claims = json.loads(base64.urlsafe_b64decode(p + "=" * (-len(p) % 4)))
        return not ("exp" in claims and float(claims["exp"]) < time.time())
    except Exception:  # noqa: BLE001 - any malformed token is simply rejected
        return False


def create_app(registry: ModelRegistry, settings: Optional[ServerSettings] = None):
    from fastapi import FastAPI
    from fastapi.responses import HTMLResponse, JSONResponse, StreamingResponse

    settings = settings or ServerSettings()
    app = FastAPI(title="deliverance-b200")

    def error(status: int, message: str):
        return JSONResponse(status_code=status, content={"error": {"message": message, "type": "invalid_request_error" if status == 400 else "error"}})

    @app.middleware("http")
    async def auth(request: Request, call_next):
        path = request.url.path
        protected = path.startswith(("/chat", "/v1/chat", "/embeddings", "/v1/embeddings", "/models", "/v1/models"))
        if protected and (settings.basic_user or settings.jwt_secret):
            hdr = request.headers.get("authorization", "")
            ok = False
            if settings.basic_user and hdr.lower().startswith("basic "):
                try:
                    user, _, pw = base64.b64decode(hdr[6:]).decode().partition(":")
                    ok = hmac.compare_digest(user, settings.basic_user) and hmac.compare_digest(pw, settings.basic_password or "")
                except Exception:  # noqa: BLE001
                    ok = False
            if not ok and settings.jwt_secret and hdr.lower().startswith("bearer "):
                ok = verify_jwt_hs256(hdr[7:].strip(), settings.jwt_secret)
            if not ok:
                return JSONResponse(status_code=401, content={"error": {"message": "unauthorized"}}, headers={"WWW-Authenticate": "Basic"})
        return await call_next(request)

    async def _body(request: Request) -> dict:
        try:
            b = await request.json()
        except Exception:  # noqa: BLE001
            raise ValueError("request body is not valid JSON")
        if not isinstance(b, dict):
            raise ValueError("request body must be a JSON object")
        return b

    def _sse(obj) -> bytes:
        return ("data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n").encode("utf-8")

    async def _stream(request: Request, runner: EngineRunner, prompt, params, session: str, make_chunk, final_chunks, has_tools: bool):
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        pending: list = []  # pieces not yet handed to the event loop (touched by the engine thread only)
        sent = {"first": True, "at": time.monotonic()}

        def flush():
            if pending:
                text = "".join(pending)
                pending.clear()
                sent["at"] = time.monotonic()
                loop.call_soon_threadsafe(q.put_nowait, ("tok", text))

        def on_event(tok, piece, text_sp, ms):
            if piece:
                pending.append(piece)
            busy = len(runner.active) > settings.coalesce_above
            if sent["first"] or not busy or len(pending) >= settings.coalesce_tokens or (time.monotonic() - sent["at"]) * 1e3 >= settings.coalesce_ms:
                if pending:
                    sent["first"] = False
                flush()

        def on_done(sub):
            flush()
            loop.call_soon_threadsafe(q.put_nowait, ("done", sub))

        sub = runner.submit(prompt, params, on_event, on_done, session)
        text = getattr(prompt, "prompt", prompt)
        splitter = ReasoningTextSplitter(isinstance(text, str) and prompt_ends_inside_reasoning(text))

        async def gen():
            try:
                while True:
                    try:
                        kind, val = await asyncio.wait_for(q.get(), timeout=settings.heartbeat_s)
                    except asyncio.TimeoutError:
                        if await request.is_disconnected():
                            sub.cancel()
                            return
                        yield b": keep-alive\n\n"
                        continue
                    if kind == "tok":
                        c, r = splitter.accept(val)
                        if r:
                            yield _sse(make_chunk({settings.reasoning_key: r}, None))
                        if c and not has_tools:  # with tools the content is buffered so tool markup never leaks
                            yield _sse(make_chunk({"content": c}, None))
                    else:
                        if val.error is not None:
                            yield _sse({"error": {"message": str(val.error)}})
                        else:
                            c, r = splitter.flush()
                            if r:
                                yield _sse(make_chunk({settings.reasoning_key: r}, None))
                            if c and not has_tools:
                                yield _sse(make_chunk({"content": c}, None))
                            for ch in final_chunks(val.response):
                                yield _sse(ch)
                        yield _sse("[DONE]")
                        return
            finally:
                if not sub.done.is_set():
                    sub.cancel()

        return StreamingResponse(gen(), media_type="text/event-stream", headers={"X-Deliverance-Session": session, "Cache-Control": "no-cache"})

    def overloaded(runner):
        if settings.max_queue > 0 and len(runner.active) + runner.inbox.qsize() >= settings.max_queue:
            return JSONResponse(status_code=429, headers={"Retry-After": "1"},
                                content={"error": {"message": f"server is at capacity ({settings.max_queue} requests in flight)", "type": "rate_limit_error"}})
        return None

    async def chat(request: Request):
        try:
            body = await _body(request)
            runner = registry.find(body.get("model"))
            busy = overloaded(runner)
            if busy is not None:
                return busy
            prompt, params = map_chat_request(body, runner)
            if settings.pre_generate is not None:
                msg = settings.pre_generate(body, params)
                if msg:
                    return error(400, msg)
        except (ValueError, KeyError, TypeError) as e:
            return error(400, (str(e.args[0]) if e.args and str(e.args[0]) else "") or f"invalid request ({type(e).__name__})")
        except Exception as e:  # noqa: BLE001 - e.g. a chat template that does not compile or render
            return error(400, f"could not prepare the request: {type(e).__name__}: {e}")
        session = request.headers.get("x-deliverance-session") or str(uuid.uuid4())
        cid, created, model = "chatcmpl-" + uuid.uuid4().hex, int(time.time()), body.get("model") or runner.clm.name
        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
            first = {"sent": False}

            def make_chunk(delta: dict, finish: Optional[str]):
                if not first["sent"]:
                    delta = {"role": "assistant", **delta}
                    first["sent"] = True
                return {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model,
                        "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}

            def final_chunks(r: Response):
                out = []
                if prompt.has_tools:
                    if r.text:
                        out.append(make_chunk({"content": r.text}, None))
                    if r.tool_calls:
                        out.append(make_chunk({"tool_calls": [{"index": i, **tc} for i, tc in enumerate(_tool_calls_json(r))]}, None))
                last = make_chunk({}, _finish(r))
                last["usage"] = _usage(r)
                out.append(last)
                if include_usage:  # OpenAI stream_options.include_usage: one more chunk with no choices, usage only
                    out.append({"id": cid, "object": "chat.completion.chunk", "created": created, "model": model, "choices": [], "usage": _usage(r)})
                return out

            return await _stream(request, runner, prompt, params, session, make_chunk, final_chunks, prompt.has_tools)
        try:
            r = await asyncio.get_running_loop().run_in_executor(None, lambda: runner.generate(prompt, params, None, session, settings.request_timeout_s))
        except Exception as e:  # noqa: BLE001
            return error(400, str(e))
        msg: dict[str, Any] = {"role": "assistant", "content": r.text}
        if r.reasoning:
            msg[settings.reasoning_key] = r.reasoning
        if r.tool_calls:
            msg["tool_calls"] = _tool_calls_json(r)
        choice = {"index": 0, "message": msg, "finish_reason": _finish(r)}
        lp = _logprobs_json(r)
        if lp:
            choice["logprobs"] = lp
        return JSONResponse({"id": cid, "object": "chat.completion", "created": created, "model": model, "choices": [choice], "usage": _usage(r)},
                            headers={"X-Deliverance-Session": session})

    async def completions(request: Request):
        try:
            body = await _body(request)
            runner = registry.find(body.get("model"))
            busy = overloaded(runner)
            if busy is not None:
                return busy
            prompt = body.get("prompt")
            if isinstance(prompt, list) and prompt and isinstance(prompt[0], str):
                prompt = prompt[0]
            if not isinstance(prompt, str) or not prompt:
                raise ValueError("'prompt' must be a non-empty string")
            params = map_params(body)
        except (ValueError, KeyError, TypeError) as e:
            return error(400, str(e.args[0]) if e.args else str(e))
        session = request.headers.get("x-deliverance-session") or str(uuid.uuid4())
        cid, created, model = "cmpl-" + str(uuid.uuid4()), int(time.time()), body.get("model") or runner.clm.name
        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
            def make_chunk(delta: dict, finish):
                return {"id": cid, "object": "text_completion", "created": created, "model": model,
                        "choices": [{"index": 0, "text": delta.get("content") or delta.get(settings.reasoning_key) or "", "finish_reason": finish}]}

            def final_chunks(r: Response):
                out = [{"id": cid, "object": "text_completion", "created": created, "model": model,
                        "choices": [{"index": 0, "text": "", "finish_reason": _finish(r)}], "usage": _usage(r)}]
                if include_usage:
                    out.append({"id": cid, "object": "text_completion", "created": created, "model": model, "choices": [], "usage": _usage(r)})
                return out

            return await _stream(request, runner, prompt, params, session, make_chunk, final_chunks, False)
        try:
            r = await asyncio.get_running_loop().run_in_executor(None, lambda: runner.generate(prompt, params, None, session, settings.request_timeout_s))
        except Exception as e:  # noqa: BLE001
            return error(400, str(e))
        text = r.text if not r.reasoning else f"<think>{r.reasoning}</think>{r.text}"
        return JSONResponse({"id": cid, "object": "text_completion", "created": created, "model": model,
                             "choices": [{"index": 0, "text": text, "finish_reason": _finish(r), "logprobs": _logprobs_json(r)}], "usage": _usage(r)})

    async def embeddings(request: Request):
        try:
            body = await _body(request)
            if not registry.embedding:
                raise KeyError("no embedding model is loaded")
            name = body.get("model")
            em = registry.embedding.get(name) or next(iter(registry.embedding.values()))
            inp = body.get("input")
            texts = [inp] if isinstance(inp, str) else list(inp or [])
            if not texts or not all(isinstance(t, str) for t in texts):
                raise ValueError("'input' must be a string or a list of strings")
        except (ValueError, KeyError, TypeError) as e:
            return error(400, str(e.args[0]) if e.args else str(e))
        from ..embedding import PoolingType

        vecs = await asyncio.get_running_loop().run_in_executor(None, lambda: em.embed_many(texts, PoolingType.AVG).tolist())
        return JSONResponse({"object": "list", "model": name or "embedding", "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                             "usage": {"prompt_tokens": 0, "total_tokens": 0}})

    async def models():
        data = [{"id": n, "object": "model", "owned_by": "deliverance", "type": "generation"} for n in registry.generation]
        data += [{"id": n, "object": "model", "owned_by": "deliverance", "type": "embedding"} for n in registry.embedding]
        return JSONResponse({"object": "list", "data": data})

    async def tp_status():
        st = dict(registry.tp_status())
        sf = os.environ.get("DLV_CLUSTER_STATUS_FILE")  # written by the rank supervisor (parallel/cluster.py --status-file)
        if sf and os.path.exists(sf):
            try:
                with open(sf) as f:
                    st["cluster"] = json.load(f)
            except (OSError, ValueError):
                pass
        st["runners"] = {n: dict(r.stats, engine=dict(r.clm.engine.metrics), prefix_cache=dict(r.clm.engine.kv.prefix.metrics)) for n, r in registry.generation.items()}
        return JSONResponse(st)

    async def tp_endpoints():
        """The ranks of the tensor-parallel group. Ranks are processes of one node that talk over NCCL / peer memory, not HTTP
        services, so an entry names the rank and its device instead of a URL (reference: /tp/endpoints lists rank-server URLs,
        web/.../TensorParallelDiagnosticsController.java:22-40)."""
        st = registry.tp_status()
        n = int(st.get("size", 1))
        return JSONResponse({"size": n, "endpoints": [{"rank": r, "device": f"cuda:{r}" if st.get("enabled") else "local",
                                                       "role": "coordinator+rank" if r == 0 else "rank"} for r in range(n)]})

    async def tp_gossip():
        """Membership view: with a gossip-managed deployment the agent's live nodes, topology, elected leader, assignment and rank
        endpoints (reference: /tp/gossip, web/.../TensorParallelDiagnosticsController.java:22-40); otherwise the group is fixed at
        launch (RANK / WORLD_SIZE) and the view is the static member list plus the supervisor's restart history."""
        if registry.membership is not None:
            return JSONResponse({"membership": "gossip", **registry.membership.diagnostics()})
        st = dict(registry.tp_status())
        out = {"membership": "static", "leader": 0, "members": list(range(int(st.get("size", 1))))}
        sf = os.environ.get("DLV_CLUSTER_STATUS_FILE")
        if sf and os.path.exists(sf):
            try:
                with open(sf) as f:
                    out["supervisor"] = json.load(f)
            except (OSError, ValueError):
                pass
        return JSONResponse(out)

    async def tp_assign(request: Request):
        """Manual rank placement ``POST /tp/assign?nodeId=..&rank=..`` for a gossip deployment in manual mode (reference:
        GossipParallelMembership.assignRankManually, core/.../tensorparallel/GossipParallelMembership.java:460-475)."""
        q = request.query_params
        m = registry.membership
        if m is None:
            return error(409, f"rank assignment is static: ranks are fixed at launch (requested nodeId={q.get('nodeId')} rank={q.get('rank')}); "
                              "restart the group with a different --nproc to change it, or run the hosts under deliverance_b200.parallel.gossip")
        try:
            return JSONResponse(m.assign_rank(str(q.get("nodeId")), int(q.get("rank", "-1"))))
        except RuntimeError as e:
            return error(409, str(e))
        except (ValueError, TypeError) as e:
            return error(400, str(e))

    async def health():
        """Liveness / readiness probe (never behind authentication): 200 while every engine runner thread is alive."""
        dead = [n for n, r in registry.generation.items() if getattr(r, "thread", None) is not None and not r.thread.is_alive()]
        body = {"status": "ok" if not dead else "degraded", "models": len(registry.generation) + len(registry.embedding), "dead_runners": dead}
        return JSONResponse(body, status_code=200 if not dead else 503)

    async def ui():
        return HTMLResponse(_UI)

    from .spec import route_docs  # request / response schemas for GET /openapi.json

    for path in ("/chat/completions", "/v1/chat/completions"):
        app.add_api_route(path, chat, methods=["POST"], **route_docs("chat"))
    for path in ("/v1/completions", "/completions"):
        app.add_api_route(path, completions, methods=["POST"], **route_docs("completions"))
    for path in ("/embeddings", "/v1/embeddings"):
        app.add_api_route(path, embeddings, methods=["POST"], **route_docs("embeddings"))
    for path in ("/models", "/v1/models"):
        app.add_api_route(path, models, methods=["GET"], **route_docs("models"))
    async def metrics():
        """Prometheus text exposition of the engine and runner counters (the reference reports through Dropwizard metrics:
        core/.../model/InferenceProfiler.java:24-161; ttft / tokens-per-second timers in GenerationEngine.java:128-175)."""
        from fastapi.responses import PlainTextResponse

        lines = []

        def emit(name, kind, help_text, samples):
            lines.append(f"# HELP {name} {help_text}")
            lines.append(f"# TYPE {name} {kind}")
            for labels, v in samples:
                lab = ",".join(f'{k}="{val}"' for k, val in labels.items())
                lines.append(f"{name}{{{lab}}} {v}")

        eng_keys = (("steps", "engine steps"), ("prefill_steps", "prefill steps"), ("decode_steps", "decode steps"),
                    ("prefill_tokens", "prompt tokens computed"), ("decode_tokens", "tokens generated by decode steps"),
                    ("graph_replays", "CUDA graph replays"), ("kernel_launches", "kernels of the extension launched"),
                    ("preemptions", "sequences preempted under KV memory pressure"))
        for key, text in eng_keys:
            emit(f"deliverance_engine_{key}_total", "counter", text,
                 [({"model": n}, r.clm.engine.metrics.get(key, 0)) for n, r in registry.generation.items()])
        for key in ("submitted", "finished", "errors", "cancelled"):
            emit(f"deliverance_requests_{key}_total", "counter", f"requests {key}", [({"model": n}, r.stats.get(key, 0)) for n, r in registry.generation.items()])
        emit("deliverance_requests_running", "gauge", "sequences in the running batch",
             [({"model": n}, len(r.clm.engine.running)) for n, r in registry.generation.items()])
        emit("deliverance_requests_waiting", "gauge", "requests waiting for admission",
             [({"model": n}, len(r.clm.engine.waiting)) for n, r in registry.generation.items()])
        emit("deliverance_kv_pages_free", "gauge", "free KV cache pages",
             [({"model": n}, r.clm.engine.kv.allocator.available()) for n, r in registry.generation.items()])
        for key in ("lookup", "hits", "misses", "evict", "stored", "hit_tokens"):
            emit(f"deliverance_prefix_cache_{key}_total", "counter", f"prefix cache {key}",
                 [({"model": n}, r.clm.engine.kv.prefix.metrics.get(key, 0)) for n, r in registry.generation.items()])
        return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

    app.add_api_route("/metrics", metrics, methods=["GET"])
    app.add_api_route("/tp/status", tp_status, methods=["GET"])
    app.add_api_route("/tp/endpoints", tp_endpoints, methods=["GET"])
    app.add_api_route("/tp/gossip", tp_gossip, methods=["GET"])
    app.add_api_route("/tp/assign", tp_assign, methods=["POST"])
    app.add_api_route("/ui", ui, methods=["GET"])
    for path in ("/health", "/healthz"):
        app.add_api_route(path, health, methods=["GET"])
    return app


_UI = """<!doctype html><meta charset=utf-8><title>deliverance</title>
<style>body{font-family:sans-serif;max-width:48em;margin:2em auto}#log{white-space:pre-wrap;border:1px solid #ccc;padding:1em;min-height:12em}</style>
<h3>chat</h3><div id=log></div><form id=f><input id=q size=60 autofocus><button>send</button></form>
<script>
const log=document.getElementById('log'),msgs=[];
document.getElementById('f').onsubmit=async e=>{e.preventDefault();const q=document.getElementById('q');msgs.push({role:'user',content:q.value});
log.textContent+='\\n> '+q.value+'\\n';q.value='';
const r=await fetch('/chat/completions',{method:'POST',headers:{'Content-Type':'application/json'},body:JSON.stringify({messages:msgs,stream:true,max_tokens:256})});
const rd=r.body.getReader(),dec=new TextDecoder();let buf='',ans='';
for(;;){const {done,value}=await rd.read();if(done)break;buf+=dec.decode(value);let i;
while((i=buf.indexOf('\\n\\n'))>=0){const line=buf.slice(0,i);buf=buf.slice(i+2);if(!line.startsWith('data: '))continue;const d=line.slice(6);if(d==='[DONE]')continue;
const c=JSON.parse(d).choices?.[0]?.delta?.content;if(c){ans+=c;log.textContent+=c;}}}
msgs.push({role:'assistant',content:ans});};
</script>"""
