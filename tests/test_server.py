"""HTTP surface against a tiny CPU model: chat / completions (blocking and SSE), embeddings, models, auth, errors."""
import base64
import json

import pytest

from deliverance_b200.api import AutoModelForCausalLM
from deliverance_b200.ckpt.tiny import write_tiny_model
from deliverance_b200.embedding import AutoModelForEmbeddings
from deliverance_b200.server.app import ModelRegistry, ServerSettings, create_app, verify_jwt_hs256
from deliverance_b200.server.runner import EngineRunner

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402


@pytest.fixture(scope="module")
def registry(tmp_path_factory):
    root = tmp_path_factory.mktemp("srv")
    d = str(root / "tiny-llama")
    write_tiny_model(d, "llama", seed=3, std=0.05)
    clm = AutoModelForCausalLM.from_pretrained(d, device="cpu")
    reg = ModelRegistry()
    reg.generation[clm.name] = EngineRunner(clm)
    b = str(root / "tiny-bert")
    write_tiny_model(b, "bert", seed=4, std=0.05)
    reg.embedding["tiny-bert"] = AutoModelForEmbeddings.from_pretrained(b, "cpu")
    yield reg
    for r in reg.generation.values():
        r.close()


def _sse(resp):
    out = []
    for line in resp.text.split("\n"):
        if line.startswith("data: "):
            out.append(line[6:])
    return out


def test_chat_blocking_and_models(registry):
    c = TestClient(create_app(registry))
    r = c.post("/chat/completions", json={"messages": [{"role": "system", "content": "s"}, {"role": "user", "content": [{"type": "text", "text": "hi"}]}],
                                          "max_tokens": 5, "logprobs": True, "top_logprobs": 2, "seed": 1})
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["object"] == "chat.completion" and j["choices"][0]["finish_reason"] == "length" and j["usage"]["completion_tokens"] == 5
    assert len(j["choices"][0]["logprobs"]["content"]) == 5 and "X-Deliverance-Session" in r.headers
    m = c.get("/models").json()["data"]
    assert {x["id"] for x in m} == {"tiny-llama", "tiny-bert"}
    assert c.get("/tp/status").json()["enabled"] is False
    assert c.get("/health").json() == {"status": "ok", "models": 2, "dead_runners": []} and c.get("/healthz").status_code == 200
    assert c.get("/tp/endpoints").json() == {"size": 1, "endpoints": [{"rank": 0, "device": "local", "role": "coordinator+rank"}]}
    assert c.get("/tp/gossip").json()["membership"] == "static" and c.post("/tp/assign?nodeId=n1&rank=1").status_code == 409


def test_chat_streaming_sse(registry):
    c = TestClient(create_app(registry))
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "stream": True},
               headers={"X-Deliverance-Session": "abc"})
    assert r.status_code == 200 and r.headers["x-deliverance-session"] == "abc"
    ev = _sse(r)
    assert ev[-1] == "[DONE]"
    chunks = [json.loads(e) for e in ev[:-1]]
    assert all(ch["object"] == "chat.completion.chunk" for ch in chunks)
    assert chunks[-1]["choices"][0]["finish_reason"] == "length" and chunks[-1]["usage"]["completion_tokens"] == 6
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"


def test_completions_and_guided(registry):
    c = TestClient(create_app(registry))
    r = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 4, "temperature": 0.7, "top_p": 0.9, "seed": 5})
    assert r.status_code == 200 and r.json()["object"] == "text_completion" and r.json()["id"].startswith("cmpl-")
    r = c.post("/completions", json={"prompt": "abc", "max_tokens": 12, "guided_regex": "[0-9]{2}x"})
    assert r.status_code == 200 and __import__("re").fullmatch("[0-9]{2}x", r.json()["choices"][0]["text"])
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "max_tokens": 30,
                                          "guided_json": {"type": "object", "properties": {"ok": {"type": "boolean"}}}})
    assert json.loads(r.json()["choices"][0]["message"]["content"]) in ({"ok": True}, {"ok": False})
    r = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 3, "stream": True})
    assert _sse(r)[-1] == "[DONE]"


def test_errors_and_embeddings(registry):
    c = TestClient(create_app(registry))
    assert c.post("/chat/completions", json={"model": "nope", "messages": [{"role": "user", "content": "x"}]}).status_code == 400
    assert c.post("/chat/completions", json={"messages": []}).status_code == 400
    assert c.post("/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "guided_regex": "a", "guided_json": {}}).status_code == 400
    assert c.post("/v1/completions", json={"prompt": ""}).status_code == 400
    assert c.post("/chat/completions", content=b"{bad").status_code == 400
    r = c.post("/embeddings", json={"input": "hello world"})
    assert r.status_code == 200 and len(r.json()["data"][0]["embedding"]) == 64


def test_auth_basic_and_jwt(registry):
    import hashlib
    import hmac
    import time

    c = TestClient(create_app(registry, ServerSettings(basic_user="u", basic_password="p", jwt_secret="s3")))
    assert c.get("/models").status_code == 401
    tok = base64.b64encode(b"u:p").decode()
    assert c.get("/models", headers={"Authorization": "Basic " + tok}).status_code == 200
    assert c.get("/models", headers={"Authorization": "Basic " + base64.b64encode(b"u:x").decode()}).status_code == 401

    def jwt(claims, secret):
        enc = lambda b: base64.urlsafe_b64encode(b).rstrip(b"=").decode()  # noqa: E731
        h, p = enc(json.dumps({"alg": "HS256", "typ": "JWT"}).encode()), enc(json.dumps(claims).encode())
        return f"{h}.{p}." + enc(hmac.new(secret.encode(), f"{h}.{p}".encode(), hashlib.sha256).digest())

    assert c.get("/models", headers={"Authorization": "Bearer " + jwt({"sub": "a", "exp": time.time() + 60}, "s3")}).status_code == 200
    assert not verify_jwt_hs256(jwt({"exp": time.time() - 5}, "s3"), "s3") and not verify_jwt_hs256(jwt({}, "other"), "s3")
    assert c.get("/tp/status").status_code == 200  # diagnostics stay open


def test_pre_generate_hook_and_reasoning_field(registry):
    c = TestClient(create_app(registry, ServerSettings(reasoning_field="vllm", pre_generate=lambda body, p: "blocked" if body.get("user") == "bad" else None)))
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "user": "bad"})
    assert r.status_code == 400 and r.json()["error"]["message"] == "blocked"
    assert ServerSettings(reasoning_field="vllm").reasoning_key == "reasoning" and ServerSettings().reasoning_key == "reasoning_content"


def test_openai_compat_fields(registry):
    """Request fields of the reference's schema that OpenAI clients send: stream_options, tool_choice, legacy functions /
    function_call, the "function" and "developer" roles, response_format json_schema."""
    from deliverance_b200.server.app import select_tools

    tools = [{"type": "function", "function": {"name": "a", "parameters": {}}}, {"type": "function", "function": {"name": "b", "parameters": {}}}]
    assert select_tools({"tools": tools}) == tools and select_tools({"tools": tools, "tool_choice": "auto"}) == tools
    assert select_tools({"tools": tools, "tool_choice": "none"}) is None and select_tools({}) is None
    assert select_tools({"tools": tools, "tool_choice": {"type": "function", "function": {"name": "b"}}}) == tools[1:]
    legacy = select_tools({"functions": [{"name": "f", "parameters": {}}], "function_call": {"name": "f"}})
    assert legacy == [{"type": "function", "function": {"name": "f", "parameters": {}}}]
    with pytest.raises(ValueError):
        select_tools({"tools": tools, "tool_choice": {"type": "function", "function": {"name": "zz"}}})

    c = TestClient(create_app(registry))
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "hello"}], "max_tokens": 4, "stream": True,
                                          "stream_options": {"include_usage": True}})
    chunks = [json.loads(e) for e in _sse(r)[:-1]]
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 4
    assert chunks[-2]["choices"][0]["finish_reason"] == "length"
    r = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 3, "stream": True, "stream_options": {"include_usage": True}})
    chunks = [json.loads(e) for e in _sse(r)[:-1]]
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 3
    r = c.post("/chat/completions", json={"messages": [{"role": "developer", "content": "be brief"}, {"role": "user", "content": "q"},
                                                       {"role": "assistant", "content": "calling"}, {"role": "function", "name": "f", "content": "42"}],
                                          "max_tokens": 3, "tool_choice": "none", "tools": tools})
    assert r.status_code == 200, r.text
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "max_tokens": 30,
                                          "response_format": {"type": "json_schema", "json_schema": {"name": "x", "schema": {
                                              "type": "object", "properties": {"ok": {"type": "boolean"}}}}}})
    assert json.loads(r.json()["choices"][0]["message"]["content"]) in ({"ok": True}, {"ok": False})
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "tools": tools, "tool_choice": {"function": {"name": "zz"}}})
    assert r.status_code == 400
    from deliverance_b200.server.app import map_chat_request

    runner = next(iter(registry.generation.values()))
    body = {"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "The answer"}], "continue_final_message": True}
    assert map_chat_request(body, runner)[0].prompt.endswith("The answer")
    assert not map_chat_request({"messages": body["messages"][:1], "add_generation_prompt": False}, runner)[0].prompt.endswith("assistant\n")


def test_malformed_requests_are_400(registry):
    """Bad field types and values are the client's fault: a 400 with a message, never a 500."""
    c = TestClient(create_app(registry), raise_server_exceptions=False)
    u = [{"role": "user", "content": "hi"}]
    for body in ({"messages": u, "max_tokens": 0}, {"messages": u, "max_tokens": "many"}, {"messages": ["hi"]}, {"messages": u, "n": 3},
                 {"messages": u, "tools": "x"}, {"messages": u, "tools": [1]}, {"messages": u, "top_logprobs": 99, "logprobs": True},
                 {"messages": u, "guided_regex": "([a-z"}, {"messages": u, "guided_regex": 5}, {"messages": u, "chat_template": "{% for %}"},
                 {"messages": u, "chat_template_kwargs": "x"}, {"messages": u, "temperature": "hot"}, {"messages": u, "seed": "abc"}):
        r = c.post("/chat/completions", json=dict(body, **({} if "max_tokens" in body else {"max_tokens": 2})))
        assert r.status_code == 400 and r.json()["error"]["message"], (body, r.status_code, r.text)
    assert c.post("/chat/completions", content="{not json", headers={"Content-Type": "application/json"}).status_code == 400
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": None}, {"role": "user", "content": 5}], "max_tokens": 2})
    assert r.status_code == 200


def test_streaming_tool_calls_never_leak_markup(tmp_path):
    """Behaviours of the reference's ChatCompletionStreamingToolCallTest on the real stack: the model is forced (guided regex)
    to emit a reasoning block and two raw <tool_call> regions; with tools in the request no markup reaches the stream, the
    calls arrive as ONE structured tool_calls delta after generation, reasoning goes to its own field, finish_reason is
    tool_calls; the blocking reply carries the same calls."""
    from deliverance_b200.guided.json_schema import escape_literal

    d = str(tmp_path / "qwen-tiny")
    write_tiny_model(d, "llama", seed=3, std=0.05, max_position_embeddings=2048)
    clm = AutoModelForCausalLM.from_pretrained(d, device="cpu")
    reg = ModelRegistry()
    reg.generation[clm.name] = EngineRunner(clm)
    try:
        c = TestClient(create_app(reg))
        call = '<tool_call>{"name":"grep","arguments":{"path":"/tmp/ed","pattern":"cat","limit":10}}</tool_call>'
        body = {"messages": [{"role": "user", "content": "grep the file"}], "max_tokens": 400, "guided_regex": escape_literal("<think>checking</think>\n" + call + call),
                "tools": [{"type": "function", "function": {"name": "grep", "parameters": {"type": "object"}}}]}
        r = c.post("/chat/completions", json=dict(body, stream=True))
        assert "<tool_call>" not in r.text and "</tool_call>" not in r.text
        chunks = [json.loads(e) for e in _sse(r)[:-1]]
        deltas = [ch["choices"][0]["delta"] for ch in chunks if ch["choices"]]
        tool_deltas = [x for x in deltas if x.get("tool_calls")]
        assert len(tool_deltas) == 1 and [t["function"]["name"] for t in tool_deltas[0]["tool_calls"]] == ["grep", "grep"]
        assert json.loads(tool_deltas[0]["tool_calls"][0]["function"]["arguments"]) == {"path": "/tmp/ed", "pattern": "cat", "limit": 10}
        assert [t["id"] for t in tool_deltas[0]["tool_calls"]] == ["101", "102"] and [t["index"] for t in tool_deltas[0]["tool_calls"]] == [0, 1]
        assert "".join(x.get("reasoning_content") or "" for x in deltas) == "checking" and "".join(x.get("content") or "" for x in deltas) == ""
        assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls"
        msg = c.post("/chat/completions", json=body).json()["choices"][0]
        assert msg["finish_reason"] == "tool_calls" and len(msg["message"]["tool_calls"]) == 2 and msg["message"]["reasoning_content"] == "checking"
        assert msg["message"]["content"] == ""
    finally:
        for r_ in reg.generation.values():
            r_.close()


def test_backpressure_429(registry, monkeypatch):
    runner = next(iter(registry.generation.values()))
    c = TestClient(create_app(registry, ServerSettings(max_queue=2)))
    assert c.post("/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "max_tokens": 2}).status_code == 200
    monkeypatch.setattr(runner.inbox, "qsize", lambda: 2)  # two requests waiting to be picked up
    r = c.post("/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "max_tokens": 2})
    assert r.status_code == 429 and r.headers["retry-after"] == "1" and r.json()["error"]["type"] == "rate_limit_error"
    assert c.post("/v1/completions", json={"prompt": "x", "max_tokens": 2}).status_code == 429
    monkeypatch.undo()
    assert c.post("/v1/completions", json={"prompt": "x", "max_tokens": 2}).status_code == 200


def test_openapi_document_describes_the_api(registry):
    """GET /openapi.json carries request and response schemas of the endpoints (clients can be generated from it), and the
    request schema accepts what the server accepts."""
    c = TestClient(create_app(registry))
    doc = c.get("/openapi.json").json()
    chat = doc["paths"]["/chat/completions"]["post"]
    req = chat["requestBody"]["content"]["application/json"]["schema"]
    assert {"messages", "tools", "guided_json", "guided_regex", "uniform_top_p", "xtc_threshold", "chat_template_kwargs", "stream_options"} <= set(req["properties"])
    assert "text/event-stream" in chat["responses"]["200"]["content"] and "429" in chat["responses"] and req["required"] == ["messages"]
    assert doc["paths"]["/v1/completions"]["post"]["requestBody"]["content"]["application/json"]["schema"]["required"] == ["prompt"]
    assert "embedding" in json.dumps(doc["paths"]["/embeddings"]["post"]["responses"]["200"])
    jsonschema = pytest.importorskip("jsonschema")
    body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}], "max_tokens": 4, "stop": ["x"], "top_logprobs": 2,
            "tools": [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}], "tool_choice": "auto"}
    jsonschema.validate(body, req)
    r = c.post("/chat/completions", json={k: v for k, v in body.items() if k not in ("tools", "tool_choice")})  # (the tiny model's context is 256 bytes)
    assert r.status_code == 200
    jsonschema.validate(r.json(), chat["responses"]["200"]["content"]["application/json"]["schema"])
    with pytest.raises(jsonschema.ValidationError):
        jsonschema.validate({"messages": [], "max_tokens": 0}, req)


def test_interrogation_game_setup_and_loop(registry):
    """The game's guided_regex name step runs through the real server; the long JSON steps and the suspect are scripted."""
    import re

    from deliverance_b200.agents import interrogation_game as g

    c = TestClient(create_app(registry))
    replies = iter(["I was at home.", "Fine, I took it. " + g.MARKER])
    seen = []

    def chat(messages, **fields):
        seen.append(fields)
        if "guided_regex" in fields:
            r = c.post("/chat/completions", json={"messages": messages, **fields})
            assert r.status_code == 200, r.text
            return r.json()["choices"][0]["message"]["content"]
        schema = fields.get("guided_json")
        if schema and "places" in schema["properties"]:
            return json.dumps({"places": [f"_place {i}" for i in range(10)]})
        if schema and "items" in schema["properties"]:
            return json.dumps({"items": [f"item {i}" for i in range(10)]})
        if schema:
            return json.dumps({"case_title": "The Missing Ledger", "setting": "a bakery", "clues": ["a", "b", "c"],
                               "hidden": {"what_happened": "w", "motive": "m", "method": "h", "mistake": "k"}})
        return next(replies)

    lines = iter(["/case", "", "/reveal", "where were you?", "you left flour on the ledger"])
    out = []
    game = g.Game(chat, lambda: next(lines, None), out.append, seed=5)
    assert game.play() == "confessed"
    name = game.case["suspect"]
    assert re.fullmatch(g.SUSPECT_NAME_REGEX, name), name
    assert seen[0]["uniform_top_p"] == 1.0 and seen[1]["temperature"] == 1.2
    text = "\n".join(out)
    assert "selected: place" in text and "HIDDEN TRUTH\nwhat happened: w" in text and text.count("CASE: The Missing Ledger") == 2
    assert g.MARKER not in text and "DEAD TO RIGHTS" in text
    msgs = [{"role": "x"}] * 40
    g.trim_conversation(msgs)
    assert len(msgs) == g.CASE_CONTEXT_MESSAGES + g.RECENT_MESSAGES
    quit_game = g.Game(chat, lambda: "/quit", out.append)
    quit_game.case = game.case
    assert quit_game.play() == "closed"


def test_server_command_line_end_to_end(tmp_path):
    """``python -m deliverance_b200.server --model DIR`` as a user starts it (CPU, tiny checkpoint): the process comes up, lists the
    model, answers a blocking and a streaming chat completion over real HTTP and exits on SIGTERM."""
    import json
    import signal
    import socket
    import subprocess
    import sys
    import time
    import urllib.request

    from deliverance_b200.ckpt.tiny import write_tiny_model

    d = str(tmp_path / "tinyllama")
    write_tiny_model(d, "llama", seed=5, std=0.05)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    proc = subprocess.Popen([sys.executable, "-m", "deliverance_b200.server", "--model", d, "--device", "cpu", "--port", str(port), "--max-seqs", "4"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"

    def call(path, body=None, timeout=60):
        req = urllib.request.Request(base + path, data=None if body is None else json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        return urllib.request.urlopen(req, timeout=timeout)

    try:
        deadline = time.time() + 120
        models = None
        while time.time() < deadline and proc.poll() is None:
            try:
                models = json.load(call("/models", timeout=2))
                break
            except OSError:
                time.sleep(0.3)
        assert models is not None, "the server did not come up"
        names = [m["id"] for m in models["data"]]
        assert names == ["tinyllama"]
        body = {"model": "tinyllama", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0}
        out = json.load(call("/chat/completions", body))
        assert out["choices"][0]["finish_reason"] in ("length", "stop") and out["usage"]["completion_tokens"] <= 6
        text = out["choices"][0]["message"]["content"]
        lines = [ln.decode() for ln in call("/v1/chat/completions", dict(body, stream=True)) if ln.startswith(b"data: ")]
        assert lines[-1].strip() == "data: [DONE]"
        streamed = "".join(json.loads(ln[6:])["choices"][0]["delta"].get("content") or "" for ln in lines[:-1] if '"delta"' in ln)
        assert streamed == text  # temperature 0: the stream carries the same text as the blocking call
    finally:
        if proc.poll() is None:
            proc.send_signal(signal.SIGTERM)
            try:
                proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                proc.kill()
                proc.wait(timeout=10)
    assert proc.returncode is not None
