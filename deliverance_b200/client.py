"""Minimal Python client for the HTTP API (the reference ships OpenAPI-generated Java clients, client/ and client-spring/).

Blocking calls return the parsed JSON; ``stream_chat`` yields (kind, text) pairs with kind in ``content`` / ``reasoning`` /
``tool_calls`` / ``finish`` as the server-sent events arrive. Only the standard library is used.
"""
from __future__ import annotations

import base64
import json
import urllib.request
from typing import Iterator, Optional


class DeliveranceClient:
    def __init__(self, base_url: str = "http://127.0.0.1:8080", basic: Optional[tuple] = None, bearer: Optional[str] = None, timeout: float = 600.0):
        self.base = base_url.rstrip("/")
        self.timeout = timeout
        self.headers = {"Content-Type": "application/json"}
        if basic:
            self.headers["Authorization"] = "Basic " + base64.b64encode(f"{basic[0]}:{basic[1]}".encode()).decode()
        elif bearer:
            self.headers["Authorization"] = "Bearer " + bearer

    def _post(self, path: str, body: dict):
        req = urllib.request.Request(self.base + path, data=json.dumps(body).encode(), headers=self.headers, method="POST")
        return urllib.request.urlopen(req, timeout=self.timeout)

    def chat(self, messages: list[dict], **params) -> dict:
        with self._post("/chat/completions", {"messages": messages, **params}) as r:
            return json.loads(r.read())

    def complete(self, prompt: str, **params) -> dict:
        with self._post("/v1/completions", {"prompt": prompt, **params}) as r:
            return json.loads(r.read())

    def embed(self, text, model: Optional[str] = None) -> list:
        with self._post("/embeddings", {"input": text, **({"model": model} if model else {})}) as r:
            return [d["embedding"] for d in json.loads(r.read())["data"]]

    def models(self) -> list[str]:
        req = urllib.request.Request(self.base + "/models", headers=self.headers)
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            return [m["id"] for m in json.loads(r.read())["data"]]

    def stream_chat(self, messages: list[dict], **params) -> Iterator[tuple]:
        with self._post("/chat/completions", {"messages": messages, "stream": True, **params}) as r:
            for raw in r:
                line = raw.decode("utf-8").rstrip("\n")
                if not line.startswith("data: "):
                    continue
                data = line[6:]
                if data == "[DONE]":
                    return
                ch = json.loads(data)
                if "error" in ch:
                    raise RuntimeError(ch["error"].get("message", "server error"))
                choice = ch["choices"][0]
                d = choice.get("delta", {})
                if d.get("content"):
                    yield "content", d["content"]
                for key in ("reasoning_content", "reasoning"):
                    if d.get(key):
                        yield "reasoning", d[key]
                if d.get("tool_calls"):
                    yield "tool_calls", d["tool_calls"]
                if choice.get("finish_reason"):
                    yield "finish", choice["finish_reason"]


def main() -> int:
    import argparse

    ap = argparse.ArgumentParser(description="terminal chat against a deliverance_b200 server")
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--max-tokens", type=int, default=512)
    a = ap.parse_args()
    c = DeliveranceClient(a.url)
    msgs: list[dict] = []
    while True:
        try:
            q = input("> ")
        except EOFError:
            return 0
        msgs.append({"role": "user", "content": q})
        ans = ""
        for kind, text in c.stream_chat(msgs, max_tokens=a.max_tokens):
            if kind == "content":
                ans += text
                print(text, end="", flush=True)
        print()
        msgs.append({"role": "assistant", "content": ans})


if __name__ == "__main__":
    raise SystemExit(main())
