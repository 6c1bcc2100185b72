"""A small terminal coding agent over ``/chat/completions`` tool calls.

Counterpart of the reference's agents: ``nanocode-deliverance`` (tools read / write / edit / glob / grep / web_fetch /
java_sandbox, streaming tool calls: nanocode-deliverance/.../NanocodeDeliverance.java) and ``deliverance-antares-cli`` (agent
loop with command approval: deliverance-antares-cli/.../AntaresAgent.java, AntaresToolExecutor.java). One loop covers both:
the model is offered file tools and a shell tool; every tool that changes something (write, edit, run) asks the approval
callback first; file access is confined to the workspace directory.

    python -m deliverance_b200.agents.nanocode --url http://127.0.0.1:8080 --workspace . [--auto-approve]
"""
from __future__ import annotations

import fnmatch
import json
import os
import re
import subprocess
from typing import Callable, Optional

TOOLS = [
    {"type": "function", "function": {"name": "read", "description": "Read a text file (optionally a line range).",
                                      "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "start": {"type": "integer"}, "end": {"type": "integer"}},
                                                     "required": ["path"]}}},
    {"type": "function", "function": {"name": "write", "description": "Create or overwrite a text file.",
                                      "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "content": {"type": "string"}}, "required": ["path", "content"]}}},
    {"type": "function", "function": {"name": "edit", "description": "Replace one exact occurrence of old with new in a file.",
                                      "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "old": {"type": "string"}, "new": {"type": "string"}},
                                                     "required": ["path", "old", "new"]}}},
    {"type": "function", "function": {"name": "glob", "description": "List files matching a glob pattern.",
                                      "parameters": {"type": "object", "properties": {"pattern": {"type": "string"}}, "required": ["pattern"]}}},
    {"type": "function", "function": {"name": "grep", "description": "Search files for a regular expression.",
                                      "parameters": {"type": "object", "properties": {"pattern": {"type": "string"}, "glob": {"type": "string"}}, "required": ["pattern"]}}},
    {"type": "function", "function": {"name": "run", "description": "Run a shell command in the workspace (asks for approval).",
                                      "parameters": {"type": "object", "properties": {"command": {"type": "string"}}, "required": ["command"]}}},
]
SYSTEM = ("You are a coding assistant working in a project directory. Use the tools to inspect and change files. "
          "Keep answers short; when the task is done, reply without calling a tool.")


class ToolExecutor:
    def __init__(self, workspace: str, approve: Callable[[str, dict], bool], max_output: int = 8000, run_timeout: float = 60.0):
        self.root = os.path.realpath(workspace)
        self.approve = approve
        self.max_output = max_output
        self.run_timeout = run_timeout

    def _path(self, p: str) -> str:
        full = os.path.realpath(os.path.join(self.root, p))
        if full != self.root and not full.startswith(self.root + os.sep):
            raise PermissionError(f"{p} is outside the workspace")
        return full

    def _files(self, pattern: str = "**/*"):
        for base, dirs, files in os.walk(self.root):
            dirs[:] = [d for d in dirs if not d.startswith(".")]
            for f in files:
                rel = os.path.relpath(os.path.join(base, f), self.root)
                if fnmatch.fnmatch(rel, pattern) or fnmatch.fnmatch(f, pattern):
                    yield rel

    def execute(self, name: str, args: dict) -> str:
        try:
            out = getattr(self, "tool_" + name)(**args)
        except AttributeError:
            out = f"error: unknown tool {name}"
        except Exception as e:  # noqa: BLE001 - the model sees the error text and can react
            out = f"error: {type(e).__name__}: {e}"
        return out if len(out) <= self.max_output else out[: self.max_output] + "\n... (truncated)"

    def tool_read(self, path: str, start: Optional[int] = None, end: Optional[int] = None) -> str:
        with open(self._path(path), errors="replace") as f:
            lines = f.readlines()
        lo, hi = (start or 1) - 1, end or len(lines)
        return "".join(f"{i + 1}\t{l}" for i, l in enumerate(lines[lo:hi], lo))

    def tool_write(self, path: str, content: str) -> str:
        if not self.approve("write", {"path": path, "bytes": len(content)}):
            return "denied by the user"
        full = self._path(path)
        os.makedirs(os.path.dirname(full) or self.root, exist_ok=True)
        with open(full, "w") as f:
            f.write(content)
        return f"wrote {len(content)} bytes to {path}"

    def tool_edit(self, path: str, old: str, new: str) -> str:
        full = self._path(path)
        with open(full) as f:
            text = f.read()
        n = text.count(old)
        if n != 1:
            return f"error: 'old' occurs {n} times, need exactly 1"
        if not self.approve("edit", {"path": path}):
            return "denied by the user"
        with open(full, "w") as f:
            f.write(text.replace(old, new, 1))
        return f"edited {path}"

    def tool_glob(self, pattern: str) -> str:
        return "\n".join(sorted(self._files(pattern))[:500]) or "(no matches)"

    def tool_grep(self, pattern: str, glob: str = "*") -> str:
        rx = re.compile(pattern)
        hits = []
        for rel in self._files(glob):
            try:
                with open(os.path.join(self.root, rel), errors="replace") as f:
                    for i, line in enumerate(f, 1):
                        if rx.search(line):
                            hits.append(f"{rel}:{i}:{line.rstrip()}")
                            if len(hits) >= 200:
                                return "\n".join(hits)
            except OSError:
                continue
        return "\n".join(hits) or "(no matches)"

    def tool_run(self, command: str) -> str:
        if not self.approve("run", {"command": command}):
            return "denied by the user"
        try:
            p = subprocess.run(command, shell=True, cwd=self.root, capture_output=True, text=True, timeout=self.run_timeout)
        except subprocess.TimeoutExpired:
            return f"error: command timed out after {self.run_timeout:.0f} s"
        return f"exit code {p.returncode}\n{p.stdout}{p.stderr}"


class Agent:
    """``chat(messages, tools=..., max_tokens=...)`` must return the server's JSON (see client.DeliveranceClient.chat)."""

    def __init__(self, chat: Callable[..., dict], executor: ToolExecutor, max_turns: int = 16, max_tokens: int = 1024,
                 on_text: Callable[[str], None] = print):
        self.chat, self.executor, self.max_turns, self.max_tokens, self.on_text = chat, executor, max_turns, max_tokens, on_text
        self.messages: list[dict] = [{"role": "system", "content": SYSTEM}]

    def ask(self, user_text: str) -> str:
        self.messages.append({"role": "user", "content": user_text})
        for _ in range(self.max_turns):
            reply = self.chat(self.messages, tools=TOOLS, max_tokens=self.max_tokens)["choices"][0]["message"]
            calls = reply.get("tool_calls") or []
            self.messages.append({"role": "assistant", "content": reply.get("content") or "", **({"tool_calls": calls} if calls else {})})
            if reply.get("content"):
                self.on_text(reply["content"])
            if not calls:
                return reply.get("content") or ""
            for c in calls:
                fn = c["function"]
                try:
                    args = fn["arguments"] if isinstance(fn["arguments"], dict) else json.loads(fn["arguments"] or "{}")
                except ValueError:
                    args = {}
                result = self.executor.execute(fn["name"], args)
                self.messages.append({"role": "tool", "tool_call_id": c.get("id"), "name": fn["name"], "content": result})
        return "(stopped: turn limit reached)"


def main() -> int:
    import argparse

    from ..client import DeliveranceClient

    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--workspace", default=".")
    ap.add_argument("--auto-approve", action="store_true")
    a = ap.parse_args()
    client = DeliveranceClient(a.url)

    def approve(kind, info):
        if a.auto_approve:
            return True
        return input(f"[approve {kind} {info}? y/N] ").strip().lower().startswith("y")

    agent = Agent(client.chat, ToolExecutor(a.workspace, approve))
    while True:
        try:
            q = input("nanocode> ")
        except EOFError:
            return 0
        if q.strip() in ("exit", "quit"):
            return 0
        agent.ask(q)


if __name__ == "__main__":
    raise SystemExit(main())
