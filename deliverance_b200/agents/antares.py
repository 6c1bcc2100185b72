"""Repository-investigation agent over the raw ``/v1/completions`` stream: the model explores a code base with read-only
tools and submits a ranked list of files.

    python -m deliverance_b200.agents.antares --url http://127.0.0.1:8080 --repo . --query "CWE-89: SQL injection" [--yes]

Unlike the chat agent (agents/nanocode.py), nothing here depends on a chat template or on server-side tool parsing: the
conversation is rendered to one text prompt with role markers, the assistant turn is prefilled with an open ``<think>`` block,
and tool calls are recovered from the generated text with a lenient parser. Behaviour follows the reference's agent
(deliverance-antares-cli/.../AntaresAgent.java:47-140, AntaresPrompt.java, ToolCallParser.java, AntaresToolExecutor.java:55-140):

* tools: ``terminal`` (read-only commands from an allow-list, each one approved by the user unless ``--yes``; 10 s limit),
  ``read_file`` (optional line bounds), ``submit_vulnerable_files`` (every path must be an existing repository-relative file)
  and ``submit_no_vulnerability_found``; ``terminal`` / ``read_file`` draw from one call budget;
* a turn without a tool call gets a nudge (at most five in a row), repeated identical calls are refused, and once the budget
  is spent the model gets ``max_submit_turns`` turns to submit before the agent falls back to the source files it has seen;
* role markers and ``<tool_response>`` delimiters inside message text are neutralised before rendering, so file contents
  cannot forge a turn boundary.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shlex
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

ROLE_OPEN, ROLE_CLOSE, END = "<|start_of_role|>", "<|end_of_role|>", "<|end_of_text|>"
CONTROL_TOKENS = (ROLE_OPEN, ROLE_CLOSE, END, "<|endoftext|>", "<|eot_id|>")
ASSISTANT_PREFILL = f"{ROLE_OPEN}assistant{ROLE_CLOSE}<think>\n"
READ_ONLY_COMMANDS = frozenset("ls tree find cat head tail sed grep rg wc sort uniq cut file stat du pwd nl basename dirname realpath diff echo true false".split())
SOURCE_SUFFIXES = (".java", ".kt", ".scala", ".py", ".js", ".ts", ".tsx", ".jsx", ".go", ".rs", ".c", ".cc", ".cpp", ".h", ".hpp", ".cs", ".rb",
                   ".php", ".sql", ".xml", ".yaml", ".yml", ".json", ".properties")
_WRAPPED = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.S | re.I)
_RAW_OBJECT = re.compile(r'\{\s*"(?:name|tool)"\s*:')
_TOOL_RESPONSE_TAG = re.compile(r"</?tool_response(?:\s+[^>]*)?>", re.I)
_PATH = re.compile(r"(?<![A-Za-z0-9_./-])(?:\./)?[A-Za-z0-9_.-]+(?:/[A-Za-z0-9_.-]+)+(?<![.,:;])")


# ------------------------------------------------------------------------------------------------------ tool-call parsing
@dataclass(frozen=True)
class ToolCall:
    name: str
    arguments: dict = field(default_factory=dict, hash=False)

    def key(self) -> str:
        return json.dumps({"name": self.name, "arguments": self.arguments}, sort_keys=True)


def _object_prefix(text: str) -> Optional[dict]:
    """The JSON object that starts at the first ``{`` of ``text``; trailing text is ignored."""
    i = text.find("{")
    if i < 0:
        return None
    try:
        obj, _ = json.JSONDecoder().raw_decode(text[i:])
    except ValueError:
        return None
    return obj if isinstance(obj, dict) else None


def _to_call(obj: Optional[dict]) -> Optional[ToolCall]:
    if obj is None:
        return None
    name = obj.get("name", obj.get("tool"))
    if name is None and "ranked_files" in obj:  # a bare answer object counts as the submit call
        return ToolCall("submit_vulnerable_files", dict(obj))
    if not isinstance(name, str):
        return None
    name = re.sub(r"[\s-]+", "_", name.strip().lower())
    args = obj.get("arguments", obj.get("args"))
    if args is None and name == "submit_vulnerable_files" and "ranked_files" in obj:
        return ToolCall(name, dict(obj))
    if args is None and name == "submit_no_vulnerability_found":
        return ToolCall(name, {})
    if not isinstance(args, dict):
        return None
    return ToolCall(name, args)


def parse_tool_calls(text: str) -> list[ToolCall]:
    """``<tool_call>{...}</tool_call>`` regions first; without any, bare ``{"name": ...}`` / ``{"tool": ...}`` objects."""
    calls = [c for c in (_to_call(_object_prefix(m.group(1))) for m in _WRAPPED.finditer(text)) if c is not None]
    if calls:
        return calls
    return [c for c in (_to_call(_object_prefix(text[m.start():])) for m in _RAW_OBJECT.finditer(text)) if c is not None]


def clean_assistant_text(text: str) -> str:
    text = _WRAPPED.sub("", text)
    for t in (END, "<|endoftext|>", "<|eot_id|>", "<think>", "</think>"):
        text = text.replace(t, "")
    return text.strip()


# ------------------------------------------------------------------------------------------------------ prompt rendering
_TOOLS = [
    {"name": "terminal", "description": "Execute a read-only terminal command in the repository. Allowed: " + ", ".join(sorted(READ_ONLY_COMMANDS))
     + ". Pipes and read-only &&, || and ; chains are fine. No interpreters, writes, redirects or network commands.",
     "parameters": {"type": "object", "properties": {"command": {"type": "string"}, "max_chars": {"type": "integer", "default": 2000}}, "required": ["command"]}},
    {"name": "read_file", "description": "Read one repository-relative file with optional line bounds.",
     "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "start_line": {"type": "integer"}, "end_line": {"type": "integer"}}, "required": ["path"]}},
    {"name": "submit_vulnerable_files", "description": "Submit your answer: a ranked list of vulnerable file paths.",
     "parameters": {"type": "object", "properties": {"ranked_files": {"type": "array", "items": {"type": "string"}}}, "required": ["ranked_files"]}},
    {"name": "submit_no_vulnerability_found", "description": "Declare that no matching vulnerability was found.",
     "parameters": {"type": "object", "properties": {}, "required": []}},
]


def system_prompt(budget: int) -> str:
    tools = "\n".join(json.dumps({"type": "function", "function": t}, separators=(",", ":")) for t in _TOOLS)
    return (
        "You are a security vulnerability localization agent with read-only terminal access to a codebase.\n\n"
        "Given a weakness description, decide whether this codebase contains a matching vulnerability and, if so, which source "
        f"file(s) are vulnerable. Explore with the `terminal` and `read_file` tools; you have up to {budget} repository tool calls.\n\n"
        "When you are done: call `submit_vulnerable_files` with a ranked list of exact file paths (most likely first), or "
        "`submit_no_vulnerability_found` if the code does not contain the weakness (it may already be patched). Only submit "
        "files you have evidence for; never globs or descriptions.\n\n"
        "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n" + tools + "\n</tools>\n\n"
        "For each tool call, return a json object with function name and arguments within <tool_call></tool_call> XML tags:\n"
        '<tool_call>\n{"name": <function-name>, "arguments": <args-json-object>}\n</tool_call>')


def _neutralise(content: str) -> str:
    for tok in CONTROL_TOKENS:
        content = content.replace(tok, f"[escaped control token: {tok[2:-2]}]")
    return content


def render(messages: Iterable[tuple]) -> str:
    """(role, content) pairs -> one completion prompt that ends inside the assistant's open ``<think>`` block."""
    out = []
    for role, content in messages:
        content = _neutralise(content)
        if role == "assistant":
            body = content if content.startswith("<think>") else "<think>\n" + content
            out.append(f"{ROLE_OPEN}assistant{ROLE_CLOSE}{body}{END}")
        elif role == "tool_response":
            content = _TOOL_RESPONSE_TAG.sub("[escaped tool-response delimiter]", content)
            out.append(f"{ROLE_OPEN}user{ROLE_CLOSE}\n<tool_response>\n{content}\n</tool_response>{END}")
        else:
            out.append(f"{ROLE_OPEN}{role}{ROLE_CLOSE}{content}{END}")
    return "\n".join(out) + ("\n" if out else "") + ASSISTANT_PREFILL


def submission_nudge(budget: int) -> str:
    return (f"\nERROR: Repository tool budget exhausted ({budget}/{budget}). Submit now using either "
            '<tool_call>{"name":"submit_vulnerable_files","arguments":{"ranked_files":["path/to/file"]}}</tool_call> or '
            '<tool_call>{"name":"submit_no_vulnerability_found","arguments":{}}</tool_call>.')


def no_tool_nudge(i: int) -> str:
    if i == 0:
        return ("You must use tools to investigate before reporting. Start by calling terminal to examine the code. When finished, "
                "submit file paths with submit_vulnerable_files or call submit_no_vulnerability_found.")
    if i >= 4:
        return "Call submit_vulnerable_files with the file paths you identified, or call submit_no_vulnerability_found if you found nothing."
    return "Continue investigating. Use terminal to read more source files."


# ------------------------------------------------------------------------------------------------------ tools
@dataclass
class AgentResult:
    status: str  # "vulnerable" | "none" | "fallback_vulnerable" | "fallback_none"
    files: list = field(default_factory=list)
    summary: str = ""


def command_is_read_only(command: str) -> Optional[str]:
    """None when every command of the pipeline / chain is on the allow-list and nothing redirects or substitutes; else why not."""
    if re.search(r"[<>`]|\$\(", command):
        return "redirects and command substitution are not allowed"
    for part in re.split(r"\|\||&&|[|;]", command):
        try:
            words = shlex.split(part)
        except ValueError as e:
            return f"cannot parse: {e}"
        if not words:
            continue
        prog = os.path.basename(words[0])
        if prog not in READ_ONLY_COMMANDS:
            return f"'{prog}' is not a read-only command"
        if prog == "sed" and any(w == "-i" or w.startswith("-i") or w == "--in-place" for w in words[1:]):
            return "sed -i writes files"
        if prog == "find" and any(w in ("-delete", "-exec", "-execdir", "-ok", "-fprint", "-fprintf", "-fls") for w in words[1:]):
            return "find actions that write or execute are not allowed"
    return None


class RepoTools:
    def __init__(self, repo: str, approve: Callable[[str], bool], max_calls: int = 20, timeout: float = 10.0):
        self.root = os.path.realpath(repo)
        if not os.path.isdir(self.root):
            raise NotADirectoryError(f"repository path is not a directory: {self.root}")
        self.approve, self.max_calls, self.timeout = approve, max_calls, timeout
        self.used = 0
        self.last_call: Optional[ToolCall] = None

    def file_error(self, path: str) -> Optional[str]:
        if not isinstance(path, str) or not path.strip():
            return "empty path"
        if any(ch in path for ch in "*?[]{}") or path.startswith("/") or ".." in path.split("/"):
            return "not an exact repository-relative path"
        full = os.path.realpath(os.path.join(self.root, path))
        if not (full == self.root or full.startswith(self.root + os.sep)):
            return "outside the repository"
        return None if os.path.isfile(full) else "no such file"

    def execute(self, call: ToolCall):
        """Returns ("submitted", AgentResult) or ("response", text)."""
        n, a = call.name, call.arguments
        if n == "submit_vulnerable_files":
            files = [f for f in (a.get("ranked_files") or []) if isinstance(f, str)] if isinstance(a.get("ranked_files"), list) else []
            bad = [f"{f} ({self.file_error(f)})" for f in files if self.file_error(f)]
            good = [f[2:] if f.startswith("./") else f for f in files if not self.file_error(f)]
            if bad or not good:
                return "response", ("submit_vulnerable_files failed: ranked_files must be existing repository-relative file paths, not "
                                    f"globs, placeholders, or descriptions. Invalid entries: {bad}")
            return "submitted", AgentResult("vulnerable", good)
        if n == "submit_no_vulnerability_found":
            return "submitted", AgentResult("none")
        if self.used >= self.max_calls:
            return "response", f"Terminal call budget exhausted ({self.max_calls}/{self.max_calls}). Submit your answer now."
        if n in ("terminal", "bash"):
            self.used += 1
            self.last_call = call
            return "response", self._terminal(a)
        if n == "read_file":
            self.used += 1
            self.last_call = call
            return "response", self._read(a)
        return "response", (f"Tool {n} failed: unknown tool. Available tools: terminal, read_file, submit_vulnerable_files, "
                            "submit_no_vulnerability_found.")

    def _terminal(self, a: dict) -> str:
        command = str(a.get("command") or "").strip()
        try:
            max_chars = int(a.get("max_chars") or 2000)
        except (TypeError, ValueError):
            max_chars = 2000
        max_chars = min(max_chars if max_chars > 0 else 2000, 20000)
        if not command:
            return "Tool terminal failed: empty command"
        why = command_is_read_only(command)
        if why:
            return f"Tool terminal refused: {why}"
        if not self.approve(command):
            return f"Tool terminal declined by user: {command}"
        try:
            p = subprocess.run(["/bin/sh", "-c", command], cwd=self.root, capture_output=True, text=True, timeout=self.timeout, errors="replace")
        except subprocess.TimeoutExpired:
            return f"Tool terminal failed: command timed out after {self.timeout:g} seconds"
        except OSError as e:
            return f"Tool terminal failed: {e}"
        out = p.stdout
        if p.stderr.strip():
            out += "\n[stderr]: " + p.stderr
        if not out.strip():
            out = f"[no output; exit={p.returncode}]"
        elif p.returncode != 0:
            out += f"\n[exit={p.returncode}]"
        return out if len(out) <= max_chars else out[:max_chars] + f"\n[truncated {len(out) - max_chars} chars]"

    def _read(self, a: dict) -> str:
        path = str(a.get("path") or a.get("file_path") or a.get("file") or "")
        err = self.file_error(path)
        if err:
            return f"Tool read_file failed: {path}: {err}"
        with open(os.path.join(self.root, path), errors="replace") as f:
            lines = f.read().split("\n")
        lo = max(1, int(a.get("start_line") or 1))
        hi = min(len(lines), int(a.get("end_line") or len(lines)))
        body = "\n".join(f"{i}: {lines[i - 1]}" for i in range(lo, hi + 1))
        return body if len(body) <= 20000 else body[:20000] + "\n[truncated]"


# ------------------------------------------------------------------------------------------------------ agent loop
class AntaresAgent:
    def __init__(self, complete: Callable[[str, Callable[[str], None]], str], tools: RepoTools, max_iterations: int = 40,
                 max_submit_turns: int = 3, on_text: Optional[Callable[[str], None]] = None, log: Optional[Callable[[str], None]] = None):
        self.complete, self.tools = complete, tools
        self.max_iterations, self.max_submit_turns = max_iterations, max_submit_turns
        self.on_text = on_text or (lambda s: None)
        self.log = log or (lambda s: None)
        self.messages: list[tuple] = []

    def _candidates(self, found: dict, text: str) -> None:
        for m in _PATH.finditer(text or ""):
            p = m.group().strip()
            p = p[2:] if p.startswith("./") else p
            if p.endswith(SOURCE_SUFFIXES) and self.tools.file_error(p) is None:
                found.setdefault(p, None)

    def _fallback(self, found: dict, summary: str) -> AgentResult:
        return AgentResult("fallback_vulnerable", list(found), summary) if found else AgentResult("fallback_none", [], summary)

    def run(self, query: str) -> AgentResult:
        budget = self.tools.max_calls
        self.messages = [("system", system_prompt(budget)), ("user", query)]
        seen: set = set()
        found: dict = {}
        no_tool_turns = submit_attempts = 0
        last = ""
        for it in range(self.max_iterations):
            spent_at_start = self.tools.used >= budget
            self.log(f"[antares] model turn {it + 1}, tool calls {self.tools.used}/{budget}")
            last = self.complete(render(self.messages), self.on_text)
            self._candidates(found, last)
            self.messages.append(("assistant", last))
            calls = parse_tool_calls(last)
            if not calls:
                if spent_at_start:
                    submit_attempts += 1
                    if submit_attempts < self.max_submit_turns:
                        note = f"Observed candidate files: {list(found)}" if found else "No candidate files have been recorded."
                        self.messages.append(("tool_response", submission_nudge(budget) + "\n" + note))
                        continue
                    return self._fallback(found, "Model did not submit after the tool budget was exhausted. Last answer: " + clean_assistant_text(last))
                if no_tool_turns < 5:
                    self.messages.append(("tool_response", no_tool_nudge(no_tool_turns)))
                    no_tool_turns += 1
                    continue
                return self._fallback(found, "Model stopped without submitting. Last answer: " + clean_assistant_text(last))
            no_tool_turns = 0
            responses, executed = [], False
            for call in calls:
                self._candidates(found, json.dumps(call.arguments))
                if call.key() in seen:
                    continue
                seen.add(call.key())
                executed = True
                self.log(f"[antares] tool {call.name} {json.dumps(call.arguments)[:200]}")
                kind, val = self.tools.execute(call)
                if kind == "submitted":
                    return val
                self._candidates(found, val)
                responses.append(val)
            if not executed:
                self.messages.append(("tool_response", "You already called these tools with these exact arguments. Please try a different approach."))
                continue
            remaining = budget - self.tools.used
            text = "\n\n".join(responses)
            if remaining <= 0:
                if spent_at_start:
                    submit_attempts += 1
                text += submission_nudge(budget) + (f"\nObserved candidate files: {list(found)}" if found else "")
            else:
                text += f"\n[{remaining} tool-calls remaining]"
            self.messages.append(("tool_response", text))
            if remaining <= 0 and submit_attempts >= self.max_submit_turns:
                return self._fallback(found, "Model did not submit after the repository tool budget was exhausted.")
        return self._fallback(found, "Maximum iterations reached. Last answer: " + clean_assistant_text(last))


def http_completer(url: str, max_tokens: int = 1024, temperature: float = 0.0, **extra) -> Callable[[str, Callable[[str], None]], str]:
    """Streams ``POST /v1/completions`` and returns the whole text; stops at the end-of-turn marker."""
    import urllib.request

    def complete(prompt: str, on_text: Callable[[str], None]) -> str:
        body = {"prompt": prompt, "stream": True, "max_tokens": max_tokens, "temperature": temperature, "stop": [END, "</tool_call>"],
                "include_stop_str_in_output": True, **extra}
        req = urllib.request.Request(url.rstrip("/") + "/v1/completions", json.dumps(body).encode(), {"Content-Type": "application/json"})
        parts = []
        with urllib.request.urlopen(req, timeout=600) as r:
            for raw in r:
                line = raw.decode("utf-8", "replace").rstrip("\n")
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ch = json.loads(line[6:])
                if "error" in ch:
                    raise RuntimeError(ch["error"].get("message", "server error"))
                t = ch["choices"][0].get("text") if ch.get("choices") else None
                if t:
                    parts.append(t)
                    on_text(t)
        text = "".join(parts)
        if "<tool_call>" in text and "</tool_call>" not in text:
            text += "</tool_call>"  # the stop string may have been cut from the stream
        return text

    return complete


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--repo", default=".")
    ap.add_argument("--query", required=True)
    ap.add_argument("--max-tool-calls", type=int, default=20)
    ap.add_argument("--max-iterations", type=int, default=40)
    ap.add_argument("--max-tokens", type=int, default=1024)
    ap.add_argument("--yes", action="store_true", help="approve every read-only command without asking")
    a = ap.parse_args()

    def approve(command: str) -> bool:
        if a.yes:
            return True
        print(f"\n[antares] run in {os.path.realpath(a.repo)}: {command}\napprove? [y/N] ", end="", file=sys.stderr, flush=True)
        return sys.stdin.readline().strip().lower() in ("y", "yes")

    agent = AntaresAgent(http_completer(a.url, a.max_tokens), RepoTools(a.repo, approve, a.max_tool_calls), a.max_iterations,
                         on_text=lambda s: (sys.stderr.write(s), sys.stderr.flush()), log=lambda s: print("\n" + s, file=sys.stderr))
    res = agent.run(a.query)
    print(json.dumps({"status": res.status, "files": res.files, "summary": res.summary}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
