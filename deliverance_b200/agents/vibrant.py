"""Spec-driven code generation and a retrieval-augmented chat loop with an embedded (in-process) model.

    python -m deliverance_b200.agents.vibrant generate --model DIR --spec vibes.json [--base .]
    python -m deliverance_b200.agents.vibrant ragchat  --model DIR --embedding-model DIR

``generate``: every enabled spec of the file (``id``, ``systemMessage`` list, ``userMessage`` list, ``generateTo`` folder,
``overwrite``, ``messageTransformer`` = ``java`` | ``python`` | ``raw``) becomes one chat request; the reply is split into
source files by its transformer and written under ``generateTo`` (existing files are kept unless ``overwrite``). The reference
does this as a Maven mojo (vibrant-maven-plugin/.../VibrantMojo.java, VibeSpec.java, JavaResponseTransformer.java:14-110): the Java
transformer takes the ```` ```java ```` region of the reply, reads one ``package`` and all ``import`` lines, and starts a new
file at each ``public class`` / ``public interface`` that ends at the next line starting with ``}``.

``ragchat``: ``index PATH [GLOB]`` splits files into overlapping chunks and embeds them; ``embedding QUERY`` retrieves the three
nearest chunks (cosine) into the context buffer; ``template QUESTION`` asks the model with that context; any other line is a
plain chat turn; ``undeliver`` quits (reference: vibrant-maven-plugin/.../RagChatMojo.java:60-150).
"""
from __future__ import annotations

import argparse
import fnmatch
import json
import os
import re
import sys
from dataclasses import dataclass, field
from typing import Callable, Optional

RAG_TEMPLATE = "Answer the following question based on the provided context.\n\nContext:\n{context}\n\nQuestion: {question}"


@dataclass
class VibeSpec:
    id: str
    user_messages: list = field(default_factory=list)
    system_messages: list = field(default_factory=list)
    enabled: bool = True
    generate_to: str = "generated-source"
    overwrite: bool = False
    transformer: str = "java"

    @classmethod
    def from_dict(cls, d: dict) -> "VibeSpec":
        def many(*keys):
            for k in keys:
                if k in d:
                    v = d[k]
                    return [v] if isinstance(v, str) else list(v)
            return []

        t = str(d.get("messageTransformer", d.get("transformer", "java")))
        if "." in t:  # a class name of the reference's plugin
            t = "java" if "Java" in t else "raw"
        return cls(str(d["id"]), many("userMessage", "userMessages", "user_messages"), many("systemMessage", "systemMessages", "system_messages"),
                   bool(d.get("enabled", True)), str(d.get("generateTo", d.get("generate_to", "generated-source"))), bool(d.get("overwrite", False)), t.lower())


def load_specs(path: str) -> list:
    with open(path) as f:
        data = json.load(f) if not path.endswith((".yaml", ".yml")) else __import__("yaml").safe_load(f)
    specs = data.get("vibeSpecs", data.get("specs", data)) if isinstance(data, dict) else data
    return [VibeSpec.from_dict(s) for s in specs]


# ------------------------------------------------------------------------------------------------------ transformers
def fenced_region(text: str, lang: str) -> str:
    """The text between the first ```` ```lang ```` and the LAST fence; the whole text when there is no such fence."""
    tag = "```" + lang
    i = text.find(tag)
    if i < 0:
        return text
    start = text.find("\n", i)
    start = len(text) if start < 0 else start + 1
    end = text.rfind("```")
    return text[start:end] if end > start else text[start:]


def _write(path: str, content: str, overwrite: bool, written: list) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    if os.path.exists(path) and not overwrite:
        raise FileExistsError(f"{path} exists and the spec does not allow overwriting")
    with open(path, "w") as f:
        f.write(content)
    written.append(path)


def transform_java(raw: str, base: str, spec: VibeSpec) -> list:
    body = fenced_region(raw, "java")
    lines = body.split("\n")
    package = None
    imports = []
    for ln in lines:
        if ln.startswith("package ") and package is None:
            package = ln.split()[1].rstrip(";")
        elif ln.startswith("import "):
            imports.append(ln)
    out_dir = os.path.join(base, *(package.split(".") if package else []))
    written: list = []
    current, buf = None, []
    for ln in lines:
        if ln.startswith(("import ", "package ")):
            continue
        m = re.search(r"\bpublic\s+(?:(?:abstract|final)\s+)*(?:class|interface|enum|record)\s+(\w+)", ln)
        if m and current is None:
            current = m.group(1)
            buf = ([f"package {package};"] if package else []) + imports
        if current is not None:
            buf.append(ln)
            if ln.startswith("}"):
                _write(os.path.join(out_dir, current + ".java"), "\n".join(buf) + "\n", spec.overwrite, written)
                current, buf = None, []
    return written


def transform_python(raw: str, base: str, spec: VibeSpec) -> list:
    """One file per ``# file: NAME.py`` marker inside the python region; without markers the region becomes ``<spec id>.py``."""
    body = fenced_region(raw, "python")
    written: list = []
    parts = re.split(r"^#\s*file:\s*(\S+)\s*$", body, flags=re.M)
    if len(parts) == 1:
        _write(os.path.join(base, spec.id + ".py"), body.strip("\n") + "\n", spec.overwrite, written)
        return written
    for name, content in zip(parts[1::2], parts[2::2]):
        if os.path.isabs(name) or ".." in name.split("/"):
            raise ValueError(f"refusing to write outside the target folder: {name}")
        _write(os.path.join(base, name), content.strip("\n") + "\n", spec.overwrite, written)
    return written


def transform_raw(raw: str, base: str, spec: VibeSpec) -> list:
    written: list = []
    _write(os.path.join(base, spec.id + ".txt"), raw, spec.overwrite, written)
    return written


TRANSFORMERS = {"java": transform_java, "python": transform_python, "raw": transform_raw}


def run_specs(chat: Callable[[list], str], specs: list, base: str = ".", log=print) -> dict:
    """``chat(messages) -> reply text``. Returns {spec id: [written paths]}."""
    out = {}
    for spec in specs:
        if not spec.enabled:
            log(f"[vibrant] {spec.id}: disabled, skipped")
            continue
        if spec.transformer not in TRANSFORMERS:
            raise ValueError(f"{spec.id}: unknown transformer '{spec.transformer}'")
        messages = [{"role": "system", "content": s} for s in spec.system_messages] + [{"role": "user", "content": u} for u in spec.user_messages]
        reply = chat(messages)
        out[spec.id] = TRANSFORMERS[spec.transformer](reply, os.path.join(base, spec.generate_to), spec)
        for p in out[spec.id]:
            log(f"[vibrant] {spec.id}: wrote {p}")
    return out


# ------------------------------------------------------------------------------------------------------ retrieval
def split_text(text: str, size: int = 1000, overlap: int = 100) -> list:
    """Chunks of at most ``size`` characters that prefer to end at a blank line, then a line end; neighbours share ``overlap``."""
    chunks, i, n = [], 0, len(text)
    while i < n:
        end = min(n, i + size)
        if end < n:
            cut = text.rfind("\n\n", i + size // 2, end)
            cut = text.rfind("\n", i + size // 2, end) if cut < 0 else cut
            end = cut + 1 if cut > 0 else end
        chunks.append(text[i:end])
        if end >= n:
            break
        i = max(end - overlap, i + 1)
    return [c for c in chunks if c.strip()]


class VectorStore:
    def __init__(self, embed: Callable[[list], "object"]):
        self.embed = embed  # list of texts -> [n, d] tensor (rows need not be normalised)
        self.meta: list = []
        self.texts: list = []
        self.vecs = None

    def add(self, texts: list, metas: list) -> None:
        import torch

        if not texts:
            return
        v = torch.nn.functional.normalize(torch.as_tensor(self.embed(texts)).float(), dim=-1)
        self.vecs = v if self.vecs is None else torch.cat([self.vecs, v])
        self.texts += texts
        self.meta += metas

    def add_path(self, root: str, pattern: str = "*.py", size: int = 1000, overlap: int = 100) -> int:
        n = 0
        for d, _, files in sorted(os.walk(root)):
            for f in sorted(files):
                if fnmatch.fnmatch(f, pattern):
                    p = os.path.join(d, f)
                    with open(p, errors="replace") as fh:
                        chunks = split_text(fh.read(), size, overlap)
                    self.add(chunks, [{"path": p, "chunk": i} for i in range(len(chunks))])
                    n += len(chunks)
        return n

    def search(self, query: str, k: int = 3) -> list:
        import torch

        if self.vecs is None:
            return []
        q = torch.nn.functional.normalize(torch.as_tensor(self.embed([query])).float(), dim=-1)[0]
        scores = self.vecs @ q
        top = torch.topk(scores, min(k, len(self.texts)))
        return [(float(s), self.meta[i], self.texts[i]) for s, i in zip(top.values.tolist(), top.indices.tolist())]


class RagChat:
    def __init__(self, chat: Callable[[list], str], store: VectorStore, out=sys.stdout):
        self.chat, self.store, self.out = chat, store, out
        self.context = ""

    def line(self, text: str) -> bool:
        """One input line; False when the session ends."""
        w = self.out.write
        if text.strip().lower() == "undeliver":
            return False
        if text.startswith("index"):
            parts = text.split()
            n = self.store.add_path(parts[1], parts[2] if len(parts) > 2 else "*.py")
            w(f"Vectorized {parts[1]} ({n} chunks)\n")
        elif text.startswith("embedding"):
            query = text[len("embedding"):].strip()
            ctx = []
            for score, meta, chunk in self.store.search(query, 3):
                w(f"{meta} relevance {score:.3f}\n{chunk[:100]}...\n")
                ctx.append(f"{meta}\n{chunk}")
            self.context = "\n".join(ctx)
        elif text.startswith("template"):
            question = text[len("template"):].strip()
            w(self.chat([{"role": "user", "content": RAG_TEMPLATE.format(context=self.context, question=question)}]) + "\n")
        else:
            w(self.chat([{"role": "user", "content": text}]) + "\n")
        return True


def _embedded_chat(model_dir: str, device: str, max_tokens: int, temperature: float = 0.2, seed: int = 99998) -> Callable[[list], str]:
    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.params import GeneratorParameters

    clm = AutoModelForCausalLM.new_builder(model_dir).with_device(device).build()

    def chat(messages: list) -> str:
        pb = clm.prompt_builder()
        for m in messages:
            pb = {"system": pb.add_system, "user": pb.add_user, "assistant": pb.add_assistant}[m["role"]](m["content"])
        return clm.generate(pb.build(), GeneratorParameters(max_tokens=max_tokens, temperature=temperature, seed=seed)).text

    return chat


def main(argv: Optional[list] = None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("--model", required=True)
    g.add_argument("--spec", required=True)
    g.add_argument("--base", default=".")
    g.add_argument("--max-tokens", type=int, default=2048)
    g.add_argument("--device", default="auto")
    r = sub.add_parser("ragchat")
    r.add_argument("--model", required=True)
    r.add_argument("--embedding-model", required=True)
    r.add_argument("--max-tokens", type=int, default=512)
    r.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    chat = _embedded_chat(a.model, a.device, a.max_tokens)
    if a.cmd == "generate":
        run_specs(chat, load_specs(a.spec), a.base)
        return 0
    from deliverance_b200.embedding import AutoModelForEmbeddings

    em = AutoModelForEmbeddings.from_pretrained(a.embedding_model, a.device)
    rag = RagChat(chat, VectorStore(em.embed_many))
    print("Chat with the model. 'index PATH [GLOB]', 'embedding QUERY', 'template QUESTION', 'undeliver' to quit.")
    for ln in sys.stdin:
        if not rag.line(ln.rstrip("\n")):
            break
        print(">> ", end="", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
