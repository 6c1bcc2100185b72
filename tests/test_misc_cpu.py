"""Model fetcher cache layout, TurboQuant codec, KV snapshots, HTTP client, profiler, LoRA hot swap."""
import json
import os
import threading

import pytest
import torch

from deliverance_b200.ckpt.fetch import FINISHED, ModelFetcher
from deliverance_b200.kv.turboquant import MseTurboQuantCodec, restore_pages, snapshot_pages
from deliverance_b200.utils.profiler import InferenceProfiler


def test_model_fetcher_layout_and_offline(tmp_path):
    calls = []

    def opener(url, headers):
        calls.append((url, headers))
        if url.endswith("/api/models/acme/tiny"):
            return json.dumps({"siblings": [{"rfilename": "config.json"}, {"rfilename": "model.safetensors"}, {"rfilename": "notes.bin"}]}).encode()
        return b"{}" if url.endswith("config.json") else b"\x00" * 16

    f = ModelFetcher.from_id("acme/tiny", home=str(tmp_path), opener=opener)
    assert f.model_dir == str(tmp_path / "acme_tiny") and not f.is_complete()
    os.environ["HF_TOKEN"] = "tok"
    try:
        d = f.maybe_download()
    finally:
        del os.environ["HF_TOKEN"]
    assert sorted(os.listdir(d)) == sorted([FINISHED, "config.json", "model.safetensors"])
    assert calls[0][1] == {"Authorization": "Bearer tok"} and calls[1][0].endswith("/acme/tiny/resolve/main/config.json")
    n = len(calls)
    assert f.maybe_download() == d and len(calls) == n  # .finished short-circuits

    def offline(url, headers):
        raise OSError("network unreachable")

    with pytest.raises(RuntimeError) as e:
        ModelFetcher("acme", "other", home=str(tmp_path), opener=offline).maybe_download()
    assert "offline" in str(e.value)
    with pytest.raises(ValueError):
        ModelFetcher.from_id("noslash")


def test_turboquant_codec_error_and_size():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 128, generator=g)
    errs = []
    for bits in (2, 3, 4, 8):
        c = MseTurboQuantCodec(128, bits)
        e = c.encode(x)
        y = c.decode(e)
        errs.append(((y - x).norm() / x.norm()).item())
        assert c.compressed_bytes(e) == 64 * 128 * bits // 8 + 64 * 4
    assert errs[0] > errs[1] > errs[2] > errs[3] and errs[1] < 0.25 and errs[3] < 0.02
    c = MseTurboQuantCodec(96, 4)  # non power-of-two rows are padded for the rotation
    z = torch.randn(5, 96, generator=g)
    assert ((c.decode(c.encode(z)) - z).norm() / z.norm()).item() < 0.15


def test_kv_snapshot_roundtrip():
    from deliverance_b200.kv.paged import PagedKVCache

    layout = {"layers": 2, "kv_heads": 2, "head_dim": 64, "layer_kinds": ["attention", "attention"]}
    kv = PagedKVCache(layout, 8, "cpu", torch.float32)
    g = torch.Generator().manual_seed(1)
    for t in kv.k + kv.v:
        t.copy_(torch.randn(t.shape, generator=g))
    k0, v0 = kv.gather_rows(1, [2, 5], 50)
    for comp, tol in (("NONE", 0.0), ("LZ4", 0.0), ("MSE_TURBOQUANT", 0.2)):
        snap = snapshot_pages(kv, [2, 5], 50, comp, bits=4)
        kv2 = PagedKVCache(layout, 8, "cpu", torch.float32)
        restore_pages(kv2, snap, [3, 4])
        k1, v1 = kv2.gather_rows(1, [3, 4], 50)
        assert ((k1 - k0).norm() / k0.norm()).item() <= tol + 1e-7 and ((v1 - v0).norm() / v0.norm()).item() <= tol + 1e-7


def test_profiler_report_format():
    p = InferenceProfiler("cpu")
    with p.stage("mlpblock.gate_up_projection"):
        sum(range(1000))
    with p.stage("mlpblock.gate_up_projection"):
        pass
    p.count("sampler.output_weight_Q4")
    s = p.summary()
    assert "[profile] mlpblock.gate_up_projection count=2 total_ms=" in s and "[profile-counter] sampler.output_weight_Q4 count=1" in s
    p.reset()
    assert p.summary() == ""


def test_python_client_against_server(tmp_path):
    import socket
    import time

    import uvicorn

    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.client import DeliveranceClient
    from deliverance_b200.server.app import ModelRegistry, create_app
    from deliverance_b200.server.runner import EngineRunner

    d = str(tmp_path / "tiny")
    write_tiny_model(d, "llama", seed=3, std=0.05)
    reg = ModelRegistry()
    runner = EngineRunner(AutoModelForCausalLM.from_pretrained(d, device="cpu"))
    reg.generation["tiny"] = runner
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    server = uvicorn.Server(uvicorn.Config(create_app(reg), host="127.0.0.1", port=port, log_level="error"))
    t = threading.Thread(target=server.run, daemon=True)
    t.start()
    for _ in range(100):
        if server.started:
            break
        time.sleep(0.05)
    try:
        c = DeliveranceClient(f"http://127.0.0.1:{port}")
        assert c.models() == ["tiny"]
        r = c.chat([{"role": "user", "content": "hi"}], max_tokens=4)
        assert r["usage"]["completion_tokens"] == 4
        kinds = [k for k, _ in c.stream_chat([{"role": "user", "content": "hi"}], max_tokens=4)]
        assert kinds[-1] == "finish"
        assert c.complete("abc", max_tokens=2)["object"] == "text_completion"
    finally:
        server.should_exit = True
        t.join(timeout=5)
        runner.close()


def test_lora_hot_swap_equals_merge(tmp_path):
    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.lora import lora_names
    from deliverance_b200.ckpt.safetensors_io import write_safetensors
    from deliverance_b200.ckpt.tiny import tiny_config, write_tiny_model
    from deliverance_b200.params import GeneratorParameters

    d = str(tmp_path / "base")
    write_tiny_model(d, "llama", seed=5, std=0.08)
    cfg = tiny_config("llama")
    hd = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    shapes = {"self_attn.q_proj": (cfg["num_attention_heads"] * hd, H), "self_attn.v_proj": (cfg["num_key_value_heads"] * hd, H),
              "self_attn.o_proj": (H, cfg["num_attention_heads"] * hd), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}
    g = torch.Generator().manual_seed(9)
    r, tensors = 4, {}
    for i in range(cfg["num_hidden_layers"]):
        for proj, (o, k) in shapes.items():
            a, b = lora_names(f"model.layers.{i}.{proj}.weight")
            tensors[a] = torch.randn(r, k, generator=g) * 0.2
            tensors[b] = torch.randn(o, r, generator=g) * 0.2
    ad = str(tmp_path / "adapter")
    os.makedirs(ad)
    write_safetensors(os.path.join(ad, "adapter_model.safetensors"), tensors)
    with open(os.path.join(ad, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": 8, "target_modules": ["q_proj", "v_proj", "o_proj", "up_proj", "down_proj"]}, f)

    p = GeneratorParameters(max_tokens=8, temperature=0.0)
    prompt = [3, 9, 27, 81, 5]
    base = AutoModelForCausalLM.from_pretrained(d, device="cpu")
    merged = AutoModelForCausalLM.new_builder(d).with_device("cpu").with_lora_adapter(ad).build()
    t_base = base.generate(prompt, p).token_ids
    t_merged = merged.generate(prompt, p).token_ids
    aid = base.register_lora(ad)
    base.activate_lora(aid)
    assert base.model.active_lora == "adapter"
    t_hot = base.generate(prompt, p).token_ids
    base.activate_lora(None)
    assert base.generate(prompt, p).token_ids == t_base
    assert t_hot == t_merged and t_hot != t_base
    with pytest.raises(KeyError):
        base.activate_lora("nope")


def test_sketches_facade_and_metrics_endpoint(tmp_path):
    import dataclasses
    from typing import Literal

    from fastapi.testclient import TestClient

    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.server.app import ModelRegistry, create_app
    from deliverance_b200.server.runner import EngineRunner
    from deliverance_b200.sketches import Sketches, schema_of

    d = str(tmp_path / "tiny")
    write_tiny_model(d, "llama", seed=3, std=0.05)
    clm = AutoModelForCausalLM.from_pretrained(d, device="cpu")
    sk = Sketches(clm, max_tokens=160)
    assert sk.choice("pick:", ["alpha", "beta"]) in ("alpha", "beta")
    import re

    assert re.fullmatch(r"[0-9]{3}-[a-c]{2}", sk.regex("code:", r"[0-9]{3}-[a-c]{2}"))

    @dataclasses.dataclass
    class Pet:
        kind: Literal["cat", "dog"]
        legs: Literal[2, 4]

    assert schema_of(Pet)["properties"]["kind"] == {"enum": ["cat", "dog"]}
    pet = sk.typed("a pet:", Pet)
    assert pet.kind in ("cat", "dog") and isinstance(pet.legs, int)

    reg = ModelRegistry()
    runner = EngineRunner(clm)
    reg.generation["tiny"] = runner
    try:
        c = TestClient(create_app(reg))
        c.post("/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
        m = c.get("/metrics")
        assert m.status_code == 200 and 'deliverance_requests_finished_total{model="tiny"} 1' in m.text
        assert "deliverance_engine_decode_tokens_total" in m.text and "deliverance_kv_pages_free" in m.text
    finally:
        runner.close()


def test_nanocode_agent_loop_with_scripted_model(tmp_path):
    """The agent executes tool calls, feeds results back, asks for approval before changes and stays inside the workspace."""
    from deliverance_b200.agents.nanocode import Agent, ToolExecutor

    (tmp_path / "a.txt").write_text("hello world\nsecond line\n")
    asked = []
    ex = ToolExecutor(str(tmp_path), lambda kind, info: (asked.append(kind), kind != "run")[1])

    def call(name, **args):
        return {"id": f"c{len(script)}", "type": "function", "function": {"name": name, "arguments": json.dumps(args)}}

    script = []
    script.append({"content": "", "tool_calls": [call("grep", pattern="hello"), call("read", path="a.txt", start=2, end=2)]})
    script.append({"content": "", "tool_calls": [call("edit", path="a.txt", old="hello", new="goodbye"), call("run", command="rm -rf /"),
                                                 call("read", path="../../etc/passwd"), call("write", path="sub/b.txt", content="x")]})
    script.append({"content": "done", "tool_calls": []})
    seen = []

    def chat(messages, **kw):
        seen.append([m["role"] for m in messages])
        assert kw["tools"]
        return {"choices": [{"message": script[len(seen) - 1]}]}

    agent = Agent(chat, ex, on_text=lambda t: None)
    assert agent.ask("change the greeting") == "done"
    tool_msgs = [m["content"] for m in agent.messages if m["role"] == "tool"]
    assert tool_msgs[0].startswith("a.txt:1:hello world") and tool_msgs[1] == "2\tsecond line\n"
    assert tool_msgs[2] == "edited a.txt" and tool_msgs[3] == "denied by the user" and "outside the workspace" in tool_msgs[4]
    assert (tmp_path / "a.txt").read_text().startswith("goodbye world") and (tmp_path / "sub" / "b.txt").read_text() == "x"
    assert asked == ["edit", "run", "write"] and seen[-1][-1] == "tool"


def test_auto_model_config_accepts_reference_json(tmp_path):
    """The reference's benchmark configs (benchmarks/configs/*.json) load unchanged; CPU-runtime knobs are recorded as ignored."""
    from deliverance_b200.api import AutoModelConfig, AutoModelForCausalLM

    c = AutoModelConfig.from_json(json.dumps({
        "outputHeadQuantization": "Q4", "maxBatchSize": 512, "workingMemoryType": "F32", "workingQuantType": "I8", "gpuPrefill": True,
        "kvBufferCache": {"maxEntries": 10000, "blockSize": 32, "maxPrefixTokensPerPrompt": 8192, "prefixCheckpointPolicy": "START_AND_END",
                          "prefixCompression": "MSE_TURBOQUANT", "prefixTurboQuantBits": 4, "maxPrefixCheckpointsPerPrompt": 4,
                          "contextRowsPerPageTarget": 32}}))
    assert c.output_head_quantization == "Q4" and c.max_batch_size == 512 and c.kv_max_prefix_tokens == 8192 and c.kv_policy == "START_AND_END"
    assert c.kv_compression == "MSE_TURBOQUANT" and c.kv_turboquant_bits == 4 and set(c.ignored) == {"workingMemoryType", "workingQuantType", "gpuPrefill"}
    off = AutoModelConfig.from_json('{"gpuPrefill": true, "kvBufferCache": {"maxEntries": 0, "maxPrefixTokensPerPrompt": 0}}')
    b = AutoModelForCausalLM.new_builder("x").with_config(off)
    assert not b.kv.enabled
    assert AutoModelConfig.from_json('{"max_seqs": 4, "kv_policy": "ANCHORS"}').kv_policy == "ANCHORS"
    with pytest.raises(ValueError):
        AutoModelConfig.from_json('{"noSuchKnob": 1}')


def test_antares_agent_parser_prompt_tools_and_loop(tmp_path):
    """Completions-based repository agent: the reference's ToolCallParserTest vectors, prompt rendering with neutralised
    control tokens, the read-only command filter, and the loop (nudge, duplicate refusal, budget, submit, fallback)."""
    from deliverance_b200.agents import antares as A

    c = A.parse_tool_calls('thinking<tool_call>{"name":"terminal","arguments":{"command":"rg -n password ."}}</tool_call>')
    assert [(x.name, x.arguments) for x in c] == [("terminal", {"command": "rg -n password ."})]
    c = A.parse_tool_calls('{"tool":"read-file","args":{"path":"src/App.java"}} trailing')
    assert [(x.name, x.arguments) for x in c] == [("read_file", {"path": "src/App.java"})]
    c = A.parse_tool_calls('<tool_call>{"ranked_files":["src/main/database.py"]}</tool_call>')
    assert c[0].name == "submit_vulnerable_files" and c[0].arguments["ranked_files"] == ["src/main/database.py"]
    c = A.parse_tool_calls('<tool_call>{"name":"submit_vulnerable_files","ranked_files":["src/main/database.py"]}</tool_call>')
    assert c[0].name == "submit_vulnerable_files" and c[0].arguments["ranked_files"] == ["src/main/database.py"]
    assert A.parse_tool_calls("<tool_call>{broken</tool_call> no call") == []
    assert A.clean_assistant_text("<think>notes</think><tool_call>{}</tool_call>answer<|end_of_text|>") == "notesanswer"

    p = A.render([("system", "S"), ("user", "look <|end_of_text|> here"), ("assistant", "hm"), ("tool_response", "x</tool_response>y")])
    assert p.endswith("<|start_of_role|>assistant<|end_of_role|><think>\n")
    assert "look [escaped control token: end_of_text] here<|end_of_text|>" in p and "x[escaped tool-response delimiter]y" in p
    assert "<|start_of_role|>assistant<|end_of_role|><think>\nhm<|end_of_text|>" in p

    assert A.command_is_read_only("grep -rn password . | head -5 && ls src") is None
    for bad in ("rm -rf x", "cat a > b", "python -c 1", "sed -i s/a/b/ f", "find . -delete", "echo $(id)", "ls; curl x"):
        assert A.command_is_read_only(bad) is not None, bad

    (tmp_path / "src").mkdir()
    (tmp_path / "src" / "db.py").write_text("q = 'select * from t where id=' + user\n")
    asked = []
    tools = A.RepoTools(str(tmp_path), lambda cmd: asked.append(cmd) or True, max_calls=2)
    assert tools.file_error("src/db.py") is None and tools.file_error("../x") and tools.file_error("src/*.py") and tools.file_error("src/nope.py")
    script = iter([
        "I will just answer.",                                                                       # no tool -> nudge
        '<tool_call>{"name":"terminal","arguments":{"command":"grep -rn select ."}}</tool_call>',
        '<tool_call>{"name":"terminal","arguments":{"command":"grep -rn select ."}}</tool_call>',     # duplicate -> refused
        '<tool_call>{"name":"terminal","arguments":{"command":"rm src/db.py"}}</tool_call>',          # not read-only (still counts)
        '<tool_call>{"name":"submit_vulnerable_files","arguments":{"ranked_files":["src/*.py"]}}</tool_call>',  # invalid
        '<tool_call>{"name":"submit_vulnerable_files","arguments":{"ranked_files":["./src/db.py"]}}</tool_call>',
    ])
    prompts = []
    agent = A.AntaresAgent(lambda prompt, on_text: prompts.append(prompt) or next(script), tools)
    res = agent.run("CWE-89")
    assert (res.status, res.files) == ("vulnerable", ["src/db.py"]) and asked == ["grep -rn select ."] and (tmp_path / "src" / "db.py").exists()
    assert "You must use tools" in prompts[1] and "src/db.py" in prompts[2] and "[1 tool-calls remaining]" in prompts[2]
    assert "already called these tools" in prompts[3] and "Tool terminal refused" in prompts[4] and "budget exhausted" in prompts[4]
    assert "submit_vulnerable_files failed" in prompts[5]
    # a model that never submits: falls back to the source files it has seen
    tools2 = A.RepoTools(str(tmp_path), lambda cmd: True, max_calls=1)
    replies = iter(['<tool_call>{"name":"read_file","arguments":{"path":"src/db.py"}}</tool_call>'] + ["nothing more"] * 10)
    res = A.AntaresAgent(lambda p, f: next(replies), tools2).run("CWE-89")
    assert res.status == "fallback_vulnerable" and res.files == ["src/db.py"]


def test_smoke_benchmarks_thinking_and_lora(tmp_path):
    """The thinking smoke benchmark's answer extraction and pass predicates, its JSONL rows on a tiny model, and the LoRA
    benchmark's base / lora-adapted rows (merge at load and hot swap generate the same adapted tokens)."""
    import io

    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.bench import smoke_benchmarks as sb
    from deliverance_b200.ckpt.lora import lora_names
    from deliverance_b200.ckpt.safetensors_io import write_safetensors
    from deliverance_b200.ckpt.tiny import tiny_config, write_tiny_model

    assert sb.final_answer("<think>maybe 10 cents</think>work...\nFinal: `0.05` dollars") == "0.05 dollars"
    bat = next(c for c in sb.CASES if c.id == "bat-ball")
    assert bat.check("0.05 dollars") and not bat.check("0.10") and not bat.check("it is 0.05, not 0.10")
    assert next(c for c in sb.CASES if c.id == "missing-dollar").check("no, nothing is missing")
    d = str(tmp_path / "base")
    write_tiny_model(d, "llama", seed=5, std=0.08, max_position_embeddings=1024)
    clm = AutoModelForCausalLM.from_pretrained(d, device="cpu")
    buf = io.StringIO()
    s = sb.run_thinking(clm, buf, max_tokens=4, cases=sb.CASES[:1] + sb.CASES[-1:])
    rows = [json.loads(l) for l in buf.getvalue().splitlines()]
    assert s["cases"] == 2 and s["max_token_warnings"] == 2 and [r["case_id"] for r in rows] == ["square-area", "follow-up"]
    assert rows[1]["generated_tokens"] == 8 and set(rows[0]) == {"timestamp", "case_id", "pass", "finish_reason", "generated_tokens", "time_ms",
                                                                 "time_to_first_token_ms", "response"}
    cfg = tiny_config("llama")
    g = torch.Generator().manual_seed(9)
    tensors = {}
    for i in range(cfg["num_hidden_layers"]):
        a, b = lora_names(f"model.layers.{i}.self_attn.q_proj.weight")
        tensors[a], tensors[b] = torch.randn(4, 64, generator=g) * 0.3, torch.randn(64, 4, generator=g) * 0.3
    ad = str(tmp_path / "adapter")
    os.makedirs(ad)
    write_safetensors(os.path.join(ad, "adapter_model.safetensors"), tensors)
    with open(os.path.join(ad, "adapter_config.json"), "w") as f:
        json.dump({"r": 4, "lora_alpha": 8, "target_modules": ["q_proj"]}, f)
    out = {}
    for mode in ("merge", "hotswap"):
        buf = io.StringIO()
        out[mode] = sb.run_lora(d, ad, buf, mode=mode, max_tokens=6, device="cpu", prompts=sb.LORA_PROMPTS[:2])
        lines = buf.getvalue().splitlines()
        assert lines[0].split(",") == sb.LORA_COLUMNS and len(lines) == 5
        assert [r["variant"] for r in out[mode]] == ["base", "base", "lora-adapted", "lora-adapted"]
    assert [r["token_ids"] for r in out["merge"]] == [r["token_ids"] for r in out["hotswap"]]
    assert out["merge"][0]["token_ids"] != out["merge"][2]["token_ids"]


def test_vibrant_codegen_transformers_and_rag(tmp_path):
    """Spec-driven generation: replies are split into source files (java: package folders, imports repeated per type; python:
    file markers), existing files are kept unless the spec allows overwriting; retrieval chat over a toy embedding."""
    import io

    from deliverance_b200.agents import vibrant as V

    reply = ("Sure!\n```java\npackage com.acme.shapes;\nimport java.util.List;\n\npublic interface Shape {\n  double area();\n}\n\n"
             "public class Square implements Shape {\n  double s;\n  public double area() { return s * s; }\n}\n```\nDone.")
    spec_file = tmp_path / "vibes.json"
    spec_file.write_text(json.dumps({"vibeSpecs": [
        {"id": "shapes", "systemMessage": ["You write Java."], "userMessage": "Make shapes.", "generateTo": "gen",
         "messageTransformer": "io.teknek.deliverance.vibrant.JavaResponseTransformer"},
        {"id": "off", "userMessage": ["x"], "enabled": False},
        {"id": "tool", "userMessage": ["py"], "generateTo": "pygen", "messageTransformer": "python", "overwrite": True}]}))
    specs = V.load_specs(str(spec_file))
    assert specs[0].transformer == "java" and specs[0].user_messages == ["Make shapes."] and not specs[1].enabled
    seen = []

    def chat(messages):
        seen.append(messages)
        return reply if "Java" in messages[0]["content"] else "```python\n# file: a.py\nx = 1\n# file: pkg/b.py\ny = 2\n```"

    out = V.run_specs(chat, specs, str(tmp_path), log=lambda s: None)
    sq = (tmp_path / "gen" / "com" / "acme" / "shapes" / "Square.java").read_text()
    assert sq.startswith("package com.acme.shapes;\nimport java.util.List;\npublic class Square implements Shape {") and sq.rstrip().endswith("}")
    assert (tmp_path / "gen" / "com" / "acme" / "shapes" / "Shape.java").exists() and len(out["shapes"]) == 2 and "off" not in out
    assert (tmp_path / "pygen" / "a.py").read_text() == "x = 1\n" and (tmp_path / "pygen" / "pkg" / "b.py").read_text() == "y = 2\n"
    assert seen[0][0] == {"role": "system", "content": "You write Java."}
    with pytest.raises(FileExistsError):  # overwrite is off for the java spec
        V.run_specs(chat, specs[:1], str(tmp_path), log=lambda s: None)
    V.run_specs(chat, specs[2:], str(tmp_path), log=lambda s: None)  # overwrite allowed
    with pytest.raises(ValueError):
        V.transform_python("```python\n# file: ../evil.py\nx\n```", str(tmp_path), specs[2])
    assert V.fenced_region("no fences", "java") == "no fences"

    chunks = V.split_text("para one\n\n" + "x" * 900 + "\n\npara three " * 30, 400, 50)
    assert all(len(c) <= 400 for c in chunks) and len(chunks) > 3
    words = ["mojo", "tensor", "socket"]
    embed = lambda texts: torch.tensor([[float(t.lower().count(w)) + 0.01 for w in words] for t in texts])  # noqa: E731
    store = V.VectorStore(embed)
    (tmp_path / "src").mkdir()
    (tmp_path / "src" / "a.py").write_text("class Plugin(Mojo):\n    '''a mojo mojo'''\n")
    (tmp_path / "src" / "b.py").write_text("def reduce(tensor):\n    return tensor.sum()\n")
    buf = io.StringIO()
    asked = []
    rag = V.RagChat(lambda m: asked.append(m[0]["content"]) or "answer", store, buf)
    assert rag.line(f"index {tmp_path / 'src'}") and "2 chunks" in buf.getvalue()
    assert rag.line("embedding which classes extend Mojo") and store.search("mojo", 1)[0][1]["path"].endswith("a.py")
    assert rag.line("template What extends Mojo?") and "class Plugin(Mojo)" in asked[0] and asked[0].endswith("Question: What extends Mojo?")
    assert rag.line("hello") and asked[1] == "hello" and not rag.line("undeliver")


def test_rank_affinity_from_fake_sysfs(tmp_path):
    """NUMA placement of rank processes, driven by a fake sysfs tree: PCI id normalisation, node lookup, core shares of ranks
    that share a node, analyze / off modes, and machines that report no node."""
    from deliverance_b200.utils import affinity as A

    assert A.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert A.normalise_pci_bus_id("00000000:1B:00.0") == "0000:1b:00.0" and A.normalise_pci_bus_id("1b:00.0") == "0000:1b:00.0"
    root = tmp_path / "sys"
    for bus, node in (("0000:1b:00.0", 0), ("0000:43:00.0", 0), ("0000:9b:00.0", 1), ("0000:c3:00.0", -1)):
        d = root / "bus" / "pci" / "devices" / bus
        d.mkdir(parents=True)
        (d / "numa_node").write_text(f"{node}\n")
    for node, cl in ((0, "0-7"), (1, "8-15")):
        d = root / "devices" / "system" / "node" / f"node{node}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cl + "\n")
    (root / "devices" / "system" / "cpu" / "cpu9" / "node1").mkdir(parents=True)
    assert A.numa_node_of_cpu(9, str(root)) == 1 and A.numa_node_of_cpu(3, str(root)) == -1
    calls = []
    bus = ["00000000:1B:00.0", "00000000:43:00.0", "00000000:9B:00.0", "00000000:C3:00.0"]
    kw = dict(sysfs_root=str(root), bus_ids=bus, setaffinity=lambda pid, cpus: calls.append(sorted(cpus)), allowed=set(range(16)))
    p0 = A.place_local_rank(0, 4, "enforce", **kw)
    p1 = A.place_local_rank(1, 4, "enforce", **kw)
    p2 = A.place_local_rank(2, 4, "enforce", **kw)
    assert (p0.numa_node, p0.cpus, p0.applied) == (0, [0, 1, 2, 3], True) and p1.cpus == [4, 5, 6, 7] and p2.cpus == list(range(8, 16))
    assert calls == [[0, 1, 2, 3], [4, 5, 6, 7], list(range(8, 16))]
    p3 = A.place_local_rank(3, 4, "enforce", **kw)
    assert not p3.applied and "no NUMA node" in p3.note and len(calls) == 3
    pa = A.place_local_rank(2, 4, "analyze", **kw)
    assert pa.cpus and not pa.applied and len(calls) == 3 and A.place_rank(0, bus[0], "off").note == "off"
    restricted = A.place_rank(2, bus[2], "enforce", str(root), setaffinity=lambda *a: None, allowed={0, 1})
    assert not restricted.applied and "no usable cores" in restricted.note
    assert p0.to_json()["cpus"] == 4


def test_server_properties_config(tmp_path):
    """The reference's .properties layout: indexed model entries (both key spellings), KV prefix settings, ${ENV:default}
    placeholders, ignored runtime-specific keys; the same keys as nested JSON."""
    from deliverance_b200.server.config import load_server_config, parse_properties

    p = tmp_path / "srv.properties"
    p.write_text("""# comment
server.port=${TP_WEB_PORT:8081}
deliverance.tensor.operations.type=simd
deliverance-model.configs[0].model-owner=edwardcapriolo
deliverance-model.configs[0].model-name=${TP_MODEL:Qwen3-4B-JQ4}
deliverance-model.configs[0].inference-type=GENERATION
deliverance-model.configs[0].output-head-quantization=Q4
deliverance-model.configs[0].tensor-parallel.enabled=true
deliverance-model.configs[0].tensor-parallel.size=${TP_SIZE:4}
deliverance-model.configs[0].tensor-parallel.seeds[0]=coordinator=udp://127.0.0.1:42606
deliverance-model.configs[1].modelName=all-MiniLM-L6-v2
deliverance-model.configs[1].modelOwner=sentence-transformers
deliverance-model.configs[1].inferenceType=EMBEDDING
deliverance.kv.prefix.max-tokens=8192
deliverance.kv.prefix.checkpoint-policy=start_and_end
deliverance.kv.prefix.max-checkpoints=12
deliverance.kv.prefix.compression=MSE_TURBOQUANT
deliverance.kv.prefix.turboquant.bits=4
deliverance.kv.context-rows-per-page-target=32
deliverance.openai.reasoning-field=vllm
deliverance.basic.auth.user=bob
""")
    c = load_server_config(str(p), env={"TP_SIZE": "8"})
    assert c.port == 8081 and len(c.models) == 2 and c.reasoning_field == "vllm" and c.basic_user == "bob"
    m0, m1 = c.models
    assert (m0.owner, m0.name, m0.output_head_quantization, m0.tp_enabled, m0.tp_size) == ("edwardcapriolo", "Qwen3-4B-JQ4", "Q4", True, 8)
    assert (m1.owner, m1.name, m1.inference_type) == ("sentence-transformers", "all-MiniLM-L6-v2", "EMBEDDING")
    kv = c.kv_settings()
    assert (kv.max_prefix_tokens, kv.policy, kv.checkpoints, kv.compression, kv.block_size) == (8192, "START_AND_END", 12, "MSE_TURBOQUANT", 32)
    assert c.kv_turboquant_bits == 4 and "deliverance.tensor.operations.type" in c.ignored and any("seeds" in k for k in c.ignored)
    (tmp_path / "root" / "edwardcapriolo_Qwen3-4B-JQ4").mkdir(parents=True)
    assert m0.resolve_dir(str(tmp_path / "root")).endswith("edwardcapriolo_Qwen3-4B-JQ4")
    assert m1.resolve_dir(str(tmp_path / "root")).endswith("sentence-transformers_all-MiniLM-L6-v2")
    assert parse_properties("a = 1\\\n  2\nb: x\n! note\n") == {"a": "12", "b": "x"}
    j = tmp_path / "srv.json"
    j.write_text(json.dumps({"server": {"port": 9000}, "deliverance-model": {"configs": [{"model-dir": "/m/x", "inferenceType": "generation"}]},
                             "deliverance": {"kv": {"prefix": {"max-tokens": 1024}}}}))
    cj = load_server_config(str(j))
    assert cj.port == 9000 and cj.models[0].model_dir == "/m/x" and cj.models[0].inference_type == "GENERATION" and cj.kv == {"max_prefix_tokens": 1024}
    bad = tmp_path / "bad.properties"
    bad.write_text("deliverance-model.configs[0].inference-type=NOPE\ndeliverance-model.configs[0].model-name=x\n")
    with pytest.raises(ValueError):
        load_server_config(str(bad))


def test_chat_model_adapters(tmp_path):
    """One ChatModel interface over HTTP and over an in-process model: option merging, the tool-execution loop (fake
    transport), guided options and streaming on a tiny embedded model."""
    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.integrations import ChatOptions, EmbeddedChatModel, HttpChatModel, ToolCallback

    add = ToolCallback("add", "adds two numbers", {"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "integer"}}}, lambda a, b: a + b)
    base = ChatOptions(temperature=0.2, max_tokens=16, tools=[add], extra={"cache_salt": "s"})
    m = base.merged(ChatOptions(temperature=0.0, guided_regex="[0-9]+", extra={"ntokens": 64}))
    assert (m.temperature, m.max_tokens, m.guided_regex, [t.name for t in m.tools]) == (0.0, 16, "[0-9]+", ["add"])
    f = m.request_fields()
    assert f["tools"][0]["function"]["name"] == "add" and f["cache_salt"] == "s" and f["ntokens"] == 64 and "top_p" not in f

    class FakeClient:
        def __init__(self):
            self.calls = []

        def chat(self, messages, **params):
            self.calls.append((messages, params))
            if len(self.calls) == 1:
                return {"choices": [{"message": {"role": "assistant", "content": "", "tool_calls": [
                    {"id": "call_101", "type": "function", "function": {"name": "add", "arguments": "{\"a\": 2, \"b\": 40}"}}]}, "finish_reason": "tool_calls"}]}
            return {"choices": [{"message": {"role": "assistant", "content": "It is 42.", "reasoning_content": "tool said 42"}, "finish_reason": "stop"}],
                    "usage": {"completion_tokens": 4}}

        def stream_chat(self, messages, **params):
            yield "content", "hi"
            yield "finish", "stop"

    fc = FakeClient()
    hm = HttpChatModel(client=fc, defaults=base)
    r = hm.call([{"role": "user", "content": "2+40?"}])
    assert (r.content, r.reasoning, r.finish_reason, r.usage) == ("It is 42.", "tool said 42", "stop", {"completion_tokens": 4})
    assert fc.calls[1][0][-1] == {"role": "tool", "tool_call_id": "call_101", "name": "add", "content": "42"} and fc.calls[1][0][-2]["tool_calls"]
    assert r.messages[-1] == {"role": "assistant", "content": "It is 42."} and list(hm.stream([{"role": "user", "content": "x"}])) == [("content", "hi"), ("finish", "stop")]
    fc2 = FakeClient()
    r2 = HttpChatModel(client=fc2).call([{"role": "user", "content": "q"}])  # no callback for "add": the call is handed to the caller
    assert r2.tool_calls and r2.finish_reason == "tool_calls" and len(fc2.calls) == 1

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=5, std=0.08, max_position_embeddings=1024)
    em = EmbeddedChatModel(AutoModelForCausalLM.from_pretrained(d, device="cpu"), ChatOptions(max_tokens=8, temperature=0.0))
    r = em.call([{"role": "system", "content": "s"}, {"role": "user", "content": "number?"}], ChatOptions(guided_regex="[0-9]{3}"))
    assert __import__("re").fullmatch("[0-9]{3}", r.content) and r.usage["completion_tokens"] >= 3
    ev = list(em.stream([{"role": "user", "content": "hello"}], ChatOptions(max_tokens=5)))
    assert ev[-1] == ("finish", "length") and sum(1 for k, _ in ev if k == "content") >= 1
    with pytest.raises(ValueError):
        em.call([{"role": "user", "content": "x"}], ChatOptions(extra={"nope": 1}))


def test_tokenizer_benchmark_and_upload_plan(tmp_path, capsys):
    from deliverance_b200.ckpt import upload
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.tokenizer import benchmark as tb
    from deliverance_b200.tokenizer.auto import AutoTokenizer

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=1)
    r = tb.run(AutoTokenizer.from_pretrained(d), tb.DEFAULT_TEXT, warmup=1, iterations=3)
    assert r["incremental_equals_decode"] and r["tokens"] > 0 and len(r["ids_sha256"]) == 64 and r["tokens_s"] > 0
    assert tb.ids_sha256([1, 2, -1]) == __import__("hashlib").sha256(bytes([0, 0, 0, 1, 0, 0, 0, 2, 255, 255, 255, 255])).hexdigest()
    assert [p for p, _ in upload.plan(d)] == ["config.json", "model.safetensors"]
    assert upload.main(["me/tiny", d, "--dry-run"]) == 0 and "2 files" in capsys.readouterr().out
    open(os.path.join(d, "deliverance-quantization.json"), "w").write("{}")
    with pytest.raises(RuntimeError):
        upload.plan(d)
    open(os.path.join(d, ".finished"), "w").close()
    assert "deliverance-quantization.json" in [p for p, _ in upload.plan(d)] and ".finished" not in [p for p, _ in upload.plan(d)]


def test_model_support_facade(tmp_path):
    from deliverance_b200 import model_support as ms
    from deliverance_b200.ckpt.tiny import write_tiny_model

    d, b = str(tmp_path / "llama"), str(tmp_path / "bert")
    write_tiny_model(d, "llama", seed=1)
    write_tiny_model(b, "bert", seed=2)
    assert ms.detect_model(d) == "llama" and ms.detect_model(os.path.join(b, "config.json")) == "bert"
    t = ms.InferenceType
    assert t.parse("generation") is t.FULL_GENERATION and t.parse("FULL_EMBEDDING").is_pooling and not t.FORWARD_PASS.is_output
    assert t.FULL_CLASSIFICATION.is_classify and t.OUTPUT_TO_TOKEN.is_output and not t.OUTPUT_TO_TOKEN.is_input
    clm = ms.load_model(d, device="cpu")
    assert clm.generate([3, 4, 5], None).generated_tokens > 0
    emb = ms.load_model(b, t.FULL_EMBEDDING, device="cpu")
    assert len(emb.embed("hello world")) == 64
    assert len(ms.load_model(d, t.FULL_EMBEDDING, device="cpu").embed("decoder as embedder")) == 64
    ms.add_model("llama", lambda model_dir, it, device, **kw: ("custom", it))
    try:
        assert ms.load_model(d, t.FORWARD_PASS) == ("custom", t.FORWARD_PASS)
    finally:
        ms._REGISTRY.clear()


def test_legacy_tokenizer_file_layouts(tmp_path):
    """Tokenizer directories without tokenizer.json: SentencePiece model, GPT-2 style vocab.json + merges.txt, BERT vocab.txt;
    each must agree with the transformers tokenizer of the same files."""
    import sentencepiece as spm

    from deliverance_b200.tokenizer.auto import AutoTokenizer, IncrementalDetokenizer

    text = "Hello world, hello tokenizers! The quick brown fox."
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join([text, "the quick brown fox jumps over the lazy dog", "hello hello world world tokenizers are quick"] * 20))
    sp_dir = tmp_path / "sp"
    sp_dir.mkdir()
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(sp_dir / "tokenizer"), vocab_size=60, model_type="bpe",
                                   bos_id=1, eos_id=2, unk_id=0, minloglevel=2)
    tok = AutoTokenizer.from_pretrained(str(sp_dir))
    ref = spm.SentencePieceProcessor(model_file=str(sp_dir / "tokenizer.model"))
    ids = tok.encode(text)
    assert ids == ref.encode(text) and tok.decode(ids) == ref.decode(ids) and (tok.bos_token, tok.eos_token) == ("<s>", "</s>")
    assert tok.bos_token_id == 1 and tok.is_special(2) and tok.decode([1] + ids[:3] + [2]).startswith("<s>") and tok.encode(text, add_special_tokens=True)[0] == 1
    det = IncrementalDetokenizer(tok, skip_special=True)
    assert "".join(det.push(i) for i in ids) == tok.decode(ids, skip_special_tokens=True)

    bpe_dir = tmp_path / "bpe"
    bpe_dir.mkdir()
    from tokenizers import ByteLevelBPETokenizer

    t = ByteLevelBPETokenizer()
    t.train([str(corpus)], vocab_size=300, min_frequency=1, special_tokens=["<|endoftext|>"])
    t.save_model(str(bpe_dir))
    tok = AutoTokenizer.from_pretrained(str(bpe_dir))
    hf = ByteLevelBPETokenizer(str(bpe_dir / "vocab.json"), str(bpe_dir / "merges.txt"))
    ids = tok.encode(text + " Ünïcödé")
    assert ids == hf.encode(text + " Ünïcödé").ids and tok.decode(ids) == text + " Ünïcödé" and tok.eos_token == "<|endoftext|>" and tok.is_special(tok.eos_token_id)

    wp_dir = tmp_path / "wp"
    wp_dir.mkdir()
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "hello", "world", "the", "quick", "brown", "fox", "token", "##izer", "##s", ",", "!", "."]
    (wp_dir / "vocab.txt").write_text("\n".join(words) + "\n")
    tok = AutoTokenizer.from_pretrained(str(wp_dir))
    from tokenizers import BertWordPieceTokenizer

    hf = BertWordPieceTokenizer(str(wp_dir / "vocab.txt"))
    assert tok.encode(text, add_special_tokens=True) == hf.encode(text).ids and tok.encode(text) == hf.encode(text, add_special_tokens=False).ids
    assert tok.decode(tok.encode("hello tokenizers")) == "hello tokenizers" and tok.pad_token == "[PAD]"


GUIDED_SUITE = [
    {"question_id": "guided-choice-nfl", "category": "guided_choice", "turns": ["Choose the better New York NFL football team."], "guided_choice": ["Giants", "Jets"]},
    {"question_id": "guided-regex-ticket", "category": "guided_regex", "turns": ["Create a support ticket identifier."], "guided_regex": "TICKET-[0-9]{4}"},
    {"question_id": "guided-regex-routing", "category": "guided_regex", "turns": ["Route a pet insurance request."], "guided_regex": "(cats|dogs|birds|fish)"},
    {"question_id": "guided-json-person", "category": "guided_json", "turns": ["Alice is 42 years old and lives in Paris."],
     "guided_json": {"type": "object", "properties": {"name": {"const": "Alice"}, "age": {"type": "integer"}, "city": {"const": "Paris"}},
                     "required": ["name", "age", "city"], "additionalProperties": False}},
    {"question_id": "guided-json-polymorphic-pet", "category": "guided_json", "turns": ["A vaccinated seven year old dog named Rex."],
     "guided_json": {"oneOf": [
         {"type": "object", "properties": {"kind": {"const": "cat"}, "name": {"const": "Misty"}, "lives_left": {"type": "integer"}}},
         {"type": "object", "properties": {"kind": {"const": "dog"}, "name": {"const": "Rex"}, "vaccinated": {"type": "boolean"}, "age": {"type": "integer"}}}]}},
    {"question_id": "guided-json-incident-report", "category": "guided_json", "turns": ["API latency was high in us-east."],
     "guided_json": {"type": "object", "properties": {
         "service": {"const": "api"}, "region": {"const": "us-east"}, "severity": {"enum": ["low", "medium", "high"]}, "impacted_users": {"type": "integer"},
         "mitigated": {"type": "boolean"}, "actions": {"type": "array", "items": {"enum": ["rollback", "scale_up", "restart", "notify"]}, "maxItems": 3}}}},
]


def test_guided_support_suite_through_the_benchmark(tmp_path):
    """The six cases of the reference's guided support suite (choice, two regexes, three JSON schemas incl. oneOf and an enum
    array), run through the single-request benchmark CLI on a tiny random model: every response must satisfy its constraint."""
    import csv
    import re
    import sys

    from deliverance_b200.bench import inference_benchmark as ib
    from deliverance_b200.ckpt.tiny import write_tiny_model

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=3, std=0.08, max_position_embeddings=1024)
    q = tmp_path / "suite.jsonl"
    q.write_text("\n".join(json.dumps(c) for c in GUIDED_SUITE) + "\n")
    assert [c[3] for c in ib.load_suite(str(q))][1] == {"guided_regex": "TICKET-[0-9]{4}"}
    out, jl = tmp_path / "out.csv", tmp_path / "out.jsonl"
    argv = sys.argv
    sys.argv = ["x", "--model", d, "--questions", str(q), "--max-tokens", "120", "--out", str(out), "--jsonl-output", str(jl), "--device", "cpu"]
    try:
        assert ib.main() == 0
    finally:
        sys.argv = argv
    rows = list(csv.DictReader(open(out)))
    texts = {json.loads(l)["case_id"]: json.loads(l)["response_text"] for l in open(jl)}
    assert [r["case_id"] for r in rows] == [c["question_id"] for c in GUIDED_SUITE]
    assert texts["guided-choice-nfl"] in ("Giants", "Jets") and re.fullmatch("TICKET-[0-9]{4}", texts["guided-regex-ticket"])
    assert texts["guided-regex-routing"] in ("cats", "dogs", "birds", "fish")
    from deliverance_b200.guided.index import RegexDFA
    from deliverance_b200.guided.json_schema import schema_to_regex

    finish = {r["case_id"]: r["finish_reason"] for r in rows}
    for case in GUIDED_SUITE[3:]:
        # a random model may write digits of an unbounded integer until max_tokens: then the text must still be a prefix the
        # schema's automaton accepts so far; a finished reply must parse and match
        cid, text = case["question_id"], texts[case["question_id"]]
        dfa = RegexDFA(schema_to_regex(case["guided_json"]))
        state, live = dfa.initial, dfa.live_states()
        for ch in text:
            state = dfa.step(state, ch)
            assert state is not None and state in live, (cid, text)
        if finish[cid] != "length":
            assert state in dfa.finals, (cid, text)
            obj = json.loads(text)
            if cid == "guided-json-person":
                assert list(obj) == ["name", "age", "city"] and obj["name"] == "Alice" and isinstance(obj["age"], int)
            elif cid == "guided-json-polymorphic-pet":
                assert (obj["kind"], obj["name"]) in (("cat", "Misty"), ("dog", "Rex"))
            else:
                assert obj["severity"] in ("low", "medium", "high") and set(obj["actions"]) <= {"rollback", "scale_up", "restart", "notify"}
    assert texts["guided-json-person"].startswith('{"name":"Alice","age":')


def test_builder_reference_methods_and_download_cache(tmp_path):
    """Builder methods of the reference that have no separate code path here are accepted and recorded; with_download resolves
    ``owner/name`` through the local model cache (a finished cache directory needs no network)."""
    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.params import GeneratorParameters

    home = tmp_path / "home"
    d = home / "acme_tiny-llama"
    write_tiny_model(str(d), "llama", seed=1)
    (d / ".finished").write_text("")
    b = (AutoModelForCausalLM.new_builder("acme/tiny-llama").with_device("cpu").with_download(True, str(home)).with_working_quant_type("I8")
         .with_gpu_prefill(True).with_gpu_decode(False).with_gpu_decode_attention(True).with_packed_prefill(True).with_tensor_runtime_mode("ENFORCE")
         .with_tensor_provider("simd").with_parallel_settings(None).with_tensor_plan_trace(False))
    clm = b.build()
    assert clm.name == "acme_tiny-llama" and clm.generate([3, 4, 5], GeneratorParameters(max_tokens=2)).generated_tokens == 2
    assert "workingQuantType=I8" in b.conf.ignored and "gpuDecode=False" in b.conf.ignored and len(b.conf.ignored) == 8
    assert AutoModelForCausalLM.new_builder(str(d)).with_tensor_plan_trace(True).conf.profile_stages
    with pytest.raises(ValueError):
        AutoModelForCausalLM.new_builder("no-slash").with_download().with_device("cpu").build()


def test_runner_isolates_engine_faults_and_oom(tmp_path):
    """A fault inside an engine step fails the requests in flight, returns their KV pages and leaves the server usable;
    a request that cannot fit into the KV pool fails alone with a message."""
    import threading

    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.params import GeneratorParameters
    from deliverance_b200.server.runner import EngineRunner

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=3, std=0.05, max_position_embeddings=1024)
    b = AutoModelForCausalLM.new_builder(d).with_device("cpu")
    b.conf.kv_pages = 8
    clm = b.build()
    clm.eos_ids, clm.engine.eos_ids = set(), frozenset((-1,))
    clm.engine.kv.settings.enabled = False
    runner = EngineRunner(clm)
    try:
        real_forward, boom = clm.model.forward, {"n": 0}

        def flaky(*a, **kw):
            boom["n"] += 1
            if boom["n"] == 3:
                raise RuntimeError("injected fault")
            return real_forward(*a, **kw)

        clm.model.forward = flaky
        errs = []

        def call(i):
            try:
                runner.generate(f"prompt {i}", GeneratorParameters(max_tokens=20), None, f"s{i}", 60)
            except Exception as e:  # noqa: BLE001
                errs.append(str(e))

        ths = [threading.Thread(target=call, args=(i,)) for i in range(3)]
        for t in ths:
            t.start()
        for t in ths:
            t.join(60)
        assert errs and all("injected fault" in e for e in errs)
        assert clm.engine.kv.allocator.available() == 7 and not clm.engine.has_work()
        assert runner.generate("after the fault", GeneratorParameters(max_tokens=3), None, "ok", 60).generated_tokens == 3
        with pytest.raises(Exception) as ei:  # 7 pages of 32 tokens cannot hold 300 tokens
            runner.generate("x" * 150, GeneratorParameters(max_tokens=200), None, "big", 60)
        assert "KV cache is too small" in str(ei.value)
        assert runner.generate("still fine", GeneratorParameters(max_tokens=3), None, "ok2", 60).generated_tokens == 3
        assert clm.engine.kv.allocator.available() == 7
    finally:
        runner.close()


def test_roofline_calculator(tmp_path):
    from deliverance_b200.bench import roofline as rf
    from deliverance_b200.ckpt.synthetic import SHAPES
    from deliverance_b200.config import parse_config

    cfg = parse_config(dict(SHAPES["qwen3-4b"]))
    c = rf.decode_step_cost(cfg, 64, 2048, "jq4", 1)
    # 36 layers x (2560 x 6144 + 4096 x 2560 + 3 x 2560 x 9728) weights + the 151936 x 2560 head, 0.625 bytes per element
    elems = 36 * (2560 * 6144 + 4096 * 2560 + 3 * 2560 * 9728) + 151936 * 2560
    assert abs(c.weight_bytes - elems * 0.625) < 1 and abs(c.kv_bytes - 64 * 36 * 2049 * 2 * 8 * 128 * 2) < 1 and c.nvlink_bytes == 0
    p = tmp_path / "peaks.json"
    p.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1400.0}))
    r = rf.report(cfg, 64, 2048, "jq4", 1, 6.0, str(p))
    assert r["bound"] == "hbm" and r["denominators"] == "of measured" and abs(r["target_ms"] - (c.hbm_bytes / 6e12 * 1e3)) < 1e-9
    assert abs(r["fraction"] - r["target_ms"] / 6.0) < 1e-12
    assert rf.load_peaks(str(tmp_path / "missing.json"))[1] == "fallback"
    c8 = rf.decode_step_cost(cfg, 64, 2048, "jq4", 8)
    assert abs(c8.weight_bytes - c.weight_bytes / 8) < 1 and c8.nvlink_bytes == 2 * 36 * 64 * 2560 * 2 * 7 and abs(c8.kv_bytes - c.kv_bytes / 8) < 1
    moe = parse_config(dict(SHAPES["mixtral-8x7b"]))
    m1, m64 = rf.decode_step_cost(moe, 1, 1024, "bf16", 1), rf.decode_step_cost(moe, 64, 1024, "bf16", 1)
    assert m1.weight_bytes < m64.weight_bytes  # one token touches two of the eight experts per layer
    g = parse_config(dict(SHAPES["gemma2-9b"]))
    assert rf.decode_step_cost(g, 1, 8000, "bf16", 1).kv_bytes < 42 * 8001 * 2 * 8 * 256 * 2  # sliding layers read at most the window


def test_runner_close_answers_waiting_callers(tmp_path):
    import threading
    import time

    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.params import GeneratorParameters
    from deliverance_b200.server.runner import EngineRunner

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=3, std=0.05, max_position_embeddings=4096)
    clm = AutoModelForCausalLM.from_pretrained(d, device="cpu")
    clm.eos_ids, clm.engine.eos_ids = set(), frozenset((-1,))
    runner = EngineRunner(clm)
    out = {}

    def call():
        try:
            out["r"] = runner.generate("long running request", GeneratorParameters(max_tokens=3000), None, "s", 120)
        except Exception as e:  # noqa: BLE001
            out["e"] = str(e)

    t = threading.Thread(target=call)
    t.start()
    while not clm.engine.running:
        time.sleep(0.01)
    runner.close()
    t.join(20)
    assert not t.is_alive() and "shutting down" in out.get("e", "") and not clm.engine.has_work()


def test_prefill_roofline_counts_every_matrix_and_half_the_attention():
    from deliverance_b200.bench.roofline import prefill_cost, prefill_report
    from deliverance_b200.ckpt.synthetic import SHAPES
    from deliverance_b200.config import parse_config

    cfg = parse_config(dict(SHAPES["qwen3-4b"]))
    c1, c2 = prefill_cost(cfg, 1, 1024), prefill_cost(cfg, 2, 1024)
    assert 1.99 < c2.flops / c1.flops < 2.01 and c1.nvlink_bytes == 0
    long = prefill_cost(cfg, 1, 2048)
    assert long.flops > 2 * c1.flops  # the attention term grows with the square of the prompt
    tp8 = prefill_cost(cfg, 64, 2048, tp=8)
    assert tp8.nvlink_bytes > 0 and abs(tp8.flops * 8 / prefill_cost(cfg, 64, 2048).flops - 1) < 0.02
    r = prefill_report(cfg, 64, 2048, "jq4", 1, measured_ms=1562.0)
    assert r["bound"] == "tensor" and 0.3 < r["fraction"] < 0.7


def test_lz4_block_format_golden_and_roundtrip():
    """The host LZ4 codec of the extension: hand-assembled blocks of the public block format decode to the expected bytes, and
    random / repetitive / empty inputs survive a round trip."""
    import os
    import random

    from deliverance_b200.ops.build import load_extension

    e = load_extension()
    if e is None:
        pytest.skip("extension not built")
    assert e.lz4_decompress(bytes([0x50]) + b"hello", 5) == b"hello"
    # 3 literals "abc", match offset 3 length 9 (overlapping copy), then a last sequence of one literal
    assert e.lz4_decompress(bytes([0x35]) + b"abc" + bytes([3, 0]) + bytes([0x10]) + b"d", 13) == b"abcabcabcabcd"
    with pytest.raises(RuntimeError):
        e.lz4_decompress(bytes([0x35]) + b"abc" + bytes([9, 0]), 12)  # offset reaches before the output start
    rnd = random.Random(3)
    for data in (b"", b"x", bytes(70000), os.urandom(3000), b"the quick brown fox " * 500 + os.urandom(17),
                 bytes(rnd.choice(b"abcd") for _ in range(30000))):
        c = e.lz4_compress(data)
        assert e.lz4_decompress(c, len(data)) == data
    assert len(e.lz4_compress(bytes(70000))) < 400


def test_guard_area_checker_on_host_memory():
    """The bounds-checking allocator of the extension: an output cut out between two guard areas, the checker passes while they are
    intact and names the output once a guard byte has changed (the change is made from the host)."""
    from deliverance_b200 import ops

    e = ops.ext()
    if e is None:
        pytest.skip("extension not built")
    e.set_bounds_check(True)
    try:
        like = torch.zeros(2, 8, dtype=torch.bfloat16)
        o = e.guarded_empty([5, 16], like)
        assert tuple(o.shape) == (5, 16) and o.dtype == torch.bfloat16
        o.fill_(1.0)
        assert e.check_guards() == []
        e.guarded_empty([3, 7], like)
        e.poke_last_guard()
        bad = e.check_guards()
        assert len(bad) == 1 and "[3, 7]" in bad[0]
    finally:
        e.set_bounds_check(False)
