"""Guided decoding automata, JSON-schema regexes, chat templates, tool-call parsers, reasoning splitter, tokenizer glue."""
import json
import re

import pytest

from deliverance_b200.guided.index import ChoiceGuide, Index, IndexGuide, LazyIndex, SketchesSettings, Vocabulary
from deliverance_b200.guided.json_schema import schema_to_regex
from deliverance_b200.prompt.chat import PromptBuilder, Tool, Function
from deliverance_b200.prompt.parsers import (LlamaToolCallParser, QwenToolCallParser, ReasoningTextSplitter, parser_for_model,
                                             split_reasoning)
from deliverance_b200.tokenizer.auto import ByteTokenizer, IncrementalDetokenizer, PreTrainedTokenizer


def _vocab():
    toks = {i + 3: chr(c) for i, c in enumerate(range(32, 127))}
    toks.update({200: "true", 201: "fal", 202: "se", 203: "12", 204: "", 205: '":'})
    return Vocabulary(toks, [2], 256), {v: k for k, v in toks.items()}


def test_lazy_index_walk_and_eos_only_in_accept():
    v, rev = _vocab()
    g = IndexGuide(LazyIndex(r"(true|false)", v))
    assert sorted(g.allowed_tokens()) == sorted([rev["t"], rev["f"], 200, 201])
    assert 204 not in g.allowed_tokens()  # empty-text tokens are never allowed
    g.accept(201)
    assert sorted(g.allowed_tokens()) == sorted([rev["s"], 202])
    g.accept(202)
    assert g.allowed_tokens() == [2]
    with pytest.raises(ValueError):
        g.accept(rev["x"])


def test_eager_index_limits():
    v, _ = _vocab()
    idx = Index(r"[0-9]{2}", v)
    assert len(idx.states) == 3
    with pytest.raises(ValueError):
        Index(r"[a-z]{40}", v, SketchesSettings(max_index_states=10))
    with pytest.raises(ValueError):
        LazyIndex("a" * 20, v, SketchesSettings(max_regex_length=10))


def test_choice_guide():
    c = ChoiceGuide([[5, 6], [5, 7, 8]], [2], 256)
    assert c.allowed_tokens() == [5]
    c.accept(5)
    assert c.allowed_tokens() == [6, 7] and not c.is_complete()
    c.accept(7)
    c.accept(8)
    assert c.is_complete() and c.allowed_tokens() == [2]


@pytest.mark.parametrize("schema,good,bad", [
    ({"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "string"}}}, ['{"a":-12,"b":"x\\n"}'], ['{"b":"x","a":1}', '{"a": 1,"b":"x"}']),
    ({"enum": ["red", 3, None]}, ['"red"', "3", "null"], ['"blue"']),
    ({"type": "array", "items": {"type": "boolean"}, "minItems": 1, "maxItems": 2}, ["[true]", "[true,false]"], ["[]", "[true,false,true]"]),
    ({"anyOf": [{"type": "number"}, {"const": "n/a"}]}, ["1.5e3", '"n/a"'], ['"x"']),
    ({"type": "string", "pattern": "^[a-z]{2}$"}, ['"ab"'], ['"abc"']),
    ({"type": "string", "maxLength": 2}, ['""', '"ab"'], ['"abc"']),
])
def test_json_schema_regex(schema, good, bad):
    rx = schema_to_regex(schema)
    for s in good:
        assert re.fullmatch(rx, s), (rx, s)
        json.loads(s)
    for s in bad:
        assert not re.fullmatch(rx, s), (rx, s)
    with pytest.raises(ValueError):
        schema_to_regex({"$ref": "#/x"})


def test_guided_json_walk_over_vocab():
    v, rev = _vocab()
    rx = schema_to_regex({"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}})
    g = IndexGuide(LazyIndex(rx, v))
    for ch in '{"ok":true,"n":12}':
        g.accept(rev[ch])
    assert g.index.is_final(g.state) and g.allowed_tokens() == [2]


def test_chatml_fallback_and_jinja():
    b = PromptBuilder().add_system("sys").add_user("hi")
    assert b.build().prompt == "<|im_start|>system\nsys<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    b = PromptBuilder().add_user("hi").with_kwargs({"enable_thinking": False})
    assert b.build().prompt.endswith("<think>\n\n</think>\n\n")
    t = PromptBuilder().add_user("q").add_tools([Tool(Function("get_weather", "w", {"type": "object"}))]).build()
    assert t.has_tools and "<tools>" in t.prompt and "get_weather" in t.prompt
    tpl = "{{ bos_token }}{% for m in messages[::-1] %}[{{ m.role }}:{{ m.content }}]{% endfor %}{% if add_generation_prompt %}>{% endif %}{% if tools %}T{% endif %}"
    p = PromptBuilder(tpl, "<s>").add_user("a").add_assistant("b").build().prompt
    assert p == "<s>[assistant:b][user:a]>"
    p = PromptBuilder().with_template("{{ messages[0].content | upper }}{{ custom }}").with_kwargs({"custom": "!"}).add_user("x").build().prompt
    assert p == "X!"
    with pytest.raises(ValueError):
        PromptBuilder().build()


def test_tool_call_parsers():
    q = QwenToolCallParser()
    text = 'Sure.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "note": "a}b"}}\n</tool_call>\n<tool_call>\n{"name": "t2", "arguments": {}}\n</tool_call>'
    calls = q.extract(text)
    assert [c.id for c in calls] == ["101", "102"] and calls[0].name == "get_weather" and calls[0].arguments["note"] == "a}b"
    assert q.strip(text) == "Sure."
    assert q.extract("no calls here") == []
    ll = LlamaToolCallParser()
    calls = ll.extract('<|start_header_id|>assistant<|end_header_id|>\n\n{"type": "function", "function": "lookup", "parameters": {"k": 1}}')
    assert calls[0].name == "lookup" and calls[0].arguments == {"k": 1}
    assert ll.should_end_turn("abc<|eot_id|>") and not ll.should_end_turn("abc")
    assert isinstance(parser_for_model("Qwen3-4B-JQ4"), QwenToolCallParser) and isinstance(parser_for_model("meta-llama/Llama-3.2-1B"), LlamaToolCallParser)


def test_reasoning_splitter_holds_back_partial_tags():
    s = ReasoningTextSplitter()
    outs = [s.accept(p) for p in ["<th", "ink>rea", "son</thi", "nk>ans", "wer <", "b>"]]
    c, r = s.flush()
    assert s.reasoning == "reason" and s.content == "answer <b>"
    assert outs[0] == ("", "") and outs[1] == ("", "rea")
    assert split_reasoning("<think>\nabc\n</think>\n\nfinal") == ("final", "abc")
    assert split_reasoning("plain") == ("plain", None)


def test_incremental_detokenizer_utf8():
    tk = PreTrainedTokenizer(ByteTokenizer(), {"bos_token": "<s>", "eos_token": "</s>"}, {"<s>": 1, "</s>": 2})
    d = IncrementalDetokenizer(tk, skip_special=True)
    ids = tk.encode("é!")
    assert len(ids) == 3
    pieces = [d.push(i) for i in ids + [2]]
    assert pieces == ["", "é", "!", ""] and d.text == "é!"
    assert tk.decode(tk.encode("héllo")) == "héllo"


def test_gemma4_tool_call_parser_vectors():
    """Golden vectors of the reference's Gemma4ToolCallParserTest (JSON arguments, the template's relaxed syntax, nesting)."""
    from deliverance_b200.prompt.parsers import Gemma4ToolCallParser, parser_for_model

    p = Gemma4ToolCallParser()
    c = p.extract('<|channel>thought\nNeed weather data<channel|><|tool_call>call:get_weather{"location":"Albany, NY","unit":"celsius"}<tool_call|>')
    assert len(c) == 1 and c[0].id == "101" and c[0].name == "get_weather" and c[0].arguments == {"location": "Albany, NY", "unit": "celsius"}
    c = p.extract('<|channel>thought\nx<channel|><|tool_call>call:get_current_temperature{detail_level:0,location:<|"|>Paris, France<|"|>,'
                  'unit:<|"|>celsius<|"|>}<tool_call|><|tool_response>')
    assert c[0].name == "get_current_temperature" and c[0].arguments == {"detail_level": 0, "location": "Paris, France", "unit": "celsius"}
    c = p.extract('<|tool_call>call:foo{bool_value:true,list_value:[<|"|>foo<|"|>,<|"|>bar<|"|>],null_value:null,number_value:1,'
                  'string_value:<|"|>foo<|"|>,struct_value:{foo:<|"|>bar<|"|>}}<tool_call|>')
    assert c[0].arguments == {"bool_value": True, "list_value": ["foo", "bar"], "null_value": None, "number_value": 1, "string_value": "foo",
                              "struct_value": {"foo": "bar"}}
    c = p.extract('<|tool_call>call:flight_searcher.get_weather{"location":"Albany, NY"}<tool_call|><|tool_call>call:b{x:2}<tool_call|>')
    assert [x.name for x in c] == ["flight_searcher.get_weather", "b"] and c[1].id == "102"
    assert p.should_end_turn("abc<tool_call|>") and not p.should_end_turn("abc")
    assert isinstance(parser_for_model("google/gemma-4-12b-it"), Gemma4ToolCallParser)


def test_reasoning_splitter_reference_vectors():
    """core/.../model/ReasoningTextSplitterTest.java: split tags across pieces, prompts that end inside <think>."""
    from deliverance_b200.prompt.parsers import ReasoningTextSplitter, prompt_ends_inside_reasoning, split_reasoning

    s = ReasoningTextSplitter()
    assert s.accept("<think>") == ("", "")
    assert s.accept("reason</") == ("", "reason")
    assert s.accept("think") == ("", "")
    assert s.accept(">answer") == ("answer", "")
    s = ReasoningTextSplitter(True)
    assert s.accept("I'll inspect files.") == ("", "I'll inspect files.")
    assert s.accept("</") == ("", "")
    assert s.accept("think>ArchiveController.java") == ("ArchiveController.java", "")
    assert prompt_ends_inside_reasoning("<|start_of_role|>assistant<|end_of_role|><think>\n")
    assert not prompt_ends_inside_reasoning("<|start_of_role|>assistant<|end_of_role|>")
    assert not prompt_ends_inside_reasoning("<think>x</think>\nassistant:")
    assert split_reasoning("plan the answer</think>\nfinal", True) == ("final", "plan the answer")


def test_gemma4_response_channels_reference_vectors():
    """Vectors of the reference's Gemma4ResponseParserTest plus the streaming splitter over the same markers."""
    from deliverance_b200.prompt.parsers import Gemma4ChannelSplitter, parse_gemma4_response

    assert parse_gemma4_response("<|channel>thought\nfirst reason second reason<channel|>Final answer",
                                 "thought\nfirst reason second reasonFinal answer") == ("Final answer", "first reason second reason")
    assert parse_gemma4_response("<|channel>thought\n<channel|>Final answer", "thought\nFinal answer") == ("Final answer", None)
    assert parse_gemma4_response("", "<|turn>plain<turn|>") == ("plain", None)
    assert parse_gemma4_response("<|channel>thought\nnever closed", "fallback text") == ("fallback text", None)
    sp = Gemma4ChannelSplitter()
    c = r = ""
    for piece in ["<|chan", "nel>thou", "ght\nwhy ", "not<chan", "nel|>Answer"]:
        dc, dr = sp.accept(piece)
        c, r = c + dc, r + dr
    dc, dr = sp.flush()
    assert (c + dc, r + dr) == ("Answer", "why not")


def test_hf_common_chat_template_behaviours():
    """The chat-template tests of transformers' common tokenizer suite that the reference ports (dummy template, raise_exception)
    and the ones it lists as unsupported there: loop controls, strftime_now, named template selection, continue_final_message."""
    import datetime

    dummy = "{% for message in messages %}{{message['role'] + message['content']}}{% endfor %}"
    p = PromptBuilder(dummy).add_system("system message").add_user("user message").add_assistant("assistant message").build().prompt
    assert p == "systemsystem messageuseruser messageassistantassistant message"
    with pytest.raises(Exception):
        PromptBuilder("{{ raise_exception('bad role') }}").add_user("hi").build()
    loop = "{%- for message in messages %}{%- if message.role == 'user' %}{{ message.content }}{%- break %}{%- endif %}{%- endfor %}"
    assert PromptBuilder(loop).add_system("s").add_user("first").add_user("second").build().prompt == "first"
    assert PromptBuilder("{{ strftime_now('%Y-%m-%d') }}").add_user("x").build().prompt == datetime.date.today().strftime("%Y-%m-%d")
    named = {"default": "D:{{ messages[0].content }}", "tool_use": "T:{{ messages[0].content }}", "rag": "R:{{ messages[0].content }}"}
    assert PromptBuilder(named).add_user("q").build().prompt == "D:q"
    assert PromptBuilder(named).add_user("q").add_tools([{"type": "function", "function": {"name": "f"}}]).build().prompt == "T:q"
    assert PromptBuilder([{"name": k, "template": v} for k, v in named.items()]).add_user("q").with_kwargs({"template_name": "rag"}).build().prompt == "R:q"
    with pytest.raises(ValueError):
        PromptBuilder(named).add_user("q").with_kwargs({"template_name": "nope"}).build()
    tpl = "{% for m in messages %}<|{{ m.role }}|>{{ m.content }}<|end|>\n{% endfor %}{% if add_generation_prompt %}<|assistant|>{% endif %}"
    b = PromptBuilder(tpl).add_user("hi").add_assistant('{"name": "')
    assert b.build().prompt.endswith('<|assistant|>{"name": "<|end|>\n<|assistant|>')
    assert b.continue_final_message().build().prompt == '<|user|>hi<|end|>\n<|assistant|>{"name": "'
    # an earlier message with the same text is not the cut point
    c = PromptBuilder(tpl).add_user("hi!").add_assistant("hi!").add_user("again").add_assistant("hi!").continue_final_message().build().prompt
    assert c == "<|user|>hi!<|end|>\n<|assistant|>hi!<|end|>\n<|user|>again<|end|>\n<|assistant|>hi!"
    assert PromptBuilder().add_user("q").add_assistant("The answer is").continue_final_message().build().prompt.endswith("<|im_start|>assistant\nThe answer is")


def test_special_text_view_equals_a_second_detokenizer(tmp_path):
    """The text-with-special-tokens view must equal a full second incremental detokeniser at every step, before and after the
    first special token, including multi-byte characters split over tokens."""
    import random

    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.tokenizer.auto import AutoTokenizer, IncrementalDetokenizer, SpecialTextView

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=1)
    tok = AutoTokenizer.from_pretrained(d)  # byte-level fallback: ids 1 / 2 are <s> / </s>
    rng = random.Random(3)
    text_ids = tok.encode("héllo wörld 你好 🙂 plain ascii tail")
    for specials_at in ([], [5], [0, 9, 10], [len(text_ids) - 1]):
        ids = list(text_ids)
        for p in specials_at:
            ids.insert(p, rng.choice([1, 2]))
        plain, ref = IncrementalDetokenizer(tok, skip_special=True), IncrementalDetokenizer(tok, skip_special=False)
        view = SpecialTextView(tok, plain)
        for t in ids:
            view.push(t)
            plain.push(t)
            ref.push(t)
            assert view.text == ref.text
        assert (view.own is None) == (not specials_at) and plain.text == "héllo wörld 你好 🙂 plain ascii tail"
