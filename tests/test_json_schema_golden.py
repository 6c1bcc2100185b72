"""Behavioural golden vectors of the reference's JSON-schema -> regex builder
(sketches-core/src/test/java/io/teknek/sketches/json/JsonSchemaRegexBuilderTest.java), checked against ``schema_to_regex``:
tight structural JSON by default, strings without raw control characters, array item bounds, string length bounds that count
escape sequences as one character, enum / const, anyOf / oneOf, nested objects; every regex must also compile to a DFA."""
import json
import re

import pytest

from deliverance_b200.guided.json_schema import schema_to_regex, validate_regex


def full(rx, text):
    return re.fullmatch(rx, text, flags=re.DOTALL) is not None


def build(schema):
    rx = schema_to_regex(schema if isinstance(schema, dict) else json.loads(schema))
    validate_regex(rx)  # compiles with the automaton library used for guided decoding
    return rx


def test_object_is_tight_json():
    rx = build({"type": "object", "properties": {"foo": {"type": "integer"}, "bar": {"type": "string"}}, "required": ["foo", "bar"]})
    assert full(rx, '{"foo":4,"bar":"baz    baz baz bar"}')
    assert not full(rx, '{"foo" : 4 ,"bar":"baz    baz baz bar"}')
    rx = build({"type": "object", "properties": {"places": {"type": "array", "items": {"type": "string"}}}, "required": ["places"]})
    assert full(rx, '{"places":[]}')
    for bad in ('{"places" :[]}', '{"places": []}', '{"places" n:[]}'):
        assert not full(rx, bad)


def test_strings_reject_raw_control_characters_and_accept_escapes():
    rx = build({"type": "string"})
    for bad in ('"bad\nvalue"', '"bad\tvalue"', '"bad\rvalue"', '"bad\x01value"', '"bad\\xvalue"', '"bad\\u12xz"'):
        assert not full(rx, bad), bad
    for good in ('"bad\\nvalue"', '"bad\\tvalue"', '"say \\"hi\\""', '"path \\\\tmp"', '"snowman \\u2603"', '"hello\\nworld"'):
        assert full(rx, good), good


def test_nested_objects_and_arrays():
    rx = build({"type": "object", "properties": {"outer": {"type": "object", "properties": {"inner": {"type": "integer"}}, "required": ["inner"]}},
                "required": ["outer"]})
    assert full(rx, '{"outer":{"inner":7}}')
    rx = build({"type": "array", "items": {"type": "integer"}})
    assert full(rx, "[]") and full(rx, "[1,2,-3]")


def test_array_item_bounds():
    rx = build({"type": "array", "minItems": 2, "maxItems": 3, "items": {"type": "integer"}})
    assert [full(rx, t) for t in ("[]", "[1]", "[1,2]", "[1,2,3]", "[1,2,3,4]")] == [False, False, True, True, False]
    rx = build({"type": "array", "minItems": 2, "maxItems": 2, "items": {"type": "string", "maxLength": 4}})
    assert [full(rx, t) for t in ("[]", '["a"]', '["a","bc"]', '["a","bc","d"]', '["aaaaa","bc"]')] == [False, False, True, False, False]


def test_string_length_and_pattern():
    rx = build({"type": "string", "maxLength": 5})
    assert full(rx, '""') and full(rx, '"abcde"') and not full(rx, '"abcdef"')
    rx = build({"type": "string", "maxLength": 2})  # an escape sequence counts as one character
    assert full(rx, '"ab"') and full(rx, '"\\na"') and full(rx, '"\\u2603a"') and not full(rx, '"abc"') and not full(rx, '"\\nab"')
    rx = build({"type": "string", "pattern": "[A-Za-z][A-Za-z ]{0,39}"})
    assert full(rx, '"cheese"') and full(rx, '"ice cream"')
    for bad in ('"} food"', '",ledger"', '"西里"'):
        assert not full(rx, bad)
    rx = build({"type": "object", "properties": {"whyCluesMatter": {"type": "string", "maxLength": 12}}, "required": ["whyCluesMatter"]})
    assert full(rx, '{"whyCluesMatter":"short"}') and not full(rx, '{"whyCluesMatter":"methodClueMattersMistakeClue"}')


def test_enum_const_anyof_oneof():
    rx = build({"enum": ["red", "blue", 7, True, None]})
    assert all(full(rx, t) for t in ('"red"', "7", "true", "null")) and not full(rx, '"green"')
    assert full(build({"const": "fixed"}), '"fixed"')
    rx = build({"anyOf": [{"type": "integer"}, {"const": "unknown"}]})
    assert full(rx, "42") and full(rx, '"unknown"')
    rx = build({"oneOf": [{"type": "boolean"}, {"type": "null"}]})
    assert full(rx, "false") and full(rx, "null")


def test_primitives():
    assert full(build({"type": "null"}), "null")
    assert full(build({"type": "boolean"}), "true") and full(build({"type": "boolean"}), "false")
    assert full(build({"type": "integer"}), "-42") and not full(build({"type": "integer"}), "4.2")
    assert full(build({"type": "number"}), "3.14e10")
    for fmt, val in (("date", "2026-07-12"), ("date-time", "2026-07-12T10:30:00Z"), ("email", "a@example.com"), ("uri", "https://example.com"),
                     ("uuid", "123e4567-e89b-12d3-a456-426614174000")):
        assert full(build({"type": "string", "format": fmt}), '"' + val + '"'), fmt


def test_large_case_schema_compiles():
    s = {"type": "string"}
    schema = {"type": "object", "additionalProperties": False, "required": ["caseTitle", "suspect", "setting", "clues", "hiddenTruth"],
              "properties": {"caseTitle": s, "suspect": s, "setting": s, "clues": {"type": "array", "minItems": 3, "maxItems": 3, "items": s},
                             "hiddenTruth": {"type": "object", "additionalProperties": False,
                                             "required": ["crime", "motive", "method", "mistakes", "whyCluesMatter", "confession"],
                                             "properties": {"crime": s, "motive": s, "method": s, "mistakes": {"type": "array", "items": s},
                                                            "whyCluesMatter": {"type": "array", "items": s}, "confession": s}}}}
    build(schema)


def test_invalid_schema_text_is_rejected():
    with pytest.raises((ValueError, TypeError)):
        schema_to_regex("{not json")
