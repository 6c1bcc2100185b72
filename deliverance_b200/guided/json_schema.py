"""JSON schema -> regular expression for guided JSON decoding.

Same coverage as the reference builder (sketches-core/src/main/java/io/teknek/sketches/json/JsonSchemaRegexBuilder.java:
22-38,59-196): ``const`` / ``enum`` literals, ``anyOf`` / ``oneOf`` alternation, ``object`` (ALL ``properties`` in schema
order, all required, no whitespace), ``string`` (JSON string, or ``pattern``, or ``{0,maxLength}``), ``integer``, ``number``,
``boolean``, ``null``, ``array`` (``items`` with optional ``minItems`` / ``maxItems``). ``required``, ``additionalProperties``,
``$ref``, ``minLength`` and numeric bounds are not supported and raise or are ignored exactly as listed there.
"""
from __future__ import annotations

import json
import re

STRING_INNER = r'([^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'
STRING = '"' + STRING_INNER + '*"'
INTEGER = r"-?(0|[1-9][0-9]*)"
NUMBER = INTEGER + r"(\.[0-9]+)?([eE][+-]?[0-9]+)?"
BOOLEAN = r"(true|false)"
NULL = r"null"
_SPECIAL = set(".^$*+?{}[]\\|()")


def escape_literal(text: str) -> str:
    return "".join("\\" + c if c in _SPECIAL else c for c in text)


def _literal(value) -> str:
    return escape_literal(json.dumps(value, ensure_ascii=False, separators=(",", ":")))


def schema_to_regex(schema, max_array_items: int = 8) -> str:
    if isinstance(schema, str):
        schema = json.loads(schema)
    if not isinstance(schema, dict):
        raise ValueError("a JSON schema must be an object")
    if "$ref" in schema:
        raise ValueError("$ref is not supported")
    if "const" in schema:
        return _literal(schema["const"])
    if "enum" in schema:
        return "(" + "|".join(_literal(v) for v in schema["enum"]) + ")"
    for key in ("anyOf", "oneOf"):
        if key in schema:
            return "(" + "|".join(schema_to_regex(s, max_array_items) for s in schema[key]) + ")"
    t = schema.get("type")
    if isinstance(t, list):
        return "(" + "|".join(schema_to_regex({**schema, "type": x}, max_array_items) for x in t) + ")"
    if t == "object" or (t is None and "properties" in schema):
        props = schema.get("properties") or {}
        parts = [escape_literal(json.dumps(k, ensure_ascii=False)) + ":" + schema_to_regex(v, max_array_items) for k, v in props.items()]
        return r"\{" + ",".join(parts) + r"\}"
    if t == "string":
        if "pattern" in schema:
            pat = schema["pattern"]
            pat = pat[1:] if pat.startswith("^") else pat
            pat = pat[:-1] if pat.endswith("$") and not pat.endswith("\\$") else pat
            return '"' + pat + '"'
        if "maxLength" in schema:
            return '"' + STRING_INNER + "{0," + str(int(schema["maxLength"])) + '}"'
        return STRING
    if t == "integer":
        return INTEGER
    if t == "number":
        return NUMBER
    if t == "boolean":
        return BOOLEAN
    if t == "null":
        return NULL
    if t == "array":
        item = schema_to_regex(schema.get("items") or {"type": "string"}, max_array_items)
        lo = int(schema.get("minItems", 0))
        hi = schema.get("maxItems")
        if hi is None:
            body = f"({item}(,{item})*)" if lo <= 1 else f"({item}(,{item}){{{lo - 1},}})"
            return r"\[" + (body if lo >= 1 else body + "?") + r"\]"
        hi = int(hi)
        if hi < lo:
            raise ValueError("maxItems < minItems")
        alts = []
        for n in range(lo, hi + 1):
            alts.append("" if n == 0 else item + ("(," + item + "){" + str(n - 1) + "}" if n > 1 else ""))
        return r"\[(" + "|".join(alts) + r")\]"
    raise ValueError(f"unsupported schema: {json.dumps(schema)[:120]}")


def validate_regex(pattern: str) -> None:
    re.compile(pattern)
