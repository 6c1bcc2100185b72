"""JSON schemas of the HTTP API, attached to the routes so that ``GET /openapi.json`` is a complete, machine-readable
description from which clients can be generated (the reference ships a hand-written OpenAPI file and generates its Java
clients from it: web/deliverance_specification.yaml, client/, client-spring/). The schemas describe what ``server/app.py``
accepts and returns; fields it ignores are not listed.
"""
from __future__ import annotations

_NUM = {"type": "number"}
_INT = {"type": "integer"}
_STR = {"type": "string"}
_BOOL = {"type": "boolean"}

SAMPLING = {
    "model": {**_STR, "description": "name of a loaded generation model (default: the first one)"},
    "temperature": {**_NUM, "minimum": 0, "default": 0.0},
    "top_p": {**_NUM, "exclusiveMinimum": 0, "maximum": 1},
    "top_k": {**_NUM, "exclusiveMinimum": 0, "description": ">= 1: that many candidates; < 1: drop that fraction of the vocabulary"},
    "uniform_top_p": {**_NUM, "exclusiveMinimum": 0, "maximum": 1, "description": "uniform pick inside the top_p nucleus (needs top_p and temperature > 0)"},
    "xtc_threshold": _NUM, "xtc_probability": _NUM,
    "max_tokens": {**_INT, "minimum": 1}, "ntokens": {**_INT, "description": "absolute position limit (prompt + generated)"},
    "seed": _INT, "stop": {"oneOf": [_STR, {"type": "array", "items": _STR}]}, "include_stop_str_in_output": _BOOL,
    "logprobs": _BOOL, "top_logprobs": {**_INT, "minimum": 0, "maximum": 20},
    "guided_regex": _STR, "guided_json": {"type": "object", "description": "JSON schema the reply must satisfy"},
    "guided_choice": {"type": "array", "items": _STR}, "cache_salt": _STR, "n": {**_INT, "enum": [1]},
    "stream": _BOOL, "stream_options": {"type": "object", "properties": {"include_usage": _BOOL}},
}

TOOL = {"type": "object", "required": ["type", "function"], "properties": {
    "type": {"enum": ["function"]},
    "function": {"type": "object", "required": ["name"], "properties": {"name": _STR, "description": _STR, "parameters": {"type": "object"}}}}}
TOOL_CALL = {"type": "object", "properties": {"id": _STR, "type": {"enum": ["function"]}, "index": _INT,
                                              "function": {"type": "object", "properties": {"name": _STR, "arguments": {**_STR, "description": "JSON text"}}}}}
MESSAGE = {"type": "object", "required": ["role"], "properties": {
    "role": {"enum": ["system", "developer", "user", "assistant", "tool", "function"]},
    "content": {"oneOf": [_STR, {"type": "null"}, {"type": "array", "items": {"type": "object", "properties": {"type": {"enum": ["text"]}, "text": _STR}}}]},
    "tool_calls": {"type": "array", "items": TOOL_CALL}, "tool_call_id": _STR, "name": _STR}}
USAGE = {"type": "object", "properties": {"prompt_tokens": _INT, "completion_tokens": _INT, "total_tokens": _INT}}
LOGPROBS = {"type": "object", "properties": {"content": {"type": "array", "items": {"type": "object", "properties": {
    "token": _STR, "logprob": _NUM, "top_logprobs": {"type": "array", "items": {"type": "object", "properties": {"token": _STR, "logprob": _NUM}}}}}}}}
ERROR = {"type": "object", "properties": {"error": {"type": "object", "properties": {"message": _STR, "type": _STR}}}}

CHAT_REQUEST = {"type": "object", "required": ["messages"], "properties": {
    **SAMPLING,
    "messages": {"type": "array", "minItems": 1, "items": MESSAGE},
    "tools": {"type": "array", "items": TOOL},
    "tool_choice": {"oneOf": [{"enum": ["auto", "none", "required"]}, {"type": "object", "properties": {"type": {"enum": ["function"]}, "function": {"type": "object", "properties": {"name": _STR}}}}]},
    "functions": {"type": "array", "items": {"type": "object"}, "description": "legacy form of tools"},
    "function_call": {"oneOf": [{"enum": ["auto", "none"]}, {"type": "object", "properties": {"name": _STR}}]},
    "response_format": {"type": "object", "properties": {"type": {"enum": ["json_schema"]}, "json_schema": {"type": "object", "properties": {"name": _STR, "schema": {"type": "object"}}}}},
    "chat_template": {**_STR, "description": "Jinja template that replaces the model's own"},
    "chat_template_kwargs": {"type": "object", "description": "extra template variables, e.g. enable_thinking"},
    "add_generation_prompt": _BOOL, "continue_final_message": _BOOL}}
ASSISTANT = {"type": "object", "properties": {"role": {"enum": ["assistant"]}, "content": _STR, "reasoning_content": _STR, "reasoning": _STR,
                                              "tool_calls": {"type": "array", "items": TOOL_CALL}}}
CHAT_RESPONSE = {"type": "object", "properties": {
    "id": _STR, "object": {"enum": ["chat.completion"]}, "created": _INT, "model": _STR, "usage": USAGE,
    "choices": {"type": "array", "items": {"type": "object", "properties": {
        "index": _INT, "message": ASSISTANT, "finish_reason": {"enum": ["stop", "length", "tool_calls"]}, "logprobs": {"oneOf": [LOGPROBS, {"type": "null"}]}}}}}}
CHAT_CHUNK = {"type": "object", "description": "one server-sent event (data: <json>); the stream ends with data: [DONE]", "properties": {
    "id": _STR, "object": {"enum": ["chat.completion.chunk"]}, "created": _INT, "model": _STR, "usage": USAGE,
    "choices": {"type": "array", "items": {"type": "object", "properties": {
        "index": _INT, "delta": ASSISTANT, "finish_reason": {"oneOf": [{"enum": ["stop", "length", "tool_calls"]}, {"type": "null"}]}}}}}}
COMPLETION_REQUEST = {"type": "object", "required": ["prompt"], "properties": {**SAMPLING, "prompt": {"oneOf": [_STR, {"type": "array", "items": _STR, "maxItems": 1}]}}}
COMPLETION_RESPONSE = {"type": "object", "properties": {
    "id": _STR, "object": {"enum": ["text_completion"]}, "created": _INT, "model": _STR, "usage": USAGE,
    "choices": {"type": "array", "items": {"type": "object", "properties": {"index": _INT, "text": _STR, "finish_reason": {"enum": ["stop", "length"]},
                                                                             "logprobs": {"oneOf": [LOGPROBS, {"type": "null"}]}}}}}}
EMBEDDING_REQUEST = {"type": "object", "required": ["input"], "properties": {"model": _STR, "input": {"oneOf": [_STR, {"type": "array", "items": _STR}]}}}
EMBEDDING_RESPONSE = {"type": "object", "properties": {"object": {"enum": ["list"]}, "model": _STR, "usage": USAGE, "data": {"type": "array", "items": {
    "type": "object", "properties": {"object": {"enum": ["embedding"]}, "index": _INT, "embedding": {"type": "array", "items": _NUM}}}}}}
MODELS_RESPONSE = {"type": "object", "properties": {"object": {"enum": ["list"]}, "data": {"type": "array", "items": {
    "type": "object", "properties": {"id": _STR, "object": {"enum": ["model"]}, "owned_by": _STR, "type": {"enum": ["generation", "embedding"]}}}}}}


def _json(schema: dict, description: str = "") -> dict:
    return {"description": description, "content": {"application/json": {"schema": schema}}}


def route_docs(kind: str) -> dict:
    """Keyword arguments for ``add_api_route``: request body and response schemas of one endpoint family."""
    session = {"X-Deliverance-Session": {"schema": _STR, "description": "echo of the request header, or a fresh id"}}
    bad = {"400": _json(ERROR, "malformed request or generation failure"), "429": _json(ERROR, "server at capacity (see Retry-After)")}
    if kind == "chat":
        ok = {"description": "a chat completion, or a stream of chat.completion.chunk events when stream is true", "headers": session,
              "content": {"application/json": {"schema": CHAT_RESPONSE}, "text/event-stream": {"schema": CHAT_CHUNK}}}
        return {"summary": "Chat completion", "openapi_extra": {"requestBody": {"required": True, **_json(CHAT_REQUEST)}}, "responses": {"200": ok, **bad}}
    if kind == "completions":
        ok = {"description": "a text completion, or a stream of text_completion events", "headers": session,
              "content": {"application/json": {"schema": COMPLETION_RESPONSE}, "text/event-stream": {"schema": COMPLETION_RESPONSE}}}
        return {"summary": "Raw-prompt completion", "openapi_extra": {"requestBody": {"required": True, **_json(COMPLETION_REQUEST)}}, "responses": {"200": ok, **bad}}
    if kind == "embeddings":
        return {"summary": "Text embeddings", "openapi_extra": {"requestBody": {"required": True, **_json(EMBEDDING_REQUEST)}},
                "responses": {"200": _json(EMBEDDING_RESPONSE, "one vector per input"), "400": bad["400"]}}
    if kind == "models":
        return {"summary": "Loaded models", "responses": {"200": _json(MODELS_RESPONSE, "generation and embedding models")}}
    raise KeyError(kind)
