"""Typed-output facade over a generation model (the reference's Outlines-like ``sketches`` module:
sketches/src/main/java/io/teknek/sketches/Sketches.java, SketchesCoreLogitsProcessor.java, DeliveranceKernel.java).

    sk = Sketches(model)
    sk.choice("Is water wet? Answer:", ["yes", "no"])                 -> "yes"
    sk.regex("A US zip code:", r"[0-9]{5}")                           -> "12203"
    sk.json("Describe a cat as JSON:", {"type": "object", ...})       -> dict
    sk.typed("Describe a cat:", Cat)                                   -> Cat (a dataclass or pydantic model)

Every call is ordinary generation with one guided-decoding constraint (choice / regex / JSON schema), so the result always
parses; ``typed`` derives the schema from a dataclass or a pydantic model and builds the object.
"""
from __future__ import annotations

import dataclasses
import json
import typing
from typing import Any, Optional, Sequence

from .params import GeneratorParameters

_PRIMS = {str: {"type": "string"}, int: {"type": "integer"}, float: {"type": "number"}, bool: {"type": "boolean"}}


def schema_of(tp) -> dict:
    """JSON schema of a dataclass, a pydantic model class, or a plain type annotation."""
    if hasattr(tp, "model_json_schema"):
        return tp.model_json_schema()
    if tp in _PRIMS:
        return dict(_PRIMS[tp])
    origin = typing.get_origin(tp)
    if origin in (list, typing.List):
        (item,) = typing.get_args(tp) or (str,)
        return {"type": "array", "items": schema_of(item)}
    if origin is typing.Literal:
        return {"enum": list(typing.get_args(tp))}
    if dataclasses.is_dataclass(tp):
        hints = typing.get_type_hints(tp)
        props = {f.name: schema_of(hints[f.name]) for f in dataclasses.fields(tp)}
        return {"type": "object", "properties": props, "required": list(props), "additionalProperties": False}
    raise TypeError(f"cannot derive a JSON schema from {tp!r}")


class Sketches:
    def __init__(self, model, max_tokens: int = 256, temperature: float = 0.0, seed: int = 42):
        self.model = model
        self.defaults = dict(max_tokens=max_tokens, temperature=temperature, seed=seed)

    def _run(self, prompt: str, **guide) -> str:
        p = GeneratorParameters(**self.defaults, **guide)
        return self.model.generate(prompt, p).text

    def choice(self, prompt: str, options: Sequence[str]) -> str:
        return self._run(prompt, guided_choice=list(options))

    def regex(self, prompt: str, pattern: str) -> str:
        return self._run(prompt, guided_regex=pattern)

    def json(self, prompt: str, schema: dict) -> Any:
        return json.loads(self._run(prompt, guided_json=schema))

    def typed(self, prompt: str, tp, schema: Optional[dict] = None):
        data = self.json(prompt, schema or schema_of(tp))
        if hasattr(tp, "model_validate"):
            return tp.model_validate(data)
        if dataclasses.is_dataclass(tp):
            return tp(**data)
        return data
