"""Legacy-style loading facade: ``detect_model`` / ``load_model`` / ``load_embedding_model`` / ``load_classifier_model`` and the
``InferenceType`` selector (reference: core/.../model/ModelSupport.java:71-342, AbstractModel.java:139-163).

In the reference ``InferenceType`` decides which sub-graphs a model instance loads (embedding table, layers, output head,
classifier, pooler), both for the kind of inference and for its older layer-split distribution scheme. Here it selects the
wrapper a model directory is loaded into; the partial types of the layer-split scheme (``INPUT_TO_EMBEDDING``,
``FORWARD_PASS``, ``OUTPUT_TO_TOKEN``) map onto the full generation model, because tensor parallelism splits every layer across
ranks instead of giving ranks different layers.
"""
from __future__ import annotations

import enum
import json
import os
from typing import Callable, Optional


class InferenceType(enum.Enum):
    # (input embedding, layers, output head, classifier, pooling)
    INPUT_TO_EMBEDDING = (True, False, False, False, False)
    OUTPUT_TO_TOKEN = (False, False, True, False, False)
    FORWARD_PASS = (True, True, False, False, False)
    FULL_GENERATION = (True, True, True, False, False)
    FULL_CLASSIFICATION = (True, True, False, True, True)
    FULL_EMBEDDING = (True, True, False, False, True)

    @property
    def is_input(self) -> bool:
        return self.value[0]

    @property
    def is_fwd_pass(self) -> bool:
        return self.value[1]

    @property
    def is_output(self) -> bool:
        return self.value[2]

    @property
    def is_classify(self) -> bool:
        return self.value[3]

    @property
    def is_pooling(self) -> bool:
        return self.value[4]

    @staticmethod
    def parse(name: str) -> "InferenceType":
        """Accepts the enum names and the short forms of the server configuration (GENERATION / EMBEDDING / CLASSIFICATION)."""
        n = name.strip().upper()
        n = {"GENERATION": "FULL_GENERATION", "EMBEDDING": "FULL_EMBEDDING", "CLASSIFICATION": "FULL_CLASSIFICATION"}.get(n, n)
        return InferenceType[n]


_REGISTRY: dict[str, Callable] = {}


def add_model(model_type: str, loader: Callable) -> None:
    """Register ``loader(model_dir, inference_type, device, **kw) -> model`` for a ``model_type`` this package does not know."""
    _REGISTRY[model_type.lower()] = loader


def detect_model(model_dir_or_config: str) -> str:
    """``model_type`` of a model directory (or of a ``config.json`` path)."""
    p = model_dir_or_config
    if os.path.isdir(p):
        p = os.path.join(p, "config.json")
    with open(p) as f:
        d = json.load(f)
    mt = d.get("model_type")
    if not mt:
        raise ValueError(f"{p} has no model_type")
    return str(mt).lower()


def load_model(model_dir: str, inference_type: InferenceType = InferenceType.FULL_GENERATION, device: str = "auto",
               output_head_quantization: Optional[str] = None, lora_adapter: Optional[str] = None, **kw):
    mt = detect_model(model_dir)
    if mt in _REGISTRY:
        return _REGISTRY[mt](model_dir, inference_type, device, **kw)
    if inference_type is InferenceType.FULL_EMBEDDING:
        return load_embedding_model(model_dir, device)
    if inference_type is InferenceType.FULL_CLASSIFICATION:
        return load_classifier_model(model_dir, device)
    from .api import AutoModelForCausalLM

    b = AutoModelForCausalLM.new_builder(model_dir).with_device(device)
    if output_head_quantization:
        b = b.with_output_head_quantization(output_head_quantization)
    if lora_adapter:
        b = b.with_lora_adapter(lora_adapter)
    return b.build()


def load_embedding_model(model_dir: str, device: str = "auto"):
    from .embedding import AutoModelForEmbeddings

    return AutoModelForEmbeddings.from_pretrained(model_dir, device)


def load_classifier_model(model_dir: str, device: str = "auto"):
    from .embedding import AutoModelForSequenceClassification

    return AutoModelForSequenceClassification.from_pretrained(model_dir, device)
