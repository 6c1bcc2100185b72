"""B200-native LLM inference and serving framework with the capabilities of Deliverance."""
from .params import FinishReason, GeneratorParameters, Response  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("AutoModelForCausalLM", "AutoModelConfig", "CausalLanguageModel"):
        from . import api

        return getattr(api, name)
    if name in ("AutoModelForEmbeddings", "AutoModelForSequenceClassification", "PoolingType"):
        from . import embedding

        return getattr(embedding, name)
    raise AttributeError(name)
