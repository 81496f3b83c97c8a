"""Model graphs.  ``ModelBase.create(path, device)`` picks the class from
``general.architecture`` (TensorSharp.Models/ModelBase.cs:1991-2007)."""
from .base import ModelBase, ModelConfig, supported_architectures  # noqa: F401


def _load_all():
    import importlib
    for m in ("qwen3", "gptoss", "qwen35", "gemma", "nemotron", "mistral3"):
        try:
            importlib.import_module(f"{__name__}.{m}")
        except ModuleNotFoundError as exc:
            if exc.name != f"{__name__}.{m}":
                raise


_load_all()
