"""`llava.model` on the B200 engine: the LLaMA/Vicuna LLaVA classes (the reference also exports an MPT variant,
llava/model/__init__.py:2, which is outside the north-star path) and the registry of every model family this package
serves, keyed by what a checkpoint's config.json calls itself (`model_type` of HF-style configurations, `architecture` of
layer-list decoders). Classes are imported on first use: a text-only model does not pay for the multimodal imports."""
import importlib
import json
import os

# name in config.json -> (module under llava.model, class)
MODEL_REGISTRY = {
    "llava": ("language_model.llava_llama", "LlavaLlamaForCausalLM"),
    "Katadra": ("language_model.katadra", "KatadraForCausalLM"),
    "Pefivik": ("language_model.pefivik", "PefivikForCausalLM"),
    "Fezuzen": ("language_model.fezuzen", "FezuzenForCausalLM"),
    "Sofopel": ("language_model.sofopel", "SofopelForCausalLM"),
}
_LAZY = {"LlavaLlamaForCausalLM": "language_model.llava_llama", "LlavaConfig": "language_model.llava_llama",
         "KatadraForCausalLM": "language_model.katadra", "KatadraConfig": "language_model.katadra",
         "PefivikForCausalLM": "language_model.pefivik", "PefivikConfig": "language_model.pefivik",
         "FezuzenForCausalLM": "language_model.fezuzen", "FezuzenConfig": "language_model.fezuzen",
         "SofopelForCausalLM": "language_model.sofopel", "SofopelConfig": "language_model.sofopel"}

__all__ = ["LlavaConfig", "LlavaLlamaForCausalLM", "KatadraConfig", "KatadraForCausalLM", "PefivikConfig", "PefivikForCausalLM", "FezuzenConfig",
           "FezuzenForCausalLM", "SofopelConfig", "SofopelForCausalLM", "MODEL_REGISTRY",
           "model_class_for"]


def __getattr__(name):
    if name in _LAZY:
        return getattr(importlib.import_module("." + _LAZY[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def model_class_for(model_path):
    """The class that serves the checkpoint directory `model_path`, chosen by its config.json."""
    with open(os.path.join(model_path, "config.json")) as f:
        cfg = json.load(f)
    name = cfg.get("architecture") or cfg.get("model_type")
    if name not in MODEL_REGISTRY:
        raise NotImplementedError(f"{model_path}: no model of this package serves {name!r} (known: {sorted(MODEL_REGISTRY)})")
    mod, cls = MODEL_REGISTRY[name]
    return getattr(importlib.import_module("." + mod, __name__), cls)
