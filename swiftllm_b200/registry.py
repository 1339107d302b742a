"""Model registry: which configuration class and which worker class serve a checkpoint, decided from its config.json.

    family      recognised by                               config class           worker class
    llama       "model_type": "llama"                       LlamaModelConfig       worker.model.LlamaModel
    bupozen     "architecture": "Bupozen"                   BupozenModelConfig     worker.bupozen_model.BupozenModel
    rivudra     "architecture": "Rivudra"                   RivudraModelConfig     worker.rivudra_model.RivudraModel
    buzarax     "architecture": "Buzarax"                   BuzaraxModelConfig     worker.buzarax_model.BuzaraxModel
    naforax     "architecture": "Naforax"                   NaforaxModelConfig     worker.naforax_model.NaforaxModel

Every worker class has the same public surface (load_weights, profile_num_blocks, init_kvcache_and_swap, forward /
forward_async with the prefill-chunks-then-decodes batch layout, free_seqs_resources), so schedulers, examples and
benchmarks are written once against `create_model`."""
from __future__ import annotations

import importlib
import json
import os
from typing import Optional

# family -> (detector(raw config) -> bool, "module:ConfigClass", "module:WorkerClass")
_FAMILIES = {
    "llama": (lambda raw: raw.get("model_type") == "llama",
              "swiftllm_b200.model_config:LlamaModelConfig", "swiftllm_b200.worker.model:LlamaModel"),
    "bupozen": (lambda raw: raw.get("architecture") == "Bupozen",
                "swiftllm_b200.model_config:BupozenModelConfig", "swiftllm_b200.worker.bupozen_model:BupozenModel"),
    "rivudra": (lambda raw: raw.get("architecture") == "Rivudra",
                "swiftllm_b200.model_config:RivudraModelConfig", "swiftllm_b200.worker.rivudra_model:RivudraModel"),
    "buzarax": (lambda raw: raw.get("architecture") == "Buzarax",
                "swiftllm_b200.model_config:BuzaraxModelConfig", "swiftllm_b200.worker.buzarax_model:BuzaraxModel"),
    "naforax": (lambda raw: raw.get("architecture") == "Naforax",
                "swiftllm_b200.model_config:NaforaxModelConfig", "swiftllm_b200.worker.naforax_model:NaforaxModel"),
}


def _resolve(path: str):
    mod, name = path.split(":")
    return getattr(importlib.import_module(mod), name)


def family_of(raw_config: dict) -> str:
    for name, (detect, _, _) in _FAMILIES.items():
        if detect(raw_config):
            return name
    raise ValueError("config.json matches no served model family (known: " + ", ".join(_FAMILIES) + ")")


def model_config_from_dict(raw_config: dict):
    return _resolve(_FAMILIES[family_of(raw_config)][1])(raw_config)


def load_model_config(model_path: str):
    with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
        return model_config_from_dict(json.load(f))


def model_class_for(model_config):
    return _resolve(_FAMILIES[model_config.family][2])


def create_model(engine_config, model_config: Optional[object] = None):
    """The worker for engine_config.model_path (or for an explicit model_config: synthetic-weight runs)."""
    if model_config is None:
        model_config = load_model_config(engine_config.model_path)
    return model_class_for(model_config)(engine_config, model_config)
