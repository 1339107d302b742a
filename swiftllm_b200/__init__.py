"""swiftllm_b200 - B200-native (sm_100a) data plane for swiftLLM's `LlamaModel`.

Mirrors the reference package surface that belongs to the hot path:
    swiftllm_b200.EngineConfig, swiftllm_b200.LlamaModel           (swiftllm/__init__.py:2,9)
    swiftllm_b200.worker.kernels.*                                 (swiftllm/worker/kernels/*)
    swiftllm_b200.swiftllm_c.swap_blocks                           (csrc/ -> module swiftllm_c)
    swiftllm_b200.create_model(engine_config)                      picks the worker class from config.json (registry.py)
The control plane (Engine, Scheduler, API server, tokenizer) is out of scope; the unmodified reference Engine can
drive this LlamaModel.
"""
from swiftllm_b200.engine_config import EngineConfig
from swiftllm_b200.model_config import (BupozenModelConfig, BuzaraxModelConfig, LlamaModelConfig, NaforaxModelConfig,
                                        RivudraModelConfig)
from swiftllm_b200.registry import create_model, load_model_config
from swiftllm_b200.worker.bupozen_model import BupozenModel
from swiftllm_b200.worker.buzarax_model import BuzaraxModel
from swiftllm_b200.worker.model import LlamaModel
from swiftllm_b200.worker.naforax_model import NaforaxModel
from swiftllm_b200.worker.rivudra_model import RivudraModel

__all__ = ["EngineConfig", "LlamaModelConfig", "LlamaModel", "BupozenModelConfig", "BupozenModel", "RivudraModelConfig", "RivudraModel",
           "BuzaraxModelConfig", "BuzaraxModel", "NaforaxModelConfig", "NaforaxModel", "create_model",
           "load_model_config"]
