"""A small model library with generation for one NVIDIA B200 (sm_100a): the Qwen3 dense decoder.

    from dryft_challenge_htn_2026_b200 import Engine
    eng = Engine("/path/to/model", dtype="bfloat16")
    for tokens in eng.generate([[1, 2, 3], [4, 5]], max_new_tokens=8):
        ...

Everything between a request's tokens and its next token: typed config and architecture registry
(``config``, ``registry``), safetensors weights and a random-weights mode (``weights``), parts and
blocks (``parts``), the paged cache (``cache``), the step function, generation loop and entry
point (``engine``), sampling (``sampling``) and the CUDA kernels (``csrc``).
"""
from .cache import Cache, CacheFull, KVRequest, StateRequest
from .config import ConfigError, ModelConfig, ModelSpec, Qwen3Config
from .engine import CausalLM, Engine, Runner, load_model, random_model
from .parts import Part, register_part
from .registry import architectures, config_from_dict, config_from_folder, register_architecture
from .sampling import SamplingParams
from .weights import WeightError, load_weights, write_random_model

__all__ = ["Cache", "CacheFull", "KVRequest", "StateRequest", "ConfigError", "ModelConfig", "ModelSpec", "Qwen3Config",
           "CausalLM", "Engine", "Runner", "load_model", "random_model", "Part", "register_part", "architectures",
           "config_from_dict", "config_from_folder", "register_architecture", "SamplingParams", "WeightError",
           "load_weights", "write_random_model"]
