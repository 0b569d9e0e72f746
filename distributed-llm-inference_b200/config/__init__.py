from .llama import LlamaConfig, RopeConfig, UnsupportedModelError, llama_model_spec
from .registry import Architecture, load_config, register_architecture, resolve_architecture, unregister_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

__all__ = [
    "Architecture", "LayerSpec", "LlamaConfig", "ModelSpec", "PartSpec", "RopeConfig", "RunStep",
    "UnsupportedModelError", "llama_model_spec", "load_config", "register_architecture",
    "resolve_architecture", "unregister_architecture",
]
