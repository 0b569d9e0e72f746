"""A small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) or seeded random weights to
generated tokens: typed configuration and architecture registry, strict weight
loading, a decoder assembled from parts, a paged cache manager, one step
function for every mix of prompt portions and decoded tokens, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels.
"""

__version__ = "0.1.0"

from .config import LlamaConfig, UnsupportedModelError, load_config, register_architecture  # noqa: E402,F401
from .weights import CheckpointError, write_model_dir  # noqa: E402,F401
from .engine import LLMEngine, Priority, SchedulerConfig, greedy_generate, load_model, random_model  # noqa: E402,F401
from .sampling import SamplingParams  # noqa: E402,F401
