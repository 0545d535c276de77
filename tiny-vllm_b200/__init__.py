"""A single-GPU inference engine for dense Qwen3 decoders on NVIDIA B200 (sm_100a).

Model folder (config.json + safetensors, or random weights from a seed) to
generated tokens: typed configuration and an architecture registry, layers put
together from parts, a paged cache with block tables and state slots, one step
function over mixed batches, a continuous-batching scheduler, sampling, a
command line (``python -m tinyvllm_b200``) and trace replay (``bin/trace_run``).
Every hot operation is a CUDA kernel of this package; there is no CPU path.
"""

from .config.engine import EngineConfig
from .config.registry import (ConfigError, architecture_names, read_model_config,
                              register_architecture)
from .config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
from . import models as _models  # noqa: F401  (registers the architectures)
from .engine.engine import Engine, GenerateRequest, RequestOutput
from .engine.llm import LLM, TextOutput
from .sampling.params import SamplingParams

__all__ = ["Engine", "GenerateRequest", "LLM", "RequestOutput", "SamplingParams", "TextOutput",
           "ConfigError", "EngineConfig", "LayerSpec", "ModelSpec", "PartSpec", "RunStep",
           "architecture_names", "read_model_config", "register_architecture"]
