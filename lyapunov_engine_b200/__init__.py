"""lyapunov_engine_b200: a small, whole LLM inference engine for one B200.

From a model folder (config.json, safetensors) or a seed to generated tokens:
typed configuration and an architecture registry, weights by tensor name,
layers assembled from parts, a paged cache with its manager, one step function
for mixed batches, a continuous scheduler, sampling on the device, a command
line (``lyapunov generate``) and trace replay (``bin/trace_run``).  All GPU work
is hand-written CUDA for sm_100a; there is no CPU path.
"""
from .engine.llm_engine import EngineConfig, LLMEngine, LoadedModel, RequestOutput, load_model
from .registry import known_architectures, register_architecture
from .sampling import SamplingParams
from .weights import write_random_model

__all__ = ["EngineConfig", "LLMEngine", "LoadedModel", "RequestOutput", "load_model", "SamplingParams",
           "register_architecture", "known_architectures", "write_random_model", "generate"]


def generate(model_dir: str, prompts, sampling_params=None, dtype="bfloat16", device="cuda:0", **engine_options):
    """Loads the model folder, generates for every prompt (lists of token ids)
    and returns the ``RequestOutput`` list."""
    engine = LLMEngine.from_pretrained(model_dir, dtype=dtype, device=device, **engine_options)
    return engine.generate(prompts, sampling_params)
