"""flyweight_b200: a small, whole, single-GPU inference engine for LFM2 on NVIDIA B200.

    from flyweight_b200 import Model, SamplingConfig
    model = Model("model_dir", dtype="bfloat16")
    runtime = model.native_runtime(context_limit=4096, parallel_sequences=8)
    tokens = runtime.generate([1, 2, 3], max_tokens=16)
"""
__version__ = "0.1.0"

from .sampling.config import GREEDY, SamplingConfig  # noqa: E402


def __getattr__(name):
    # the engine pulls in torch and the CUDA library; load it on first use
    if name in ("Model", "Runtime", "GenerationResult", "EngineConfig"):
        from .engine import runtime as _runtime
        return getattr(_runtime, name)
    raise AttributeError(name)


__all__ = ["GREEDY", "SamplingConfig", "Model", "Runtime", "GenerationResult", "EngineConfig", "__version__"]
