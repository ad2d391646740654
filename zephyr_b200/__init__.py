"""zephyr_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

    from zephyr_b200 import Engine
    engine = Engine("/path/to/model", dtype="bfloat16")
    out = engine.generate([1, 2, 3], max_tokens=16, temperature=0.0)
    print(out.token_ids)

Importing the package needs neither a GPU nor the compiled kernels; building an ``Engine`` does.
"""

__version__ = "0.1.0"

_LAZY = {
    "Engine": "engine", "GenerationParams": "engine", "GenerationOutput": "engine", "KvCacheOptions": "engine",
    "PagedSchedulerConfig": "engine", "FinishReason": "engine", "RequestStatus": "engine", "ModelRunner": "engine",
    "StepEntry": "engine", "SamplingParams": "sampling", "Qwen3Config": "config", "load_model_config": "config",
    "register_architecture": "config", "write_random_model": "weights",
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib

        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = sorted(_LAZY)
