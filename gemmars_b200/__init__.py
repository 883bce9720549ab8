"""gemmars_b200: Qwen3 text generation on one NVIDIA B200, from token ids to the next token.

    from gemmars_b200 import Engine
    eng = Engine.load("/path/to/model", "dtype=bfloat16;max_batch=8")
    replies = eng.generate([[1, 2, 3], [4, 5]], max_tokens=16)
"""
__version__ = "0.1.0"

_LAZY = {
    "Engine": ("gemmars_b200.engine.engine", "Engine"),
    "EngineOptions": ("gemmars_b200.engine.engine", "EngineOptions"),
    "SamplingParams": ("gemmars_b200.sampling.sampler", "SamplingParams"),
    "build_model": ("gemmars_b200.engine.model", "build_model"),
    "Runner": ("gemmars_b200.engine.step", "Runner"),
    "StepItem": ("gemmars_b200.engine.step", "StepItem"),
    "write_random_model": ("gemmars_b200.weights.random_init", "write_random_model"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)
