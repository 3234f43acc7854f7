"""A GPT-2 inference engine for one NVIDIA B200, in the manner of mlx-lm.

``load``, ``generate``, ``stream_generate``, ``generate_step`` and ``batch_generate`` are the entry points
(mlx_lm/__init__.py:9-20); they are imported on first use so that configuration, weights and the
cache manager can be used without a CUDA device.
"""

__version__ = "0.1.0"

_API = {"load", "generate", "stream_generate", "generate_step", "batch_generate", "BatchGenerator",
        "GenerationResponse"}


def __getattr__(name):
    if name in _API:
        import importlib

        mod = importlib.import_module(__name__ + ".generate")
        for n in _API:     # as in mlx-lm, the name ``generate`` is the function, not the module
            globals()[n] = getattr(mod, n)
        return globals()[name]
    raise AttributeError(f"module 'mlx_lm_b200' has no attribute {name!r}")
