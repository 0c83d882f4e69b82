"""infer_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

Everything between a request's tokens and its next token: typed configuration and architecture
registry, safetensors weights, layers put together from parts, a paged cache manager, one step
function for mixed batches, a scheduler, sampling, and hand-written CUDA kernels underneath.
"""
__version__ = "0.1.0"


def __getattr__(name):
    # Lazy, so that importing the package (for the configuration or the cache manager alone) does not load torch kernels.
    if name in ("LLM", "GenerationEngine"):
        from .engine import generation
        return getattr(generation, name)
    if name in ("Engine", "StepEntry"):
        from . import engine
        return getattr(engine, name)
    if name in ("Request", "SampleParams", "Scheduler", "SchedulerConfig", "Completed", "StopReason"):
        from .engine import scheduler
        return getattr(scheduler, name)
    raise AttributeError(name)
