"""kapel_b200: a small, whole inference engine for one GPU (sm_100a), after smallbard/kapel.

From a model folder (config.json, model.safetensors) to generated tokens: typed configuration
and registry (`config`), weights by name (`weights`), layer parts (`parts`), the paged cache
(`cache`), the step function, scheduler and generation (`engine`), sampling (`sampling`), and
hand-written CUDA kernels (`csrc`, called through `kernels`).
"""
__version__ = "0.1.0"


def __getattr__(name):
    # `Model` and the scheduler's records are imported on first use, so that importing the
    # package (for its configuration or cache classes, say) does not need torch.cuda.
    if name in ("Model", "KapelError"):
        from . import model

        return getattr(model, name)
    if name in ("Sampling",):
        from .sampling import Sampling

        return Sampling
    if name in ("Request", "Scheduler", "EngineOptions", "Event", "EngineStats"):
        from .engine import scheduler

        return getattr(scheduler, name)
    raise AttributeError(name)
