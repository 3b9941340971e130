"""kapel_b200: a small, whole inference engine for one GPU (sm_100a), after smallbard/kapel.

From a model folder (config.json, model.safetensors) to generated tokens: typed configuration
and registry (`config`), weights by name (`weights`), layer parts (`parts`), the paged cache
(`cache`), the step function, scheduler and generation (`engine`), sampling (`sampling`), and
hand-written CUDA kernels (`csrc`, called through `kernels`).
"""
__version__ = "0.1.0"
