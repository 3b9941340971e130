"""The step function, the model as built parts, the scheduler and generation."""
from .batch import StepBatch
from .model import ModelParts
from .step import PAGE_SIZE, Engine, StepEntry, parse_dtype, require_device
