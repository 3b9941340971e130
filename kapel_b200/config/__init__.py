"""Typed configurations, the model-as-data records, and the architecture registry."""
from .gemma2 import ConfigError, Gemma2Config
from .registry import (
    architectures,
    config_class_for,
    config_from_dir,
    config_from_json,
    presets,
    read_config_file,
    register_architecture,
    unregister_architecture,
)
from .spec import (
    AttentionSpec,
    BlockSpec,
    EmbedSpec,
    GatedMLPSpec,
    HeadSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
    default_schedule,
)
