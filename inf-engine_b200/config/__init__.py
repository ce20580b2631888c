from .barerax import BareraxConfig
from .fovunex import FovunexConfig
from .gavatar import GavatarConfig
from .kipezen import KipezenConfig
from .llama import ConfigError, LlamaConfig
from .registry import (
    ARCHITECTURES,
    Architecture,
    detect_config,
    get_architecture,
    get_llama_config,
    get_preset,
    parse_config_dict,
    preset_names,
    register_architecture,
)
from .spec import (
    AttentionSpec,
    DifferentialAttentionSpec,
    LatentAttentionSpec,
    MinGRUSpec,
    ReinjectDecoderSpec,
    YarnScaling,
    BigramDecoderSpec,
    BlockSpec,
    FeedForwardSpec,
    GatedDeltaSpec,
    GatedLinearRecurrenceSpec,
    GatedMLPSpec,
    GeneralDeltaSpec,
    HeadNormSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    ParallelMixerSpec,
    PolyNormMLPSpec,
    PositionSpec,
    RopeScaling,
    RoutedExpertsSpec,
    ScheduleEntry,
    ShortConvSpec,
)
