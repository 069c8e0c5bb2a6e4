from nanotron_b200.config.config import *  # noqa: F401,F403
from nanotron_b200.config.config import (  # noqa: F401
    AdamWOptimizerArgs, BenchArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, KernelArgs,
    LoggingArgs, LRSchedulerArgs, MetricsLoggingArgs, ModelArgs, NanosetDatasetsArgs, OptimizerArgs,
    PretrainDatasetsArgs, ProfilerArgs, S3UploadArgs, SFTDatasetsArgs, SGDOptimizerArgs, TokenizerArgs, TokensArgs,
    get_config_from_dict, get_config_from_file, model_config_from_dict,
)
from nanotron_b200.config.lighteval_config import *  # noqa: F401,F403
from nanotron_b200.config.lighteval_config import GenerationArgs, LightEvalConfig  # noqa: F401
from nanotron_b200.config.models_config import *  # noqa: F401,F403
from nanotron_b200.config.models_config import (  # noqa: F401
    ExistingCheckpointInit, LlamaConfig, MoEConfig, NanotronConfigs, Qwen2Config, RandomInit, SpectralMupInit, Starcoder2Config,
)
from nanotron_b200.config.parallelism_config import ParallelismArgs  # noqa: F401
from nanotron_b200.config.utils_config import *  # noqa: F401,F403
from nanotron_b200.config.utils_config import InitScalingMethod, RecomputeGranularity, SamplerType, serialize  # noqa: F401
