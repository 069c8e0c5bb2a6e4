from nanotron_b200.serialize.main import *  # noqa: F401,F403
from nanotron_b200.serialize.main import load, parse_ckpt_path, save  # noqa: F401
from nanotron_b200.serialize.metadata import CheckpointMetadata, DataStageMetadata, TensorMetadata, TrainingMetadata, load_meta, save_meta  # noqa: F401
from nanotron_b200.serialize.optimizer import load_lr_scheduler, load_optimizer, save_lr_scheduler, save_optimizer  # noqa: F401
from nanotron_b200.serialize.random import load_random_states, save_random_states  # noqa: F401
from nanotron_b200.serialize.weights import load_weights, save_weights  # noqa: F401
