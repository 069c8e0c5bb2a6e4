"""Trainer of the Mamba example (capability parity: reference examples/mamba/trainer.py): the framework's ``DistributedTrainer``
with this example's config classes and model class plugged into its extension points."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from config import MambaConfig, MambaInit, MambaModelConfig  # noqa: E402
from mamba import MambaForTraining  # noqa: E402

from nanotron_b200 import logging  # noqa: E402
from nanotron_b200.config import ExistingCheckpointInit  # noqa: E402
from nanotron_b200.logging import log_rank  # noqa: E402
from nanotron_b200.serialize import load_weights  # noqa: E402
from nanotron_b200.trainer import DistributedTrainer  # noqa: E402

logger = logging.get_logger(__name__)


class MambaTrainer(DistributedTrainer):
    def __init__(self, config_or_config_file, config_class=MambaConfig, model_config_class=MambaModelConfig, model_class=MambaForTraining):
        super().__init__(config_or_config_file, config_class=config_class, model_config_class=model_config_class, model_class=model_class)

    def _load_model_checkpoint(self, model):
        init = self.config.model.init_method
        if self.init_checkpoint_path is not None or isinstance(init, ExistingCheckpointInit):
            return super()._load_model_checkpoint(model)
        assert isinstance(init, MambaInit), f"unsupported init method {init}"
        log_rank("Mamba initialisation (S4D-real A, log-uniform dt, depth-scaled output projections)", logger=logger, level=logging.INFO, rank=0)
        model.init_model_randomly(config=self.config)
        self._sync_initial_parameters(model)  # replicas start identical
        return model


__all__ = ["MambaTrainer", "load_weights"]
