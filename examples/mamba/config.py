"""Configuration of the Mamba example (capability parity: reference examples/mamba/config.py).

``MambaModelConfig`` describes the architecture, ``MambaInit`` its initialisation, and ``MambaConfig`` is the framework's
``Config`` whose ``model`` section carries the two.  ``DistributedTrainer`` reads it with
``config_class=MambaConfig, model_config_class=MambaModelConfig``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Union

import torch

from nanotron_b200.config import Config, ExistingCheckpointInit
from nanotron_b200.config.utils_config import cast_str_to_torch_dtype


@dataclass
class MambaInit:
    initializer_range: float = 0.02
    rescale_prenorm_residual: bool = True
    n_residuals_per_layer: int = 1  # 2 for models with an MLP next to the mixer


@dataclass
class MambaModelConfig:
    is_mamba_config: bool = True  # discriminator in YAML files
    d_model: int = 2560
    num_hidden_layers: int = 64
    vocab_size: int = 50277
    ssm_cfg: Optional[dict] = None  # d_state, d_conv, expand, dt_rank, dt_min, dt_max, dt_init, dt_scale, dt_init_floor, conv_bias, bias
    rms_norm: bool = True
    residual_in_fp32: bool = True
    pad_vocab_size_multiple: int = 8
    rms_norm_eps: float = 1e-5
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    tie_word_embeddings: bool = True
    scan_chunk: int = 32  # steps the state-space scan handles at once
    # accepted so that configuration files of the reference example load: the parameter dtype comes from ``model.dtype``, and the
    # residual add is always done together with the norm
    dtype: Optional[str] = None
    fused_add_norm: bool = True

    def ssm(self) -> dict:
        """The mixer's hyper-parameters with their defaults filled in."""
        c = dict(d_state=16, d_conv=4, expand=2, dt_rank="auto", dt_min=0.001, dt_max=0.1, dt_init="random", dt_scale=1.0, dt_init_floor=1e-4, conv_bias=True, bias=False)
        c.update(self.ssm_cfg or {})
        if c["dt_rank"] == "auto":
            c["dt_rank"] = math.ceil(self.d_model / 16)
        return c

    @property
    def hidden_size(self) -> int:
        return self.d_model

    def __post_init__(self):
        if self.vocab_size % self.pad_vocab_size_multiple:
            self.vocab_size += self.pad_vocab_size_multiple - self.vocab_size % self.pad_vocab_size_multiple


@dataclass
class MambaModelArgs:
    model_config: MambaModelConfig
    init_method: Union[MambaInit, ExistingCheckpointInit] = field(default_factory=MambaInit)
    dtype: Optional[torch.dtype] = None
    make_vocab_size_divisible_by: int = 1
    ddp_bucket_cap_mb: int = 25

    def __post_init__(self):
        if self.dtype is None:
            self.dtype = torch.bfloat16
        if isinstance(self.dtype, str):
            self.dtype = cast_str_to_torch_dtype(self.dtype)
        if isinstance(self.model_config, dict):
            self.model_config = MambaModelConfig(**self.model_config)
        self.model_config._is_using_mup = False


@dataclass
class MambaConfig(Config):
    model: Optional[MambaModelArgs] = None
