"""Checkpoint-level and tensor-level metadata (format parity: reference src/nanotron/serialize/metadata.py)."""
from __future__ import annotations

import dataclasses
import json
import re
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
from packaging.version import Version

from nanotron_b200 import distributed as dist
from nanotron_b200.constants import CHECKPOINT_FILE_NAME, CHECKPOINT_VERSION
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import SlicesPair


@dataclasses.dataclass
class DataStageMetadata:
    """consumed_train_samples / consumed_tokens_per_dataset_folder count within this stage only."""

    name: str
    start_training_step: int
    consumed_train_samples: int
    sequence_length: Optional[int] = None
    consumed_tokens_per_dataset_folder: Dict[str, int] = dataclasses.field(default_factory=dict)

    def __post_init__(self):
        if self.sequence_length is None:
            self.sequence_length = 4096

    def sanity_consumed_train_samples(self):
        assert self.consumed_train_samples * self.sequence_length == sum(self.consumed_tokens_per_dataset_folder.values()), (
            f"Mismatch between consumed samples and per-folder consumed tokens: {self.consumed_train_samples=} {self.sequence_length=} {self.consumed_tokens_per_dataset_folder=}"
        )

    @property
    def consumed_tokens_all_datasets(self):
        return sum(self.consumed_tokens_per_dataset_folder.values())


@dataclasses.dataclass
class TrainingMetadata:
    consumed_train_samples: int
    last_train_step: int
    consumed_tokens_total: Optional[int] = None
    last_stage_idx: Optional[int] = None
    data_stages: Optional[List[DataStageMetadata]] = None

    def __post_init__(self):
        if self.data_stages is not None:
            assert self.consumed_train_samples == sum(s.consumed_train_samples for s in self.data_stages), "Mismatch between the total consumed samples and the sum of consumed samples across stages! Something went wrong in the training."
            total = sum(s.consumed_tokens_all_datasets for s in self.data_stages)
            if self.consumed_tokens_total is not None and total > 0:
                assert self.consumed_tokens_total == total, "Mismatch between the total consumed tokens and the sum of consumed tokens across stages!"
            elif self.consumed_tokens_total is None:
                self.consumed_tokens_total = total
        if self.last_stage_idx is not None:
            assert self.data_stages is not None, "data_stages should not be None if last_stage_idx is not None"

    @property
    def consumed_tokens_per_dataset_folder_total(self):
        consumed = defaultdict(int)
        for stage in self.data_stages or []:
            for folder, tokens in stage.consumed_tokens_per_dataset_folder.items():
                consumed[folder] += tokens
        return consumed

    @property
    def current_stage(self) -> DataStageMetadata:
        return self.data_stages[self.last_stage_idx]


@dataclasses.dataclass
class CheckpointMetadata:
    version: Version
    tp: int
    dp: int
    metas: TrainingMetadata
    cp: int = 1
    custom_metas: Optional[Dict[str, Any]] = None


def _parse_shape(text: str) -> Tuple[int, ...]:
    out = []
    for piece in text.strip("()[] ").split(","):
        piece = piece.strip()
        if not piece:
            continue
        m = re.search(r"\((\d+)\)", piece)  # "np.int64(12)"
        out.append(int(m.group(1)) if m else int(piece))
    return tuple(out)


@dataclasses.dataclass
class TensorMetadata:
    """Stored as safetensors string metadata beside every parameter shard."""

    version: Version
    local_global_slices_pairs: Tuple[SlicesPair, ...]
    unsharded_shape: Tuple[int, ...]

    def to_str_dict(self) -> Dict[str, str]:
        return {
            "version": str(self.version),
            "local_global_slices_pairs": SlicesPair.tuple_to_str(self.local_global_slices_pairs),
            "unsharded_shape": str(tuple(int(s) for s in self.unsharded_shape)),
        }

    @classmethod
    def from_str_dict(cls, dictionary: Dict[str, str]) -> "TensorMetadata":
        extra = set(dictionary) - {"version", "local_global_slices_pairs", "unsharded_shape"}
        assert not extra, f"unknown tensor metadata keys {extra}"
        return cls(
            version=Version(dictionary["version"]),
            local_global_slices_pairs=SlicesPair.tuple_from_str(dictionary["local_global_slices_pairs"]),
            unsharded_shape=torch.Size(_parse_shape(dictionary["unsharded_shape"])),
        )


def save_meta(parallel_context: ParallelContext, root_folder: Path, training_metadata: TrainingMetadata):
    assert isinstance(training_metadata, TrainingMetadata)
    if dist.get_rank(parallel_context.world_pg) != 0:
        return
    root_folder = Path(root_folder)
    root_folder.mkdir(exist_ok=True, parents=True)
    meta = CheckpointMetadata(version=CHECKPOINT_VERSION, tp=parallel_context.tp_pg.size(), dp=parallel_context.dp_pg.size(), cp=parallel_context.cp_pg.size(), metas=training_metadata)
    d = dataclasses.asdict(meta)
    d["version"] = str(meta.version)
    with open(root_folder / CHECKPOINT_FILE_NAME, mode="w") as fo:
        json.dump(d, fo, indent=2, sort_keys=True)


def load_meta(parallel_context: Optional[ParallelContext], root_folder: Path) -> CheckpointMetadata:
    with open(Path(root_folder) / CHECKPOINT_FILE_NAME) as fi:
        d = json.load(fi)
    metas = d["metas"]
    stages = metas.get("data_stages")
    if stages is not None:
        stages = [DataStageMetadata(**s) for s in stages]
    tm = TrainingMetadata(
        consumed_train_samples=metas["consumed_train_samples"], last_train_step=metas["last_train_step"],
        consumed_tokens_total=metas.get("consumed_tokens_total"), last_stage_idx=metas.get("last_stage_idx"), data_stages=stages,
    )
    return CheckpointMetadata(version=Version(d["version"]), tp=d["tp"], dp=d["dp"], cp=d.get("cp", 1), metas=tm, custom_metas=d.get("custom_metas"))
