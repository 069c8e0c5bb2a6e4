#!/usr/bin/env python
"""Training entry point (parity: reference run_train.py).

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 run_train.py --config-file examples/config_tiny_llama.yaml

Builds one dataloader per data stage: the dummy generator when ``data.dataset`` is null, a HuggingFace text dataset
(tokenised and packed) for ``PretrainDatasetsArgs`` / ``SFTDatasetsArgs``, or pre-tokenised token files
(``NanosetDatasetsArgs``).  Stages are created lazily so only the active one holds memory.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import Dict, Optional

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from nanotron_b200 import logging  # noqa: E402
from nanotron_b200.config import DataArgs, DatasetStageArgs, LlamaConfig, NanosetDatasetsArgs, PretrainDatasetsArgs, SFTDatasetsArgs, Starcoder2Config  # noqa: E402
from nanotron_b200.data.dataloader import dummy_infinite_data_generator, get_train_dataloader  # noqa: E402
from nanotron_b200.helpers import compute_remain_train_steps_of_a_data_stage_from_ckp, get_consumed_train_samples_of_a_data_stage_from_ckp  # noqa: E402
from nanotron_b200.logging import log_rank  # noqa: E402
from nanotron_b200.parallel.pipeline_parallel.utils import get_input_output_pp_ranks  # noqa: E402
from nanotron_b200.trainer import DistributedTrainer  # noqa: E402

logger = logging.get_logger("nanotron_b200.run_train")


def get_dataloader_from_data_stage(trainer: DistributedTrainer, data: DataArgs, consumed_train_samples_stage: int, consumed_tokens_per_dataset_folder: Dict[str, int], num_remaining_train_steps: int, sequence_length: Optional[int] = None):
    assert consumed_train_samples_stage >= 0 and num_remaining_train_steps >= 0
    input_pp_rank, output_pp_rank = get_input_output_pp_ranks(model=trainer.model)
    seq = sequence_length or trainer.sequence_length
    uses_mask = isinstance(trainer.model_config, (LlamaConfig, Starcoder2Config))
    if data.dataset is None:
        log_rank("Using dummy data generator", logger=logger, level=logging.INFO, rank=0)
        return dummy_infinite_data_generator(
            micro_batch_size=trainer.micro_batch_size, sequence_length=seq, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank,
            vocab_size=trainer.model_config.vocab_size, seed=data.seed, parallel_context=trainer.parallel_context, use_position_ids=not uses_mask,
            skip_batches=consumed_train_samples_stage // (trainer.parallel_context.dp_pg.size() * trainer.micro_batch_size),
        )()
    if isinstance(data.dataset, (PretrainDatasetsArgs, SFTDatasetsArgs)):
        from transformers import AutoTokenizer

        from nanotron_b200.data.processing import clm_process, get_datasets
        from nanotron_b200.utils import main_rank_first

        tokenizer_path = trainer.config.tokenizer.tokenizer_name_or_path
        log_rank(f"Loading tokenizer from {tokenizer_path}", logger=logger, level=logging.INFO, rank=0)
        with main_rank_first(trainer.parallel_context.world_pg):
            raw = get_datasets(hf_dataset_or_datasets=data.dataset.hf_dataset_or_datasets, hf_dataset_config_name=data.dataset.hf_dataset_config_name, splits=data.dataset.hf_dataset_splits)["train"]
            tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
            tokenizer.pad_token = tokenizer.pad_token or tokenizer.eos_token
            tokenizer.padding_side = "left"
            assert tokenizer.vocab_size <= trainer.model_config.vocab_size, f"tokenizer vocab ({tokenizer.vocab_size}) larger than the model's ({trainer.model_config.vocab_size})"
            if isinstance(data.dataset, SFTDatasetsArgs):
                from nanotron_b200.data.sft_processing import prepare_sft_dataset

                train_dataset = prepare_sft_dataset(raw, tokenizer, seq, debug_max_samples=data.dataset.debug_max_samples, num_proc=data.dataset.dataset_processing_num_proc_per_process)
            else:
                train_dataset = clm_process(raw_dataset=raw, tokenizer=tokenizer, text_column_name=data.dataset.text_column_name, dataset_processing_num_proc_per_process=data.dataset.dataset_processing_num_proc_per_process, dataset_overwrite_cache=data.dataset.dataset_overwrite_cache, sequence_length=seq)
        if isinstance(data.dataset, SFTDatasetsArgs):
            from torch.utils.data import DataLoader

            from nanotron_b200.data.clm_collator import DataCollatorForSFT
            from nanotron_b200.data.samplers import get_sampler
            import nanotron_b200.distributed as dist

            ctx = trainer.parallel_context
            sampler = get_sampler(dl_ranks_size=ctx.dp_pg.size(), dl_rank=dist.get_rank(ctx.dp_pg), train_dataset=train_dataset, consumed_train_samples=consumed_train_samples_stage, seed=data.seed)
            return DataLoader(train_dataset.with_format("numpy"), batch_size=trainer.micro_batch_size, sampler=sampler, collate_fn=DataCollatorForSFT(seq, input_pp_rank, output_pp_rank, ctx), num_workers=data.num_loading_workers, drop_last=True)
        dataloader = get_train_dataloader(
            train_dataset=train_dataset, sequence_length=seq, parallel_context=trainer.parallel_context, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank,
            micro_batch_size=trainer.micro_batch_size, consumed_train_samples=consumed_train_samples_stage, dataloader_num_workers=data.num_loading_workers,
            seed_worker=data.seed, dataloader_drop_last=True, use_position_ids=not uses_mask,
        )
        total_tokens_dataset = len(dataloader.dataset) * seq
        needed = num_remaining_train_steps * trainer.global_batch_size * seq
        assert needed < total_tokens_dataset, f"Dataset is too small for steps ({total_tokens_dataset} < {needed}), try train_steps<={len(dataloader.dataset) // trainer.global_batch_size + trainer.iteration_step}"
        return dataloader
    if isinstance(data.dataset, NanosetDatasetsArgs) and (data.dataset.use_old_brrr_dataloader or data.dataset.dataset_read_path):
        # streamed token files / folders mirrored under another root: blended folders + the Megatron batch sampler
        from nanotron_b200.data.tokenized_bytes import get_tb_dataloader, get_tb_datasets

        if data.dataset.token_size_in_bytes is None:
            data.dataset.token_size_in_bytes = 4 if trainer.model_config.vocab_size > 65535 else 2
        train_dataset, data_log = get_tb_datasets(
            data.dataset, sequence_length=seq, global_batch_size=trainer.global_batch_size, train_steps=trainer.config.tokens.train_steps,
            current_iteration=trainer.iteration_step, parallel_context=trainer.parallel_context, eos_token_id=getattr(trainer.model_config, "eos_token_id", None),
            shuffle=bool(data.dataset.shuffle_files), seed=data.seed, consumed_samples=consumed_train_samples_stage,
            consumed_tokens_per_dataset_folder=consumed_tokens_per_dataset_folder,
        )
        log_rank(f"[tokenized bytes] {data_log.human_total_train_tokens} training tokens in {data_log.train_num_samples} samples", logger=logger, level=logging.INFO, rank=0)
        return get_tb_dataloader(
            train_dataset, sequence_length=seq, micro_batch_size=trainer.micro_batch_size, global_batch_size=trainer.global_batch_size, cfg=data.dataset,
            num_workers=data.num_loading_workers, consumed_samples=consumed_train_samples_stage, num_samples=len(train_dataset), parallel_context=trainer.parallel_context,
            input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank, use_position_ids=not uses_mask and bool(data.dataset.return_positions),
            use_doc_masking=getattr(trainer.model_config, "_use_doc_masking", False),
        )
    if isinstance(data.dataset, NanosetDatasetsArgs):
        from nanotron_b200.data.nanoset import Nanoset
        from nanotron_b200.utils import main_rank_first

        with main_rank_first(trainer.parallel_context.world_pg):
            train_dataset = Nanoset(
                dataset_folders=data.dataset.dataset_folder, dataset_weights=data.dataset.dataset_weights, sequence_length=seq,
                token_size=data.dataset.token_size_in_bytes or (4 if trainer.model_config.vocab_size > 65535 else 2),
                train_split_num_samples=trainer.config.tokens.train_steps * trainer.global_batch_size, random_seed=data.seed,
                return_positions=bool(data.dataset.return_positions), eos_token_id=getattr(trainer.model_config, "eos_token_id", None),
            )
        return get_train_dataloader(
            train_dataset=train_dataset, sequence_length=seq, parallel_context=trainer.parallel_context, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank,
            micro_batch_size=trainer.micro_batch_size, consumed_train_samples=consumed_train_samples_stage, dataloader_num_workers=data.num_loading_workers,
            seed_worker=data.seed, dataloader_drop_last=True, use_position_ids=not uses_mask, use_doc_masking=getattr(trainer.model_config, "_use_doc_masking", False),
        )
    raise ValueError(f"Unhandled case of `self.config.data.dataset`. Got: {data.dataset}")


def log_batches_every(dataloader, interval: int, tokenizer_path: Optional[str], stage_name: str):
    """Pass the batches of ``dataloader`` through and describe every ``interval``-th one on rank 0: shapes, the first tokens of
    the first row (decoded when the configuration names a tokenizer), where its documents start, how many labels count
    (``--sanity-check-dataloader-interval``; capability parity: reference run_train.py:302-307).  Nothing is consumed twice."""
    tokenizer = None
    if tokenizer_path is not None:
        try:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
        except Exception as e:  # a debugging aid must not stop the run
            log_rank(f"[dataloader sample] tokenizer {tokenizer_path} not usable ({type(e).__name__}): printing ids", logger=logger, level=logging.WARNING, rank=0)
    for index, batch in enumerate(dataloader):
        if index % interval == 0:
            lines = [f"[dataloader sample] stage {stage_name!r}, micro-batch {index}"]
            for key, value in batch.items():
                if hasattr(value, "shape"):
                    lines.append(f"  {key}: shape {tuple(value.shape)} dtype {getattr(value, 'dtype', '?')}")
                else:
                    lines.append(f"  {key}: {value}")
            ids = batch.get("input_ids")
            if hasattr(ids, "shape"):
                row = [int(t) for t in ids[0][:32]]
                lines.append("  first row: " + (repr(tokenizer.decode(row)) if tokenizer is not None else str(row)))
            positions = batch.get("position_ids")
            if hasattr(positions, "shape"):
                lines.append(f"  documents of the first row start at {[i for i, p in enumerate(positions[0].tolist()) if p == 0][:16]}")
            mask = batch.get("label_mask")
            if hasattr(mask, "shape"):
                lines.append(f"  labels that count: {int(mask.sum())} of {int(np.prod(mask.shape))}")  # (numpy from the collators, tensors from generators)
            log_rank("\n".join(lines), logger=logger, level=logging.INFO, rank=0)
        yield batch


def get_dataloader(trainer: DistributedTrainer, sanity_check_dataloader_interval: Optional[int] = None):
    """{stage name: dataloader or zero-argument factory}.  The stage to resume is built now, later stages lazily."""
    dataloaders = {}
    stages = sorted(trainer.config.data_stages, key=lambda s: s.start_training_step)
    for stage_idx, stage in enumerate(stages):
        stage: DatasetStageArgs
        consumed = get_consumed_train_samples_of_a_data_stage_from_ckp(stage, trainer.metadata)
        assert consumed is not None, f"Cannot find consumed_train_samples for stage {stage.start_training_step} in the checkpoint"
        remaining = compute_remain_train_steps_of_a_data_stage_from_ckp(stage, trainer.config, trainer.metadata)
        meta_stage = next(s for s in trainer.metadata.data_stages if s.start_training_step == stage.start_training_step)
        log_rank(f"[Training Plan] Stage {stage.name} has {remaining} remaining training steps and has consumed {consumed} samples", logger=logger, level=logging.INFO, rank=0)

        def build(stage=stage, consumed=consumed, remaining=remaining, meta_stage=meta_stage):
            dl = get_dataloader_from_data_stage(trainer, stage.data, consumed_train_samples_stage=consumed, consumed_tokens_per_dataset_folder=meta_stage.consumed_tokens_per_dataset_folder, num_remaining_train_steps=remaining, sequence_length=stage.sequence_length)
            if sanity_check_dataloader_interval:
                tokenizer_path = trainer.config.tokenizer.tokenizer_name_or_path if trainer.config.tokenizer is not None else None
                return _Described(dl, sanity_check_dataloader_interval, tokenizer_path, stage.name)
            return dl

        is_current = stage_idx == (trainer.metadata.last_stage_idx or 0)
        dataloaders[stage.name] = build() if is_current else build
    return dataloaders


class _Described:
    """A dataloader whose batches are described now and then; keeps ``dataset`` visible (the trainer reads consumption
    statistics from it)."""

    def __init__(self, dataloader, interval: int, tokenizer_path: Optional[str], stage_name: str):
        self.dataloader, self.interval, self.tokenizer_path, self.stage_name = dataloader, interval, tokenizer_path, stage_name
        if hasattr(dataloader, "dataset"):
            self.dataset = dataloader.dataset

    def __iter__(self):
        return log_batches_every(self.dataloader, self.interval, self.tokenizer_path, self.stage_name)


def get_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--config-file", type=str, required=True, help="Path to the YAML or python config file")
    parser.add_argument("--sanity-check-dataloader-interval", type=int, default=None, help="Log a decoded batch every N steps (debug)")
    return parser.parse_args()


def wait_for_debugger_if_asked():
    """``NANOTRON_DEBUG_RANK=<r>``: rank r announces its pid and stops itself (SIGSTOP) before anything is initialised, so a
    debugger can attach; ``kill -CONT <pid>`` lets it go on.  The other ranks wait for it at the first collective."""
    import signal

    want = os.environ.get("NANOTRON_DEBUG_RANK")
    if want is not None and want == os.environ.get("RANK", "0"):
        print(f"[rank {want}] pid {os.getpid()} stopped for a debugger; resume with: kill -CONT {os.getpid()}", flush=True)
        os.kill(os.getpid(), signal.SIGSTOP)


if __name__ == "__main__":
    args = get_args()
    wait_for_debugger_if_asked()
    trainer = DistributedTrainer(args.config_file)
    dataloader = get_dataloader(trainer, sanity_check_dataloader_interval=args.sanity_check_dataloader_interval)
    trainer.train(dataloader)
