"""Training with a dataloader of your own (capability parity: reference examples/custom-dataloader/run_train.py).

``DistributedTrainer.train`` takes ``{data-stage name: iterable of micro-batches}``.  A micro-batch is a dict with the keys
the model's forward expects -- ``input_ids / input_mask / label_ids / label_mask`` for Llama and Starcoder2,
``input_ids / position_ids / label_ids / label_mask`` for Qwen2 -- where a pipeline rank that does not consume a key holds a
``TensorPointer`` to the rank that does.  The stock collators (``nanotron_b200.data.clm_collator``) build exactly that from
examples of ``sequence_length + 1`` token ids, so a custom pipeline is: any ``torch.utils.data.Dataset`` that returns
``{"input_ids": ids}``, a sampler that splits it over data-parallel ranks, one of those collators.

The dataset here is synthetic and learnable (so the loss visibly falls): every sequence counts upwards modulo the vocabulary
from a random start with a random stride out of a small set.

    torchrun --nproc-per-node 2 examples/custom_dataloader/run_train.py --config-file examples/config_tiny_llama.yaml
"""
import argparse
import os
import sys

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nanotron_b200 import logging  # noqa: E402
from nanotron_b200.config import LlamaConfig, Starcoder2Config  # noqa: E402
from nanotron_b200.data.clm_collator import DataCollatorForCLM, DataCollatorForCLMWithPositionIds  # noqa: E402
from nanotron_b200.data.dataloader import get_dataloader_worker_init  # noqa: E402
from nanotron_b200.data.samplers import get_sampler  # noqa: E402
from nanotron_b200.logging import log_rank  # noqa: E402
from nanotron_b200.parallel.pipeline_parallel.utils import get_input_output_pp_ranks  # noqa: E402
from nanotron_b200.trainer import DistributedTrainer  # noqa: E402

logger = logging.get_logger(__name__)


class CountingSequences(Dataset):
    """``num_samples`` sequences of ``length`` tokens: ``(start + i * stride) mod vocab``; sample ``i`` is a pure function of ``i``."""

    STRIDES = (1, 2, 3, 5)

    def __init__(self, num_samples: int, length: int, vocab_size: int, seed: int = 0):
        self.num_samples, self.length, self.vocab_size, self.seed = num_samples, length, vocab_size, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx: int):
        rng = np.random.default_rng(self.seed * 1_000_003 + idx)
        start = int(rng.integers(0, self.vocab_size))
        stride = self.STRIDES[int(rng.integers(0, len(self.STRIDES)))]
        return {"input_ids": (start + stride * np.arange(self.length, dtype=np.int64)) % self.vocab_size}


def build_dataloader(trainer: DistributedTrainer, num_steps: int, consumed_train_samples: int = 0, seed: int = 0) -> DataLoader:
    ctx = trainer.parallel_context
    input_pp_rank, output_pp_rank = get_input_output_pp_ranks(model=trainer.unwrapped_model)
    dataset = CountingSequences(num_samples=trainer.global_batch_size * num_steps, length=trainer.sequence_length + 1, vocab_size=trainer.model_config.vocab_size, seed=seed)
    uses_mask = isinstance(trainer.model_config, (LlamaConfig, Starcoder2Config))
    collator_cls = DataCollatorForCLM if uses_mask else DataCollatorForCLMWithPositionIds
    collator = collator_cls(sequence_length=trainer.sequence_length, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank, parallel_context=ctx)
    from nanotron_b200 import distributed as dist

    sampler = get_sampler(
        dl_ranks_size=ctx.dp_pg.size(), dl_rank=dist.get_rank(ctx.dp_pg), train_dataset=dataset, consumed_train_samples=consumed_train_samples,
        seed=seed, micro_batch_size=trainer.micro_batch_size, drop_last=True, shuffle=False,
    )
    return DataLoader(
        dataset, batch_size=trainer.micro_batch_size, sampler=sampler, collate_fn=collator, drop_last=True, num_workers=0,
        pin_memory=ctx.device.type == "cuda", worker_init_fn=get_dataloader_worker_init(dp_rank=dist.get_rank(ctx.dp_pg)),
    )


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-file", type=str, required=True, help="Path to the YAML or python config file")
    args = ap.parse_args()
    trainer = DistributedTrainer(args.config_file)
    stages = trainer.config.data_stages
    assert stages is not None and len(stages) >= 1
    remaining = trainer.config.tokens.train_steps - trainer.metadata.last_train_step
    log_rank(f"custom dataloader: {remaining} steps of {trainer.global_batch_size} counting sequences", logger=logger, level=logging.INFO, rank=0)
    # one loader for the stage that is active at resume; later stages could be given as zero-argument factories
    loaders = {stages[-1].name: build_dataloader(trainer, num_steps=remaining, consumed_train_samples=trainer.metadata.consumed_train_samples, seed=stages[-1].data.seed)}
    for s in stages[:-1]:
        loaders[s.name] = loaders[stages[-1].name]
    trainer.train(loaders)


if __name__ == "__main__":
    main()
