"""Trains the Mamba example (capability parity: reference examples/mamba/train_mamba.py).

    torchrun --nproc-per-node 1 --master-addr 127.0.0.1 examples/mamba/train_mamba.py --config-file examples/mamba/config_mamba.yaml

Without a dataset in the config the run uses a synthetic *repetition* task: every sequence repeats its first ``--period`` random
tokens, which a recurrent model can only predict by carrying them in its state (the convolution sees 3 positions back) - the
loss on the repeated part falls well below the uniform level within a few dozen steps of the tiny config.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import Optional

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from trainer import MambaTrainer  # noqa: E402

from nanotron_b200 import distributed as dist  # noqa: E402
from nanotron_b200.parallel.pipeline_parallel.block import TensorPointer  # noqa: E402


def copy_task_batches(trainer: MambaTrainer, seed: int = 0, period: Optional[int] = None):
    """Micro-batches in the framework's batch format.  Every sequence repeats its first ``period`` random tokens over and over
    (default: half the sequence, i.e. [first half | same tokens again]); only positions whose target is a repetition are scored."""
    ctx = trainer.parallel_context
    cfg = trainer.config
    seq, mbs, vocab = cfg.tokens.sequence_length, cfg.tokens.micro_batch_size, trainer.model_config.vocab_size
    period = period or (seq + 1) // 2 + 1
    model = trainer.unwrapped_model
    in_rank, out_rank = model.model.token_position_embeddings.rank, model.loss.rank
    pp_rank = dist.get_rank(ctx.pp_pg)
    gen = torch.Generator().manual_seed(seed + 1000 * dist.get_rank(ctx.dp_pg))
    device = ctx.device
    reps = (seq + 1 + period - 1) // period
    while True:
        first = torch.randint(2, vocab, (mbs, period), generator=gen)
        tokens = first.repeat(1, reps)[:, : seq + 1]
        mask = torch.zeros(mbs, seq, dtype=torch.bool)
        mask[:, period - 1 :] = True  # label t is token t + 1: scored from the first repeated token on
        yield {
            "input_ids": tokens[:, :-1].to(device) if pp_rank == in_rank else TensorPointer(group_rank=in_rank),
            "input_mask": torch.ones(mbs, seq, dtype=torch.bool, device=device) if pp_rank == in_rank else TensorPointer(group_rank=in_rank),
            "label_ids": tokens[:, 1:].contiguous().to(device) if pp_rank == out_rank else TensorPointer(group_rank=out_rank),
            "label_mask": mask.to(device) if pp_rank == out_rank else TensorPointer(group_rank=out_rank),
        }


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-file", type=str, required=True)
    ap.add_argument("--period", type=int, default=6, help="synthetic task: length of the repeated token pattern")
    args = ap.parse_args()
    trainer = MambaTrainer(args.config_file)
    if trainer.config.data_stages and trainer.config.data_stages[0].data.dataset is not None:
        from run_train import get_dataloader  # the framework's dataset -> dataloader path (nanoset / tokenized text)

        trainer.train(get_dataloader(trainer))
    else:
        trainer.train({trainer.config.data_stages[0].name: copy_task_batches(trainer, period=args.period)})
