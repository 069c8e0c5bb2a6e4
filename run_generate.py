#!/usr/bin/env python
"""Text generation from a checkpoint (parity: reference run_generate.py).

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 run_generate.py --ckpt-path checkpoints/10 --tp 2 --max-new-tokens 32
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

from nanotron_b200 import distributed as dist  # noqa: E402
from nanotron_b200 import logging  # noqa: E402
from nanotron_b200.config import GenerationArgs, LoggingArgs, ParallelismArgs, get_config_from_file  # noqa: E402
from nanotron_b200.generation.decode import GenerationInput, TokenizerConfig, decode_text, decode_tokenized  # noqa: E402
from nanotron_b200.logging import log_rank, set_ranks_logging_level  # noqa: E402
from nanotron_b200.models import build_model  # noqa: E402
from nanotron_b200.parallel import ParallelContext  # noqa: E402
from nanotron_b200.parallel.parameters import sanity_check  # noqa: E402
from nanotron_b200.parallel.pipeline_parallel.engine import OneForwardOneBackwardPipelineEngine  # noqa: E402
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode  # noqa: E402
from nanotron_b200.random import RandomStates, get_current_random_state, get_synced_random_state, set_random_seed  # noqa: E402
from nanotron_b200.serialize import load_weights  # noqa: E402
from nanotron_b200.trainer import CONFIG_TO_MODEL_CLASS, mark_tied_parameters  # noqa: E402

logger = logging.get_logger("nanotron_b200.run_generate")


def get_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--ckpt-path", type=Path, required=True, help="Checkpoint step folder")
    parser.add_argument("--dp", type=int, default=1)
    parser.add_argument("--pp", type=int, default=0)
    parser.add_argument("--tp", type=int, default=0)
    parser.add_argument("--max-new-tokens", type=int, default=128)
    parser.add_argument("--use-cache", action="store_true")
    parser.add_argument("--prompt", action="append", default=None, help="May be given several times")
    return parser.parse_args()


def main():
    args = get_args()
    assert args.ckpt_path.exists(), f"Checkpoint path {args.ckpt_path} does not exist"
    config = get_config_from_file(str(args.ckpt_path / "config.yaml"))
    model_config = config.model.model_config
    tokenizer_path = config.tokenizer.tokenizer_name_or_path if config.tokenizer is not None else None
    parallel_config = ParallelismArgs(
        dp=args.dp, pp=args.pp or config.parallelism.pp, tp=args.tp or config.parallelism.tp, pp_engine=OneForwardOneBackwardPipelineEngine(),
        tp_mode=TensorParallelLinearMode.ALL_REDUCE, tp_linear_async_communication=False,
    )
    ctx = ParallelContext(data_parallel_size=parallel_config.dp, pipeline_parallel_size=parallel_config.pp, tensor_parallel_size=parallel_config.tp)
    set_ranks_logging_level(parallel_context=ctx, logging_config=LoggingArgs(log_level="info", log_level_replica="info"))
    log_rank(f"model_config: {model_config}", logger=logger, level=logging.INFO, rank=0)
    set_random_seed(42)
    random_states = RandomStates({"tp_synced": get_synced_random_state(random_state=get_current_random_state(), pg=ctx.tp_pg)})
    model_cls = CONFIG_TO_MODEL_CLASS[model_config.__class__.__name__]
    model = build_model(model_builder=lambda: model_cls(config=model_config, parallel_context=ctx, parallel_config=parallel_config, random_states=random_states), dtype=config.model.dtype, parallel_context=ctx)
    mark_tied_parameters(model=model, parallel_context=ctx, parallel_config=parallel_config)
    sanity_check(root_module=model)
    log_rank(f"Loading checkpoint from {args.ckpt_path}:", logger=logger, level=logging.INFO, rank=0)
    load_weights(model=model, parallel_context=ctx, root_folder=args.ckpt_path)
    model.eval()
    prompts = args.prompt or ["The future of AI is", "def fib(n)", "Passage: Daniel went back to the garden. Mary travelled to the kitchen.\nQuestion: Where is Mary?\nAnswer:"]
    gen_cfg = GenerationArgs(sampler="greedy", use_cache=args.use_cache)
    if tokenizer_path is not None:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
        outputs = decode_text(
            input_iter=(GenerationInput(text=t) for t in prompts), tokenizer=tokenizer, model=model.model, parallel_context=ctx, max_new_tokens=args.max_new_tokens,
            max_micro_batch_size=2, generation_config=gen_cfg, tokenizer_config=TokenizerConfig(max_input_length=None), use_cache=args.use_cache,
            is_bench=os.environ.get("USE_BENCH", "0") == "1",  # also logs the decoding throughput of every micro-batch
        )
        for out in outputs:
            log_rank(f"input: {tokenizer.decode(out.input_ids, clean_up_tokenization_spaces=False)[:1000]}", logger=logger, level=logging.INFO, rank=0)
            log_rank(f"generation: {tokenizer.decode(out.generation_ids, clean_up_tokenization_spaces=False)}", logger=logger, level=logging.INFO, rank=0)
            log_rank("--------------------------------------------------", logger=logger, level=logging.INFO, rank=0)
    else:
        # no tokenizer in the config: generate from random token ids (smoke run)
        ids = torch.randint(0, model_config.vocab_size, (2, 8), generator=torch.Generator().manual_seed(0))
        out = decode_tokenized(ids, torch.ones_like(ids, dtype=torch.bool), model=model.model, parallel_context=ctx, generation_config=gen_cfg, max_new_tokens=args.max_new_tokens, use_cache=args.use_cache,
                               is_bench=os.environ.get("USE_BENCH", "0") == "1")
        for i in range(ids.shape[0]):
            log_rank(f"input: {ids[i].tolist()}", logger=logger, level=logging.INFO, rank=0)
            log_rank(f"generation: {out.generation_ids[i].tolist()}", logger=logger, level=logging.INFO, rank=0)
    dist.barrier()
    ctx.destroy()


if __name__ == "__main__":
    main()
