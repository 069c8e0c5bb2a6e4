#!/usr/bin/env python
"""Evaluate a checkpoint on the multiple-choice tasks of ``nanotron_b200.eval.evaluation_tasks`` (entry-point parity: reference
run_evals.py, which hands the checkpoint to the ``lighteval`` package; here the scoring runs in-tree).

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 run_evals.py --checkpoint-config-path ckpt/10/config.yaml \\
        --tasks "arc_cf:easy,hellaswag_cf,mmlu_mcf:*" --data-dir eval_data --max-samples 500 --output results.json

Documents come from ``<data-dir>/<task family>[:<subset>].<split>.jsonl`` when ``--data-dir`` is given (one JSON object per line with
the fields of the original dataset; the way to evaluate on a machine without network access), otherwise from the HuggingFace hub
through the ``datasets`` package.  The tokenizer is the one named in the checkpoint's config (``--tokenizer`` overrides it).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def get_parser():
    p = argparse.ArgumentParser()
    p.add_argument("--checkpoint-config-path", type=str, required=True, help="config.yaml inside the checkpoint folder")
    p.add_argument("--tasks", type=str, default="arc_cf:easy,arc_cf:challenge,hellaswag_cf,piqa_cf,winogrande_cf,openbookqa_cf,commonsenseqa_cf")
    p.add_argument("--data-dir", type=str, default=None, help="folder with <family>[:<subset>].<split>.jsonl files")
    p.add_argument("--tokenizer", type=str, default=None)
    p.add_argument("--max-samples", type=int, default=None)
    p.add_argument("--num-fewshot", type=int, default=0)
    p.add_argument("--batch-size", type=int, default=8)
    p.add_argument("--max-length", type=int, default=2048)
    p.add_argument("--dp", type=int, default=1)
    p.add_argument("--pp", type=int, default=0)
    p.add_argument("--tp", type=int, default=0)
    p.add_argument("--output", type=str, default=None, help="write the results as JSON here (rank 0)")
    p.add_argument("--lighteval-override", type=str, default=None, help="accepted for command-line compatibility with the reference; unused")
    p.add_argument("--cache-dir", type=str, default=None)
    return p


def load_lines(task, split: str, data_dir, cache_dir=None):
    family = task.name.split("_" + task.formulation.value)[0]
    subset = task.name.split(":", 1)[1] if ":" in task.name else None
    if data_dir is not None:
        path = Path(data_dir) / (f"{family}:{subset}.{split}.jsonl" if subset else f"{family}.{split}.jsonl")
        assert path.exists(), f"{path} not found (expected the {split} split of {task.hf_repo} / {task.hf_subset} as JSON lines)"
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    try:
        import datasets
    except ImportError as e:
        raise SystemExit("no --data-dir given and the `datasets` package is not installed") from e
    return list(datasets.load_dataset(task.hf_repo, task.hf_subset, split=split, revision=task.hf_revision, cache_dir=cache_dir))


def main():
    args = get_parser().parse_args()
    import torch  # noqa: F401

    from nanotron_b200 import distributed as dist
    from nanotron_b200 import logging
    from nanotron_b200.config import LoggingArgs, ParallelismArgs, get_config_from_file
    from nanotron_b200.eval.evaluation_tasks import get_tasks
    from nanotron_b200.eval.harness import LogLikelihoodScorer, evaluate_task
    from nanotron_b200.logging import log_rank, set_ranks_logging_level
    from nanotron_b200.models import build_model
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.pipeline_parallel.engine import OneForwardOneBackwardPipelineEngine
    from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
    from nanotron_b200.random import RandomStates, get_current_random_state, get_synced_random_state, set_random_seed
    from nanotron_b200.serialize import load_weights
    from nanotron_b200.trainer import CONFIG_TO_MODEL_CLASS, mark_tied_parameters

    logger = logging.get_logger("nanotron_b200.run_evals")
    ckpt = Path(args.checkpoint_config_path).parent
    config = get_config_from_file(args.checkpoint_config_path)
    model_config = config.model.model_config
    par = ParallelismArgs(dp=args.dp, pp=args.pp or config.parallelism.pp, tp=args.tp or config.parallelism.tp, pp_engine=OneForwardOneBackwardPipelineEngine(),
                          tp_mode=TensorParallelLinearMode.ALL_REDUCE, tp_linear_async_communication=False)
    ctx = ParallelContext(data_parallel_size=par.dp, pipeline_parallel_size=par.pp, tensor_parallel_size=par.tp)
    set_ranks_logging_level(parallel_context=ctx, logging_config=LoggingArgs(log_level="info", log_level_replica="warning"))
    set_random_seed(42)
    random_states = RandomStates({"tp_synced": get_synced_random_state(random_state=get_current_random_state(), pg=ctx.tp_pg)})
    model_cls = CONFIG_TO_MODEL_CLASS[model_config.__class__.__name__]
    model = build_model(model_builder=lambda: model_cls(config=model_config, parallel_context=ctx, parallel_config=par, random_states=random_states), dtype=config.model.dtype, parallel_context=ctx)
    mark_tied_parameters(model=model, parallel_context=ctx, parallel_config=par)
    load_weights(model=model, parallel_context=ctx, root_folder=ckpt)
    tokenizer_path = args.tokenizer or (config.tokenizer.tokenizer_name_or_path if config.tokenizer is not None else None)
    assert tokenizer_path is not None, "the checkpoint's config names no tokenizer: pass --tokenizer"
    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
    scorer = LogLikelihoodScorer(model.model, ctx, tokenizer, max_length=args.max_length, batch_size=args.batch_size)
    results = {}
    for task in get_tasks(args.tasks):
        few = []
        if args.num_fewshot > 0 and task.few_shots_split is not None:
            few = load_lines(task, task.few_shots_split, args.data_dir, args.cache_dir)[: args.num_fewshot]
        for split in task.evaluation_splits:
            lines = load_lines(task, split, args.data_dir, args.cache_dir)
            results[f"{task.name}|{split}"] = evaluate_task(scorer, task, lines, few_shot_lines=few, max_samples=args.max_samples)
            log_rank(f"{task.name} [{split}]: {results[f'{task.name}|{split}']}", logger=logger, level=logging.INFO, rank=0)
    if dist.get_rank(ctx.world_pg) == 0:
        text = json.dumps({"config": str(args.checkpoint_config_path), "results": results}, indent=2, sort_keys=True)
        print(text)
        if args.output:
            Path(args.output).write_text(text)
    dist.barrier()
    ctx.destroy()


if __name__ == "__main__":
    main()
