"""Reference arm of ``bench.py``: runs the UNMODIFIED huggingface/nanotron installed under ``baseline/_ref`` through its
own ``DistributedTrainer`` on the same model / batch / parallelism as the native arm and prints the same JSON line.

Nothing of this repository's models, kernels or engine is on that path.  The only additions are import stand-ins under
``baseline/shims`` for third-party packages that cannot be installed offline (``dacite``, ``torchtyping``,
``grouped_gemm``; the latter two are import-time only for a dense Llama).  Timing: the trainer's public
``post_train_step`` hook is used to place CUDA events after the last warm-up step and after the last timed step,
with a barrier + synchronize at both points; max over ranks.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")


def _unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def run_reference(args):
    if not os.path.isdir(os.path.join(REF, "nanotron")):
        return _unavailable("baseline/_ref is missing: install with `pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy of the reference source tree>`")
    sys.path.insert(0, SHIMS)
    sys.path.insert(0, REF)
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    # the reference's data-parallel path (replicated fp32 optimizer + DDP buckets) sits within a few GB of the 180 GB of a B200 for
    # an 8B model: let the caching allocator grow segments instead of fragmenting, so that it gets every byte it can use
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1"), os.environ.setdefault("LOCAL_RANK", "0")
    try:
        import torch

        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
        import flash_attn_compat

        flash_attn_compat.apply()
        import nanotron  # noqa: F401
        from nanotron import distributed as dist
        from nanotron.config import (
            AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LoggingArgs, Qwen2Config,
            LRSchedulerArgs, ModelArgs, OptimizerArgs, ParallelismArgs, RandomInit, TokenizerArgs, TokensArgs,
        )
        from nanotron.data.dataloader import dummy_infinite_data_generator
        from nanotron.parallel.pipeline_parallel.utils import get_input_output_pp_ranks
        from nanotron.trainer import DistributedTrainer
    except Exception as e:  # import problems of the reference or of its dependencies
        return _unavailable(f"reference does not import here: {type(e).__name__}: {str(e)[:200]}")

    from bench import BASELINE_TOK_S_PER_GPU, MODELS, ClockSampler

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    m = dict(MODELS[args.model])
    # The reference's `LlamaForTraining.init_model_randomly` fails on its stock path (models/llama.py:1095 hands
    # `config.model` to a parametrizator that reads `config.model.init_method`: AttributeError), so the Llama-3-8B shape
    # is run through its maintained decoder implementation, `Qwen2ForTraining`, which without attention bias is the same
    # architecture (RMSNorm, RoPE, GQA, SwiGLU) with the same parameter count and FLOPs.
    model_config = Qwen2Config(bos_token_id=1, eos_token_id=2, hidden_act="silu", initializer_range=0.02, pretraining_tp=1, rope_scaling=None, use_cache=True, rope_interleaved=False, attention_bias=False, log_attn_probs=False, **m)
    total_steps = args.warmup + args.steps
    ckpt_dir = tempfile.mkdtemp(prefix="ref_ckpt_")
    config = Config(
        general=GeneralArgs(project="bench", run="reference", seed=42, ignore_sanity_checks=True),
        checkpoints=CheckpointsArgs(checkpoints_path=ckpt_dir, checkpoint_interval=10**9, save_final_state=False),
        parallelism=ParallelismArgs(dp=world, pp=1, tp=1, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=False, recompute_layer=bool(args.recompute)),
        model=ModelArgs(init_method=RandomInit(std=0.02), model_config=model_config),
        tokenizer=TokenizerArgs(tokenizer_name_or_path=None),
        optimizer=OptimizerArgs(
            # ZeRO-1 together with fp32 gradient accumulation and dp > 1 is not runnable in the reference: its DDP hook raises
            # NotImplementedError("Not implemented") on the reduce-scatter branch (optim/gradient_accumulator.py:354-355, selected by
            # helpers.py:460 whenever the optimizer is a ZeroDistributedOptimizer).  Its working data-parallel path is the fp32
            # all-reduce with a replicated optimizer, so that is what runs here at every N.
            zero_stage=0, weight_decay=0.01, clip_grad=1.0, accumulate_grad_in_fp32=True,
            learning_rate_scheduler=LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=3e-5),
            optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
        ),
        logging=LoggingArgs(log_level="warning", log_level_replica="error", iteration_step_info_interval=1),
        tokens=TokensArgs(sequence_length=args.seq, train_steps=total_steps, micro_batch_size=args.mbs, batch_accumulation_per_replica=args.accum),
        data_stages=[DatasetStageArgs(name="bench", start_training_step=1, data=DataArgs(dataset=None, seed=42, num_loading_workers=0))],
    )
    # the reference trainer wants a file path; every rank writes its own (identical) copy into its own scratch directory
    cfg_path = os.path.join(ckpt_dir, "config.yaml")
    config.save_as_yaml(cfg_path)
    state = {"start": None, "end": None, "sampler": None, "clocks": None}

    class TimedTrainer(DistributedTrainer):
        def post_train_step(self):
            super().post_train_step()
            done = self.iteration_step - self.initial_iter_step + 1
            if done == args.warmup or done == total_steps:
                dist.barrier()
                torch.cuda.synchronize()
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                if done == args.warmup:
                    state["start"] = ev
                    state["sampler"] = ClockSampler(int(os.environ["LOCAL_RANK"]))
                    state["sampler"].start()
                else:
                    state["end"] = ev
                    torch.cuda.synchronize()
                    state["clocks"] = state["sampler"].stop()

    try:
        trainer = TimedTrainer(cfg_path)
        input_pp_rank, output_pp_rank = get_input_output_pp_ranks(model=trainer.model)
        dataloader = dummy_infinite_data_generator(
            micro_batch_size=trainer.micro_batch_size, sequence_length=trainer.sequence_length, input_pp_rank=input_pp_rank,
            output_pp_rank=output_pp_rank, vocab_size=trainer.model_config.vocab_size, seed=42, parallel_context=trainer.parallel_context,
            use_position_ids=True, cp_pg=trainer.parallel_context.cp_pg,
        )()
        trainer.train({"bench": dataloader})
    except torch.cuda.OutOfMemoryError as e:
        return _unavailable(f"reference ran out of GPU memory on this config: {str(e)[:160]}")
    except Exception as e:
        import traceback

        traceback.print_exc(file=sys.stderr)
        return _unavailable(f"reference failed on its stock path: {type(e).__name__}: {str(e)[:300]}")
    ms = torch.tensor([state["start"].elapsed_time(state["end"])], dtype=torch.float64, device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    tokens_per_step = args.mbs * args.seq * args.accum * world
    value = tokens_per_step / (ms / args.steps / 1000.0)
    if rank == 0:
        out = {
            "metric": "Llama-3-8B training tokens/sec (whole job), bf16, seq 4096" if args.model == "llama3-8b" else f"{args.model} training tokens/sec",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": value / world / BASELINE_TOK_S_PER_GPU if args.model == "llama3-8b" else None,
            "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights", "impl": "reference", "tokens_per_sec_per_gpu": value / world,
            "config": {"model": args.model, "global_batch": args.mbs * args.accum * world, "seq_len": args.seq, "micro_batch": args.mbs, "grad_accum": args.accum,
                       "parallelism": f"dp{world}" + ("+zero1" if world > 1 else ""), "fp32_grad_accum": True, "optimizer": "AdamW (torch fused)", "clip_grad": 1.0,
                       "l2": "inputs larger than L2; no explicit flush"},
            "clocks": state["clocks"],
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4, "note": "the reference's stock loop: tokens drawn on the device by its dummy generator, loss read on the host every step"},
            "gpu_launches": 0,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
        }
        print(json.dumps(out), flush=True)
    return 0
