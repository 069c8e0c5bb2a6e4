"""Reference arm of ``bench.py``: runs the UNMODIFIED huggingface/nanotron installed under ``baseline/_ref`` through its
own ``DistributedTrainer`` on the same model, batch and parallel layout (tp / pp by GPU count, sequence-parallel tensor
parallelism with its asynchronous-communication linears, 1F1B) as the native arm and prints the same JSON line.

Where the native arm's layout has pipeline stages (8 GPUs: tp4 x pp2) the reference runs tensor parallelism over all the GPUs
instead: its Qwen2 model, the only one that random-initialises on its stock path, raises on every stage but the first
(see ``run_reference``).  A failure of one rank ends the whole job with the ``unavailable`` line (``_Guard``).

Nothing of this repository's models, kernels or engine is on that path.  The only additions are import stand-ins under
``baseline/shims`` for third-party packages that cannot be installed offline (``dacite``, ``torchtyping``,
``grouped_gemm``; the latter two are import-time only for a dense Llama), and the dataloader handed to
``DistributedTrainer.train``: the reference accepts any iterator of batches, and this one builds every micro-batch in
pinned host memory and copies it to the device (the same end-to-end input path as the native arm) in the batch format
of the reference's own dummy generator.  Timing: the trainer's public ``post_train_step`` hook places CUDA events after
the last warm-up step and after the last timed step, with a barrier + synchronize at both points; max over ranks.  The
reference reads the loss on the host every step (``iteration_step_info_interval=1``), so its timed region is end to end.
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


class _Guard:
    """Keeps a failure of one rank from leaving the others waiting in a collective until someone kills the job.

    A rank whose training loop raised publishes the reason in the job's rendezvous store (host side, no collective); a daemon
    thread on every rank polls the store and also watches a wall-clock deadline.  When either fires, rank 0 prints the
    ``unavailable`` line and every rank leaves with ``os._exit(0)``: the ranks stuck in a collective never return to Python,
    so nothing gentler would end them."""

    KEY = "ntb_reference_failed"

    def __init__(self, deadline_s: float):
        self.deadline_s = deadline_s
        self._stop = False
        self._thread = None

    @staticmethod
    def _store():
        import torch.distributed as tdist
        from torch.distributed import distributed_c10d as c10d

        return c10d._get_default_store() if tdist.is_initialized() else None

    def start(self):
        """Starts the watcher.  The job's process group may not exist yet (the reference trainer creates it): the watcher waits
        for it, the deadline runs from now."""
        import threading
        import time

        if int(os.environ.get("WORLD_SIZE", "1")) == 1:
            return
        t_end = time.monotonic() + self.deadline_s

        def watch():
            store = None
            while not self._stop:
                time.sleep(2.0)
                why = None
                try:
                    store = store or self._store()
                    if store is not None and store.check([self.KEY]):
                        why = store.get(self.KEY).decode(errors="replace")
                except Exception:
                    pass
                if why is None and time.monotonic() > t_end:
                    why = f"the reference did not finish within {self.deadline_s:.0f} s on this layout (a rank is waiting in a collective)"
                if why is not None and not self._stop:
                    _unavailable(why)
                    sys.stdout.flush()
                    os._exit(0)

        self._thread = threading.Thread(target=watch, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop = True

    def fail(self, why: str):
        """Called by the rank that failed: tell the others, give their watchers time to act, report."""
        import time

        self._stop = True
        store = None
        try:
            store = self._store()
        except Exception:
            pass
        if store is not None and int(os.environ.get("WORLD_SIZE", "1")) > 1:
            try:
                store.set(self.KEY, why)
            except Exception:
                pass
            if int(os.environ.get("RANK", "0")) != 0:
                time.sleep(6.0)  # rank 0's watcher prints the line
                os._exit(0)
        _unavailable(why)
        sys.stdout.flush()
        if store is not None and int(os.environ.get("WORLD_SIZE", "1")) > 1:
            time.sleep(6.0)
            os._exit(0)
        return 0


def _host_batches(trainer, input_pp_rank: int, output_pp_rank: int, counter: dict):
    """Micro-batches in the format of the reference's ``dummy_infinite_data_generator(use_position_ids=True)``
    (src/nanotron/data/dataloader.py:100-227: the first row packs documents of 4, 6 and seq - 10 tokens), built on the host in
    pinned memory and copied to the device; ``counter`` accumulates the bytes copied."""
    import torch
    from nanotron import distributed as dist
    from nanotron.parallel.pipeline_parallel.tensor_pointer import TensorPointer

    ctx = trainer.parallel_context
    mbs, seq, vocab = trainer.micro_batch_size, trainer.sequence_length, trainer.model_config.vocab_size
    pp_rank = dist.get_rank(ctx.pp_pg)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(42 * (1 + dist.get_rank(ctx.dp_pg)))
    lengths = [[4, 6, seq - 10]] + [[seq]] * (mbs - 1)
    position_ids = torch.cat([torch.cat([torch.arange(n) for n in row]).unsqueeze(0) for row in lengths]).long()

    def to_device(t):
        counter["bytes"] += t.numel() * t.element_size()
        return t.pin_memory().to("cuda", non_blocking=True)

    while True:
        tokens = torch.randint(0, vocab, (mbs, seq + 1), dtype=torch.long, generator=gen)
        batch = {}
        if pp_rank == input_pp_rank:
            batch["input_ids"] = to_device(tokens[:, :-1].contiguous())
            batch["position_ids"] = to_device(position_ids)
        else:
            batch["input_ids"] = TensorPointer(group_rank=input_pp_rank)
            batch["position_ids"] = TensorPointer(group_rank=input_pp_rank)
        if pp_rank == output_pp_rank:
            batch["label_ids"] = to_device(tokens[:, 1:].contiguous())
            batch["label_mask"] = to_device(torch.ones(mbs, seq, dtype=torch.bool))
        else:
            batch["label_ids"] = TensorPointer(group_rank=output_pp_rank)
            batch["label_mask"] = TensorPointer(group_rank=output_pp_rank)
        counter["batches"] += 1
        yield batch


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
        from nanotron.parallel.pipeline_parallel.utils import get_input_output_pp_ranks
        from nanotron.trainer import DistributedTrainer
    except Exception as e:  # import problems of the reference or of its dependencies
        return _unavailable(f"reference does not import here: {type(e).__name__}: {str(e)[:200]}")

    from bench import BASELINE_TOK_S_PER_GPU, MODELS, ClockSampler, layout_label, resolve_layout

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    tp, pp, dp = resolve_layout(args, world)
    if args.model == "qwen-moe":
        return _unavailable("the reference has no expert parallelism in src/ (nn/moe.py never communicates, parallel/context.py asserts tp*pp*cp*dp == world) and needs the grouped_gemm package, which cannot be installed offline")
    if world // (tp * pp * dp) > 1:
        return _unavailable("the reference cannot random-init a model under context parallelism (trainer.py:1052-1053 raises) and there is no checkpoint to load offline")
    if dp > 1 and args.model == "llama3-8b":
        # measured on this pool: with fp32 accumulation the reference's ZeRO-1 hook raises NotImplementedError
        # (optim/gradient_accumulator.py:354-355) and its replicated-optimizer path needs more than the 180 GB of a B200 for 8B parameters
        return _unavailable("the reference cannot hold a data-parallel replica of an 8B model on a 180 GB GPU (ZeRO-1 with fp32 accumulation is not implemented in its DDP hook; the replicated optimizer runs out of memory)")
    layout_note = None
    if pp > 1:
        # The reference's only model that random-initialises on its stock path, Qwen2, cannot run on more than one pipeline stage:
        # Qwen2Model.forward calls position_ids.numel() on every stage (models/qwen.py:766) while its data path hands every stage
        # but the first a TensorPointer (data/dataloader.py:164-166, data/clm_collator.py:194), so stage 1 raises
        # AttributeError: 'TensorPointer' object has no attribute 'numel' and stage 0 waits for it forever (seen on 8 GPUs at
        # tp4 x pp2).  The arm therefore spends the same GPUs on the layout it can run: tensor parallelism over all of them.
        layout_note = f"requested tp{tp}xpp{pp}; the reference's Qwen2 model raises AttributeError on pipeline stages > 0 (models/qwen.py:766), so its arm runs tp{tp * pp}"
        tp, pp = tp * pp, 1
    m = dict(MODELS[args.model])
    if m["num_key_value_heads"] % tp or m["num_attention_heads"] % tp:
        return _unavailable(f"the reference cannot split {m['num_key_value_heads']} key/value heads over tp={tp}")
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
        parallelism=ParallelismArgs(dp=dp, pp=pp, tp=tp, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=tp > 1, recompute_layer=bool(args.recompute)),
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

    guard = _Guard(deadline_s=float(os.environ.get("NTB_REFERENCE_DEADLINE_S", "300")))
    guard.start()
    try:
        trainer = TimedTrainer(cfg_path)
        input_pp_rank, output_pp_rank = get_input_output_pp_ranks(model=trainer.model)
        h2d = {"bytes": 0, "batches": 0}
        dataloader = _host_batches(trainer, input_pp_rank, output_pp_rank, h2d)
        trainer.train({"bench": dataloader})
    except torch.cuda.OutOfMemoryError as e:
        return guard.fail(f"reference ran out of GPU memory on this config: {str(e)[:160]}")
    except Exception as e:
        import traceback

        traceback.print_exc(file=sys.stderr)
        return guard.fail(f"reference failed on its stock path: {type(e).__name__}: {str(e)[:300]}")
    guard.stop()
    ms = torch.tensor([state["start"].elapsed_time(state["end"])], dtype=torch.float64, device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    tokens_per_step = args.mbs * args.seq * args.accum * dp
    value = tokens_per_step / (ms / args.steps / 1000.0)
    per_batch = torch.tensor([h2d["bytes"] / max(h2d["batches"], 1)], dtype=torch.float64, device="cuda")
    dist.all_reduce(per_batch, op=dist.ReduceOp.MAX)  # the rank that feeds both inputs and labels (or the larger of the two stages)
    h2d_per_step = int(per_batch.item()) * args.accum
    if rank == 0:
        out = {
            "metric": "Llama-3-8B training tokens/sec (whole job), bf16, seq 4096" if args.model == "llama3-8b" else f"{args.model} training tokens/sec",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak" if dp == world else "strong", "vs_baseline": value / world / BASELINE_TOK_S_PER_GPU if args.model == "llama3-8b" else None,
            "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights", "impl": "reference", "tokens_per_sec_per_gpu": value / world,
            "config": {"model": args.model, "global_batch": args.mbs * args.accum * dp, "seq_len": args.seq, "micro_batch": args.mbs, "grad_accum": args.accum,
                       "parallelism": layout_label(tp, pp, dp, 0), **({"layout_note": layout_note} if layout_note else {}), "fp32_grad_accum": True, "fp32_master_weights": True, "optimizer": "AdamW", "clip_grad": 1.0,
                       "recompute_layer": bool(args.recompute), "l2": "inputs larger than L2 (per-step working set is tens of GB); no explicit flush"},
            "clocks": state["clocks"],
            "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms / args.steps, "h2d_bytes_per_step": h2d_per_step, "d2h_bytes_per_step": 4,
                    "note": "the reference's training loop has one mode: inputs copied from pinned host memory every micro-batch, loss read on the host every step; value and e2e are the same measurement"},
            "gpu_launches": 0,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
        }
        print(json.dumps(out), flush=True)
    return 0
