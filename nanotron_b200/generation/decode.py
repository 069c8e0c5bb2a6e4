"""Autoregressive decoding through the pipeline (capability parity: reference src/nanotron/generation/decode.py).

``decode_tokenized`` takes left-padded ``input_ids`` / ``input_mask`` and generates up to ``max_new_tokens`` tokens;
``decode_text`` tokenises ``GenerationInput`` items, batches them and yields ``GenerationOutput`` objects.
Every pipeline rank runs the same loop: the model call moves activations stage to stage (``PipelineEvalBatchState``),
the last stage samples, and the new tokens are broadcast over the pipeline group so the first stage can embed them.
With ``use_cache`` each attention layer keeps its keys/values in a ``Store`` (Llama models), so a step only runs the new
token; without it the whole prefix is recomputed each step (what the reference does for text decoding).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Dict, Generator, Iterable, List, Optional, Union

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.config import GenerationArgs
from nanotron_b200.config.utils_config import SamplerType
from nanotron_b200.generation.generate_store import Store, attach_store
from nanotron_b200.generation.sampler import BasicSampler, GreedySampler, TopKSampler, TopPSampler
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.pipeline_parallel.context_manager import attach_pipeline_state_to_model
from nanotron_b200.parallel.pipeline_parallel.state import PipelineEvalBatchState
from nanotron_b200.logging import log_rank
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

logger = logging.get_logger(__name__)


@dataclasses.dataclass
class GenerationInput:
    text: str


@dataclasses.dataclass
class GenerationInputs:
    input_ids: Union[torch.Tensor, TensorPointer]  # [b, s]
    input_masks: Union[torch.Tensor, TensorPointer]


@dataclasses.dataclass
class GenerationOutput:
    input_ids: Union[torch.Tensor, TensorPointer]
    generation_ids: Union[torch.Tensor, TensorPointer]
    return_logits: Optional[Union[torch.Tensor, TensorPointer]] = None


@dataclasses.dataclass
class TokenizerConfig:
    max_input_length: Optional[int]
    truncation: Optional[Union[str, bool]] = None
    padding: Optional[Union[str, bool]] = None


def chunks(iterable, chunk_size: int) -> Generator[List, None, None]:
    assert chunk_size >= 1
    chunk = []
    for item in iterable:
        chunk.append(item)
        if len(chunk) == chunk_size:
            yield chunk
            chunk = []
    if chunk:
        yield chunk


def _make_sampler(cfg: Optional[GenerationArgs], tp_pg):
    kind = cfg.sampler if cfg is not None and cfg.sampler is not None else SamplerType.GREEDY
    if isinstance(kind, str):
        kind = SamplerType[kind.upper()]
    if kind == SamplerType.GREEDY:
        return GreedySampler(pg=tp_pg)
    if kind == SamplerType.TOP_K:
        return TopKSampler(pg=tp_pg, k=cfg.top_k or 50, temperature=cfg.temperature or 1.0)
    if kind == SamplerType.TOP_P:
        return TopPSampler(pg=tp_pg, p=cfg.top_p or 0.9, temperature=cfg.temperature or 1.0)
    if kind == SamplerType.BASIC:
        return BasicSampler(pg=tp_pg)
    raise NotImplementedError(f"Sampler type {kind} is not implemented")


def _model_takes_position_ids(model) -> bool:
    import inspect

    return "position_ids" in inspect.signature(model.forward).parameters


def _forward_logits(model, input_ids, mask_or_pos, takes_pos: bool):
    if takes_pos:
        out = model(input_ids=input_ids, position_ids=mask_or_pos)
    else:
        out = model(input_ids=input_ids, input_mask=mask_or_pos)
    return out[0] if isinstance(out, tuple) else out


@torch.inference_mode()
def decode_tokenized(
    input_ids: torch.Tensor,
    input_mask: torch.Tensor,
    model,
    parallel_context: ParallelContext,
    generation_config: Optional[GenerationArgs] = None,
    max_new_tokens: int = 16,
    use_cache: bool = False,
    eos_token_id: Optional[int] = None,
    returns_logits: bool = False,
    is_bench: bool = False,
) -> GenerationOutput:
    """``model`` is the bare transformer (``trainer.unwrapped_model.model``).  Inputs are [b, s], left padded, present on
    every rank (tiny).  Returns the generated ids [b, <= max_new_tokens] on every rank.  ``is_bench`` logs the decoding
    throughput of the call (the first step, which reads the whole prompt, is timed apart; reference generation/decode.py:277-449)."""
    ctx = parallel_context
    device = ctx.device
    input_ids, input_mask = input_ids.to(device), input_mask.to(device).bool()
    pp_pg = ctx.pp_pg
    last = pp_pg.size() - 1
    is_first, is_last = dist.get_rank(pp_pg) == 0, dist.get_rank(pp_pg) == last
    sampler = _make_sampler(generation_config, ctx.tp_pg)
    takes_pos = _model_takes_position_ids(model)
    if takes_pos:
        use_cache = False
    b = input_ids.shape[0]
    was_training = model.training
    model.eval()
    generated = torch.empty((b, 0), dtype=torch.long, device=device)
    finished = torch.zeros(b, dtype=torch.bool, device=device)
    all_logits = []
    store = Store()
    cur_ids, cur_mask = input_ids, input_mask
    state = PipelineEvalBatchState()
    with attach_pipeline_state_to_model(model, state), (attach_store(model, store) if use_cache else _null()):
        clock = _DecodeClock(device) if is_bench else None
        for step in range(max_new_tokens):
            if clock is not None:
                clock.step_begins(step)
            if use_cache and step > 0:
                step_ids, step_mask = generated[:, -1:], torch.ones((b, 1), dtype=torch.bool, device=device)
            else:
                step_ids, step_mask = cur_ids, cur_mask
            if takes_pos:
                second = (step_mask.long().cumsum(-1) - 1).clamp_(min=0)
            else:
                second = step_mask
            ids_arg = step_ids if is_first else TensorPointer(0)
            sec_arg = second if is_first else TensorPointer(0)
            logits = _forward_logits(model, ids_arg, sec_arg, takes_pos)
            new_tokens = torch.empty((b, 1), dtype=torch.long, device=device)
            if is_last:
                q = step_ids.shape[1]
                rows = logits.view(b, q, -1)
                # left padding: the last position of every row is its newest real token
                last_logits = rows[:, -1, :]
                if returns_logits:
                    all_logits.append(last_logits.float())
                new_tokens = sampler(last_logits).to(torch.long)
            if pp_pg.size() > 1:
                dist.broadcast(new_tokens, src=dist.get_global_rank(pp_pg, last), group=pp_pg)
            if eos_token_id is not None:
                new_tokens = torch.where(finished.unsqueeze(1), torch.full_like(new_tokens, eos_token_id), new_tokens)
                finished |= new_tokens.squeeze(1) == eos_token_id
            generated = torch.cat([generated, new_tokens], dim=1)
            cur_ids = torch.cat([cur_ids, new_tokens], dim=1)
            cur_mask = torch.cat([cur_mask, torch.ones((b, 1), dtype=torch.bool, device=device)], dim=1)
            if eos_token_id is not None and bool(finished.all()):
                break
    if clock is not None:
        clock.report(batch=b, steps=generated.shape[1], replicas=ctx.dp_pg.size(), world=ctx.world_pg.size(), use_cache=use_cache)
    model.train(was_training)
    return GenerationOutput(input_ids=input_ids, generation_ids=generated, return_logits=torch.stack(all_logits, 1) if all_logits else None)


class _DecodeClock:
    """Wall-clock of a decoding loop, synchronised with the device at the two points that are read."""

    def __init__(self, device):
        self.device = device
        self.start = self.after_first = None
        self.last: Optional[Dict[str, float]] = None

    def _now(self) -> float:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        return time.perf_counter()

    def step_begins(self, step: int):
        if step == 0:
            self.start = self._now()
        elif step == 1:
            self.after_first = self._now()

    def report(self, batch: int, steps: int, replicas: int, world: int, use_cache: bool):
        end = self._now()
        first = (self.after_first if self.after_first is not None else end) - self.start
        rest = end - (self.after_first if self.after_first is not None else end)
        later_steps = max(steps - 1, 0)
        tokens_per_sec = batch * replicas * later_steps / rest if rest > 0 and later_steps else 0.0
        self.last = {"first_step_s": first, "later_steps_s": rest, "tokens_per_sec": tokens_per_sec, "tokens_per_sec_per_gpu": tokens_per_sec / world}
        _DecodeClock.last_report = self.last
        log_rank(
            f"[decode bench] batch {batch} x {steps} new tokens ({'cached' if use_cache else 'recomputed'} keys / values): first step {first * 1e3:.1f} ms, "
            f"{later_steps} later steps {rest * 1e3:.1f} ms -> {tokens_per_sec:.1f} tokens/s ({tokens_per_sec / world:.1f} per process)",
            logger=logger, level=logging.INFO, rank=0,
        )


class _null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


@torch.inference_mode()
def decode_text(
    input_iter: Iterable[GenerationInput],
    tokenizer,
    model,
    parallel_context: ParallelContext,
    max_new_tokens: int,
    max_micro_batch_size: int,
    generation_config: Optional[GenerationArgs] = None,
    tokenizer_config: Optional[TokenizerConfig] = None,
    returns_logits: bool = False,
    use_cache: bool = False,
    is_bench: bool = False,
) -> Generator[GenerationOutput, None, None]:
    """Yields one ``GenerationOutput`` per input text (ids are trimmed of padding)."""
    if getattr(tokenizer, "pad_token_id", None) is None:
        tokenizer.pad_token_id = tokenizer.eos_token_id if getattr(tokenizer, "eos_token_id", None) is not None else 0
    tokenizer.padding_side = "left"
    for batch in chunks(input_iter, max_micro_batch_size):
        enc = tokenizer(
            [e.text for e in batch], return_tensors="pt", return_attention_mask=True, padding=True if tokenizer_config is None or tokenizer_config.padding is None else tokenizer_config.padding,
            truncation=tokenizer_config.truncation if tokenizer_config is not None and tokenizer_config.truncation is not None else False,
            max_length=tokenizer_config.max_input_length if tokenizer_config is not None else None,
        )
        out = decode_tokenized(
            enc["input_ids"], enc["attention_mask"], model=model, parallel_context=parallel_context, generation_config=generation_config,
            max_new_tokens=max_new_tokens, use_cache=use_cache, eos_token_id=getattr(tokenizer, "eos_token_id", None), returns_logits=returns_logits, is_bench=is_bench,
        )
        mask = enc["attention_mask"].bool()
        for i in range(len(batch)):
            yield GenerationOutput(
                input_ids=out.input_ids[i][mask[i].to(out.input_ids.device)], generation_ids=out.generation_ids[i],
                return_logits=out.return_logits[i] if out.return_logits is not None else None,
            )
