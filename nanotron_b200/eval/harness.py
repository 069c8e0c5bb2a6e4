"""Log-likelihood evaluation of multiple-choice tasks with this framework's own models (no external evaluation package).

``LogLikelihoodScorer`` turns (prompt, continuation) pairs into summed log-probabilities of the continuation tokens: prompts and
continuations are tokenised separately, concatenated, left-padded into batches and pushed through the model exactly as generation
does (pipeline stages exchange activations through ``PipelineEvalBatchState``; the last stage holds the vocabulary-sharded logits,
whose per-token cross entropy is computed without gathering the vocabulary).  ``evaluate_task`` applies the task's prompt
formulation to every document and aggregates accuracy under the token / character / PMI normalisations.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.eval.evaluation_tasks import EvalTask, Request, accuracy, aggregate, build_request, choice_scores
from nanotron_b200.generation.decode import _forward_logits, _model_takes_position_ids
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.pipeline_parallel.context_manager import attach_pipeline_state_to_model
from nanotron_b200.parallel.pipeline_parallel.state import PipelineEvalBatchState
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer
from nanotron_b200.parallel.tensor_parallel.functional import sharded_cross_entropy


class LogLikelihoodScorer:
    def __init__(self, model, parallel_context: ParallelContext, tokenizer, max_length: int = 2048, batch_size: int = 8):
        """``model``: the bare transformer (``trainer.unwrapped_model.model``).  ``tokenizer``: anything with
        ``encode(text, add_special_tokens=False) -> List[int]`` (a HuggingFace tokenizer, or a test double)."""
        self.model, self.ctx, self.tok = model, parallel_context, tokenizer
        self.max_length, self.batch_size = max_length, batch_size
        self.takes_pos = _model_takes_position_ids(model)

    def _encode(self, text: str) -> List[int]:
        try:
            return list(self.tok.encode(text, add_special_tokens=False))
        except TypeError:
            return list(self.tok.encode(text))

    @torch.inference_mode()
    def loglikelihoods(self, pairs: Sequence[Tuple[str, str]]) -> List[Tuple[float, int]]:
        """For every (context, continuation): (sum of log p(continuation token | everything before it), number of continuation
        tokens).  The same values on every rank."""
        ctx, device = self.ctx, self.ctx.device
        pp_pg = ctx.pp_pg
        last = pp_pg.size() - 1
        is_first, is_last = dist.get_rank(pp_pg) == 0, dist.get_rank(pp_pg) == last
        encoded = []
        for context, continuation in pairs:
            c, t = self._encode(context), self._encode(continuation)
            assert len(t) > 0, f"empty continuation after tokenisation: {continuation!r}"
            c = c if c else [getattr(self.tok, "bos_token_id", None) or 0]
            keep = self.max_length - len(t)
            assert keep >= 1, "continuation longer than max_length"
            encoded.append((c[-keep:], t))
        order = sorted(range(len(encoded)), key=lambda i: -(len(encoded[i][0]) + len(encoded[i][1])))  # similar lengths share a batch
        results: List[Optional[Tuple[float, int]]] = [None] * len(encoded)
        was_training = self.model.training
        self.model.eval()
        state = PipelineEvalBatchState()
        with attach_pipeline_state_to_model(self.model, state):
            for start in range(0, len(order), self.batch_size):
                idx = order[start : start + self.batch_size]
                rows = [encoded[i][0] + encoded[i][1] for i in idx]
                width = max(len(r) for r in rows)
                ids = torch.zeros((len(rows), width), dtype=torch.long)
                mask = torch.zeros((len(rows), width), dtype=torch.bool)
                for r, row in enumerate(rows):  # left padding, as in generation
                    ids[r, width - len(row) :] = torch.tensor(row)
                    mask[r, width - len(row) :] = True
                ids, mask = ids.to(device), mask.to(device)
                second = (mask.long().cumsum(-1) - 1).clamp_(min=0) if self.takes_pos else mask
                logits = _forward_logits(self.model, ids if is_first else TensorPointer(0), second if is_first else TensorPointer(0), self.takes_pos)
                sums = torch.zeros(len(rows), dtype=torch.float32, device=device)
                if is_last:
                    # position p predicts token p + 1: score the continuation tokens only
                    targets = torch.roll(ids, shifts=-1, dims=1).reshape(-1)
                    nll = sharded_cross_entropy(logits.reshape(ids.numel(), -1), targets.contiguous(), group=ctx.tp_pg, dtype=torch.float).view(len(rows), width)
                    for r, i in enumerate(idx):
                        n = len(encoded[i][1])
                        sums[r] = -nll[r, width - n - 1 : width - 1].sum()
                if pp_pg.size() > 1:
                    dist.broadcast(sums, src=dist.get_global_rank(pp_pg, last), group=pp_pg)
                for r, i in enumerate(idx):
                    results[i] = (float(sums[r]), len(encoded[i][1]))
        self.model.train(was_training)
        return results  # type: ignore[return-value]

    def score_request(self, request: Request, with_pmi: bool = True) -> Dict[str, List[float]]:
        pairs = [(request.prompt, c) for c in request.continuations]
        if with_pmi:
            pairs += [(request.unconditioned_prompt, c) for c in request.continuations]
        out = self.loglikelihoods(pairs)
        n = len(request.continuations)
        return choice_scores([o[0] for o in out[:n]], request.continuations, [o[1] for o in out[:n]], [o[0] for o in out[n:]] if with_pmi else None)


def evaluate_task(scorer: LogLikelihoodScorer, task: EvalTask, lines: Iterable[Dict[str, Any]], few_shot_lines: Sequence[Dict[str, Any]] = (), max_samples: Optional[int] = None) -> Dict[str, float]:
    per_doc = []
    for n, line in enumerate(lines):
        if max_samples is not None and n >= max_samples:
            break
        request = build_request(task, line, few_shots=few_shot_lines)
        scores = scorer.score_request(request, with_pmi="acc_pmi" in task.metrics)
        per_doc.append({k: v for k, v in accuracy(scores, request.gold_idx).items() if k in task.metrics})
    out = aggregate(per_doc)
    out["num_samples"] = float(len(per_doc))
    return out
