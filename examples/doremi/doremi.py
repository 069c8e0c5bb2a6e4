"""DoReMi (domain reweighting with minimax optimisation) on top of the framework's extension points
(capability parity: reference examples/doremi/doremi/{config,doremi_context,loss,llama,trainer}.py; the domain-weighted
sampler and collator live in ``dataloader.py`` beside this file).

A small *proxy* model is trained with a loss that re-weights data domains; the weights follow the per-domain *excess loss*
of the proxy over a frozen *reference* model:

    excess_d = mean over tokens of domain d of  max(loss_proxy - loss_reference, 0)
    w       <- w * exp(step_size * excess)          (then normalise, then mix with the uniform distribution: smoothing)
    loss     = sum_d  w_d * (sum of proxy token losses of domain d) / (tokens of the batch)

What this file shows about the framework:
  * ``DoReMiConfig`` extends ``Config`` with a ``doremi`` section and is handed to the trainer as ``config_class``;
  * ``LlamaForDoReMiTraining`` reuses the stock Llama decoder and replaces only the loss ``PipelineBlock``; the trainer gets it
    as ``model_class`` (the batch carries two extra keys, ``domain_idxs`` and ``ref_losses``);
  * ``DoReMiTrainer`` subclasses ``DistributedTrainer``: ``_init_model_instance`` builds the frozen reference model next to the
    proxy, and the dataloader is wrapped so every micro-batch is scored by the reference first; the history of the domain
    weights is written beside every checkpoint (``doremi_domain_weights_<step>.pt``) and read back on resume;
  * ``ReferenceTrainer`` trains a plain model on a fixed mixture (step 1 and step 4 of the recipe) and logs the loss of every
    domain.
Pipeline parallelism is not supported by this example (the reference model's per-token losses are fed back as an input).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Union

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.config import Config
from nanotron_b200.logging import log_rank
from nanotron_b200.models.llama import LlamaForTraining
from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock
from nanotron_b200.parallel.tensor_parallel.functional import sharded_cross_entropy
from nanotron_b200.serialize import load_weights
from nanotron_b200.trainer import DistributedTrainer

logger = logging.get_logger(__name__)


# ---------------------------------------------------------------------------- configuration
@dataclass
class DoReMiArgs:
    domain_names: Union[List[str], str] = field(default_factory=lambda: ["a", "b"])  # a comma-separated string also works
    domain_weights: Optional[List[float]] = None  # initial weights (uniform when omitted)
    step_size: float = 1.0
    smoothing_param: float = 1e-3
    ref_model_resume_checkpoint_path: Optional[str] = None  # weights of the reference model; None: random init with ref_model_seed
    ref_model_seed: int = 1234
    # True: the sampler follows the weights as they move (what the reference implementation does); False: the mixture of the
    # batches stays at the initial weights and only the loss is re-weighted (Algorithm 1 of the paper)
    sample_with_current_weights: bool = False
    # one folder of tokenised ``.ds`` files per domain (same order as domain_names); None: the synthetic domains of ``utils.py``
    domain_folders: Optional[List[str]] = None
    token_size: int = 2  # bytes per token in those files
    samples_per_synthetic_domain: int = 4096

    def __post_init__(self):
        if isinstance(self.domain_names, str):
            self.domain_names = [name.strip() for name in self.domain_names.split(",")]
        if self.domain_folders is not None:
            assert len(self.domain_folders) == len(self.domain_names), "one folder per domain"
        if self.domain_weights is not None:
            assert len(self.domain_weights) == len(self.domain_names)
            assert abs(sum(self.domain_weights) - 1.0) < 1e-3, "domain weights must sum to 1"


@dataclass
class DoReMiConfig(Config):
    doremi: Optional[DoReMiArgs] = None


class DoReMiContext:
    """Current domain weights (same values on every rank) and their history."""

    def __init__(self, args: DoReMiArgs, device):
        n = len(args.domain_names)
        w = torch.tensor(args.domain_weights, dtype=torch.float32) if args.domain_weights is not None else torch.full((n,), 1.0 / n)
        self.domain_names = list(args.domain_names)
        self.domain_weights = w.to(device)
        self.step_size, self.smoothing_param = args.step_size, args.smoothing_param
        self.history: List[torch.Tensor] = [self.domain_weights.clone()]

    @property
    def num_domains(self) -> int:
        return len(self.domain_names)

    def history_records(self) -> List[Dict[str, object]]:
        return [{"update": i, "domain_names": self.domain_names, "domain_weights": w.detach().cpu()} for i, w in enumerate(self.history)]

    def load_history(self, records: List[Dict[str, object]]) -> None:
        assert list(records[0]["domain_names"]) == self.domain_names, "the saved weights belong to other domains"
        device = self.domain_weights.device
        self.history = [r["domain_weights"].to(device) for r in records]
        self.domain_weights = self.history[-1].clone()

    def update(self, excess_per_domain: torch.Tensor):
        w = self.domain_weights * torch.exp(self.step_size * excess_per_domain)
        w = w / w.sum()
        uniform = torch.full_like(w, 1.0 / w.numel())
        self.domain_weights = (1 - self.smoothing_param) * w + self.smoothing_param * uniform
        self.history.append(self.domain_weights.clone())


# ---------------------------------------------------------------------------- losses
def per_token_losses(sharded_logits: torch.Tensor, label_ids: torch.Tensor, tp_pg) -> torch.Tensor:
    """[b, s] cross entropy of every token (fp32), from vocabulary-sharded logits [b*s, V/tp]."""
    loss = sharded_cross_entropy(sharded_logits, label_ids.reshape(-1).contiguous(), group=tp_pg, dtype=torch.float)
    return loss.view(label_ids.shape)


class ReferenceLoss(nn.Module):
    """Loss block of the frozen reference model: returns the token losses instead of their mean."""

    def __init__(self, tp_pg):
        super().__init__()
        self.tp_pg = tp_pg

    def forward(self, sharded_logits, label_ids, label_mask):
        losses = per_token_losses(sharded_logits, label_ids, self.tp_pg)
        return {"losses": losses * label_mask}


class DoReMiLoss(nn.Module):
    """Loss block of the proxy model: domain-weighted cross entropy; the weights are updated from the excess loss of this batch
    (summed over the data-parallel group so every rank applies the same update)."""

    def __init__(self, tp_pg, dp_pg, doremi_context: DoReMiContext):
        super().__init__()
        self.tp_pg, self.dp_pg, self.ctx = tp_pg, dp_pg, doremi_context

    def forward(self, sharded_logits, label_ids, label_mask, domain_idxs, ref_losses):
        losses = per_token_losses(sharded_logits, label_ids, self.tp_pg) * label_mask  # [b, s]
        n = self.ctx.num_domains
        dom = domain_idxs.reshape(-1).long()
        training_forward = self.training and torch.is_grad_enabled()
        with torch.no_grad():
            excess = (losses.detach() - ref_losses).clamp_(min=0).sum(-1)  # [b]
            tokens = label_mask.sum(-1).float()
            stats = torch.zeros(2, n, dtype=torch.float32, device=losses.device)
            stats[0].index_add_(0, dom, excess)
            stats[1].index_add_(0, dom, tokens)
            if self.dp_pg is not None and self.dp_pg.size() > 1:
                dist.all_reduce(stats, group=self.dp_pg)
            excess_per_domain = torch.where(stats[1] > 0, stats[0] / stats[1].clamp(min=1), torch.zeros_like(stats[0]))
            if training_forward:
                self.ctx.update(excess_per_domain)
            weights = self.ctx.domain_weights
        sample_loss = losses.sum(-1)  # [b]
        weighted = (weights[dom] * sample_loss).sum() * n / label_mask.sum().clamp(min=1)  # equals the plain mean for uniform weights
        ce = sample_loss.sum().detach() / label_mask.sum().clamp(min=1)
        return {"loss": weighted, "ce_loss": ce, "excess_losses": excess_per_domain}


# ---------------------------------------------------------------------------- models
class LlamaReferenceForDoReMi(LlamaForTraining):
    """Frozen scorer: ``forward`` returns the per-token losses of a micro-batch."""

    def __init__(self, config, parallel_context, parallel_config, random_states=None):
        super().__init__(config=config, parallel_context=parallel_context, parallel_config=parallel_config, random_states=random_states)
        self.loss = PipelineBlock(
            p2p=self.model.p2p, module_builder=ReferenceLoss, module_kwargs={"tp_pg": parallel_context.tp_pg},
            module_input_keys={"sharded_logits", "label_ids", "label_mask"}, module_output_keys={"losses"},
        )

    def forward(self, input_ids, input_mask, label_ids, label_mask):
        logits = self.model(input_ids=input_ids, input_mask=input_mask)
        return self.loss(sharded_logits=logits, label_ids=label_ids, label_mask=label_mask)


class PerDomainLoss(nn.Module):
    """Plain mean cross entropy (what is optimised) plus the loss sum and token count of every domain (what is logged)."""

    def __init__(self, tp_pg, num_domains: int):
        super().__init__()
        self.tp_pg, self.num_domains = tp_pg, num_domains

    def forward(self, sharded_logits, label_ids, label_mask, domain_idxs):
        losses = per_token_losses(sharded_logits, label_ids, self.tp_pg) * label_mask
        loss = losses.sum() / label_mask.sum().clamp(min=1)
        with torch.no_grad():
            dom = domain_idxs.reshape(-1).long()
            sums = torch.zeros(self.num_domains, dtype=torch.float32, device=losses.device).index_add_(0, dom, losses.detach().sum(-1))
            tokens = torch.zeros(self.num_domains, dtype=torch.float32, device=losses.device).index_add_(0, dom, label_mask.sum(-1).float())
        return {"loss": loss, "domain_loss_sums": sums, "domain_tokens": tokens}


class LlamaForReferenceTraining(LlamaForTraining):
    """The stock Llama trained on a fixed mixture; its loss block also reports every domain's loss."""

    num_domains: Optional[int] = None  # set by ReferenceTrainer before the model is built

    def __init__(self, config, parallel_context, parallel_config, random_states=None):
        super().__init__(config=config, parallel_context=parallel_context, parallel_config=parallel_config, random_states=random_states)
        assert type(self).num_domains is not None, "ReferenceTrainer sets LlamaForReferenceTraining.num_domains before building the model"
        self.loss = PipelineBlock(
            p2p=self.model.p2p, module_builder=PerDomainLoss, module_kwargs={"tp_pg": parallel_context.tp_pg, "num_domains": type(self).num_domains},
            module_input_keys={"sharded_logits", "label_ids", "label_mask", "domain_idxs"}, module_output_keys={"loss", "domain_loss_sums", "domain_tokens"},
        )

    def forward(self, input_ids, input_mask, label_ids, label_mask, domain_idxs):
        logits = self.model(input_ids=input_ids, input_mask=input_mask)
        return self.loss(sharded_logits=logits, label_ids=label_ids, label_mask=label_mask, domain_idxs=domain_idxs)


class LlamaForDoReMiTraining(LlamaForTraining):
    doremi_context: Optional[DoReMiContext] = None  # set by the trainer before the model is built

    def __init__(self, config, parallel_context, parallel_config, random_states=None):
        super().__init__(config=config, parallel_context=parallel_context, parallel_config=parallel_config, random_states=random_states)
        assert type(self).doremi_context is not None, "DoReMiTrainer sets LlamaForDoReMiTraining.doremi_context before building the model"
        self.loss = PipelineBlock(
            p2p=self.model.p2p, module_builder=DoReMiLoss,
            module_kwargs={"tp_pg": parallel_context.tp_pg, "dp_pg": parallel_context.dp_pg, "doremi_context": type(self).doremi_context},
            module_input_keys={"sharded_logits", "label_ids", "label_mask", "domain_idxs", "ref_losses"},
            module_output_keys={"loss", "ce_loss", "excess_losses"},
        )

    def forward(self, input_ids, input_mask, label_ids, label_mask, domain_idxs, ref_losses):
        logits = self.model(input_ids=input_ids, input_mask=input_mask)
        return self.loss(sharded_logits=logits, label_ids=label_ids, label_mask=label_mask, domain_idxs=domain_idxs, ref_losses=ref_losses)


# ---------------------------------------------------------------------------- trainer
class DoReMiTrainer(DistributedTrainer):
    def __init__(self, config_or_config_file: Union[DoReMiConfig, str]):
        super().__init__(config_or_config_file, config_class=DoReMiConfig, model_class=LlamaForDoReMiTraining)

    def pre_init(self):
        super().pre_init()
        assert self.config.doremi is not None, "the config needs a `doremi` section"
        assert self.parallel_context.pp_pg.size() == 1, "the DoReMi example feeds reference losses back as an input: pp must be 1"
        self.doremi_context = DoReMiContext(self.config.doremi, self.parallel_context.device)
        LlamaForDoReMiTraining.doremi_context = self.doremi_context

    def _init_model_instance(self):
        model = super()._init_model_instance()  # the proxy (model_class was registered by __init__)
        args = self.config.doremi
        self.ref_model = self._init_model(model_builder=lambda: LlamaReferenceForDoReMi(config=self.model_config, parallel_context=self.parallel_context, parallel_config=self.config.parallelism, random_states=self.random_states))
        if args.ref_model_resume_checkpoint_path is not None:
            log_rank(f"[DoReMi] loading the reference model from {args.ref_model_resume_checkpoint_path}", logger=logger, level=logging.INFO, rank=0)
            load_weights(model=self.ref_model, parallel_context=self.parallel_context, root_folder=args.ref_model_resume_checkpoint_path)
        else:
            state = torch.random.get_rng_state()
            torch.manual_seed(args.ref_model_seed + dist.get_rank(self.parallel_context.tp_pg))
            self.ref_model.init_model_randomly(config=self.config)
            torch.random.set_rng_state(state)
            self._sync_initial_parameters(self.ref_model)
        self.ref_model.eval()
        for p in self.ref_model.parameters():
            p.requires_grad_(False)
        return model

    def _score_with_reference(self, batches: Iterator[Dict]) -> Iterator[Dict]:
        for batch in batches:
            with torch.no_grad():
                out = self.ref_model(input_ids=batch["input_ids"], input_mask=batch["input_mask"], label_ids=batch["label_ids"], label_mask=batch["label_mask"])
            yield {**batch, "ref_losses": out["losses"].detach()}

    def _wrap(self, dl):
        return self._score_with_reference(super()._wrap(dl))

    def sampling_weights(self) -> torch.Tensor:
        """What a ``dataloader.DomainWeightedSampler`` of this run follows (its ``weights_fn``)."""
        if self.config.doremi.sample_with_current_weights:
            return self.doremi_context.domain_weights
        return self.doremi_context.history[0]

    def train_step_logs(self, outputs, loss_avg, z_loss_avg=None):
        super().train_step_logs(outputs=outputs, loss_avg=loss_avg, z_loss_avg=z_loss_avg)
        w = ", ".join(f"{n}={float(v):.4f}" for n, v in zip(self.doremi_context.domain_names, self.doremi_context.domain_weights))
        log_rank(f"[DoReMi] domain weights: {w}", logger=logger, level=logging.INFO, rank=0)

    # the weights are the product of proxy training: one file per checkpoint with every value they took so far
    def post_init(self):
        super().post_init()
        if self.init_checkpoint_path is not None:
            path = _weights_file(self.init_checkpoint_path.parent, self.metadata.last_train_step)
            if path.exists():
                self.doremi_context.load_history(torch.load(path, map_location="cpu"))
                log_rank(f"[DoReMi] resumed the domain weights from {path}", logger=logger, level=logging.INFO, rank=0)

    def post_save_checkpoint(self):
        if dist.get_rank(self.parallel_context.world_pg) == 0:
            torch.save(self.doremi_context.history_records(), _weights_file(self.config.checkpoints.checkpoints_path, self.iteration_step))
        super().post_save_checkpoint()


def _weights_file(checkpoints_path, step: int):
    from pathlib import Path

    return Path(checkpoints_path) / f"doremi_domain_weights_{step}.pt"


def average_domain_weights(path) -> torch.Tensor:
    """The tuned mixture: the mean of the weights over all updates of a proxy run (what the larger run is trained with)."""
    records = torch.load(path, map_location="cpu")
    return torch.stack([r["domain_weights"] for r in records]).mean(0)


class ReferenceTrainer(DistributedTrainer):
    """Training on a fixed mixture of the domains with per-domain loss logging: the small reference model of step 1, and the
    large model of step 4 with the tuned weights (capability parity: reference examples/doremi/doremi/trainer.py:200-270)."""

    def __init__(self, config_or_config_file: Union[DoReMiConfig, str], domain_weights: Optional[torch.Tensor] = None):
        self._given_weights = domain_weights
        super().__init__(config_or_config_file, config_class=DoReMiConfig, model_class=LlamaForReferenceTraining)

    def pre_init(self):
        super().pre_init()
        assert self.config.doremi is not None, "the config needs a `doremi` section"
        self.doremi_context = DoReMiContext(self.config.doremi, self.parallel_context.device)
        if self._given_weights is not None:  # e.g. weights from the token counts of the datasets
            w = torch.as_tensor(self._given_weights, dtype=torch.float32, device=self.parallel_context.device)
            assert w.numel() == self.doremi_context.num_domains and abs(float(w.sum()) - 1.0) < 1e-3
            self.doremi_context.domain_weights = w
            self.doremi_context.history = [w.clone()]
        LlamaForReferenceTraining.num_domains = self.doremi_context.num_domains
        self.domain_losses: Optional[torch.Tensor] = None

    def sampling_weights(self) -> torch.Tensor:
        return self.doremi_context.domain_weights

    def train_step_logs(self, outputs, loss_avg, z_loss_avg=None):
        super().train_step_logs(outputs=outputs, loss_avg=loss_avg, z_loss_avg=z_loss_avg)
        if not isinstance(outputs[0]["loss"], torch.Tensor):
            return  # not the pipeline rank that holds the loss
        stats = torch.stack([torch.stack([o["domain_loss_sums"] for o in outputs]).sum(0), torch.stack([o["domain_tokens"] for o in outputs]).sum(0)])
        pg = self.parallel_context.dp_pg
        if pg.size() > 1:
            dist.all_reduce(stats, group=pg)
        self.domain_losses = torch.where(stats[1] > 0, stats[0] / stats[1].clamp(min=1e-9), torch.full_like(stats[0], float("nan")))
        if self.iteration_step % self.config.logging.iteration_step_info_interval == 0:
            text = ", ".join(f"{n}={float(v):.4f}" for n, v in zip(self.doremi_context.domain_names, self.domain_losses))
            log_rank(f"[DoReMi] domain losses: {text}", logger=logger, level=logging.INFO, rank=self.logger_ranks[0] if hasattr(self, "logger_ranks") else 0)
