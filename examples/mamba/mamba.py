"""Mamba (selective state-space) language model on the framework's building blocks
(capability parity: reference examples/mamba/mamba.py).

Per layer:  h <- h + Mixer(RMSNorm(h)),  Mixer(x):
    xz   = in_proj(x)                       column-parallel, the x and z halves are each split over tp
    x    = silu(causal depthwise conv(x))   per-channel, so local channels need nothing from other ranks
    dt, B, C = x_proj(x)                    row-parallel (summed over tp): these are shared by all channels
    dt   = dt_proj(dt)                      column-parallel from the replicated low-rank dt
    y    = selective_scan(x, dt, A, B, C, D, z)   independent per channel
    out  = out_proj(y)                      row-parallel
Tensor parallelism uses the all-reduce mode (the scan needs whole sequences per channel, not sequence shards); pipeline
parallelism works as for every model of the framework (each layer is a ``PipelineBlock``).  Activations travel token-flat
``[batch * seq, d_model]`` between blocks, like the framework's other models; the mixer reshapes with the batch size it reads from
``sequence_mask``.
"""
from __future__ import annotations

import math
import os
import sys
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from config import MambaModelConfig  # noqa: E402
from selective_scan import selective_scan, selective_state_update  # noqa: E402

from nanotron_b200 import distributed as dist  # noqa: E402
from nanotron_b200.config import ParallelismArgs  # noqa: E402
from nanotron_b200.models.base import NanotronModel  # noqa: E402
from nanotron_b200.models.qwen import Loss  # noqa: E402
from nanotron_b200.nn.layer_norm import TritonRMSNorm  # noqa: E402
from nanotron_b200.parallel import ParallelContext  # noqa: E402
from nanotron_b200.parallel.parameters import NanotronParameter  # noqa: E402
from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock  # noqa: E402
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P  # noqa: E402
from nanotron_b200.parallel.sharded_parameters import SplitConfig, create_sharded_parameter_from_config, mark_all_parameters_in_module_as_sharded  # noqa: E402
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode  # noqa: E402
from nanotron_b200.parallel.tensor_parallel.nn import TensorParallelColumnLinear, TensorParallelEmbedding, TensorParallelRowLinear  # noqa: E402
from nanotron_b200.random import RandomStates  # noqa: E402


class MambaMixer(nn.Module):
    def __init__(self, config: MambaModelConfig, tp_pg: dist.ProcessGroup, layer_idx: int):
        super().__init__()
        c = config.ssm()
        tp = tp_pg.size()
        self.d_model, self.d_state, self.d_conv, self.dt_rank = config.d_model, c["d_state"], c["d_conv"], c["dt_rank"]
        self.d_inner = c["expand"] * config.d_model
        assert self.d_inner % tp == 0, f"tp={tp} must divide d_inner={self.d_inner}"
        self.d_inner_local = self.d_inner // tp
        self.tp_pg, self.layer_idx, self.chunk = tp_pg, layer_idx, config.scan_chunk
        mode = TensorParallelLinearMode.ALL_REDUCE
        self.in_proj = TensorParallelColumnLinear(config.d_model, 2 * self.d_inner, pg=tp_pg, mode=mode, bias=c["bias"], contiguous_chunks=(self.d_inner, self.d_inner))
        self.conv1d = nn.Conv1d(self.d_inner_local, self.d_inner_local, kernel_size=self.d_conv, groups=self.d_inner_local, padding=self.d_conv - 1, bias=c["conv_bias"])
        mark_all_parameters_in_module_as_sharded(self.conv1d, pg=tp_pg, split_config=SplitConfig(split_dim=0))
        self.x_proj = TensorParallelRowLinear(self.d_inner, self.dt_rank + 2 * self.d_state, pg=tp_pg, mode=mode, bias=False)
        self.dt_proj = TensorParallelColumnLinear(self.dt_rank, self.d_inner, pg=tp_pg, mode=mode, bias=True)
        # A = -exp(A_log) starts at -(1 .. d_state) for every channel (the S4D-real initialisation); D is a skip gain of 1
        A_log = torch.log(torch.arange(1, self.d_state + 1, dtype=torch.float32)).repeat(self.d_inner_local, 1)
        self.A_log = create_sharded_parameter_from_config(nn.Parameter(A_log), pg=tp_pg, split_config=SplitConfig(split_dim=0))
        self.D = create_sharded_parameter_from_config(nn.Parameter(torch.ones(self.d_inner_local)), pg=tp_pg, split_config=SplitConfig(split_dim=0))
        self.out_proj = TensorParallelRowLinear(self.d_inner, config.d_model, pg=tp_pg, mode=mode, bias=c["bias"])
        self._dt_init = (c["dt_init"], c["dt_scale"], c["dt_min"], c["dt_max"], c["dt_init_floor"])

    @torch.no_grad()
    def init_dt(self):
        """dt_proj: weights so that dt starts near its fan-in scale, bias so that softplus(bias) is log-uniform in [dt_min, dt_max]."""
        kind, scale, dt_min, dt_max, floor = self._dt_init
        std = self.dt_rank**-0.5 * scale
        if kind == "constant":
            nn.init.constant_(self.dt_proj.weight, std)
        else:
            nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt = torch.exp(torch.rand(self.d_inner_local) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=floor)
        self.dt_proj.bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(self.dt_proj.bias.dtype))  # inverse of softplus

    def _ssm_inputs(self, x_flat: torch.Tensor):
        dbc = self.x_proj(x_flat)  # summed over tp: identical on every rank
        dt, B, C = torch.split(dbc, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        dt = F.linear(dt, self.dt_proj.weight)  # the bias goes into the scan, before the softplus
        return dt, B, C

    def forward(self, hidden_states: torch.Tensor, sequence_mask: torch.Tensor) -> torch.Tensor:
        b, l = sequence_mask.shape
        xz = self.in_proj(hidden_states)  # [b*l, 2 * d_inner / tp]
        x, z = xz.view(b, l, 2, self.d_inner_local).unbind(dim=2)
        x = x.transpose(1, 2)  # [b, d, l]
        x = F.silu(self.conv1d(x)[..., :l])  # padding d_conv - 1 on the left, the right overhang is cut: causal
        dt, B, C = self._ssm_inputs(x.transpose(1, 2).reshape(b * l, self.d_inner_local))
        dt = dt.view(b, l, self.d_inner_local).transpose(1, 2)
        B = B.view(b, l, self.d_state).transpose(1, 2)
        C = C.view(b, l, self.d_state).transpose(1, 2)
        y = selective_scan(x, dt, -torch.exp(self.A_log.float()), B, C, self.D.float(), z=z.transpose(1, 2), delta_bias=self.dt_proj.bias.float(), delta_softplus=True, chunk=self.chunk)
        return self.out_proj(y.transpose(1, 2).reshape(b * l, self.d_inner_local))

    # ---- decoding: one token per call, state = (last d_conv inputs of the convolution, state-space state)
    def allocate_state(self, batch: int, device, dtype):
        return torch.zeros(batch, self.d_inner_local, self.d_conv, device=device, dtype=dtype), torch.zeros(batch, self.d_inner_local, self.d_state, device=device, dtype=torch.float32)

    def step(self, hidden_states: torch.Tensor, conv_state: torch.Tensor, ssm_state: torch.Tensor):
        """hidden_states: [b, d_model] (one position).  Returns (out [b, d_model], conv_state, ssm_state)."""
        x, z = self.in_proj(hidden_states).view(-1, 2, self.d_inner_local).unbind(dim=1)
        conv_state = torch.cat([conv_state[:, :, 1:], x.unsqueeze(-1)], dim=-1)
        x = (conv_state * self.conv1d.weight.squeeze(1)).sum(-1)
        if self.conv1d.bias is not None:
            x = x + self.conv1d.bias
        x = F.silu(x)
        dt, B, C = self._ssm_inputs(x)
        y, ssm_state = selective_state_update(ssm_state, x, dt, -torch.exp(self.A_log.float()), B, C, self.D.float(), z=z, dt_bias=self.dt_proj.bias.float(), dt_softplus=True)
        return self.out_proj(y), conv_state, ssm_state


class MambaBlock(nn.Module):
    def __init__(self, config: MambaModelConfig, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, layer_idx: int):
        super().__init__()
        self.norm = TritonRMSNorm(config.d_model, eps=config.rms_norm_eps)
        self.mixer = MambaMixer(config, tp_pg, layer_idx)
        self.residual_in_fp32 = config.residual_in_fp32

    def forward(self, hidden_states: torch.Tensor, sequence_mask: torch.Tensor) -> Dict[str, torch.Tensor]:
        out = self.mixer(self.norm(hidden_states), sequence_mask)
        return {"hidden_states": hidden_states + out.to(hidden_states.dtype), "sequence_mask": sequence_mask}


class Embedding(nn.Module):
    def __init__(self, tp_pg: dist.ProcessGroup, config: MambaModelConfig):
        super().__init__()
        self.token_embedding = TensorParallelEmbedding(num_embeddings=config.vocab_size, embedding_dim=config.d_model, pg=tp_pg, mode=TensorParallelLinearMode.ALL_REDUCE)

    def forward(self, input_ids: torch.Tensor, input_mask: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {"input_embeds": self.token_embedding(input_ids.reshape(-1))}


class MambaModel(nn.Module):
    def __init__(self, config: MambaModelConfig, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs], random_states: Optional[RandomStates] = None):
        super().__init__()
        self.p2p = P2P(parallel_context.pp_pg, device=parallel_context.device)
        self.config, self.parallel_context, self.parallel_config = config, parallel_context, parallel_config
        tp_pg = parallel_context.tp_pg
        self.token_position_embeddings = PipelineBlock(p2p=self.p2p, module_builder=Embedding, module_kwargs={"tp_pg": tp_pg, "config": config}, module_input_keys={"input_ids", "input_mask"}, module_output_keys={"input_embeds"})
        self.decoder = nn.ModuleList(
            [
                PipelineBlock(p2p=self.p2p, module_builder=MambaBlock, module_kwargs={"config": config, "parallel_config": parallel_config, "tp_pg": tp_pg, "layer_idx": i}, module_input_keys={"hidden_states", "sequence_mask"}, module_output_keys={"hidden_states", "sequence_mask"})
                for i in range(config.num_hidden_layers)
            ]
        )
        self.final_layer_norm = PipelineBlock(p2p=self.p2p, module_builder=TritonRMSNorm, module_kwargs={"hidden_size": config.d_model, "eps": config.rms_norm_eps}, module_input_keys={"input"}, module_output_keys={"hidden_states"})
        self.lm_head = PipelineBlock(
            p2p=self.p2p, module_builder=TensorParallelColumnLinear,
            module_kwargs={"in_features": config.d_model, "out_features": config.vocab_size, "pg": tp_pg, "bias": False, "mode": TensorParallelLinearMode.ALL_REDUCE},
            module_input_keys={"x"}, module_output_keys={"logits"},
        )

    def forward(self, input_ids, input_mask):
        state = {"hidden_states": self.token_position_embeddings(input_ids=input_ids, input_mask=input_mask)["input_embeds"], "sequence_mask": input_mask}
        for layer in self.decoder:
            state = layer(**state)
        h = self.final_layer_norm(input=state["hidden_states"])["hidden_states"]
        return self.lm_head(x=h)["logits"]  # [b*s, vocab / tp]

    def get_block_compute_costs(self):
        c = self.config.ssm()
        d_inner = c["expand"] * self.config.d_model
        per_layer = 3 * d_inner * self.config.d_model + d_inner * (c["dt_rank"] + 2 * c["d_state"]) + c["dt_rank"] * d_inner
        return {MambaBlock: per_layer, TensorParallelColumnLinear: self.config.vocab_size * self.config.d_model}

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        """Model FLOPs: the projections (2 FLOPs per weight and token), the convolution and 9 FLOPs per state element of the scan; x3 for forward + backward."""
        c = self.config.ssm()
        d, n = self.config.d_model, c["d_state"]
        d_inner = c["expand"] * d
        per_token_layer = 2 * (3 * d_inner * d + d_inner * (c["dt_rank"] + 2 * n) + c["dt_rank"] * d_inner) + 2 * d_inner * c["d_conv"] + 9 * d_inner * n
        per_token = self.config.num_hidden_layers * per_token_layer + 2 * d * self.config.vocab_size
        flops = 3 * per_token * sequence_length * global_batch_size
        world = self.parallel_context.world_pg.size()
        tflops = flops / (iteration_time_in_sec * world * 1e12)
        return tflops, tflops


class MambaForTraining(NanotronModel):
    def __init__(self, config: MambaModelConfig, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs], random_states: Optional[RandomStates] = None):
        super().__init__()
        self.model = MambaModel(config=config, parallel_context=parallel_context, parallel_config=parallel_config, random_states=random_states)
        self.loss = PipelineBlock(p2p=self.model.p2p, module_builder=Loss, module_kwargs={"tp_pg": parallel_context.tp_pg}, module_input_keys={"sharded_logits", "label_ids", "label_mask"}, module_output_keys={"loss"})
        self.config, self.parallel_config, self.parallel_context = config, parallel_config, parallel_context

    def forward(self, input_ids, input_mask, label_ids, label_mask):
        logits = self.model(input_ids=input_ids, input_mask=input_mask)
        return {"loss": self.loss(sharded_logits=logits, label_ids=label_ids, label_mask=label_mask)["loss"]}

    def get_named_params_without_weight_decay(self) -> List[str]:
        """A_log, D and the dt bias parametrise the dynamics directly (decaying them changes the time scales), norms are gains."""
        return [name for name, _ in self.named_parameters() if name.endswith(("A_log", ".D", "dt_proj.bias", "norm.weight", "final_layer_norm.pp_block.weight"))]

    @torch.no_grad()
    def init_model_randomly(self, config):
        init = config.model.init_method
        std = getattr(init, "initializer_range", getattr(init, "std", 0.02))
        rescale = getattr(init, "rescale_prenorm_residual", True)
        n_res = getattr(init, "n_residuals_per_layer", 1)
        done = set()
        for name, p in sorted(self.named_parameters(), key=lambda x: x[0]):
            full = p.get_tied_info().get_full_name_from_module_id_to_prefix(self.module_id_to_prefix) if getattr(p, "is_tied", False) else name
            if full in done:
                continue
            done.add(full)
            module_name, _, local = name.rpartition(".")
            module = self.get_submodule(module_name)
            if isinstance(module, TritonRMSNorm):
                p.fill_(1)
            elif local in ("A_log", "D"):
                continue  # set by the mixer's constructor
            elif module_name.endswith("dt_proj"):
                continue  # set below, weight and bias together
            elif module_name.endswith("conv1d"):
                if local == "bias":
                    p.zero_()
                else:
                    bound = 1.0 / math.sqrt(p.shape[1] * p.shape[2])
                    nn.init.uniform_(p, -bound, bound)
            elif local == "bias":
                p.zero_()
            elif isinstance(module, TensorParallelEmbedding):
                nn.init.normal_(p, mean=0.0, std=std)
            elif module_name.endswith("out_proj") and rescale:
                # the residual stream sums one mixer output per layer: keep its variance independent of depth
                nn.init.normal_(p, mean=0.0, std=std / math.sqrt(n_res * self.config.num_hidden_layers))
            else:
                nn.init.normal_(p, mean=0.0, std=std)
        for m in self.modules():
            if isinstance(m, MambaMixer):
                m.init_dt()

    def get_embeddings_lm_head_tied_names(self) -> List[str]:
        if not self.config.tie_word_embeddings:
            return []
        return ["model.token_position_embeddings.pp_block.token_embedding.weight", "model.lm_head.pp_block.weight"]

    def get_block_compute_costs(self):
        return self.model.get_block_compute_costs()

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        return self.model.get_flops_per_sec(iteration_time_in_sec, sequence_length, global_batch_size)


@torch.no_grad()
def greedy_decode(model: MambaForTraining, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
    """Recurrent decoding on one pipeline stage and tp = 1: the prompt is consumed position by position through ``MambaMixer.step``
    (constant memory in the sequence length), then tokens are generated greedily.  input_ids: [b, prompt_len]."""
    blocks = [blk.pp_block for blk in model.model.decoder]
    emb = model.model.token_position_embeddings.pp_block.token_embedding
    norm, head = model.model.final_layer_norm.pp_block, model.model.lm_head.pp_block
    b = input_ids.shape[0]
    dtype = emb.weight.dtype
    states = [blk.mixer.allocate_state(b, input_ids.device, dtype) for blk in blocks]
    out = input_ids
    logits = None
    for t in range(input_ids.shape[1] + max_new_tokens - 1):
        tok = out[:, t]
        h = emb(tok)
        for i, blk in enumerate(blocks):
            y, cs, ss = blk.mixer.step(blk.norm(h), *states[i])
            states[i] = (cs, ss)
            h = h + y.to(h.dtype)
        logits = head(norm(h))
        if t >= input_ids.shape[1] - 1:
            out = torch.cat([out, logits.argmax(-1, keepdim=True)], dim=1)
    return out
