"""Unit tests of components that the end-to-end tests only exercise indirectly: parameter initialisation rules, model
construction contexts, coalesced collectives, samplers, text packing and collators, small utilities, the FLOP count
(test strategy parity: reference tests/test_parametrization.py, test_base_model.py, test_distributed.py, test_sft.py)."""
import math

import numpy as np
import pytest
import torch

from helpers import make_config, run_distributed, single_process_env, tiny_llama_config, tiny_qwen_config


# ---------------------------------------------------------------------------- initialisation rules
def _std(t):
    return float(t.detach().float().std())


def test_standard_parametrization_scales_output_projections_by_depth():
    import nanotron_b200.config as c
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    cfg = make_config(tiny_llama_config(hidden_size=128, intermediate_size=256, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=3, vocab_size=512), seq=16)
    cfg.model.init_method = c.RandomInit(std=0.04)
    t = DistributedTrainer(cfg)
    named = dict(t.unwrapped_model.named_parameters())
    scaled = 0.04 / math.sqrt(2 * 3)
    for name, p in named.items():
        if "layernorm" in name or name.endswith("final_layer_norm.pp_block.weight"):
            assert torch.equal(p.detach(), torch.ones_like(p)), name
        elif "o_proj" in name or "down_proj" in name:
            assert abs(_std(p) - scaled) < 0.06 * scaled, (name, _std(p))
        elif name.endswith("weight"):
            assert abs(_std(p) - 0.04) < 0.06 * 0.04, (name, _std(p))
    t.parallel_context.destroy()
    # without depth scaling every matrix gets the plain std
    single_process_env()
    cfg.model.init_method = c.RandomInit(std=0.04, scaling_method=c.InitScalingMethod.NONE)
    t = DistributedTrainer(cfg)
    p = dict(t.unwrapped_model.named_parameters())["model.decoder.0.pp_block.mlp.down_proj.weight"]
    assert abs(_std(p) - 0.04) < 0.06 * 0.04
    t.parallel_context.destroy()


def test_spectral_mup_initialisation_and_learning_rates():
    import nanotron_b200.config as c
    from nanotron_b200.scaling.parametrization import LearningRateForSpectralMup, SpectralMupParametrizator
    from nanotron_b200.trainer import DistributedTrainer

    assert SpectralMupParametrizator._compute_spectral_std(1.0, fan_in=256, fan_out=64) == pytest.approx((1 / 16) * 0.5)
    assert SpectralMupParametrizator._compute_spectral_std(1.0, fan_in=64, fan_out=256) == pytest.approx(1 / 8)
    single_process_env()
    cfg = make_config(tiny_llama_config(hidden_size=128, intermediate_size=512, num_attention_heads=4, num_key_value_heads=4, vocab_size=512), seq=16, lr=1e-2)
    cfg.model.init_method = c.SpectralMupInit(use_mup=True)
    t = DistributedTrainer(cfg)
    named = dict(t.unwrapped_model.named_parameters())
    up = named["model.decoder.0.pp_block.mlp.gate_up_proj.weight"]  # 128 -> 1024: fan_out > fan_in
    down = named["model.decoder.0.pp_block.mlp.down_proj.weight"]  # 512 -> 128
    assert abs(_std(up) - 1 / math.sqrt(128)) < 0.05 / math.sqrt(128)
    expect = (1 / math.sqrt(512)) * math.sqrt(128 / 512)
    assert abs(_std(down) - expect) < 0.05 * expect
    assert abs(_std(named["model.token_position_embeddings.pp_block.token_embedding.weight"]) - 1.0) < 0.05
    # learning rate of a matrix = base * fan_out / fan_in; the optimizer's groups carry them
    modules = dict(t.unwrapped_model.named_modules())
    rule = LearningRateForSpectralMup(lr=1e-2, names_to_modules=modules)
    assert rule.get_lr("x.weight", modules["model.decoder.0.pp_block.mlp.down_proj"]) == pytest.approx(1e-2 * 128 / 512)
    assert rule.get_lr("x.weight", modules["model.decoder.0.pp_block.mlp.gate_up_proj"]) == pytest.approx(1e-2 * 1024 / 128)
    lrs = sorted({round(g["lr"], 8) for g in t.optimizer.get_base_optimizer().param_groups})
    assert len(lrs) >= 3 and round(1e-2 * 128 / 512, 8) in lrs and round(1e-2 * 8, 8) in lrs, lrs
    t.parallel_context.destroy()


def test_models_are_built_on_the_requested_device_and_dtype_except_where_they_opt_out():
    from nanotron_b200.models.base import ignore_init_on_device_and_dtype, init_on_device_and_dtype

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(4, 4)
            self.register_buffer("table", torch.zeros(3))
            self.scratch = torch.ones(2)
            self.router = self._fp32_linear()

        @ignore_init_on_device_and_dtype
        def _fp32_linear(self):
            return torch.nn.Linear(4, 2, bias=False)

    with init_on_device_and_dtype(device=torch.device("cpu"), dtype=torch.bfloat16):
        block = Block()
    assert block.lin.weight.dtype == torch.bfloat16 and block.lin.bias.dtype == torch.bfloat16
    assert block.table.dtype == torch.float32  # buffers (rotary tables, ...) keep the precision they were built with
    assert block.router.weight.dtype == torch.float32
    with init_on_device_and_dtype(device=torch.device("meta"), dtype=torch.float32):
        on_meta = Block()
    assert on_meta.lin.weight.device.type == "meta" and on_meta.table.device.type == "meta" and on_meta.scratch.device.type == "meta"
    assert on_meta.router.weight.device.type == "meta"  # opting out of the dtype does not opt out of the device
    assert torch.nn.Linear(2, 2).weight.device.type == "cpu" and torch.ones(1).device.type == "cpu"  # the patch is gone afterwards


def _stage_assignment(out_file):
    from nanotron_b200.trainer import DistributedTrainer

    t = DistributedTrainer(make_config(tiny_llama_config(num_hidden_layers=6, vocab_size=64), pp=2, seq=16))
    model = t.unwrapped_model.model
    mine = sorted(int(name.split(".")[1]) for name, m in model.named_modules() if name.startswith("decoder.") and name.count(".") == 1 and hasattr(m, "pp_block"))
    ranks = [m.rank for m in model.decoder]
    if t.parallel_context.world_pg.rank() == 0:
        torch.save({"mine": mine, "ranks": ranks, "emb": model.token_position_embeddings.rank, "head": model.lm_head.rank}, out_file)
    t.parallel_context.destroy()


def test_pipeline_stages_are_contiguous_and_balanced_by_cost(tmp_path):
    out = str(tmp_path / "stages.pt")
    run_distributed(_stage_assignment, 2, out_file=out)
    res = torch.load(out)
    assert res["ranks"] == sorted(res["ranks"]) and set(res["ranks"]) == {0, 1}  # contiguous, both stages used
    assert res["emb"] == 0 and res["head"] == 1
    assert abs(res["ranks"].count(0) - res["ranks"].count(1)) <= 2
    assert res["mine"] == [i for i, r in enumerate(res["ranks"]) if r == 0]  # rank 0 instantiated exactly its own layers


# ---------------------------------------------------------------------------- collectives
def _coalesced(out_file):
    import nanotron_b200.distributed as dist

    dist.initialize_torch_distributed()
    rank, world = dist.get_rank(), dist.get_world_size()
    group = dist.new_group(list(range(world)))
    # all-reduce of views into one buffer (flat path) and of unrelated tensors with two dtypes (packed path)
    flat = torch.arange(10, dtype=torch.float32) * (rank + 1)
    dist.all_reduce_coalesced([flat[:4].view(2, 2), flat[4:]], group=group)
    assert torch.equal(flat, torch.arange(10, dtype=torch.float32) * 3)
    a, b, c = torch.full((3,), float(rank + 1)), torch.full((2, 2), 2.0 * (rank + 1), dtype=torch.float64), torch.full((5,), 1.0)
    dist.all_reduce_coalesced([a, b, c], group=group)
    assert torch.equal(a, torch.full((3,), 3.0)) and torch.equal(b, torch.full((2, 2), 6.0, dtype=torch.float64)) and torch.equal(c, torch.full((5,), 2.0))
    # all-gather of slices that differ in size between ranks (ZeRO's parameter slices)
    sizes = [[3, 1], [2, 4]]  # sizes[tensor][rank]
    outs = [[torch.empty(sizes[i][r]) for r in range(world)] for i in range(2)]
    ins = [torch.full((sizes[i][rank],), float(10 * i + rank)) for i in range(2)]
    dist.all_gather_coalesced(outs, ins, group=group)
    for i in range(2):
        for r in range(world):
            assert torch.equal(outs[i][r], torch.full((sizes[i][r],), float(10 * i + r)))
    # reduce-scatter of lists: every rank ends with the sum of its own column
    ins = [[torch.full((2,), float((rank + 1) * (r + 1))) for r in range(world)], [torch.full((3,), float(rank + r)) for r in range(world)]]
    outs = [torch.empty(2), torch.empty(3)]
    dist.reduce_scatter_coalesced(outs, ins, group=group)
    assert torch.equal(outs[0], torch.full((2,), 3.0 * (rank + 1))) and torch.equal(outs[1], torch.full((3,), 1.0 + 2 * rank))
    # single-member groups are a copy; asking for the rank in a group one is not part of is an error
    singles = [dist.new_group([0]), dist.new_group([1])]
    x, y = torch.ones(4), torch.empty(4)
    dist.all_gather_into_tensor(y, x, group=singles[rank])
    assert torch.equal(y, x)
    dist.reduce_scatter_tensor(y, x * 2, group=singles[rank])
    assert torch.equal(y, torch.full((4,), 2.0))
    assert list(dist.get_global_ranks(group)) == [0, 1] and dist.get_global_rank(singles[1], 0) == 1
    with pytest.raises(Exception):
        dist.get_rank(singles[1 - rank])
    if rank == 0:
        torch.save(True, out_file)
    dist.barrier()
    dist.destroy_process_group()


def test_coalesced_collectives(tmp_path):
    out = str(tmp_path / "ok.pt")
    run_distributed(_coalesced, 2, out_file=out)
    assert torch.load(out) is True


# ---------------------------------------------------------------------------- samplers, packing, collators
def test_samplers_partition_the_data_and_resume():
    from nanotron_b200.data.samplers import MegatronPretrainingCyclicSampler, MegatronPretrainingRandomSampler, MegatronPretrainingSampler, get_sampler

    data = list(range(20))
    per_rank = [list(get_sampler(dl_ranks_size=2, dl_rank=r, train_dataset=data, consumed_train_samples=0, shuffle=False)) for r in range(2)]
    assert sorted(per_rank[0] + per_rank[1]) == data and not set(per_rank[0]) & set(per_rank[1])
    resumed = [list(get_sampler(dl_ranks_size=2, dl_rank=r, train_dataset=data, consumed_train_samples=8, shuffle=False)) for r in range(2)]
    assert resumed[0] == per_rank[0][4:] and resumed[1] == per_rank[1][4:]  # 8 samples of the job = 4 per rank
    shuffled = [list(get_sampler(2, r, data, 0, seed=5, shuffle=True)) for r in range(2)]
    assert sorted(shuffled[0] + shuffled[1]) == data and shuffled[0] != per_rank[0]
    looped = list(get_sampler(2, 0, list(range(7)), 0, use_loop_to_round_batch_size=True, micro_batch_size=4, drop_last=False))
    assert len(looped) % 4 == 0
    # Megatron-style: rank r takes slice r of every global micro-batch; consumed samples shift the start
    seq = [list(MegatronPretrainingSampler(total_samples=20, consumed_samples=4, micro_batch_size=2, data_parallel_rank=r, data_parallel_size=2)) for r in range(2)]
    assert seq[0][0] == [4, 5] and seq[1][0] == [6, 7] and len(seq[0]) == 4
    last = list(MegatronPretrainingSampler(total_samples=10, consumed_samples=0, micro_batch_size=2, data_parallel_rank=1, data_parallel_size=2, drop_last=False, pad_samples_to_global_batch_size=True))
    assert last[-1] == [-1, -1]  # ten samples: the third global micro-batch has two real samples, both on rank 0
    rnd = [MegatronPretrainingRandomSampler(total_samples=16, consumed_samples=0, micro_batch_size=2, data_parallel_rank=r, data_parallel_size=2, seed=1) for r in range(2)]
    drawn = [list(s) for s in rnd]
    assert sorted(i for batches in drawn for b in batches for i in b) == list(range(16))
    again = MegatronPretrainingRandomSampler(total_samples=16, consumed_samples=8, micro_batch_size=2, data_parallel_rank=0, data_parallel_size=2, seed=1)
    assert list(again) == drawn[0][2:]  # same epoch, same permutation, continued after 8 samples of the job
    cyc = iter(MegatronPretrainingCyclicSampler(total_samples=6, consumed_samples=4, micro_batch_size=2, data_parallel_rank=0, data_parallel_size=2))
    assert [next(cyc) for _ in range(2)] == [[4, 5], [2, 3]]


def test_text_packing_and_collators():
    from nanotron_b200.data.clm_collator import DataCollatorForCLM, DataCollatorForCLMWithPositionIds
    from nanotron_b200.data.processing import group_texts
    from nanotron_b200.parallel.context import ParallelContext
    from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

    # windows of sequence_length + 1 tokens that overlap by one: every token but the first is a label exactly once
    docs = [list(range(0, 7)), list(range(7, 12)), list(range(12, 23))]
    windows = group_texts(docs, sequence_length=5)["input_ids"]
    assert [w.tolist() for w in windows] == [[0, 1, 2, 3, 4, 5], [5, 6, 7, 8, 9, 10], [10, 11, 12, 13, 14, 15], [15, 16, 17, 18, 19, 20]]
    assert group_texts([[1, 2, 3]], sequence_length=5)["input_ids"] == []
    single_process_env()
    ctx = ParallelContext(tensor_parallel_size=1, pipeline_parallel_size=1, data_parallel_size=1)
    examples = [{"input_ids": np.arange(9)}, {"input_ids": np.arange(9) + 100}]
    batch = DataCollatorForCLM(sequence_length=8, input_pp_rank=0, output_pp_rank=0, parallel_context=ctx)(examples)
    assert batch["input_ids"].tolist()[0] == list(range(8)) and batch["label_ids"].tolist()[0] == list(range(1, 9))
    assert batch["input_mask"].all() and batch["label_mask"].all()
    with pytest.raises(AssertionError):
        DataCollatorForCLM(sequence_length=7, input_pp_rank=0, output_pp_rank=0, parallel_context=ctx)(examples)
    # packed documents: positions restart at a boundary, and the first token of a document is never a label
    positions = np.array([0, 1, 2, 3, 0, 1, 2, 0, 1])
    packed = [{"input_ids": np.arange(9), "positions": positions}]
    batch = DataCollatorForCLMWithPositionIds(sequence_length=8, input_pp_rank=0, output_pp_rank=0, parallel_context=ctx)(packed)
    assert batch["position_ids"].tolist() == [positions[:-1].tolist()]
    assert batch["label_mask"].tolist() == [[True, True, True, False, True, True, False, True]]
    plain = DataCollatorForCLM(sequence_length=8, input_pp_rank=0, output_pp_rank=0, parallel_context=ctx)(packed)
    assert plain["label_mask"].tolist() == batch["label_mask"].tolist()
    # a pipeline rank that is neither first nor last only gets pointers
    other = DataCollatorForCLM(sequence_length=8, input_pp_rank=1, output_pp_rank=2, parallel_context=ctx)([{}, {}])
    assert all(isinstance(v, TensorPointer) for v in other.values()) and other["input_ids"].group_rank == 1 and other["label_ids"].group_rank == 2
    ctx.destroy()


# ---------------------------------------------------------------------------- utilities
def test_small_utilities():
    from nanotron_b200.parallel.utils import MemoryBuffer
    from nanotron_b200.utils import ContextManagers, checkpoint_method, find_free_port, get_parameter_and_parent_module, tensor_from_untyped_storage

    buf = MemoryBuffer()
    a = buf.get("gather", (4, 8), dtype=torch.float32, device="cpu")
    b = buf.get("gather", (2, 8), dtype=torch.float32, device="cpu")
    assert a.data_ptr() == b.data_ptr() and MemoryBuffer() is buf  # one pool, the smaller request reuses the storage
    c = buf.get("gather", (8, 8), dtype=torch.float32, device="cpu")
    assert c.shape == (8, 8) and buf.get("other", (4,), dtype=torch.float32, device="cpu").data_ptr() != c.data_ptr()
    buf.clear()

    order = []

    class CM:
        def __init__(self, name):
            self.name = name

        def __enter__(self):
            order.append("in " + self.name)

        def __exit__(self, *a):
            order.append("out " + self.name)

    with ContextManagers([CM("a"), CM("b")]):
        order.append("body")
    assert order == ["in a", "in b", "body", "out b", "out a"]

    class Layer(torch.nn.Module):
        def __init__(self, recompute):
            super().__init__()
            self.lin = torch.nn.Linear(8, 8)
            self.recompute = recompute
            self.calls = 0

        @checkpoint_method("recompute")
        def forward(self, x, scale=1.0):
            self.calls += 1
            return torch.tanh(self.lin(x)) * scale

    torch.manual_seed(0)
    plain, ckpt = Layer(False), Layer(True)
    ckpt.load_state_dict(plain.state_dict())
    x = torch.randn(3, 8)
    g = []
    for layer in (plain, ckpt):
        xi = x.clone().requires_grad_(True)
        layer(xi, scale=2.0).sum().backward()
        g.append((xi.grad, layer.lin.weight.grad))
    assert torch.equal(g[0][0], g[1][0]) and torch.equal(g[0][1], g[1][1])
    assert plain.calls == 1 and ckpt.calls == 2  # the checkpointed one ran its forward again in the backward

    p, mod, name = get_parameter_and_parent_module("lin.weight", plain)
    assert p is plain.lin.weight and mod is plain.lin and name == "weight"
    with pytest.raises(AttributeError):
        get_parameter_and_parent_module("lin.nothing", plain)
    raw = torch.arange(6, dtype=torch.float32)
    assert torch.equal(tensor_from_untyped_storage(raw.untyped_storage(), torch.float32), raw)
    assert 2000 <= find_free_port() <= 65000


def test_flop_count_of_dense_and_mixture_models():
    from nanotron_b200.config.models_config import MoEConfig
    from nanotron_b200.models.qwen import get_flops

    kw = dict(num_layers=2, hidden_size=64, num_heads=4, num_key_value_heads=2, vocab_size=1000, seq_len=128, ffn_hidden_size=256, batch_size=3)
    T, h, d = 3 * 128, 64, 16
    attention = 2 * T * h * (4 + 2 * 2) * d + 2 * (2 * 4 * T * 128 * d) + 2 * T * 4 * d * h
    fwd = 2 * (attention + 6 * T * h * 256) + 2 * T * h * 1000
    model, hardware = get_flops(**kw)
    assert model == hardware == 3 * fwd
    _, hardware = get_flops(**kw, recompute_layer=True)
    assert hardware == 3 * fwd + 2 * (attention + 6 * T * h * 256)
    # one of the two layers is a mixture of experts: 2 of 8 experts of width 32 per token, a router, a gated shared expert
    moe = MoEConfig(num_experts=8, top_k=2, moe_intermediate_size=32, shared_expert_intermediate_size=64, enable_shared_expert=True)
    model, _ = get_flops(**kw, moe_config=moe, num_moe_layers=1)
    moe_mlp = 6 * T * h * 32 * 2 + 2 * T * h * 8 + 6 * T * h * 64 + 2 * T * h
    assert model == 3 * (2 * attention + 6 * T * h * 256 + moe_mlp + 2 * T * h * 1000)


# ---------------------------------------------------------------------------- less common options of the trainer
def test_initial_checkpoint_weights_only_start_sgd_and_validation(tmp_path):
    import os

    import nanotron_b200.config as c
    from helpers import dummy_dataloader
    from nanotron_b200.trainer import DistributedTrainer

    # save_initial_state writes step 0 before the first update
    single_process_env()
    cfg = make_config(tiny_llama_config(), seq=16, steps=3, ckpt_path=str(tmp_path / "a"), ckpt_interval=3)
    cfg.checkpoints.save_initial_state = True
    t = DistributedTrainer(cfg)
    t.train(dummy_dataloader(t))
    assert sorted(os.listdir(tmp_path / "a")) == ["0", "3", "latest.txt"] and open(tmp_path / "a" / "latest.txt").read() == "3"
    trained = {k: v.detach().clone() for k, v in t.unwrapped_model.named_parameters()}
    t.parallel_context.destroy()
    # init_method.path starts a NEW run from those weights: step 0, fresh schedule and optimizer
    single_process_env()
    cfg = make_config(tiny_llama_config(), seq=16, steps=2, ckpt_path=str(tmp_path / "b"))
    cfg.model.init_method = c.ExistingCheckpointInit(path=str(tmp_path / "a" / "3"))
    t = DistributedTrainer(cfg)
    assert all(torch.equal(v, dict(t.unwrapped_model.named_parameters())[k]) for k, v in trained.items())
    assert t.iteration_step == 0 and t.metadata.consumed_train_samples == 0 and len(t.optimizer.get_base_optimizer().state) == 0
    # validation: limit_val_batches forward passes without gradients; their outputs add up to the mean loss
    t.config.tokens.limit_val_batches = t.limit_val_batches = 2
    t.prepare_training()
    outputs = t.validation_step(dummy_dataloader(t))
    assert len(outputs) == 2 and all(not o["loss"].requires_grad for o in outputs) and 3.0 < float(sum(o["loss"] for o in outputs)) < 7.0
    assert all(p.grad is None for p in t.unwrapped_model.parameters())
    t.parallel_context.destroy()
    # plain SGD from the config
    single_process_env()
    cfg = make_config(tiny_llama_config(), seq=16, steps=8, lr=0.5)
    cfg.optimizer.optimizer_factory = c.SGDOptimizerArgs()
    t = DistributedTrainer(cfg)
    assert type(t.optimizer.get_base_optimizer()).__name__ == "SGD"
    t.prepare_training()
    batch = [next(dummy_dataloader(t))]
    losses = []
    for _ in range(6):
        losses.append(float(t.training_step(iter(batch))[1]))
        t.iteration_step += 1
    assert losses[-1] < losses[0] - 0.5, losses
    t.parallel_context.destroy()


def test_rotary_options_layers_without_rope_and_frequency_scaling():
    from helpers import dummy_dataloader
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    t = DistributedTrainer(make_config(tiny_qwen_config(no_rope_layer=2), seq=16, steps=2))
    assert [blk.pp_block.attn.use_rope for blk in t.unwrapped_model.model.decoder] == [True, False]  # every second layer is position-free
    t.prepare_training()
    assert torch.isfinite(t.training_step(dummy_dataloader(t))[1])
    t.parallel_context.destroy()
    single_process_env()
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    t = DistributedTrainer(make_config(tiny_llama_config(rope_scaling=scaling, max_position_embeddings=256, num_attention_heads=2, num_key_value_heads=2, hidden_size=64), seq=16, steps=2))
    rot = t.unwrapped_model.model.decoder[0].pp_block.attn.rotary_emb
    t.prepare_training()
    assert torch.isfinite(t.training_step(dummy_dataloader(t))[1])
    # long wavelengths are stretched by the factor, short ones are kept (the Llama-3.1 rule)
    plain = 1.0 / (10000.0 ** (torch.arange(0, 32, 2).float() / 32))
    got = rot.inv_freq.float().cpu() if hasattr(rot, "inv_freq") else None
    if got is not None:
        assert torch.allclose(got[0], plain[0]) and torch.allclose(got[-1], plain[-1] / 8.0, rtol=1e-4)
    t.parallel_context.destroy()


def test_fp32_accumulator_keeps_what_half_precision_would_lose():
    """Gradients of bf16 parameters are summed in fp32 over the micro-batches, the optimizer works on fp32 masters, and the step
    writes the masters back to the bf16 parameters: small updates that bf16 alone would round away survive."""
    from nanotron_b200.optim.gradient_accumulator import FP32GradientAccumulator
    from nanotron_b200.parallel.parameters import NanotronParameter

    torch.manual_seed(0)
    lin = torch.nn.Linear(16, 8, bias=True).to(torch.bfloat16)
    for name in ("weight", "bias"):
        setattr(lin, name, NanotronParameter(getattr(lin, name).data))
    named = list(lin.named_parameters())
    acc = FP32GradientAccumulator(named)
    reference = {n: p.detach().double().clone().requires_grad_(True) for n, p in named}
    xs = [torch.randn(4, 16) for _ in range(3)]
    for x in xs:  # three micro-batches
        acc.backward(lin(x.to(torch.bfloat16)).float().pow(2).mean())
        (x.double() @ reference["weight"].t() + reference["bias"]).pow(2).mean().backward()
    for n, p in named:
        assert p.grad is None  # the half-precision gradient is consumed at once
        got, exp = acc.get_grad_buffer(n), reference[n].grad
        assert got.dtype == torch.float32 and got.shape == p.shape
        torch.testing.assert_close(got.double(), exp, rtol=0.05, atol=2e-2)  # bf16 forward, fp32 sum
    # one flat buffer behind all slots
    flat = acc._contiguous_fp32_grad_buffer
    assert flat.numel() >= sum(p.numel() for _, p in named) and acc.get_grad_buffer("weight").data_ptr() == flat.data_ptr() + acc._grad_offsets["weight"] * 4
    # an update far below bf16 resolution, applied 64 times: the masters move, and so (eventually) do the parameters
    master = acc.get_parameter_for_optimizer("weight")
    assert master.dtype == torch.float32 and master.grad is not None
    before_master, before_half = master.detach().clone(), lin.weight.detach().clone()
    for _ in range(64):
        with torch.no_grad():
            master.add_(1e-4)  # |w| ~ 0.1: one bf16 step there is ~5e-4
        acc.step()
    torch.testing.assert_close(master.detach(), before_master + 64e-4, rtol=0, atol=1e-6)
    assert float((lin.weight.detach().float() - before_half.float()).mean()) == pytest.approx(64e-4, rel=0.2)
    in_bf16 = before_half.clone()
    for _ in range(64):
        in_bf16 += 1e-4
    assert float((in_bf16.float() - before_half.float()).abs().mean()) < 0.5 * 64e-4  # what accumulating in bf16 would have kept
    acc.zero_grad()
    assert float(flat.abs().sum()) == 0.0
    # the masters are the state that a checkpoint carries
    state = acc.state_dict()
    assert set(state) == {"weight", "bias"} and state["weight"].dtype == torch.float32
    fresh = FP32GradientAccumulator(named)
    fresh.load_state_dict(state)
    torch.testing.assert_close(fresh.get_parameter_for_optimizer("weight").detach(), master.detach(), rtol=0, atol=0)
