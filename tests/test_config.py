import pytest
import torch

import nanotron_b200.config as c
from helpers import make_config, tiny_llama_config, tiny_qwen_config


def test_yaml_round_trip(tmp_path):
    cfg = make_config(tiny_llama_config(), tp=1, pp=1, dp=1, pp_engine="1f1b", tp_mode="reduce_scatter")
    path = tmp_path / "cfg.yaml"
    cfg.save_as_yaml(path)
    back = c.get_config_from_file(str(path))
    assert isinstance(back.model.model_config, c.LlamaConfig)
    assert back.parallelism.tp_mode.name == "REDUCE_SCATTER"
    assert type(back.parallelism.pp_engine).__name__ == "OneForwardOneBackwardPipelineEngine"
    assert back.model.dtype == torch.float32
    assert c.serialize(back) == c.serialize(cfg)


def test_qwen_moe_config_round_trip(tmp_path):
    mc = tiny_qwen_config(moe_config=c.MoEConfig(num_experts=4, top_k=2, moe_intermediate_size=32, enable_shared_expert=True, shared_expert_intermediate_size=64))
    cfg = make_config(mc)
    path = tmp_path / "cfg.yaml"
    cfg.save_as_yaml(path)
    back = c.get_config_from_file(str(path))
    assert isinstance(back.model.model_config, c.Qwen2Config)
    assert back.model.model_config.moe_config.layers == [0, 1]
    assert back.model.model_config.is_moe_model


def test_strict_loader_rejects_unknown_keys(tmp_path):
    cfg = make_config(tiny_llama_config())
    d = c.serialize(cfg)
    d["tokens"]["not_a_field"] = 1
    with pytest.raises(ValueError):
        c.get_config_from_dict(d)


def test_cross_field_validation():
    with pytest.raises(AssertionError):
        make_config(tiny_llama_config(num_attention_heads=4, num_key_value_heads=4), tp=3, dp=1)
    cfg = make_config(tiny_llama_config(), mbs=2, accum=3, dp=1)
    assert cfg.global_batch_size == 6
    cfg.data_stages.append(c.DatasetStageArgs(name="stable", start_training_step=5, data=c.DataArgs(dataset=None, seed=1)))
    with pytest.raises(ValueError):
        cfg.__post_init__()


def test_lr_scheduler_shapes():
    from nanotron_b200.helpers import lr_scheduler_builder

    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=1.0)
    args = c.LRSchedulerArgs(learning_rate=1.0, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="cosine", lr_decay_steps=4, min_decay_lr=0.1)
    sched = lr_scheduler_builder(opt, args, total_training_steps=10)
    lrs = []
    for _ in range(9):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    assert lrs[0] == 0.0 and abs(lrs[1] - 0.5) < 1e-9 and abs(lrs[2] - 1.0) < 1e-9
    assert abs(lrs[4] - 0.55) < 1e-9  # halfway through the cosine
    assert abs(lrs[6] - 0.1) < 1e-9 and abs(lrs[8] - 0.1) < 1e-9


def test_older_spellings_of_the_reference_schema_still_load(tmp_path):
    """AdamW settings directly under ``optimizer``, ``dataset_folder`` as {folder: weight}, ``interleaved_rotary``: files written for
    older versions of the reference (several of its own examples among them) load with a warning and mean the same."""
    import warnings

    import yaml

    from nanotron_b200.config.config import upgrade_legacy_config_dict

    cfg = make_config(tiny_llama_config(), seq=16)
    path = tmp_path / "new.yaml"
    cfg.save_as_yaml(str(path))
    new = yaml.safe_load(open(path))
    old = yaml.safe_load(open(path))
    factory = old["optimizer"].pop("optimizer_factory")
    factory.pop("name")
    old["optimizer"].update(factory)  # adam_beta1 / adam_beta2 / adam_eps / torch_adam_is_fused at the top level
    old["model"]["model_config"]["interleaved_rotary"] = old["model"]["model_config"].pop("rope_interleaved")
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    for d in (new, old):
        d["data_stages"][0]["data"]["dataset"] = {"dataset_folder": [str(tmp_path / "a"), str(tmp_path / "b")], "dataset_weights": [0.75, 0.25]}
    old["data_stages"][0]["data"]["dataset"] = {"dataset_folder": {str(tmp_path / "a"): 0.75, str(tmp_path / "b"): 0.25}}
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        loaded_old = c.get_config_from_dict(old)
    assert len([w for w in seen if str(w.message).startswith("config:")]) == 3
    assert loaded_old == c.get_config_from_dict(new)
    assert loaded_old.optimizer.optimizer_factory.adam_beta2 == 0.95 and loaded_old.data_stages[0].data.dataset.dataset_weights == [0.75, 0.25]
    assert upgrade_legacy_config_dict(new) == new  # the current schema passes through untouched
    with pytest.raises(Exception):
        c.get_config_from_dict({**old, "optimizer": {**old["optimizer"], "adam_beta3": 0.5}})  # unknown keys are still errors


def test_parallelism_section_validates_sizes_and_describes_the_layout():
    from nanotron_b200.parallel.pipeline_parallel.engine import AllForwardAllBackwardPipelineEngine, OneForwardOneBackwardPipelineEngine
    from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode

    p = c.ParallelismArgs(dp=2, pp=1, tp=1)
    assert isinstance(p.pp_engine, AllForwardAllBackwardPipelineEngine) and p.tp_mode == TensorParallelLinearMode.ALL_REDUCE and p.tp_linear_async_communication is False
    assert p.world_size == 2 and p.describe() == "dp2"
    p = c.ParallelismArgs(dp=8, pp=2, tp=4, pp_engine="1f1b", tp_mode="reduce_scatter", tp_linear_async_communication=True, expert_parallel_size=4, context_parallel_size=2)
    assert isinstance(p.pp_engine, OneForwardOneBackwardPipelineEngine) and p.tp_mode == TensorParallelLinearMode.REDUCE_SCATTER
    assert p.world_size == 128 and p.describe() == "dp8 (ep4) x cp2 x tp4 (sequence parallel) x pp2 (OneForwardOneBackwardPipelineEngine)"
    for bad in (dict(dp=0, pp=1, tp=1), dict(dp=1, pp=1, tp=-2), dict(dp=6, pp=1, tp=1, expert_parallel_size=4), dict(dp=1, pp=1, tp=1, context_parallel_size=0)):
        with pytest.raises(ValueError):
            c.ParallelismArgs(**bad)


def test_evaluation_section_accepts_the_reference_keys_and_round_trips(tmp_path):
    cfg = make_config(tiny_llama_config(), seq=16)
    cfg.lighteval = c.LightEvalConfig(
        batch_size=16, s3_save_path="s3://bucket/evals", upload_to_wandb=True, wandb_project="p", eval_interval=200,
        logging=c.LightEvalLoggingArgs(local_output_path="eval_out", push_results_to_tensorboard=True, hub_repo_results="org/results", tensorboard_metric_prefix="e"),
        tasks=c.LightEvalTasksArgs(tasks="early-signal", max_samples=1000, no_multichoice_continuations_start_space=True),
        generation=c.GenerationArgs(sampler="top_p", top_p=0.9, temperature=0.7),
    )
    assert cfg.lighteval.output_dir == "eval_out" and str(cfg.lighteval.logging.local_output_path) == "eval_out" and cfg.lighteval.generation.seed == 42
    path = tmp_path / "with_eval.yaml"
    cfg.save_as_yaml(str(path))
    again = c.get_config_from_file(str(path))
    assert again.lighteval == cfg.lighteval and again.lighteval.parallelism.world_size == 1
    assert c.LightEvalLoggingArgs(output_dir="x").local_output_path.name == "x"  # the newer spelling fills the reference's field
    with pytest.raises(AssertionError):
        c.LightEvalConfig(upload_to_wandb=True, wandb_project="p")  # nowhere to read the results from
    with pytest.raises(ValueError):
        c.LightEvalTasksArgs(multichoice_continuations_start_space=True, no_multichoice_continuations_start_space=True)
