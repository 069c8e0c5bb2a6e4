"""Checkpoints: the on-disk layout (file names the reference uses), exact resume of a run (weights, fp32 masters, optimizer
moments, lr schedule, step / sample counters), and resuming under a different topology (tp 2 -> 1, dp 2 + ZeRO-1 -> 1)."""
import json
import os

import torch

from helpers import make_config, run_distributed, tiny_llama_config
from test_distributed_cpu import _deterministic_init, _fixed_batches


def _run(out_file, ckpt_dir, steps, first_step=0, save=False, resume=None, total_mbs=4, **topology):
    import nanotron_b200.distributed as dist
    from nanotron_b200.trainer import DistributedTrainer as _Base

    class DistributedTrainer(_Base):
        def _load_model_checkpoint(self, model):
            if self.init_checkpoint_path is not None:
                return super()._load_model_checkpoint(model)
            _deterministic_init(model)
            return model

    dp = topology.get("dp", 1)
    accum = total_mbs // dp
    uses_mask = True
    if topology.pop("moe", False):
        import nanotron_b200.config as c
        from helpers import tiny_qwen_config

        mc = tiny_qwen_config(moe_config=c.MoEConfig(num_experts=4, top_k=2, moe_intermediate_size=16, shared_expert_intermediate_size=32, enable_shared_expert=True, router_aux_loss_coef=0.01))
        uses_mask = False
    else:
        mc = tiny_llama_config(tie_word_embeddings=topology.pop("tied", False))
    cfg = make_config(mc, seq=16, mbs=1, accum=accum, steps=8, lr=1e-2, ckpt_path=ckpt_dir, **topology)
    if resume is not None:
        cfg.checkpoints.resume_checkpoint_path = resume
    t = DistributedTrainer(cfg)
    t.prepare_training()
    assert t.iteration_step == first_step + 1, (t.iteration_step, first_step)  # the step about to run
    all_batches = _fixed_batches(t, first_step + steps, total_mbs, 16, mc.vocab_size, uses_mask=uses_mask)
    per_step = len(all_batches) // (first_step + steps)
    batches = iter(all_batches[first_step * per_step :])
    losses = []
    for i in range(steps):
        _, loss, _ = t.training_step(batches)
        t.metadata.last_train_step = t.iteration_step
        t.metadata.consumed_train_samples += t.global_batch_size
        t.metadata.data_stages[0].consumed_train_samples += t.global_batch_size
        if loss is not None:
            losses.append(float(loss))
        if save and i == steps - 1:
            t.save_checkpoint()
        t.iteration_step += 1
    if dist.get_rank(t.parallel_context.world_pg) == t.logger_ranks[0]:
        torch.save(losses, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def _losses(tmp_path, name, world, **kw):
    f = str(tmp_path / f"{name}.pt")
    run_distributed(_run, world, out_file=f, **kw)
    return torch.load(f)


def test_resume_continues_the_same_run_and_layout_matches(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    full = _losses(tmp_path, "full", 1, ckpt_dir=str(tmp_path / "unused"), steps=4)
    first = _losses(tmp_path, "first", 1, ckpt_dir=ckpt, steps=2, save=True)
    assert first == full[:2]
    step_dir = os.path.join(ckpt, "2")
    # layout
    assert open(os.path.join(ckpt, "latest.txt")).read().strip() == "2"
    meta = json.load(open(os.path.join(step_dir, "checkpoint_metadata.json")))
    assert meta["metas"]["last_train_step"] == 2 and meta["tp"] == 1 and meta["dp"] == 1
    assert os.path.isfile(os.path.join(step_dir, "config.yaml"))
    assert os.path.isfile(os.path.join(step_dir, "model", "model", "token_position_embeddings", "pp_block", "token_embedding", "model_weight_pp-rank-0-of-1_tp-rank-0-of-1.safetensors"))
    assert os.path.isfile(os.path.join(step_dir, "model", "model", "decoder", "0", "pp_block", "attn", "qkv_proj", "model_weight_pp-rank-0-of-1_tp-rank-0-of-1.safetensors"))
    assert os.path.isfile(os.path.join(step_dir, "model", "model", "final_layer_norm", "pp_block", "model_weight.safetensors"))  # replicated: no suffix
    assert os.path.isfile(os.path.join(step_dir, "optimizer", "optimizer_config.json"))
    assert any(f.startswith("optimizer_pp-0-of-1") and f.endswith(".pt") for f in os.listdir(os.path.join(step_dir, "optimizer")))
    assert os.listdir(os.path.join(step_dir, "lr_scheduler")) == ["lr_scheduler_pp-0-of-1_tp-0-of-1_exp-0-of-1.pt"]
    assert os.listdir(os.path.join(step_dir, "random")) == ["tp-0-of-1_dp-0-of-1_pp-0-of-1.pt"]
    # exact continuation
    resumed = _losses(tmp_path, "resumed", 1, ckpt_dir=ckpt, steps=2, first_step=2, resume=ckpt)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 1e-6, (resumed, full)


def test_resume_under_another_topology(tmp_path):
    full = _losses(tmp_path, "full", 1, ckpt_dir=str(tmp_path / "unused"), steps=4)
    # tensor parallel 2 -> 1: sharded weights and optimizer moments are merged on load
    ckpt_tp = str(tmp_path / "ckpt_tp")
    _losses(tmp_path, "tp_first", 2, ckpt_dir=ckpt_tp, steps=2, save=True, tp=2, tp_mode="reduce_scatter")
    names = os.listdir(os.path.join(ckpt_tp, "2", "model", "model", "decoder", "0", "pp_block", "attn", "qkv_proj"))
    assert sorted(names) == ["model_weight_pp-rank-0-of-1_tp-rank-0-of-2.safetensors", "model_weight_pp-rank-0-of-1_tp-rank-1-of-2.safetensors"]
    resumed = _losses(tmp_path, "tp_resumed", 1, ckpt_dir=ckpt_tp, steps=2, first_step=2, resume=ckpt_tp)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)
    # data parallel 2 with ZeRO-1 -> single process: optimizer shards are concatenated on load
    ckpt_dp = str(tmp_path / "ckpt_dp")
    _losses(tmp_path, "dp_first", 2, ckpt_dir=ckpt_dp, steps=2, save=True, dp=2, zero=1)
    resumed = _losses(tmp_path, "dp_resumed", 1, ckpt_dir=ckpt_dp, steps=2, first_step=2, resume=ckpt_dp)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)


def test_resume_same_tp_other_optimizer_layout(tmp_path):
    """tp stays 2 while the optimizer layout changes (ZeRO-1 over dp 2 -> one replica, and -> no ZeRO): every tp rank must get
    its own shard of the moments and fp32 masters back, not tp rank 0's."""
    full = _losses(tmp_path, "full", 1, ckpt_dir=str(tmp_path / "unused"), steps=4)
    ckpt = str(tmp_path / "ckpt_tp2dp2")
    _losses(tmp_path, "first", 4, ckpt_dir=ckpt, steps=2, save=True, tp=2, dp=2, zero=1, tp_mode="reduce_scatter")
    resumed = _losses(tmp_path, "resumed_dp1", 2, ckpt_dir=ckpt, steps=2, first_step=2, resume=ckpt, tp=2, tp_mode="reduce_scatter")
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)
    resumed = _losses(tmp_path, "resumed_dp2_zero0", 4, ckpt_dir=ckpt, steps=2, first_step=2, resume=ckpt, tp=2, dp=2, zero=0, tp_mode="reduce_scatter")
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)


def test_resume_with_embeddings_tied_across_pipeline_stages(tmp_path):
    """Embedding (first stage) and lm head (last stage) share one weight: only the first member of the tie writes it, under the
    embedding's name, and the lm head's stage must find it there when the run resumes, on the same layout and on a single process."""
    full = _losses(tmp_path, "full", 1, ckpt_dir=str(tmp_path / "unused"), steps=4, tied=True)
    ckpt = str(tmp_path / "ckpt_pp")
    first = _losses(tmp_path, "pp_first", 2, ckpt_dir=ckpt, steps=2, save=True, pp=2, tied=True)
    for a, b in zip(first, full[:2]):
        assert abs(a - b) < 3e-4, (first, full)
    model_dir = os.path.join(ckpt, "2", "model", "model")
    assert os.path.isdir(os.path.join(model_dir, "token_position_embeddings")) and not os.path.isdir(os.path.join(model_dir, "lm_head"))
    same = _losses(tmp_path, "pp_resumed", 2, ckpt_dir=ckpt, steps=2, first_step=2, resume=ckpt, pp=2, tied=True)
    single = _losses(tmp_path, "single_resumed", 1, ckpt_dir=ckpt, steps=2, first_step=2, resume=ckpt, tied=True)
    for got in (same, single):
        for a, b in zip(got, full[2:]):
            assert abs(a - b) < 3e-4, (got, full)


def test_resume_from_another_pipeline_and_combined_layout(tmp_path):
    """pp 2 -> 1 and (tp 2 x pp 2) -> dp 2 with ZeRO-1: file names carry the writer's pipeline rank, the reader finds the shards anyway."""
    full = _losses(tmp_path, "full", 1, ckpt_dir=str(tmp_path / "unused"), steps=4)
    ckpt_pp = str(tmp_path / "ckpt_pp")
    _losses(tmp_path, "pp_first", 2, ckpt_dir=ckpt_pp, steps=2, save=True, pp=2)
    resumed = _losses(tmp_path, "pp_to_one", 1, ckpt_dir=ckpt_pp, steps=2, first_step=2, resume=ckpt_pp)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)
    ckpt_4 = str(tmp_path / "ckpt_4")
    _losses(tmp_path, "tp2pp2_first", 4, ckpt_dir=ckpt_4, steps=2, save=True, tp=2, pp=2, tp_mode="reduce_scatter")
    resumed = _losses(tmp_path, "to_dp2", 2, ckpt_dir=ckpt_4, steps=2, first_step=2, resume=ckpt_4, dp=2, zero=1)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)


def test_resume_into_larger_layouts(tmp_path):
    """Growing instead of shrinking: ZeRO-1 over 2 ranks -> over 4, and a single process -> tp 2 x dp 2 with ZeRO-1 (weights and
    optimizer moments are cut along tp, then partitioned over dp)."""
    full = _losses(tmp_path, "full", 1, ckpt_dir=str(tmp_path / "unused"), steps=4)
    ckpt_dp = str(tmp_path / "ckpt_dp2")
    _losses(tmp_path, "dp2_first", 2, ckpt_dir=ckpt_dp, steps=2, save=True, dp=2, zero=1)
    resumed = _losses(tmp_path, "dp4", 4, ckpt_dir=ckpt_dp, steps=2, first_step=2, resume=ckpt_dp, dp=4, zero=1)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)
    ckpt_one = str(tmp_path / "ckpt_one")
    _losses(tmp_path, "one_first", 1, ckpt_dir=ckpt_one, steps=2, save=True)
    resumed = _losses(tmp_path, "tp2dp2", 4, ckpt_dir=ckpt_one, steps=2, first_step=2, resume=ckpt_one, tp=2, dp=2, zero=1, tp_mode="reduce_scatter")
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)


def test_expert_parallel_checkpoint_resumes(tmp_path):
    """Experts split over two ranks (and replicated over two tp ranks): every expert rank writes its own expert shard, and the run
    continues exactly after a resume on the same layout."""
    kw = dict(dp=2, ep=2, tp=2, tp_mode="reduce_scatter", moe=True)
    full = _losses(tmp_path, "moe_full", 4, ckpt_dir=str(tmp_path / "unused"), steps=4, **kw)
    ckpt = str(tmp_path / "ckpt_moe")
    first = _losses(tmp_path, "moe_first", 4, ckpt_dir=ckpt, steps=2, save=True, **kw)
    assert first == full[:2]
    experts = os.path.join(ckpt, "2", "model", "model", "decoder", "0", "pp_block", "mlp", "experts")
    names = sorted(os.listdir(experts))
    assert any("exp-rank-0-of-2" in n for n in names) and any("exp-rank-1-of-2" in n for n in names), names
    resumed = _losses(tmp_path, "moe_resumed", 4, ckpt_dir=ckpt, steps=2, first_step=2, resume=ckpt, **kw)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 1e-5, (resumed, full)
