"""Starcoder2 on CPU / gloo: multi-query and grouped-query attention under tensor parallelism against one process, sliding-window
layers, the tied key/value projection of multi-query attention in checkpoints, and cached decoding."""
import os

import torch

from helpers import make_config, run_distributed, single_process_env
from test_distributed_cpu import _deterministic_init, _fixed_batches


def _config(mq: bool, **over):
    from nanotron_b200.config import Starcoder2Config

    base = dict(hidden_size=32, num_attention_heads=4, num_hidden_layers=2, intermediate_size=64, vocab_size=128, max_position_embeddings=64, multi_query=mq, grouped_query=not mq,
                num_kv_heads=None if mq else 2, sliding_window_size=8, global_attn_layers=[1], attn_pdrop=0.0, resid_pdrop=0.0, embd_pdrop=0.0, use_rotary_embeddings=True)
    base.update(over)
    return Starcoder2Config(**base)


def _train(out_file, mq, steps=3, ckpt=None, resume=None, sanity=False, clip=1.0, **topology):
    import nanotron_b200.distributed as dist
    from nanotron_b200.trainer import DistributedTrainer as Base

    class T(Base):
        def _load_model_checkpoint(self, model):
            if self.init_checkpoint_path is not None:
                return super()._load_model_checkpoint(model)
            _deterministic_init(model)
            return model

    dp = topology.get("dp", 1)
    cfg = make_config(_config(mq), seq=16, mbs=1, accum=4 // dp, steps=8, lr=1e-2, ckpt_path=ckpt, sanity=sanity, clip=clip, **topology)
    if resume:
        cfg.checkpoints.resume_checkpoint_path = resume
    t = T(cfg)
    t.prepare_training()
    first = t.iteration_step - 1
    batches = iter(_fixed_batches(t, first + steps, 4, 16, 128, uses_mask=True)[first * 4 :])
    losses = []
    for i in range(steps):
        _, loss, _ = t.training_step(batches)
        t.metadata.last_train_step = t.iteration_step
        t.metadata.consumed_train_samples += t.global_batch_size
        t.metadata.data_stages[0].consumed_train_samples += t.global_batch_size
        if ckpt and not resume and i == steps - 1:
            t.save_checkpoint()
        t.iteration_step += 1
        if loss is not None:
            losses.append(float(loss))
    if dist.get_rank(t.parallel_context.world_pg) == t.logger_ranks[0]:
        torch.save(losses, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def _losses(tmp_path, name, world, **kw):
    f = str(tmp_path / f"{name}.pt")
    run_distributed(_train, world, out_file=f, **kw)
    return torch.load(f)


def test_mqa_and_gqa_match_one_process_under_tensor_parallelism(tmp_path):
    # (the other mode of each attention kind runs in the 3D test below)
    for mq, mode in ((True, "all_reduce"), (False, "reduce_scatter")):
        base = _losses(tmp_path, f"base{mq}", 1, mq=mq)
        got = _losses(tmp_path, f"tp{mq}{mode}", 2, mq=mq, tp=2, tp_mode=mode)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-4, (mq, mode, got, base)


def test_mqa_and_gqa_match_one_process_under_3d_layouts_with_the_invariant_checks_on(tmp_path):
    """Tied embeddings across pipeline stages, the single replicated kv head under tensor parallelism and sharded optimizer
    states together, with active clipping and the runtime invariant checks."""
    base = _losses(tmp_path, "base_mq", 1, mq=True, clip=0.05)
    got = _losses(tmp_path, "mq_3d", 8, mq=True, dp=2, tp=2, pp=2, tp_mode="reduce_scatter", zero=1, pp_engine="1f1b", sanity=True, clip=0.05)
    for a, b in zip(got, base):
        assert abs(a - b) < 3e-4, (got, base)
    base = _losses(tmp_path, "base_gq", 1, mq=False, clip=0.05)
    got = _losses(tmp_path, "gq_pp2_tp2", 4, mq=False, tp=2, pp=2, tp_mode="all_reduce", pp_engine="afab", sanity=True, clip=0.05)
    for a, b in zip(got, base):
        assert abs(a - b) < 3e-4, (got, base)


def test_mqa_checkpoint_has_one_replicated_kv_projection_and_resumes(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    full = _losses(tmp_path, "full", 1, mq=True, steps=4)
    _losses(tmp_path, "first", 2, mq=True, steps=2, ckpt=ckpt, tp=2, tp_mode="reduce_scatter")
    attn = os.path.join(ckpt, "2", "model", "model", "decoder", "0", "pp_block", "attn", "qkv")
    # q is sharded over tp (one file per rank), the single kv head is one tied, replicated tensor (one file, no rank suffix)
    assert sorted(os.listdir(os.path.join(attn, "q"))) == ["model_bias_pp-rank-0-of-1_tp-rank-0-of-2.safetensors", "model_bias_pp-rank-0-of-1_tp-rank-1-of-2.safetensors", "model_weight_pp-rank-0-of-1_tp-rank-0-of-2.safetensors", "model_weight_pp-rank-0-of-1_tp-rank-1-of-2.safetensors"]
    assert sorted(os.listdir(os.path.join(attn, "kv"))) == ["model_bias.safetensors", "model_weight.safetensors"]
    resumed = _losses(tmp_path, "resumed", 1, mq=True, steps=2, ckpt=ckpt, resume=ckpt)
    for a, b in zip(resumed, full[2:]):
        assert abs(a - b) < 3e-4, (resumed, full)


def test_sliding_window_layers_and_cached_decoding():
    from nanotron_b200.generation.decode import decode_tokenized
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    t = DistributedTrainer(make_config(_config(True, sliding_window_size=4, global_attn_layers=[]), seq=32))
    model = t.unwrapped_model.model
    model.eval()
    layer0 = model.decoder[0].pp_block.attn
    assert layer0.window == 4
    # a token further back than the window cannot influence the logits of the last position
    torch.manual_seed(0)
    ids = torch.randint(0, 128, (1, 20))
    other = ids.clone()
    other[0, 2] = (other[0, 2] + 1) % 128  # 17 positions before the last one, two layers x window 4 reach at most 6 back
    mask = torch.ones(1, 20, dtype=torch.bool)
    with torch.no_grad():
        a = model(input_ids=ids, input_mask=mask)[-1]
        b = model(input_ids=other, input_mask=mask)[-1]
    torch.testing.assert_close(a, b)
    # cached decoding == recomputing the prefix, with left padding in the batch
    ids = torch.randint(0, 128, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.bool)
    mask[1, :4] = False
    x = decode_tokenized(ids, mask, model, t.parallel_context, max_new_tokens=5, use_cache=False)
    y = decode_tokenized(ids, mask, model, t.parallel_context, max_new_tokens=5, use_cache=True)
    assert torch.equal(x.generation_ids, y.generation_ids)
    t.parallel_context.destroy()
