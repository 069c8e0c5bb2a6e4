import pytest
import torch

from helpers import make_config, single_process_env, tiny_llama_config, tiny_qwen_config


def _build(model_config):
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    t = DistributedTrainer(make_config(model_config, seq=32))
    return t


def test_greedy_decode_cache_matches_recompute():
    from nanotron_b200.generation.decode import decode_tokenized

    t = _build(tiny_llama_config())
    ids = torch.randint(0, 256, (2, 7))
    mask = torch.ones(2, 7, dtype=torch.bool)
    mask[1, :3] = False  # left padding on row 1
    a = decode_tokenized(ids, mask, t.unwrapped_model.model, t.parallel_context, max_new_tokens=6, use_cache=False)
    b = decode_tokenized(ids, mask, t.unwrapped_model.model, t.parallel_context, max_new_tokens=6, use_cache=True)
    assert a.generation_ids.shape == (2, 6)
    # with and without the key/value cache, for the unpadded row and for the left-padded one (padding takes no part in attention)
    assert torch.equal(a.generation_ids, b.generation_ids)
    # a row decoded alone gives what it gives inside the padded batch
    alone = decode_tokenized(ids[1:, 3:], mask[1:, 3:], t.unwrapped_model.model, t.parallel_context, max_new_tokens=6, use_cache=True)
    assert torch.equal(alone.generation_ids[0], b.generation_ids[1])
    # the timed mode changes nothing but reports the decoding rate of the call
    from nanotron_b200.generation.decode import _DecodeClock

    timed = decode_tokenized(ids, mask, t.unwrapped_model.model, t.parallel_context, max_new_tokens=6, use_cache=True, is_bench=True)
    assert torch.equal(timed.generation_ids, b.generation_ids)
    report = _DecodeClock.last_report
    assert report["first_step_s"] > 0 and report["later_steps_s"] > 0 and report["tokens_per_sec"] == pytest.approx(2 * 5 / report["later_steps_s"])
    t.parallel_context.destroy()


def test_qwen_decode_and_samplers():
    from nanotron_b200.config import GenerationArgs
    from nanotron_b200.generation.decode import decode_tokenized
    from nanotron_b200.generation.sampler import BasicSampler, GreedySampler, TopKSampler, TopPSampler

    t = _build(tiny_qwen_config())
    ids = torch.randint(0, 256, (2, 5))
    out = decode_tokenized(ids, torch.ones(2, 5, dtype=torch.bool), t.unwrapped_model.model, t.parallel_context, generation_config=GenerationArgs(sampler="top_k", top_k=5), max_new_tokens=4)
    assert out.generation_ids.shape == (2, 4)
    logits = torch.randn(3, 50)
    assert torch.equal(GreedySampler(pg=None)(logits).squeeze(1), logits.argmax(-1))
    top = torch.topk(logits, 5, dim=-1).indices
    tk = TopKSampler(pg=None, k=5)(logits)
    assert all(tk[i, 0] in top[i] for i in range(3))
    peaked = torch.full((2, 50), -20.0)
    peaked[:, 7] = 20.0
    assert TopPSampler(pg=None, p=0.9)(peaked).squeeze(1).tolist() == [7, 7]
    assert BasicSampler(pg=None)(peaked).squeeze(1).tolist() == [7, 7]
    t.parallel_context.destroy()


def _pp_decode(out_file, tp, pp, use_cache):
    import nanotron_b200.distributed as dist
    from nanotron_b200.generation.decode import decode_tokenized
    from nanotron_b200.trainer import DistributedTrainer
    from test_distributed_cpu import _deterministic_init

    class T(DistributedTrainer):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    t = T(make_config(tiny_llama_config(), tp=tp, pp=pp, seq=32))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (3, 8), generator=g)
    mask = torch.ones(3, 8, dtype=torch.bool)
    mask[0, :5] = False
    mask[2, :2] = False
    out = decode_tokenized(ids, mask, t.unwrapped_model.model, t.parallel_context, max_new_tokens=7, use_cache=use_cache, returns_logits=True)
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save(out.generation_ids.cpu(), out_file)
    # every rank (first stage, last stage, every tp rank) ends up with the same tokens
    ref = out.generation_ids.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, out.generation_ids)
    dist.barrier()
    t.parallel_context.destroy()


def test_decoding_through_pipeline_and_tensor_parallel_stages(tmp_path):
    """Generation with the model split over two pipeline stages (activations cross stages every step, new tokens travel back to the
    first stage) and two tensor-parallel ranks (sharded logits, sharded sampling) gives the tokens of a single process."""
    from helpers import run_distributed

    outs = {}
    for name, world, kw in [("single", 1, dict(tp=1, pp=1, use_cache=False)), ("pp2", 2, dict(tp=1, pp=2, use_cache=False)), ("pp2_cache", 2, dict(tp=1, pp=2, use_cache=True)), ("tp2pp2", 4, dict(tp=2, pp=2, use_cache=True))]:
        f = str(tmp_path / f"{name}.pt")
        run_distributed(_pp_decode, world, out_file=f, **kw)
        outs[name] = torch.load(f)
    for name in ("pp2", "pp2_cache", "tp2pp2"):
        assert torch.equal(outs[name], outs["single"]), (name, outs[name], outs["single"])


def _moe_decode(out_file, **topology):
    import nanotron_b200.config as c
    import nanotron_b200.distributed as dist
    from nanotron_b200.generation.decode import decode_tokenized
    from nanotron_b200.trainer import DistributedTrainer
    from test_distributed_cpu import _deterministic_init

    class T(DistributedTrainer):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    moe = c.MoEConfig(num_experts=4, top_k=2, moe_intermediate_size=16, shared_expert_intermediate_size=32, enable_shared_expert=True)
    t = T(make_config(tiny_qwen_config(moe_config=moe), seq=16, **topology))
    ids = torch.randint(0, 256, (2, 6), generator=torch.Generator().manual_seed(0))
    out = decode_tokenized(ids, torch.ones_like(ids, dtype=torch.bool), t.unwrapped_model.model, t.parallel_context, max_new_tokens=5)
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save(out.generation_ids.cpu(), out_file)
    dist.barrier()
    t.parallel_context.destroy()


def test_mixture_of_experts_decodes_the_same_with_experts_split_over_ranks(tmp_path):
    """Greedy decoding of a Qwen2 mixture-of-experts model: experts split over two expert-parallel ranks (tokens are dispatched
    and combined at every step) and a tensor-parallel split give the tokens of one process."""
    from helpers import run_distributed

    outs = {}
    for name, world, kw in (("single", 1, {}), ("ep2", 2, dict(dp=2, ep=2)), ("tp2", 2, dict(tp=2))):
        f = str(tmp_path / f"{name}.pt")
        run_distributed(_moe_decode, world, out_file=f, **kw)
        outs[name] = torch.load(f)
    assert torch.equal(outs["ep2"], outs["single"]) and torch.equal(outs["tp2"], outs["single"]), outs
