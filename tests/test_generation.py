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
    # row 0 has no padding: the cached and recomputed paths must agree exactly
    assert torch.equal(a.generation_ids[0], b.generation_ids[0])
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
