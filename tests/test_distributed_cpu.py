"""Multi-rank behaviour on CPU/gloo: process-group topology, TP layers vs an unsharded oracle, ZeRO-1 vs plain
data parallelism, pipeline engines vs a single stage, checkpoint round trip across topologies."""
import os

import pytest
import torch

from helpers import dummy_dataloader, make_config, run_distributed, tiny_llama_config, tiny_qwen_config


# --------------------------------------------------------------------------- topology
def _check_context(tp, pp, dp, cp, ep):
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext

    ctx = ParallelContext(tensor_parallel_size=tp, pipeline_parallel_size=pp, data_parallel_size=dp, context_parallel_size=cp, expert_parallel_size=ep)
    rank = dist.get_rank(ctx.world_pg)
    assert ctx.tp_pg.size() == tp and ctx.pp_pg.size() == pp and ctx.dp_pg.size() == dp and ctx.cp_pg.size() == cp and ctx.ep_pg.size() == ep
    local = ctx.get_local_ranks(rank)
    assert ctx.get_global_rank(ep_rank=local["ep"], pp_rank=local["pp"], dp_rank=local["dp"], cp_rank=local["cp"], tp_rank=local["tp"]) == rank
    # tp ranks are adjacent
    assert dist.get_global_ranks(ctx.tp_pg) == tuple(range(rank - local["tp"], rank - local["tp"] + tp))
    assert ctx.expert_dp_pg.size() == dp // ep
    assert local["ep"] == dist.get_rank(ctx.ep_pg)
    ctx.destroy()


@pytest.mark.parametrize("tp,pp,dp,cp,ep", [(2, 1, 2, 1, 1), (1, 2, 2, 1, 2), (2, 2, 1, 1, 1), (1, 1, 2, 2, 1), (1, 1, 4, 1, 2)])
def test_parallel_context(tp, pp, dp, cp, ep):
    run_distributed(_check_context, tp * pp * dp * cp, tp=tp, pp=pp, dp=dp, cp=cp, ep=ep)


# --------------------------------------------------------------------------- TP layers
def _check_tp_linear(mode, async_comm):
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
    from nanotron_b200.parallel.tensor_parallel.nn import TensorParallelColumnLinear, TensorParallelEmbedding, TensorParallelRowLinear

    ctx = ParallelContext(tensor_parallel_size=2, pipeline_parallel_size=1, data_parallel_size=1)
    tp_mode = TensorParallelLinearMode[mode]
    rank = dist.get_rank(ctx.tp_pg)
    torch.manual_seed(0)
    H, F, T = 8, 12, 6
    w1 = torch.randn(F, H, dtype=torch.float64)
    w2 = torch.randn(H, F, dtype=torch.float64)
    x_full = torch.randn(T, H, dtype=torch.float64)
    col = TensorParallelColumnLinear(H, F, pg=ctx.tp_pg, mode=tp_mode, bias=False, dtype=torch.float64, async_communication=async_comm, contiguous_chunks=(8, 4))
    row = TensorParallelRowLinear(F, H, pg=ctx.tp_pg, mode=tp_mode, bias=False, dtype=torch.float64, async_communication=False)
    with torch.no_grad():
        shard = torch.cat([w1[0:8].chunk(2)[rank], w1[8:12].chunk(2)[rank]])
        col.weight.copy_(shard)
        cols = torch.cat([torch.arange(0, 8).chunk(2)[rank], torch.arange(8, 12).chunk(2)[rank]])
        row.weight.copy_(w2[:, cols])
    x_in = x_full.chunk(2)[rank].clone().requires_grad_(True) if tp_mode is TensorParallelLinearMode.REDUCE_SCATTER else x_full.clone().requires_grad_(True)
    y = row(torch.tanh(col(x_in)))
    # oracle
    xo = x_full.clone().requires_grad_(True)
    w1o, w2o = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    yo = torch.tanh(xo @ w1o.t()) @ w2o.t()
    y_exp = yo.chunk(2)[rank] if tp_mode is TensorParallelLinearMode.REDUCE_SCATTER else yo
    torch.testing.assert_close(y, y_exp)
    g = torch.randn_like(yo)
    yo.backward(g)
    y.backward(g.chunk(2)[rank] if tp_mode is TensorParallelLinearMode.REDUCE_SCATTER else g)
    torch.testing.assert_close(x_in.grad, xo.grad.chunk(2)[rank] if tp_mode is TensorParallelLinearMode.REDUCE_SCATTER else xo.grad)
    torch.testing.assert_close(col.weight.grad, torch.cat([w1o.grad[0:8].chunk(2)[rank], w1o.grad[8:12].chunk(2)[rank]]))
    torch.testing.assert_close(row.weight.grad, w2o.grad[:, cols])
    # embedding
    emb = TensorParallelEmbedding(10, 4, pg=ctx.tp_pg, mode=tp_mode, dtype=torch.float64)
    table = torch.randn(10, 4, dtype=torch.float64)
    with torch.no_grad():
        emb.weight.copy_(table.chunk(2)[rank])
    ids = torch.tensor([0, 9, 4, 5, 5, 2])
    out = emb(ids)
    exp = table[ids]
    torch.testing.assert_close(out, exp.chunk(2)[rank] if tp_mode is TensorParallelLinearMode.REDUCE_SCATTER else exp)
    ctx.destroy()


@pytest.mark.parametrize("mode,async_comm", [("ALL_REDUCE", False), ("REDUCE_SCATTER", False), ("REDUCE_SCATTER", True)])
def test_tp_layers_match_unsharded(mode, async_comm):
    run_distributed(_check_tp_linear, 2, mode=mode, async_comm=async_comm)


def _check_sharded_ce():
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.tensor_parallel.functional import sharded_cross_entropy_with_z_loss

    ctx = ParallelContext(tensor_parallel_size=2, pipeline_parallel_size=1, data_parallel_size=1)
    rank = dist.get_rank(ctx.tp_pg)
    torch.manual_seed(0)
    logits = torch.randn(5, 16)
    tgt = torch.randint(0, 16, (5,))
    local = logits.chunk(2, dim=-1)[rank].clone().requires_grad_(True)
    ce, z = sharded_cross_entropy_with_z_loss(local, tgt, group=ctx.tp_pg, z_loss_coef=1e-2)
    (ce + z).mean().backward()
    full = logits.clone().requires_grad_(True)
    lz = torch.logsumexp(full, -1)
    exp = torch.nn.functional.cross_entropy(full, tgt, reduction="none")
    (exp + 1e-2 * lz**2).mean().backward()
    torch.testing.assert_close(ce, exp, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(local.grad, full.grad.chunk(2, dim=-1)[rank], atol=1e-6, rtol=1e-4)
    ctx.destroy()


def test_vocab_parallel_cross_entropy():
    run_distributed(_check_sharded_ce, 2)


# --------------------------------------------------------------------------- trainer-level equivalences
def _packed_positions(rows, seq, generator):
    """Position ids of rows packed with several documents (a 0 starts one); the first document of a row may have begun earlier."""
    out = []
    for _ in range(rows):
        cuts = sorted(set(torch.randint(1, seq, (3,), generator=generator).tolist()))
        bounds = [0] + cuts + [seq]
        pos = torch.cat([torch.arange(b - a) for a, b in zip(bounds[:-1], bounds[1:])])
        pos[: bounds[1]] += int(torch.randint(0, 5, (1,), generator=generator))
        out.append(pos)
    return torch.stack(out)


def _fixed_batches(trainer, n, total_mbs, seq, vocab, uses_mask=True, seed=123, packed=False):
    """The same global batch for every topology: ``total_mbs`` sequences per step, this rank takes its dp slice."""
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

    ctx = trainer.parallel_context
    g = torch.Generator().manual_seed(seed)
    dp, dp_rank = ctx.dp_pg.size(), dist.get_rank(ctx.dp_pg)
    pp_rank = dist.get_rank(ctx.pp_pg)
    per_rank = total_mbs // dp
    mbs = trainer.micro_batch_size
    out = []
    for _ in range(n):
        tokens = torch.randint(0, vocab, (total_mbs, seq + 1), generator=g)
        positions = _packed_positions(total_mbs, seq, g) if packed else torch.arange(seq).unsqueeze(0).expand(total_mbs, -1)
        mine = tokens[dp_rank * per_rank : (dp_rank + 1) * per_rank]
        for i in range(0, per_rank, mbs):
            t = mine[i : i + mbs]
            b = {}
            if pp_rank == trainer.unwrapped_model.input_pp_rank:
                b["input_ids"] = t[:, :-1].contiguous()
                if uses_mask:
                    b["input_mask"] = torch.ones(mbs, seq, dtype=torch.bool)
                else:
                    b["position_ids"] = positions[dp_rank * per_rank + i : dp_rank * per_rank + i + mbs].contiguous()
            else:
                b["input_ids"] = TensorPointer(trainer.unwrapped_model.input_pp_rank)
                b["input_mask" if uses_mask else "position_ids"] = TensorPointer(trainer.unwrapped_model.input_pp_rank)
            if pp_rank == trainer.unwrapped_model.output_pp_rank:
                b["label_ids"] = t[:, 1:].contiguous()
                b["label_mask"] = torch.ones(mbs, seq, dtype=torch.bool)
            else:
                b["label_ids"] = TensorPointer(trainer.unwrapped_model.output_pp_rank)
                b["label_mask"] = TensorPointer(trainer.unwrapped_model.output_pp_rank)
            cp, cp_rank = ctx.cp_pg.size(), dist.get_rank(ctx.cp_pg)
            if cp > 1:
                from nanotron_b200.parallel.context_parallel.zigzag import zigzag_slice

                b = {k: (zigzag_slice(v, cp_rank, cp, dim=1).contiguous() if isinstance(v, torch.Tensor) else v) for k, v in b.items()}
            out.append(b)
    return out


def _deterministic_init(model):
    """Every topology gets the same unsharded weights: values depend only on the parameter's canonical name and on
    the element's position in the unsharded tensor."""
    import zlib

    tied_names = getattr(model, "get_embeddings_lm_head_tied_names", lambda: [])()
    tied_matrix = bool(tied_names) or getattr(getattr(model, "config", None), "tie_word_embeddings", False)
    with torch.no_grad():
        for name, p in model.get_named_params_with_correct_tied():
            shape = tuple(p.get_sharded_info().unsharded_shape) if p.is_sharded else tuple(p.shape)
            seed_name = name
            if tied_matrix and ("token_embedding" in name or "lm_head" in name):
                seed_name = "tied_word_embeddings"  # one matrix under two names (one per pipeline stage)
            g = torch.Generator().manual_seed(zlib.crc32(seed_name.encode()))
            full = torch.randn(shape, generator=g, dtype=torch.float32) * 0.05
            if "layernorm" in name or "layer_norm" in name or "ln_" in name:
                full = 1.0 + full
            if p.is_sharded:
                for sp in p.get_sharded_info().local_global_slices_pairs:
                    p[sp.local_slices] = full[sp.global_slices].to(p.dtype)
            else:
                p.copy_(full.to(p.dtype))


def _train_losses(out_file, steps=4, total_mbs=4, model="llama", norms_file=None, **topology):
    import nanotron_b200.distributed as dist
    from nanotron_b200.trainer import DistributedTrainer as _Base

    class DistributedTrainer(_Base):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    dp = topology.get("dp", 1)
    mbs = topology.pop("mbs", 1)
    if topology.get("cp", 1) > 1:
        topology["fp32_accum"] = True
    accum = total_mbs // (dp * mbs)
    tie = topology.pop("tie", False)
    packed = topology.pop("packed", False)
    layers = topology.pop("layers", 2)
    if model == "moe":
        import nanotron_b200.config as c

        moe = c.MoEConfig(num_experts=4, top_k=2, moe_intermediate_size=16, shared_expert_intermediate_size=32, enable_shared_expert=True, router_aux_loss_coef=0.01)
        mc = tiny_qwen_config(tie_word_embeddings=tie, moe_config=moe)
    else:
        mc = tiny_llama_config(tie_word_embeddings=tie, num_hidden_layers=layers) if model == "llama" else tiny_qwen_config(tie_word_embeddings=tie, _use_doc_masking=packed, num_hidden_layers=layers)
    cfg = make_config(mc, seq=16, mbs=mbs, accum=accum, steps=steps, lr=1e-2, **topology)
    t = DistributedTrainer(cfg)
    t.prepare_training()
    batches = iter(_fixed_batches(t, steps, total_mbs, 16, mc.vocab_size, uses_mask=(model == "llama"), packed=packed))
    losses, norms = [], []
    for _ in range(steps):
        _, loss, _ = t.training_step(batches)
        t.iteration_step += 1
        if loss is not None:
            losses.append(float(loss))
        norms.append(float(t.grad_norm_unclipped))
    if norms_file is not None and dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save(norms, norms_file)
    if tie and t.parallel_context.pp_pg.size() > 1:
        # the two copies of the tied matrix (embedding on the first stage, lm head on the last) must still be equal
        pp_pg = t.parallel_context.pp_pg
        mine = [p for n, p in t.unwrapped_model.named_parameters() if "token_embedding" in n or "lm_head" in n]
        assert len(mine) == 1, [n for n, _ in t.unwrapped_model.named_parameters()]
        copies = [torch.empty_like(mine[0].data) for _ in range(pp_pg.size())]
        dist.all_gather(copies, mine[0].data.contiguous(), group=pp_pg)
        torch.testing.assert_close(copies[0], copies[-1], atol=0, rtol=0)
    if dist.get_rank(t.parallel_context.world_pg) == t.logger_ranks[0]:
        torch.save(losses, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def _losses_for(tmp_path, world, name, **kw):
    f = str(tmp_path / f"{name}.pt")
    kw.setdefault("norms_file", str(tmp_path / f"{name}_norms.pt"))
    run_distributed(_train_losses, world, out_file=f, **kw)
    return torch.load(f)


def _norms_for(tmp_path, name):
    """Unclipped gradient norms of the steps of a run made by ``_losses_for`` (what gradient clipping would have used)."""
    return torch.load(str(tmp_path / f"{name}_norms.pt"))


def _same_norms(tmp_path, name, ref_name):
    got, ref = _norms_for(tmp_path, name), _norms_for(tmp_path, ref_name)
    for a, b in zip(got, ref):
        assert abs(a - b) < 2e-4 * b, (name, got, ref)


def test_topologies_agree_on_loss_curve(tmp_path):
    """dp / zero-1 / tp (both modes) / pp (both engines) give the same loss curve as one process on the same data."""
    base = _losses_for(tmp_path, 1, "base")
    assert base[-1] < base[0]
    cases = {
        "dp2": dict(dp=2),
        "dp2_zero1": dict(dp=2, zero=1),
        "tp2_ar": dict(tp=2, tp_mode="all_reduce"),
        "tp2_sp_async": dict(tp=2, tp_mode="reduce_scatter", async_tp=True),  # (the synchronous form runs in the bf16 / accumulator tests)
        "pp2_1f1b": dict(pp=2, pp_engine="1f1b"),  # (all-forward-all-backward: tests/test_pipeline_cpu.py and the Starcoder2 layouts)
    }
    for name, kw in cases.items():
        world = kw.get("dp", 1) * kw.get("tp", 1) * kw.get("pp", 1)
        got = _losses_for(tmp_path, world, name, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-4, (name, got, base)
        # the norm gradient clipping uses counts every weight once under every layout (shards summed, replicas counted once)
        _same_norms(tmp_path, name, "base")


def test_3d_and_qwen_topologies(tmp_path):
    # clip far below the gradient norm, so that every step really clips: a weight that is scaled on one rank and not on another shows
    base = _losses_for(tmp_path, 1, "qbase", model="qwen", clip=0.05)
    got = _losses_for(tmp_path, 4, "q3d", model="qwen", dp=2, tp=2, tp_mode="reduce_scatter", zero=1, sanity=True, clip=0.05)  # with the runtime invariant checks on
    for a, b in zip(got, base):
        assert abs(a - b) < 2e-4, (got, base)
    got = _losses_for(tmp_path, 4, "qpp", model="qwen", pp=2, tp=2, pp_engine="1f1b", clip=0.05)
    for a, b in zip(got, base):
        assert abs(a - b) < 2e-4, (got, base)
    got = _losses_for(tmp_path, 2, "qcp", model="qwen", cp=2, clip=0.05)
    for a, b in zip(got, base):
        assert abs(a - b) < 2e-4, (got, base)


def test_tied_embeddings_across_stages_with_zero1(tmp_path):
    """Embedding and lm head tied across two pipeline stages, each stage data-parallel with ZeRO-1: the tie-group sum of the
    gradients must see whole (not reduce-scattered) gradients, or the two copies drift apart."""
    base = _losses_for(tmp_path, 1, "tbase", tie=True)
    got = _losses_for(tmp_path, 4, "tpp2dp2", tie=True, pp=2, dp=2, zero=1, pp_engine="1f1b", sanity=True)
    for a, b in zip(got, base):
        assert abs(a - b) < 2e-4, (got, base)
    _same_norms(tmp_path, "tpp2dp2", "tbase")  # the tied matrix is counted once, not once per stage


def test_single_process_overfits_fixed_batch():
    """Guards the optimizer wiring: the fp32 masters must keep receiving gradients after ``zero_grad``."""
    from helpers import single_process_env
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    t = DistributedTrainer(make_config(tiny_llama_config(), seq=32, steps=8, lr=1e-2))
    t.prepare_training()
    batch = next(dummy_dataloader(t))
    losses = []
    for _ in range(8):
        _, loss, _ = t.training_step(iter([batch]))
        t.iteration_step += 1
        losses.append(float(loss))
    t.parallel_context.destroy()
    assert all(b < a for a, b in zip(losses, losses[1:])), losses
    assert losses[-1] < losses[0] - 0.5, losses


def test_expert_parallel_training_matches_replicated_experts(tmp_path):
    """A Qwen2-MoE model on 2 data-parallel ranks: with the experts split over the two ranks (ep 2: tokens travel to their
    experts, expert gradients are averaged over expert_dp and already contain both ranks' tokens) the loss curve is the one of
    replicated experts (ep 1), also together with tensor parallelism.  ZeRO-1 over ranks that own different experts is refused."""
    rep = _losses_for(tmp_path, 2, "moe_dp2", model="moe", dp=2)
    assert rep[-1] < rep[0]
    got = _losses_for(tmp_path, 2, "moe_ep2", model="moe", dp=2, ep=2)
    for a, b in zip(got, rep):
        assert abs(a - b) < 3e-4, (got, rep)
    _same_norms(tmp_path, "moe_ep2", "moe_dp2")  # expert shards summed over the expert ranks, dense weights counted once
    # with sequence-parallel tp every rank routes its own token shard (the load-balance loss is a statistic of that shard), so the
    # like-for-like comparison is the same tp layout with replicated experts
    rep_tp = _losses_for(tmp_path, 4, "moe_dp2_tp2", model="moe", dp=2, tp=2, tp_mode="reduce_scatter")
    got = _losses_for(tmp_path, 4, "moe_ep2_tp2", model="moe", dp=2, tp=2, ep=2, tp_mode="reduce_scatter", sanity=True)  # invariant checks know which ranks replicate an expert
    for a, b in zip(got, rep_tp):
        assert abs(a - b) < 3e-4, (got, rep_tp)
    _same_norms(tmp_path, "moe_ep2_tp2", "moe_dp2_tp2")  # the tp copies of an expert count once
    assert abs(rep_tp[0] - rep[0]) < 5e-3  # the two layouts differ only in that statistic
    with pytest.raises(AssertionError, match="cannot be combined with expert_parallel_size"):
        _losses_for(tmp_path, 2, "moe_ep2_zero1", model="moe", dp=2, ep=2, zero=1)


def test_expert_parallelism_with_pipeline_and_context_parallelism(tmp_path):
    """Experts split over the data-parallel ranks inside a 2-stage pipeline, and under context parallelism (every cp rank routes
    its own sequence shard): the same curves as with replicated experts."""
    rep = _losses_for(tmp_path, 2, "moe_dp2_b", model="moe", dp=2)
    got = _losses_for(tmp_path, 4, "moe_pp2_ep2", model="moe", dp=2, ep=2, pp=2, pp_engine="1f1b")
    for a, b in zip(got, rep):
        assert abs(a - b) < 3e-4, (got, rep)
    rep_cp = _losses_for(tmp_path, 4, "moe_cp2", model="moe", dp=2, cp=2)
    got = _losses_for(tmp_path, 4, "moe_cp2_ep2", model="moe", dp=2, ep=2, cp=2)
    for a, b in zip(got, rep_cp):
        assert abs(a - b) < 3e-4, (got, rep_cp)


def _two_stage_lengths(out_file, ckpt=None, resume=None, **topology):
    import importlib.util

    import nanotron_b200.config as c
    import nanotron_b200.distributed as dist
    from helpers import tiny_qwen_config
    from nanotron_b200.trainer import DistributedTrainer

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("run_train_for_stage_test", os.path.join(root, "run_train.py"))
    run_train = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(run_train)
    cfg = make_config(tiny_qwen_config(max_position_embeddings=64), seq=16, mbs=2, accum=2, steps=5, lr=1e-2, sanity=True, ckpt_path=ckpt, ckpt_interval=4, **topology)
    cfg.checkpoints.resume_checkpoint_path = resume
    cfg.data_stages = [
        c.DatasetStageArgs(name="short", start_training_step=1, data=c.DataArgs(dataset=None, seed=3)),
        c.DatasetStageArgs(name="long", start_training_step=3, data=c.DataArgs(dataset=None, seed=4), sequence_length=32),
    ]
    t = DistributedTrainer(cfg)
    seen = []
    step = t.training_step

    def spy(dataloader):
        result = step(dataloader)
        seen.append((t.iteration_step, t.sequence_length) + ((round(float(result[1]), 5),) if result[1] is not None else ()))
        return result

    t.training_step = spy
    t.train(run_train.get_dataloader(t))
    if dist.get_rank(t.parallel_context.world_pg) == t.logger_ranks[0]:
        torch.save({"seen": seen, "tokens": t.metadata.consumed_tokens_total, "stages": [(s.name, s.consumed_train_samples, s.sequence_length) for s in t.metadata.data_stages]}, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def test_data_stages_may_change_the_sequence_length_under_pipeline_parallelism(tmp_path):
    """The second stage doubles the sequence length: pipeline stages that replay learnt activation shapes must learn the new ones
    at the switch, and the token accounting follows the stage's length."""
    out, ckpt = str(tmp_path / "stages.pt"), str(tmp_path / "ckpt")
    layout = dict(pp=2, tp=2, tp_mode="reduce_scatter", pp_engine="1f1b")
    run_distributed(_two_stage_lengths, 4, out_file=out, ckpt=ckpt, **layout)
    res = torch.load(out)
    assert [(step, length) for step, length, _ in res["seen"]] == [(1, 16), (2, 16), (3, 32), (4, 32), (5, 32)]
    assert res["tokens"] == 2 * 4 * 16 + 3 * 4 * 32 and res["stages"] == [("short", 8, 16), ("long", 12, 32)]
    # resumed inside the second stage (checkpoint of step 4): the synthetic stream continues where it stopped, so step 5 repeats exactly
    run_distributed(_two_stage_lengths, 4, out_file=out, ckpt=ckpt, resume=ckpt, **layout)
    again = torch.load(out)
    assert again["seen"] == res["seen"][4:] and again["tokens"] == res["tokens"] and again["stages"] == res["stages"]


def test_training_without_the_fp32_accumulator_agrees_across_layouts(tmp_path):
    """``accumulate_grad_in_fp32: false``: gradients live on the parameters, the data-parallel exchange and the ZeRO slices work on
    them directly; same loss curve as one process, with clipping active and the invariant checks on."""
    base = _losses_for(tmp_path, 1, "plain_base", fp32_accum=False, sanity=True, clip=0.05)
    with_accumulator = _losses_for(tmp_path, 1, "accum_base", sanity=True, clip=0.05)
    for a, b in zip(base, with_accumulator):
        assert abs(a - b) < 1e-5  # float32 parameters: the two gradient paths are the same arithmetic
    for name, world, kw in (("plain_dp2_zero1", 2, dict(dp=2, zero=1)), ("plain_tp2_pp2", 4, dict(tp=2, pp=2, tp_mode="reduce_scatter", pp_engine="1f1b"))):
        got = _losses_for(tmp_path, world, name, fp32_accum=False, sanity=True, clip=0.05, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-4, (name, got, base)


def test_bfloat16_parameters_with_fp32_masters_agree_across_layouts(tmp_path):
    """bf16 parameters, fp32 gradient accumulation and master weights (the production precision) on CPU ranks: sharding the
    optimizer does not change the arithmetic; tensor / pipeline parallelism only reorders bf16 roundings."""
    kw = dict(dtype="bfloat16", sanity=True, clip=0.05)
    base = _losses_for(tmp_path, 1, "bf16_base", **kw)
    zero = _losses_for(tmp_path, 2, "bf16_dp2_zero1", dp=2, zero=1, **kw)
    for a, b in zip(zero, base):
        assert abs(a - b) < 2e-4, (zero, base)
    model_parallel = _losses_for(tmp_path, 4, "bf16_tp2_pp2", tp=2, pp=2, tp_mode="reduce_scatter", pp_engine="1f1b", **kw)
    for a, b in zip(model_parallel, base):
        assert abs(a - b) < 5e-3, (model_parallel, base)


def test_packed_documents_train_the_same_under_context_parallelism(tmp_path):
    """Qwen2 with document masking on rows packed with several documents: splitting every sequence over 2 ranks (alone, and
    together with tensor parallelism) gives the loss curve of one process; without the masking the curve is a different one."""
    base = _losses_for(tmp_path, 1, "docs_base", model="qwen", packed=True, sanity=True)
    unmasked = _losses_for(tmp_path, 1, "docs_unmasked", model="qwen", sanity=True)
    assert max(abs(a - b) for a, b in zip(base, unmasked)) > 1e-4
    for name, world, kw in (("docs_cp2", 2, dict(cp=2)), ("docs_cp2_tp2", 4, dict(cp=2, tp=2, tp_mode="reduce_scatter"))):
        got = _losses_for(tmp_path, world, name, model="qwen", packed=True, sanity=True, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-4, (name, got, base)
