"""The examples that show the extension API run end to end on CPU: a user-defined dataloader, and trainers that subclass
``DistributedTrainer`` with their own model / config classes."""
import importlib.util
import os
import sys

import pytest

import torch

from helpers import make_config, run_distributed, single_process_env, tiny_llama_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _custom_dataloader_run(out_file):
    from nanotron_b200.trainer import DistributedTrainer

    ex = _load("examples/custom_dataloader/run_train.py", "custom_dl_example")
    cfg = make_config(tiny_llama_config(vocab_size=64), dp=2, seq=32, mbs=2, accum=1, steps=30, lr=3e-3)
    cfg.logging.iteration_step_info_interval = 1
    t = DistributedTrainer(cfg)
    losses = []

    orig = t.train_step_logs

    def record(outputs, loss_avg, z_loss_avg=None):
        if loss_avg is not None:
            losses.append(float(loss_avg))
        return orig(outputs=outputs, loss_avg=loss_avg, z_loss_avg=z_loss_avg)

    t.train_step_logs = record
    loader = ex.build_dataloader(t, num_steps=30, seed=1)
    # the two data-parallel ranks must see different samples
    first = next(iter(loader))["input_ids"]
    import nanotron_b200.distributed as dist

    gathered = [torch.empty_like(torch.as_tensor(first)) for _ in range(2)]
    dist.all_gather(gathered, torch.as_tensor(first).contiguous(), group=t.parallel_context.dp_pg)
    assert not torch.equal(gathered[0], gathered[1])
    t.train({"stable": ex.build_dataloader(t, num_steps=30, seed=1)})
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save(losses, out_file)
    t.parallel_context.destroy()


def test_custom_dataloader_example_trains(tmp_path):
    out = str(tmp_path / "losses.pt")
    run_distributed(_custom_dataloader_run, 2, out_file=out)
    losses = torch.load(out)
    assert len(losses) == 30
    assert losses[-1] < losses[0] - 0.25, losses  # counting sequences are learnable


def _doremi_run(out_file):
    sys.path.insert(0, os.path.join(ROOT, "examples", "doremi"))
    import doremi as dr
    import nanotron_b200.distributed as dist

    train = _load("examples/doremi/train_doremi.py", "train_doremi_example")
    os.chdir(os.path.dirname(out_file))  # the example's relative checkpoints_path lands in the test's scratch directory
    t = dr.DoReMiTrainer(os.path.join(ROOT, "examples", "doremi", "config_tiny_doremi.yaml"))  # YAML with the extra section
    assert isinstance(t.config, dr.DoReMiConfig) and t.config.doremi.domain_names == ["counting", "noise"]
    assert isinstance(t.unwrapped_model, dr.LlamaForDoReMiTraining) and isinstance(t.ref_model, dr.LlamaReferenceForDoReMi)
    assert all(not p.requires_grad for p in t.ref_model.parameters())
    # proxy and reference start from different weights
    a = next(iter(t.unwrapped_model.parameters())).detach().float()
    b = next(iter(t.ref_model.parameters())).detach().float()
    assert not torch.equal(a, b)
    t.config.tokens.train_steps = 25
    t.train({"proxy": train.domain_batches(t, seed=7)})
    w = t.doremi_context.domain_weights
    # same weights on both data-parallel ranks, still a distribution, moved away from uniform
    both = [torch.empty_like(w) for _ in range(2)]
    dist.all_gather(both, w.contiguous(), group=t.parallel_context.dp_pg)
    torch.testing.assert_close(both[0], both[1])
    assert abs(float(w.sum()) - 1.0) < 1e-5 and float((w - 0.5).abs().max()) > 1e-3, w
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save({"weights": w.cpu(), "n_updates": len(t.doremi_context.history)}, out_file)
    t.parallel_context.destroy()


def test_doremi_trainer_subclass_example(tmp_path):
    out = str(tmp_path / "doremi.pt")
    run_distributed(_doremi_run, 2, out_file=out)
    res = torch.load(out)
    assert res["n_updates"] == 26  # the initial weights + one update per step


def _mamba_run(out_file, tp=1, pp=1, steps=80):
    sys.path.insert(0, os.path.join(ROOT, "examples", "mamba"))
    import nanotron_b200.distributed as dist

    create = _load("examples/mamba/create_config_mamba.py", "create_config_mamba_example")
    train = _load("examples/mamba/train_mamba.py", "train_mamba_example")
    import mamba as mb
    from trainer import MambaTrainer

    os.chdir(os.path.dirname(out_file))
    cfg = create.build(d_model=32, layers=2, vocab=16, seq=32, mbs=8, steps=steps, tp=tp, pp=pp, lr=3e-2)
    path = os.path.join(os.path.dirname(out_file), f"mamba_{os.environ.get('RANK', '0')}.yaml")  # one file per rank: they are written concurrently
    cfg.save_as_yaml(path)  # the extended config survives the YAML round trip without naming its classes
    t = MambaTrainer(path)
    assert isinstance(t.unwrapped_model, mb.MambaForTraining) and t.model_config.ssm()["dt_rank"] == 2
    t.prepare_training()
    data = train.copy_task_batches(t, seed=3, period=6)
    losses = []
    for _ in range(steps):
        _, loss, _ = t.training_step(data)
        t.iteration_step += 1
        if loss is not None:
            losses.append(float(loss))
    rank = dist.get_rank(t.parallel_context.world_pg)
    if losses and rank == dist.get_world_size(t.parallel_context.world_pg) - 1:
        torch.save({"losses": losses}, out_file)
    if tp > 1:
        # the mixer's own sharded parameters (A_log, D, convolution) go through the checkpoint like the linears' weights
        from nanotron_b200.serialize import load_weights

        t.config.checkpoints.checkpoints_path = type(t.config.checkpoints.checkpoints_path)(os.path.dirname(out_file)) / "ckpt"
        ck = t.save_checkpoint()
        model = t.unwrapped_model
        before = {n: p.detach().clone() for n, p in model.named_parameters()}
        with torch.no_grad():
            for p in model.parameters():
                p.zero_()
        load_weights(model=model, parallel_context=t.parallel_context, root_folder=ck)
        for n, p in model.named_parameters():
            assert torch.equal(p, before[n]), n
    if tp == 1 and pp == 1:
        # recurrent decoding (one position per step, constant state) continues a prompt exactly like the full forward
        model = t.unwrapped_model.eval()
        prompt = torch.randint(2, 16, (2, 9))
        out = mb.greedy_decode(model, prompt, max_new_tokens=4)
        mask = torch.ones(2, out.shape[1] - 1, dtype=torch.bool)
        logits = model.model(input_ids=out[:, :-1], input_mask=mask).view(2, out.shape[1] - 1, -1)
        assert torch.equal(logits[:, 8:].argmax(-1), out[:, 9:])
    t.parallel_context.destroy()


def test_mamba_example_learns_the_copy_task(tmp_path):
    """The selective-scan model of examples/mamba trains through the framework's trainer: on sequences that repeat a 6-token
    pattern the loss falls well below the uniform level log(14) = 2.64; step-by-step decoding agrees with the parallel forward."""
    out = str(tmp_path / "mamba.pt")
    run_distributed(_mamba_run, 1, out_file=out)
    losses = torch.load(out)["losses"]
    assert losses[0] > 2.3 and min(losses[-5:]) < 0.7 * losses[0], losses[::10]


def test_mamba_example_under_tensor_and_pipeline_parallelism(tmp_path):
    out = str(tmp_path / "mamba_tp.pt")
    run_distributed(_mamba_run, 4, out_file=out, tp=2, pp=2, steps=30)
    losses = torch.load(out)["losses"]
    assert losses[-1] < losses[0] and all(l == l for l in losses), losses[::5]


def test_mup_example_keeps_logits_stable_across_widths(tmp_path, monkeypatch):
    """examples/mup: under the spectral parametrisation the output logits of a freshly initialised model have the same size at
    width 64 and at width 256; under the standard one (one std for every matrix) they grow with sqrt(width)."""
    from helpers import dummy_dataloader, single_process_env

    from nanotron_b200.trainer import DistributedTrainer

    mup = _load("examples/mup/config_mup_llama.py", "config_mup_llama_example")
    monkeypatch.chdir(tmp_path)
    single_process_env()
    stds = {}
    for use_mup in (True, False):
        for width in (64, 256):
            cfg = mup.build(use_mup, hidden_size=width, layers=2, heads=4, vocab=512, seq=32, mbs=2, acc=1, dp=1, steps=2, lr=1e-3, dtype="float32")
            cfg.checkpoints.checkpoint_interval = 10**6
            cfg.checkpoints.save_final_state = False
            t = DistributedTrainer(cfg)
            assert t.model_config.is_using_mup == use_mup
            torch.manual_seed(0)
            ids = torch.randint(0, 512, (2, 32))
            with torch.no_grad():
                logits = t.unwrapped_model.model(input_ids=ids, input_mask=torch.ones(2, 32, dtype=torch.bool))
            stds[(use_mup, width)] = float(logits.float().std())
            if use_mup and width == 64:
                t.prepare_training()
                _, loss, _ = t.training_step(dummy_dataloader(t))
                assert torch.isfinite(loss)
            t.parallel_context.destroy()
    assert 0.8 < stds[(True, 256)] / stds[(True, 64)] < 1.25, stds
    assert 1.6 < stds[(False, 256)] / stds[(False, 64)] < 2.4, stds


def _llamoe_run(out_file):
    sys.path.insert(0, os.path.join(ROOT, "examples", "moe"))
    import nanotron_b200.distributed as dist
    from helpers import dummy_dataloader

    cfgmod = _load("examples/moe/config_llamoe.py", "config_llamoe")
    sys.modules["config_llamoe"] = cfgmod  # train_moe imports it by this name
    train = _load("examples/moe/train_moe.py", "train_moe_example")
    import llamoe

    os.chdir(os.path.dirname(out_file))
    cfg = cfgmod.build(hidden_size=32, layers=2, heads=4, experts=4, top_k=2, expert_size=32, vocab=64, seq=32, mbs=2, dp=2, ep=2, steps=12, dtype="float32", lr=3e-3)
    path = os.path.join(os.path.dirname(out_file), f"llamoe_{os.environ.get('RANK', '0')}.yaml")  # one file per rank: they are written concurrently
    cfg.save_as_yaml(path)
    t = train.make_trainer(path)  # from the YAML file: the extra model-config fields survive the round trip
    model = t.unwrapped_model
    assert isinstance(model, llamoe.LlaMoEForTraining) and isinstance(t.model_config, cfgmod.LlaMoEConfig) and t.model_config.log_expert_load
    no_decay = model.get_named_params_without_weight_decay()
    assert any(".router." in n for n in no_decay)
    t.prepare_training()
    data = dummy_dataloader(t)
    losses = []
    for _ in range(12):
        _, loss, _ = t.training_step(data)
        t.iteration_step += 1
        losses.append(float(loss))
    report = model.expert_load_report()
    assert len(report) == 2 and all(0.25 <= v <= 1.0 for v in report.values()), report  # one router per layer, 4 experts
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save({"losses": losses}, out_file)
    t.parallel_context.destroy()


def test_llamoe_example_trains_with_expert_parallelism(tmp_path):
    out = str(tmp_path / "llamoe.pt")
    run_distributed(_llamoe_run, 2, out_file=out)
    losses = torch.load(out)["losses"]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses


def test_every_shipped_configuration_file_loads():
    """All YAML files under examples/ parse with the strict loader (a renamed or removed config field shows up here), including
    the ones with their own config classes."""
    import glob

    from nanotron_b200.config import Config, get_config_from_file

    sys.path.insert(0, os.path.join(ROOT, "examples", "mamba"))
    sys.path.insert(0, os.path.join(ROOT, "examples", "doremi"))
    special = {}
    from config import MambaConfig  # examples/mamba

    special["config_mamba.yaml"] = dict(config_class=MambaConfig)
    import doremi as dr

    special["config_tiny_doremi.yaml"] = dict(config_class=dr.DoReMiConfig)
    llamoe = _load("examples/moe/config_llamoe.py", "config_llamoe_for_load")
    special["config_llamoe.yaml"] = dict(model_config_class=llamoe.LlaMoEConfig)
    files = sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.yaml"), recursive=True))
    assert len(files) >= 14, files
    for path in files:
        cfg = get_config_from_file(path, **special.get(os.path.basename(path), {}))
        assert isinstance(cfg, Config) and cfg.parallelism.dp >= 1, path
    variants = _load("examples/config_variants.py", "config_variants_example")
    assert variants.resume().checkpoints.resume_checkpoint_path is not None
    assert variants.s3_upload().s3_upload.upload_s3_path.startswith("s3://")
    assert variants.nanoset().data_stages[1].data.dataset.dataset_weights == [0.8, 0.2]


def test_doremi_quotas_and_domain_weighted_sampler():
    sys.path.insert(0, os.path.join(ROOT, "examples", "doremi"))
    import numpy as np
    from dataloader import CombinedDataset, DomainWeightedSampler, apportion, domain_weights_from_token_count
    from utils import SyntheticDomain

    # quotas: sum to the batch, within one sample of the exact share unless the floor binds, every domain keeps one sample
    assert apportion([0.5, 0.3, 0.2], 10) == [5, 3, 2]
    assert apportion([0.98, 0.01, 0.01], 16) == [14, 1, 1]
    assert sum(apportion([0.37, 0.33, 0.30], 7)) == 7
    rng = np.random.default_rng(0)
    wins = np.zeros(3)
    for _ in range(300):  # equal weights, 4 samples: the extra sample goes to every domain equally often with a random tie-break
        wins += np.asarray(apportion([1, 1, 1], 4, rng=rng)) - 1
    assert wins.sum() == 300 and wins.min() > 60
    with pytest.raises(ValueError):
        apportion([0.5, 0.5], 1)
    # the sampler: both data-parallel ranks draw from one global batch that follows the weights; domains never repeat an item
    # inside a pass; a change of the weights shows in the next global batch
    domains = [SyntheticDomain("counting", 40, 9, 32), SyntheticDomain("noise", 24, 9, 32), SyntheticDomain("repeat", 16, 9, 32)]
    combined = CombinedDataset(domains)
    assert len(combined) == 80 and combined.locate(40) == (1, 0) and combined[63]["domain_idx"] == 1 and combined[64]["domain_idx"] == 2
    torch.testing.assert_close(domain_weights_from_token_count(domains), torch.tensor([0.5, 0.3, 0.2]))
    weights = {"w": [0.5, 0.25, 0.25]}
    samplers = [DomainWeightedSampler(combined.lengths, micro_batch_size=2, num_microbatches=2, dp_size=2, dp_rank=r, weights_fn=lambda: weights["w"], seed=3) for r in range(2)]
    its = [iter(s) for s in samplers]
    seen = [[], [], []]
    for step in range(4):
        batch = [i for it in its for _ in range(2) for i in next(it)]  # 2 ranks x 2 micro-batches x 2 samples
        assert len(batch) == 8 and len(set(batch)) == 8
        doms = [combined.locate(i)[0] for i in batch]
        assert [doms.count(d) for d in range(3)] == [4, 2, 2] == samplers[0].last_quotas
        for i, d in zip(batch, doms):
            seen[d].append(i)
    assert all(len(set(s)) == len(s) for s in seen)
    weights["w"] = [0.125, 0.75, 0.125]
    batch = [i for it in its for _ in range(2) for i in next(it)]
    assert [[combined.locate(i)[0] for i in batch].count(d) for d in range(3)] == [1, 6, 1]
    # resumable: a new sampler with the saved counters continues with the same batches
    state = samplers[0].state_dict()
    fresh = DomainWeightedSampler(combined.lengths, 2, 2, 2, 0, lambda: weights["w"], seed=3)
    fresh.load_state_dict(state)
    assert [next(its[0]) for _ in range(4)] == [b for _, b in zip(range(4), iter(fresh))]
    # an exhausted domain starts a new pass (default) or ends the epoch
    stop = DomainWeightedSampler([3, 100], 2, 1, 1, 0, lambda: [0.5, 0.5], seed=0, on_exhausted="stop")
    assert len(list(stop)) == 3
    wrap = DomainWeightedSampler([3, 100], 2, 1, 1, 0, lambda: [0.5, 0.5], seed=0)
    got = [b for _, b in zip(range(6), iter(wrap))]
    assert wrap.passes[0] == 1 and sorted(i for b in got for i in b if i < 3) == [0, 0, 1, 1, 2, 2]


def _doremi_reference_run(out_file, ckpt):
    sys.path.insert(0, os.path.join(ROOT, "examples", "doremi"))
    import doremi as dr
    import nanotron_b200.distributed as dist
    from dataloader import get_dataloader
    from utils import get_domain_datasets

    os.chdir(os.path.dirname(out_file))
    cfg_path = os.path.join(ROOT, "examples", "doremi", "config_tiny_doremi.yaml")
    # step 1 of the recipe: a reference model on a fixed 3:1 mixture, with the loss of every domain
    ref = dr.ReferenceTrainer(cfg_path, domain_weights=torch.tensor([0.75, 0.25]))
    ref.config.tokens.train_steps = 30
    ref.config.checkpoints.checkpoints_path = ckpt + "/ref"
    datasets = get_domain_datasets(ref)
    ref.train({"proxy": get_dataloader(ref, datasets, weights_fn=ref.sampling_weights)})
    assert ref.doremi_sampler.last_quotas == [6, 2]  # global batch 8
    losses = ref.domain_losses
    assert float(losses[0]) < float(losses[1]) - 0.5, losses  # counting is learnable, noise is not
    del ref
    # step 2: the proxy scores against that checkpoint; its weight history lands beside its own checkpoints and is resumed
    t = dr.DoReMiTrainer(cfg_path)
    assert t.config.doremi.ref_model_resume_checkpoint_path is None
    t.config.doremi.ref_model_resume_checkpoint_path = ckpt + "/ref/30"
    dr.load_weights(model=t.ref_model, parallel_context=t.parallel_context, root_folder=ckpt + "/ref/30")
    t.config.tokens.train_steps = 6
    t.config.checkpoints.checkpoints_path = ckpt + "/proxy"
    t.train({"proxy": get_dataloader(t, get_domain_datasets(t), weights_fn=t.sampling_weights)})
    assert t.doremi_sampler.last_quotas == [4, 4]  # sampling keeps the starting mixture, the loss is re-weighted
    final = t.doremi_context.domain_weights.clone()
    n = len(t.doremi_context.history)
    dist.barrier()
    avg = dr.average_domain_weights(ckpt + "/proxy/doremi_domain_weights_6.pt")
    torch.testing.assert_close(avg, torch.stack(t.doremi_context.history).mean(0).cpu())
    del t
    from nanotron_b200.config import get_config_from_file

    cfg = get_config_from_file(cfg_path, config_class=dr.DoReMiConfig)
    cfg.checkpoints.checkpoints_path = ckpt + "/proxy"
    cfg.checkpoints.resume_checkpoint_path = ckpt + "/proxy"
    cfg.doremi.ref_model_resume_checkpoint_path = ckpt + "/ref/30"
    resumed = dr.DoReMiTrainer(cfg)
    torch.testing.assert_close(resumed.doremi_context.domain_weights, final)
    assert len(resumed.doremi_context.history) == n and resumed.iteration_step == 6
    if dist.get_rank(resumed.parallel_context.world_pg) == 0:
        torch.save({"ref_domain_losses": losses.cpu(), "weights": final.cpu()}, out_file)
    resumed.parallel_context.destroy()


def test_doremi_reference_then_proxy_with_saved_domain_weights(tmp_path):
    out = str(tmp_path / "doremi_ref.pt")
    run_distributed(_doremi_reference_run, 2, out_file=out, ckpt=str(tmp_path / "ckpt"))
    res = torch.load(out)
    assert abs(float(res["weights"].sum()) - 1.0) < 1e-5


def test_doremi_loss_updates_the_domain_weights_as_specified():
    """excess_d = mean over the tokens of domain d of max(proxy - reference, 0); w <- normalise(w * exp(step * excess)) mixed with the
    uniform distribution; loss = sum_d w_d * (token losses of d) * n_domains / tokens."""
    sys.path.insert(0, os.path.join(ROOT, "examples", "doremi"))
    import doremi as dr
    from nanotron_b200.parallel.context import ParallelContext

    single_process_env()
    ctx = ParallelContext(tensor_parallel_size=1, pipeline_parallel_size=1, data_parallel_size=1)
    args = dr.DoReMiArgs(domain_names=["a", "b", "c"], domain_weights=[0.5, 0.3, 0.2], step_size=0.7, smoothing_param=0.01)
    state = dr.DoReMiContext(args, torch.device("cpu"))
    loss_block = dr.DoReMiLoss(ctx.tp_pg, ctx.dp_pg, state)
    torch.manual_seed(0)
    b, s, v = 4, 6, 11
    logits = torch.randn(b * s, v, requires_grad=True)
    labels = torch.randint(0, v, (b, s))
    mask = torch.ones(b, s, dtype=torch.bool)
    mask[1, 4:] = False
    domains = torch.tensor([0, 2, 0, 1])
    ref_losses = torch.rand(b, s) * 2.5 * mask
    out = loss_block(logits, labels, mask, domains, ref_losses)
    token_losses = torch.nn.functional.cross_entropy(logits.detach(), labels.reshape(-1), reduction="none").view(b, s) * mask
    excess = (token_losses - ref_losses).clamp(min=0)
    per_domain = torch.stack([excess[domains == d].sum() / mask[domains == d].sum() for d in range(3)])
    torch.testing.assert_close(out["excess_losses"], per_domain)
    w = torch.tensor([0.5, 0.3, 0.2]) * torch.exp(0.7 * per_domain)
    w = 0.99 * w / w.sum() + 0.01 / 3
    torch.testing.assert_close(state.domain_weights, w)
    assert len(state.history) == 2 and abs(float(state.domain_weights.sum()) - 1) < 1e-6
    expected = sum(w[d] * token_losses[domains == d].sum() for d in range(3)) * 3 / mask.sum()
    torch.testing.assert_close(out["loss"], expected)
    torch.testing.assert_close(out["ce_loss"], token_losses.sum() / mask.sum())
    out["loss"].backward()
    assert logits.grad is not None and float(logits.grad.view(b, s, v)[1, 4:].abs().sum()) == 0  # masked tokens carry no gradient
    # evaluation (no gradient) reads the weights without moving them
    with torch.no_grad():
        loss_block(logits, labels, mask, domains, ref_losses)
    assert len(state.history) == 2
    # uniform weights reduce to the plain mean
    uniform = dr.DoReMiContext(dr.DoReMiArgs(domain_names=["a", "b", "c"], step_size=0.0, smoothing_param=0.0), torch.device("cpu"))
    plain = dr.DoReMiLoss(ctx.tp_pg, ctx.dp_pg, uniform)(logits, labels, mask, domains, ref_losses)
    torch.testing.assert_close(plain["loss"], plain["ce_loss"])
    ctx.destroy()
