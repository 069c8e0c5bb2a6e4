"""Unit tests of the distributed building blocks on gloo / CPU ranks: P2P wire protocol, random-state branching and syncing,
tied parameters, gradient clipping against torch's own, ZeRO-1 against the replicated optimizer, activation recomputation,
SFT masking, tensor metadata and random-state serialisation, the S3 mover state machine, dtype-invariant buffers."""
import os
import stat

import numpy as np
import pytest
import torch

from helpers import dummy_dataloader, make_config, run_distributed, single_process_env, tiny_llama_config


# ------------------------------------------------------------------------------------------------ P2P
def _p2p_rank():
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.pipeline_parallel.p2p import P2P, BatchTensorSendRecvState

    ctx = ParallelContext(1, 2, 1)
    rank = dist.get_rank(ctx.pp_pg)
    p2p = P2P(ctx.pp_pg, device=torch.device("cpu"))
    torch.manual_seed(0)
    base = torch.randn(6, 8)
    cases = [
        base.clone(),                                  # contiguous fp32
        base.t(),                                      # transposed view
        base[1:5, ::2],                                # sliced, strided, with storage offset
        base.to(torch.bfloat16),                       # another dtype
        torch.arange(10, dtype=torch.int64),           # integer
        base.clone().requires_grad_(True),             # requires_grad travels in the header
        torch.tensor(3.5),                             # 0-dim
    ]
    if rank == 0:
        p2p.send_tensors(cases, to_rank=1)
        back = p2p.recv_tensors(1, from_rank=1)[0]
        assert torch.equal(back, base * 2)
    else:
        got = p2p.recv_tensors(len(cases), from_rank=0)
        for g, e in zip(got, cases):
            assert g.shape == e.shape and g.dtype == e.dtype and g.requires_grad == e.requires_grad, (g.shape, e.shape, g.dtype)
            assert torch.equal(g.detach(), e.detach())
        p2p.send_tensors([got[0] * 2], to_rank=0)
    # batched exchange in both directions at once
    batch = BatchTensorSendRecvState(p2p)
    other = 1 - rank
    batch.add_send(torch.full((4,), float(rank)), to_rank=other)
    batch.add_recv(from_rank=other)
    out = batch.flush()
    assert torch.equal(out[0], torch.full((4,), float(other)))
    # fixed-shape streams may skip re-reading the header
    p2p.expect_static(True)
    for i in range(3):
        if rank == 0:
            p2p.send_tensors([base + i], to_rank=1, tag=7)
        else:
            assert torch.equal(p2p.recv_tensors(1, from_rank=0, tag=7)[0], base + i)
    ctx.destroy()


def test_p2p_protocol():
    run_distributed(_p2p_rank, 2)


# ------------------------------------------------------------------------------------------------ random states
def _random_rank():
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.random import RandomStates, branch_random_state, get_current_random_state, get_synced_random_state, set_random_seed

    ctx = ParallelContext(2, 1, 1)
    rank = dist.get_rank(ctx.tp_pg)
    set_random_seed(100 + rank)  # ranks start apart
    synced = get_synced_random_state(get_current_random_state(), ctx.tp_pg)
    states = RandomStates({"tp_synced": synced})
    a_before = torch.rand(3)  # ambient stream: differs between ranks
    with branch_random_state(states, "tp_synced", enabled=True):
        b1 = torch.rand(3)
    with branch_random_state(states, "tp_synced", enabled=True):
        b2 = torch.rand(3)
    a_after = torch.rand(3)
    gathered = [torch.zeros(3) for _ in range(2)]
    dist.all_gather(gathered, b1, group=ctx.tp_pg)
    assert torch.equal(gathered[0], gathered[1])          # branch is the same on both ranks
    assert not torch.equal(b1, b2)                         # and advances between uses
    dist.all_gather(gathered, a_before, group=ctx.tp_pg)
    assert not torch.equal(gathered[0], gathered[1])      # ambient streams stay different
    # the branch did not disturb the ambient stream
    set_random_seed(100 + rank)
    get_synced_random_state(get_current_random_state(), ctx.tp_pg)
    assert torch.equal(torch.rand(3), a_before) and torch.equal(torch.rand(3), a_after)
    ctx.destroy()


def test_random_state_branch_and_sync():
    run_distributed(_random_rank, 2)


def test_random_states_serialise(tmp_path):
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.random import RandomStates, get_current_random_state, set_random_seed
    from nanotron_b200.serialize.random import load_random_states, save_random_states

    single_process_env()
    ctx = ParallelContext(1, 1, 1)
    set_random_seed(5)
    rs = RandomStates({"tp_synced": get_current_random_state()})
    save_random_states(rs, ctx, tmp_path)
    back = load_random_states(ctx, tmp_path)
    assert back == rs
    ctx.destroy()


# ------------------------------------------------------------------------------------------------ tied parameters
def _tied_rank():
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.tied_parameters import create_pg_for_tied_weights, get_tied_id_to_param, sync_tied_weights_gradients, tie_parameters

    ctx = ParallelContext(1, 2, 1)
    rank = dist.get_rank(ctx.pp_pg)
    # same-process tie: two modules end up sharing one Parameter object
    m = torch.nn.ModuleDict({"a": torch.nn.Linear(4, 4, bias=False), "b": torch.nn.Linear(4, 4, bias=False)})
    me = dist.get_rank(ctx.world_pg)
    tie_parameters(m, [("a.weight", (me,)), ("b.weight", (me,))], ctx, dist.ReduceOp.SUM)
    assert m["a"].weight is m["b"].weight and m["a"].weight.is_tied
    # cross-process tie: each pipeline rank holds one copy; gradients are summed over the tie group
    torch.manual_seed(0)
    lin = torch.nn.Linear(4, 4, bias=False)
    root = torch.nn.ModuleDict({"emb" if rank == 0 else "head": lin})
    name = ("emb" if rank == 0 else "head") + ".weight"
    tie_parameters(root, [("emb.weight", (0,)), ("head.weight", (1,))], ctx, dist.ReduceOp.SUM)
    create_pg_for_tied_weights(root, ctx)
    p = dict(root.named_parameters())[name]
    assert p.is_tied and p.get_tied_info().global_ranks == (0, 1)
    p.grad = torch.full_like(p, float(rank + 1))
    sync_tied_weights_gradients(root, ctx, grad_accumulator=None)
    assert torch.equal(p.grad, torch.full_like(p, 3.0))
    assert len(get_tied_id_to_param(list(root.parameters()), root)) == 1
    ctx.destroy()


def test_tied_parameters():
    run_distributed(_tied_rank, 2)


# ------------------------------------------------------------------------------------------------ clipping, ZeRO, recompute
def _trainer(world_kw, **kw):
    from nanotron_b200.trainer import DistributedTrainer
    from test_distributed_cpu import _deterministic_init

    class T(DistributedTrainer):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    cfg = make_config(tiny_llama_config(), seq=16, mbs=2, steps=4, lr=1e-2, **world_kw, **kw)
    t = T(cfg)
    t.prepare_training()
    return t


def _clip_rank(out_file, tp):
    import nanotron_b200.distributed as dist

    t = _trainer(dict(tp=tp, tp_mode="all_reduce"), clip=0.05)
    from test_distributed_cpu import _fixed_batches

    batches = iter(_fixed_batches(t, 1, 2, 16, 256, uses_mask=True))
    t.training_step(batches)
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save(float(t.grad_norm_unclipped), out_file)
    dist.barrier()
    t.parallel_context.destroy()


def test_clipped_norm_is_topology_independent_and_matches_torch(tmp_path):
    f1, f2 = str(tmp_path / "n1.pt"), str(tmp_path / "n2.pt")
    run_distributed(_clip_rank, 1, out_file=f1, tp=1)
    run_distributed(_clip_rank, 2, out_file=f2, tp=2)
    n1, n2 = torch.load(f1), torch.load(f2)
    assert n1 > 0.05 and abs(n1 - n2) < 1e-4 * n1, (n1, n2)


def test_clip_grad_norm_equals_torch_on_one_process():
    from nanotron_b200.optim.clip_grads import clip_grad_norm
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.parameters import NanotronParameter

    single_process_env()
    ctx = ParallelContext(1, 1, 1)
    torch.manual_seed(0)
    params = [NanotronParameter(torch.randn(5, 7)), NanotronParameter(torch.randn(11))]
    for p in params:
        p.grad = torch.randn_like(p)
    ref = [torch.nn.Parameter(p.detach().clone()) for p in params]
    for r, p in zip(ref, params):
        r.grad = p.grad.clone()
    exp = torch.nn.utils.clip_grad_norm_(ref, max_norm=0.3)
    got = clip_grad_norm(ctx.mp_pg, [(f"p{i}", p) for i, p in enumerate(params)], max_norm=0.3, grad_accumulator=None)
    torch.testing.assert_close(got, exp, atol=1e-6, rtol=1e-6)
    for r, p in zip(ref, params):
        torch.testing.assert_close(p.grad, r.grad, atol=1e-6, rtol=1e-5)
    ctx.destroy()


def _zero_rank(out_file, zero):
    import nanotron_b200.distributed as dist
    from test_distributed_cpu import _fixed_batches

    t = _trainer(dict(dp=2, zero=zero), accum=1)
    batches = iter(_fixed_batches(t, 3, 4, 16, 256, uses_mask=True))
    for _ in range(3):
        t.training_step(batches)
        t.iteration_step += 1
    flat = torch.cat([p.detach().float().reshape(-1) for _, p in sorted(t.unwrapped_model.named_parameters())])
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save(flat, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def test_zero1_is_bit_exact_with_the_replicated_optimizer(tmp_path):
    f0, f1 = str(tmp_path / "z0.pt"), str(tmp_path / "z1.pt")
    run_distributed(_zero_rank, 2, out_file=f0, zero=0)
    run_distributed(_zero_rank, 2, out_file=f1, zero=1)
    assert torch.equal(torch.load(f0), torch.load(f1))


def test_activation_recomputation_changes_nothing():
    from test_distributed_cpu import _fixed_batches

    res = []
    for recompute in (False, True):
        single_process_env()
        t = _trainer({}, recompute=recompute)
        batches = iter(_fixed_batches(t, 2, 2, 16, 256, uses_mask=True))
        losses = []
        for _ in range(2):
            _, loss, _ = t.training_step(batches)
            t.iteration_step += 1
            losses.append(float(loss))
        res.append((losses, torch.cat([p.detach().reshape(-1) for _, p in sorted(t.unwrapped_model.named_parameters())])))
        t.parallel_context.destroy()
    assert res[0][0] == res[1][0]
    torch.testing.assert_close(res[0][1], res[1][1], atol=1e-7, rtol=0)


# ------------------------------------------------------------------------------------------------ data / metadata / misc
class _Tok:
    eos_token_id = 1
    pad_token_id = 0

    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": [10 + (ord(c) % 50) for c in text]}


def test_sft_masks_only_the_completion():
    from nanotron_b200.data.sft_processing import process_sft

    out = process_sft({"prompt": ["abc", "a much longer prompt than fits"], "completion": ["xy", "z"]}, _Tok(), sequence_length=8)
    ids, mask, pos = out["input_ids"][0], out["label_mask"][0], out["position_ids"][0]
    assert len(ids) == 9 and ids[5] == 1 and ids[6] == 0            # prompt(3) + completion(2) + eos, then padding
    assert mask.tolist() == [False] * 3 + [True] * 3 + [False] * 3   # loss on completion + eos only
    assert pos.tolist() == [0, 1, 2, 3, 4, 5, 0, 1, 2]               # padding restarts the positions (its own document)
    assert not out["label_mask"][1].any()                             # prompt alone fills the window: nothing to learn from


def test_tensor_metadata_round_trip():
    from nanotron_b200.constants import CHECKPOINT_VERSION
    from nanotron_b200.parallel.parameters import SlicesPair
    from nanotron_b200.serialize.metadata import TensorMetadata

    pairs = (SlicesPair(local_slices=(slice(0, 4), slice(None)), global_slices=(slice(8, 12), slice(None))),
             SlicesPair(local_slices=(slice(4, 6), slice(None)), global_slices=(slice(20, 22), slice(None))))
    meta = TensorMetadata(version=CHECKPOINT_VERSION, local_global_slices_pairs=pairs, unsharded_shape=(32, 16))
    d = meta.to_str_dict()
    assert all(isinstance(v, str) for v in d.values())
    back = TensorMetadata.from_str_dict(d)
    assert back.local_global_slices_pairs == pairs and tuple(back.unsharded_shape) == (32, 16) and back.version == CHECKPOINT_VERSION
    with pytest.raises(AssertionError):
        TensorMetadata.from_str_dict({**d, "surprise": "1"})


def test_dtype_invariant_tensor_keeps_its_dtype():
    from nanotron_b200.models.base import DTypeInvariantTensor

    t = DTypeInvariantTensor(torch.arange(4, dtype=torch.float32))
    assert t.to("cpu").dtype == torch.float32  # device moves are allowed
    with pytest.raises(RuntimeError):
        t.to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        t.to(dtype=torch.float32)  # any dtype argument is refused, even the current one
    with pytest.raises(RuntimeError):
        t.half()
    m = torch.nn.Module()
    m.register_buffer("inv_freq", t)
    m.to(torch.device("cpu"))  # device moves are fine


def test_s3_mover_state_machine_with_a_fake_s5cmd(tmp_path):
    from nanotron_b200.s3_checkpoints import S3Mover

    local = tmp_path / "ckpt"
    (local / "10").mkdir(parents=True)
    (local / "10" / "w.bin").write_bytes(b"x" * 10)
    fake = tmp_path / "s5cmd"
    log = tmp_path / "calls.txt"
    fake.write_text(f"#!/bin/sh\necho \"$@\" >> {log}\ncase \"$*\" in *fail*) exit 3;; esac\nexit 0\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    done = []
    mover = S3Mover(local_path=str(local), s3_path="s3://bucket/run", post_upload_callback=lambda uploaded_files=None: done.append(1), remove_after_upload=True, s5cmd_path=str(fake))
    assert mover.state == S3Mover.S3MoverState.IDLE and mover.is_previous_save_finished()
    mover.start_uploading()
    assert mover.state in (S3Mover.S3MoverState.UPLOADING, S3Mover.S3MoverState.REMOVING_CHECKPOINT, S3Mover.S3MoverState.IDLE)
    mover.wait_for_completion()
    assert mover.state == S3Mover.S3MoverState.IDLE
    calls = log.read_text()
    assert "cp" in calls and "s3://bucket/run" in calls
    assert not (local / "10" / "w.bin").exists()  # removed after the upload
    assert done == [1]
    # a failing transfer is reported and leaves the mover usable
    bad = S3Mover(local_path=str(local), s3_path="s3://bucket/fail", remove_after_upload=False, s5cmd_path=str(fake))
    (local / "11").mkdir()
    (local / "11" / "w.bin").write_bytes(b"y")
    bad.start_uploading()
    bad.wait_for_completion()
    assert bad.state == S3Mover.S3MoverState.IDLE and (local / "11" / "w.bin").exists()


# ------------------------------------------------------------------------------------------------ optimizer parameter groups
def test_param_groups_get_their_weight_decay_and_learning_rate(tmp_path):
    """Norm gains (the model's own no-decay list) and names matched by ``weight_decay_exclude_named_params`` sit in groups with
    weight decay 0, everything else decays; one AdamW step with zero gradients therefore shrinks exactly the decayed
    parameters; under the spectral parametrisation matrices get learning rates scaled by their fan-in / fan-out."""
    from nanotron_b200.config import SpectralMupInit
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    cfg = make_config(tiny_llama_config(hidden_size=32, intermediate_size=64), seq=16, mbs=2, steps=2, dtype="float32", lr=1e-2)
    cfg.optimizer.weight_decay = 0.5
    cfg.optimizer.weight_decay_exclude_named_params = [r".*down_proj.*"]
    cfg.optimizer.zero_stage = 0
    cfg.optimizer.accumulate_grad_in_fp32 = False
    cfg.checkpoints.checkpoints_path = tmp_path
    t = DistributedTrainer(cfg)
    base = t.optimizer.get_base_optimizer()
    id_to_name = {id(p): n for n, p in t.unwrapped_model.named_parameters()}
    decayed, spared = set(), set()
    for group in base.param_groups:
        for p in group["params"]:
            (decayed if group["weight_decay"] > 0 else spared).add(id_to_name[id(p)])
        assert group["lr"] == pytest.approx(1e-2) or group["lr"] == 0.0  # standard parametrisation: one learning rate (0 before warm-up starts)
    assert any("down_proj" in n for n in spared) and not any("down_proj" in n for n in decayed)
    assert all("norm" in n or "down_proj" in n for n in spared), spared
    assert any("qkv_proj" in n for n in decayed) and any("token_embedding" in n for n in decayed)
    before = {n: p.detach().clone() for n, p in t.unwrapped_model.named_parameters()}
    for p in t.unwrapped_model.parameters():
        p.grad = torch.zeros_like(p)
    for group in base.param_groups:
        group["lr"] = 1e-2
    t.optimizer.step()
    for n, p in t.unwrapped_model.named_parameters():
        if n in spared:
            assert torch.equal(p, before[n]), n  # zero gradient, no decay: untouched
        else:
            torch.testing.assert_close(p, before[n] * (1 - 1e-2 * 0.5))
    t.parallel_context.destroy()
    # spectral muP: per-matrix learning rates
    cfg2 = make_config(tiny_llama_config(hidden_size=32, intermediate_size=128), seq=16, mbs=2, steps=2, dtype="float32", lr=1e-2)
    cfg2.model.init_method = SpectralMupInit(use_mup=True)
    cfg2.model.model_config._is_using_mup = True
    cfg2.optimizer.zero_stage = 0
    cfg2.optimizer.accumulate_grad_in_fp32 = False
    cfg2.checkpoints.checkpoints_path = tmp_path
    t2 = DistributedTrainer(cfg2)
    lrs = {}
    names = {id(p): n for n, p in t2.unwrapped_model.named_parameters()}
    for group in t2.optimizer.get_base_optimizer().param_groups:
        for p in group["params"]:
            lrs[names[id(p)]] = group.get("initial_lr", group["lr"])
    up = next(v for n, v in lrs.items() if "gate_up_proj" in n)  # fan_out 256 / fan_in 32
    down = next(v for n, v in lrs.items() if "down_proj" in n)  # fan_out 32 / fan_in 128
    assert up > down, (up, down)
    t2.parallel_context.destroy()


def test_fsspec_helpers_copy_between_file_systems(tmp_path):
    from nanotron_b200.s3_checkpoints import check_path_is_local, fs_copy, fs_open

    src = tmp_path / "a.bin"
    payload = bytes(range(256)) * 5000  # larger than nothing, smaller than a block
    src.write_bytes(payload)
    fs_copy(src, "memory://bucket/run/a.bin")
    with fs_open("memory://bucket/run/a.bin", mode="rb") as f:
        assert f.read() == payload
    fs_copy("memory://bucket/run/a.bin", tmp_path / "back.bin")
    assert (tmp_path / "back.bin").read_bytes() == payload
    assert check_path_is_local(tmp_path) and not check_path_is_local("memory://bucket/run")


def test_learning_rate_schedules_have_the_documented_shapes():
    """Linear / constant warm-up, then cosine / linear / 1-sqrt decay to ``min_decay_lr`` over ``lr_decay_steps`` from ``lr_decay_starting_step``,
    then flat; the default decay length is what is left of training after the warm-up."""
    import math

    import nanotron_b200.config as c
    from nanotron_b200.helpers import lr_scheduler_builder

    def curve(total=20, **kw):
        p = torch.nn.Parameter(torch.zeros(1))
        opt = torch.optim.SGD([p], lr=1.0)
        sched = lr_scheduler_builder(opt, c.LRSchedulerArgs(learning_rate=1.0, **kw), total_training_steps=total)
        out = []
        for _ in range(total + 3):
            out.append(opt.param_groups[0]["lr"])
            opt.step()
            sched.step()
        return out

    cos = curve(lr_warmup_steps=4, lr_warmup_style="linear", lr_decay_style="cosine", lr_decay_steps=10, lr_decay_starting_step=6, min_decay_lr=0.1)
    assert cos[:5] == pytest.approx([0.0, 0.25, 0.5, 0.75, 1.0]) and cos[5] == cos[6] == pytest.approx(1.0)  # warm-up, then the plateau before the decay starts
    assert cos[11] == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 5 / 10)))  # half way down the cosine
    assert cos[16] == pytest.approx(0.1) and cos[-1] == pytest.approx(0.1)  # floor, kept after the decay ends
    assert all(a >= b - 1e-12 for a, b in zip(cos[6:], cos[7:]))  # monotone from the plateau on
    lin = curve(lr_warmup_steps=2, lr_warmup_style="constant", lr_decay_style="linear", lr_decay_steps=8, min_decay_lr=0.2)
    assert lin[0] == lin[1] == pytest.approx(1.0)  # constant warm-up stays at the peak
    assert lin[2 + 4] == pytest.approx(0.2 + 0.8 * 0.5) and lin[10] == pytest.approx(0.2)
    sq = curve(lr_warmup_steps=0, lr_decay_style="1-sqrt", lr_decay_steps=16, min_decay_lr=0.0)
    assert sq[4] == pytest.approx(1 - math.sqrt(4 / 16)) and sq[16] == pytest.approx(0.0)
    # default decay length: total steps minus the warm-up
    default = curve(total=12, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="linear", min_decay_lr=0.0)
    assert default[2] == pytest.approx(1.0) and default[12] == pytest.approx(0.0) and default[7] == pytest.approx(0.5)


_FAKE_S5CMD = r'''#!/usr/bin/env python3
"""Stands in for s5cmd: ``cp [--exclude P]... SRC DST`` where ``s3://bucket/key`` lives under $FAKE_S3_ROOT/bucket/key."""
import fnmatch, os, shutil, sys
root = os.environ["FAKE_S3_ROOT"]
args = [a for a in sys.argv[1:]]
local = lambda p: os.path.join(root, p[len("s3://"):]) if p.startswith("s3://") else p
while args[0] not in ("cp", "cat"):
    args.pop(0) if args[0] == "--json" else (args.pop(0), args.pop(0))
if args.pop(0) == "cat":
    path = local(args[0])
    if not os.path.exists(path):
        sys.exit(1)
    sys.stdout.write(open(path).read())
    sys.exit(0)
exclude = []
while args[0].startswith("--"):
    flag, value = args.pop(0), args.pop(0)
    if flag == "--exclude":
        exclude.append(value)
src, dst = local(args[0]), local(args[1])
if src.endswith("*"):  # everything under a prefix, hierarchy kept
    src = os.path.dirname(src)
for folder, _, files in os.walk(src):
    for name in files:
        if any(fnmatch.fnmatch(name, pattern) for pattern in exclude):
            continue
        out = os.path.join(dst, os.path.relpath(os.path.join(folder, name), src))
        os.makedirs(os.path.dirname(out), exist_ok=True)
        shutil.copy(os.path.join(folder, name), out)
        print('{"operation":"cp","success":true,"source":"%s","destination":"%s"}' % (os.path.join(folder, name), out))
'''


def _train_with_upload(ckpt, tool, steps=4, resume=None, out_file=None):
    import nanotron_b200.config as c
    import nanotron_b200.distributed as dist
    from helpers import dummy_dataloader, make_config, tiny_llama_config
    from nanotron_b200.trainer import DistributedTrainer

    cfg = make_config(tiny_llama_config(), dp=2, seq=16, steps=steps, ckpt_path=ckpt, ckpt_interval=2)
    cfg.s3_upload = c.S3UploadArgs(upload_s3_path="s3://bucket/run1", remove_after_upload=True, s5cmd_numworkers=2, s5cmd_concurrency=2, s5cmd_path=tool)
    cfg.checkpoints.resume_checkpoint_path = resume
    t = DistributedTrainer(cfg)
    start = t.iteration_step
    t.train(dummy_dataloader(t))
    if out_file is not None and dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save({"start": start, "end": t.iteration_step, "samples": t.metadata.consumed_train_samples}, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def test_trainer_uploads_every_checkpoint_and_removes_the_local_copy(tmp_path):
    """``s3_upload`` in the configuration: after every save the checkpoint folder is copied to the bucket in the background (first
    rank of the node only), the next save waits for it, the local step folders are removed, and training ends after the last copy."""
    from helpers import run_distributed

    tool = tmp_path / "s5cmd"
    tool.write_text(_FAKE_S5CMD)
    tool.chmod(tool.stat().st_mode | stat.S_IEXEC)
    os.environ["FAKE_S3_ROOT"] = str(tmp_path / "object_store")
    remote = tmp_path / "object_store" / "bucket" / "run1"
    try:
        run_distributed(_train_with_upload, 2, ckpt=str(tmp_path / "ckpt"), tool=str(tool))
        assert sorted(os.listdir(remote)) == ["2", "4", "latest.txt"] and (remote / "latest.txt").read_text() == "4"
        for step in ("2", "4"):
            assert sorted(os.listdir(remote / step)) == ["checkpoint_metadata.json", "config.yaml", "lr_scheduler", "model", "model_config.json", "optimizer", "random"]
        assert sorted(os.listdir(tmp_path / "ckpt")) == ["latest.txt"]  # the step folders are gone
        # a new job on an empty disk resumes from the bucket: latest.txt is read remotely, step 4 is fetched, training goes on to 6
        out = str(tmp_path / "resumed.pt")
        run_distributed(_train_with_upload, 2, ckpt=str(tmp_path / "fresh_disk"), tool=str(tool), steps=6, resume="s3://bucket/run1", out_file=out)
    finally:
        os.environ.pop("FAKE_S3_ROOT")
    assert torch.load(out) == {"start": 4, "end": 6, "samples": 6 * 4}
    assert sorted(os.listdir(remote)) == ["2", "4", "6", "latest.txt"] and (remote / "latest.txt").read_text() == "6"
