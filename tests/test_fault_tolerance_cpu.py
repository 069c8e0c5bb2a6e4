"""Failure detection without touching a GPU: failures are made on the host (a rank that exits between steps, a rank that
raises, a missing checkpoint shard, a dataloader worker that raises, a kill-switch file) and must surface as clear errors or
clean stops on the other ranks, never as a hang."""
import os
import time

import pytest
import torch

from helpers import dummy_dataloader, make_config, run_distributed, single_process_env, tiny_llama_config


def _silent_rank(hb_dir, marker_dir):
    """Rank 2 leaves between steps (no collective in flight); ranks 0 and 1 must notice within the heartbeat timeout."""
    import nanotron_b200.distributed as dist
    from nanotron_b200.fault_tolerance import Heartbeat, RankFailureError, Watchdog
    from nanotron_b200.parallel import ParallelContext

    ctx = ParallelContext(1, 1, 3)
    rank = dist.get_rank(ctx.world_pg)
    hb = Heartbeat(hb_dir, rank, interval=0.1).start()
    wd = Watchdog(hb_dir, rank, 3, timeout=3.0, startup_timeout=30.0)  # generous against a loaded test machine: healthy ranks beat every 0.1 s
    t = torch.ones(1)
    for step in range(1, 4):  # three healthy steps
        wd.raise_if_failed()
        hb.beat(step)
        dist.all_reduce(t, group=ctx.world_pg)
    if rank == 2:
        hb._stop.set()  # the process goes away without saying goodbye: its beats simply stop
        time.sleep(0.3)
        os._exit(0)
    t0 = time.time()
    try:
        while time.time() - t0 < 25:
            wd.raise_if_failed()  # the check every rank makes before launching the next step
            time.sleep(0.1)
        raise AssertionError("dead rank was not detected")
    except RankFailureError as e:
        # the other survivor may already have seen the failure and said so in its own heartbeat file
        assert "last heartbeat" in e.failed[2] and all("reported failure" in why for r, why in e.failed.items() if r != 2)
        open(os.path.join(marker_dir, f"detected_{rank}"), "w").write(f"{time.time() - t0:.2f}")
    hb.stop("failed")
    os._exit(0)  # do not enter a destroy-barrier with a dead peer


def test_rank_that_stops_between_steps_is_detected(tmp_path):
    hb, marks = tmp_path / "hb", tmp_path / "marks"
    hb.mkdir()
    marks.mkdir()
    run_distributed(_silent_rank, 3, hb_dir=str(hb), marker_dir=str(marks))
    assert sorted(os.listdir(marks)) == ["detected_0", "detected_1"]
    assert all(float(open(marks / f).read()) < 20 for f in os.listdir(marks))


def _raising_rank(marker_dir):
    """Rank 1 raises inside a step; rank 0 is waiting in a collective of a group with a short timeout and must get an
    error instead of waiting forever."""
    import datetime

    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext

    ctx = ParallelContext(1, 1, 2)
    rank = dist.get_rank(ctx.world_pg)
    short = torch.distributed.new_group(ranks=[0, 1], timeout=datetime.timedelta(seconds=3), backend="gloo")
    t = torch.ones(1)
    dist.all_reduce(t, group=short)
    if rank == 1:
        open(os.path.join(marker_dir, "raised_1"), "w").write("x")
        os._exit(0)  # stands for an exception that unwinds the process: it never joins the next collective
    t0 = time.time()
    try:
        dist.all_reduce(t, group=short)
        raise AssertionError("collective with a missing peer returned")
    except RuntimeError as e:
        open(os.path.join(marker_dir, "error_0"), "w").write(f"{time.time() - t0:.2f} {type(e).__name__}")
    os._exit(0)


def test_collective_with_a_missing_peer_errors_out(tmp_path):
    run_distributed(_raising_rank, 2, marker_dir=str(tmp_path))
    assert sorted(os.listdir(tmp_path)) == ["error_0", "raised_1"]
    assert float(open(tmp_path / "error_0").read().split()[0]) < 30


def test_reported_failure_and_missing_heartbeat(tmp_path):
    from nanotron_b200.fault_tolerance import Heartbeat, RankFailureError, StepDeadline, StepDeadlineExceeded, Watchdog

    a = Heartbeat(str(tmp_path), 0, interval=0.05).start()
    b = Heartbeat(str(tmp_path), 1, interval=0.05).start()
    wd = Watchdog(str(tmp_path), 0, 3, timeout=5.0, startup_timeout=0.3)
    assert wd.failed_ranks() == {}  # rank 2 has not appeared yet, but is still within its start-up allowance
    time.sleep(0.4)
    assert list(wd.failed_ranks()) == [2] and "no heartbeat" in wd.failed_ranks()[2]
    b.beat(7)
    b.stop("failed")
    with pytest.raises(RankFailureError) as ei:
        wd.raise_if_failed()
    assert ei.value.failed[1] == "reported failure at step 7"
    assert wd.slowest().step == 0
    a.stop()
    with pytest.raises(StepDeadlineExceeded):
        with StepDeadline(0.05):
            time.sleep(0.1)
    with StepDeadline(None):
        pass


def test_kill_switch_saves_and_stops(tmp_path):
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    switch = tmp_path / "stop_now"
    os.environ["NANOTRON_KILL_SWITCH"] = str(switch)
    try:
        cfg = make_config(tiny_llama_config(), seq=16, mbs=1, steps=50, ckpt_path=str(tmp_path / "ckpt"), ckpt_interval=1000)
        t = DistributedTrainer(cfg)
        inner = dummy_dataloader(t)

        def dl():
            for i, b in enumerate(inner):
                if i == 3:
                    switch.write_text("stop")  # an operator touches the file while step 4 is being prepared
                yield b

        t.train({"stable": dl()})
        assert t.iteration_step < 10, t.iteration_step
        saved = int(open(tmp_path / "ckpt" / "latest.txt").read())
        assert saved == t.iteration_step and (tmp_path / "ckpt" / str(saved) / "checkpoint_metadata.json").exists()
        t.parallel_context.destroy()
    finally:
        del os.environ["NANOTRON_KILL_SWITCH"]


def test_missing_checkpoint_shard_is_a_clear_error(tmp_path):
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    ckpt = tmp_path / "ckpt"
    cfg = make_config(tiny_llama_config(), seq=16, mbs=1, steps=2, ckpt_path=str(ckpt), ckpt_interval=2)
    t = DistributedTrainer(cfg)
    t.train({"stable": dummy_dataloader(t)})
    t.parallel_context.destroy()
    victim = next((ckpt / "2" / "model").rglob("qkv_proj/*.safetensors"))
    victim.unlink()
    single_process_env()
    cfg2 = make_config(tiny_llama_config(), seq=16, mbs=1, steps=4, ckpt_path=str(ckpt), ckpt_interval=100)
    cfg2.checkpoints.resume_checkpoint_path = ckpt
    with pytest.raises((FileNotFoundError, ValueError, AssertionError)) as ei:
        DistributedTrainer(cfg2)
    assert "qkv_proj" in str(ei.value)
    torch.distributed.destroy_process_group()


class _Exploding(torch.utils.data.Dataset):
    def __len__(self):
        return 8

    def __getitem__(self, i):
        if i == 5:
            raise OSError("disk went away")
        return {"input_ids": torch.zeros(17, dtype=torch.long).numpy()}


def test_dataloader_worker_failure_propagates():
    # a spawned worker: forking this (by now multi-threaded) test process can deadlock the child; the timeout turns a stuck
    # worker into an error instead of a hang
    dl = torch.utils.data.DataLoader(_Exploding(), batch_size=1, num_workers=1, multiprocessing_context="spawn", timeout=120)
    with pytest.raises(Exception) as ei:
        for _ in dl:
            pass
    assert "disk went away" in str(ei.value)


def test_trainer_writes_heartbeats(tmp_path):
    import json

    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    os.environ["NANOTRON_HEARTBEAT_DIR"] = str(tmp_path / "hb")
    os.environ["NANOTRON_HEARTBEAT_INTERVAL"] = "0.05"
    try:
        cfg = make_config(tiny_llama_config(), seq=16, mbs=1, steps=3, ckpt_path=str(tmp_path / "ckpt"), ckpt_interval=1000)
        t = DistributedTrainer(cfg)
        t.train({"stable": dummy_dataloader(t)})
        beat = json.load(open(tmp_path / "hb" / "rank_0.json"))
        assert beat["state"] == "done" and beat["step"] == 3 and beat["rank"] == 0
        t.parallel_context.destroy()
    finally:
        del os.environ["NANOTRON_HEARTBEAT_DIR"], os.environ["NANOTRON_HEARTBEAT_INTERVAL"]


def _reference_arm_guard(marker_dir):
    """Rank 1's "training loop" raises; rank 0 sits in a receive that nobody will match.  The guard of the benchmark's
    reference arm must end both ranks with exit code 0 and rank 0 must be the one that reports."""
    import sys

    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    import run_reference

    ctx = ParallelContext(1, 1, 2)
    rank = dist.get_rank(ctx.world_pg)
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), "2"
    run_reference._unavailable = lambda why: open(os.path.join(marker_dir, f"reported_{rank}"), "w").write(why)
    guard = run_reference._Guard(deadline_s=60.0)
    guard.start()
    if rank == 1:
        guard.fail("reference failed on its stock path: Boom")
        raise AssertionError("fail() returned on a rank other than 0 of a multi-rank job")
    t = torch.ones(1)
    torch.distributed.recv(t, src=1)  # never matched: only the guard's watcher can end this rank
    raise AssertionError("unmatched receive returned")


def test_reference_arm_guard_ends_every_rank_when_one_fails(tmp_path):
    t0 = time.time()
    run_distributed(_reference_arm_guard, 2, marker_dir=str(tmp_path))
    assert time.time() - t0 < 60
    assert os.listdir(tmp_path) == ["reported_0"]
    assert "Boom" in open(tmp_path / "reported_0").read()
