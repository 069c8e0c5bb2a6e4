"""Stand-alone scripts: evaluation curves replayed for logging, dataset warm-up on tiered storage."""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_eval_results_are_replayed_in_step_order(tmp_path):
    mod = _load("scripts/log_lighteval_to_wandb.py", "log_evals")
    for step, base in ((10000, 0.5), (5000, 0.25)):
        d = tmp_path / str(step)
        d.mkdir()
        results = {
            "custom|mmlu:anatomy|0": {"acc": base, "acc_stderr": 0.01},
            "custom|mmlu:law|0": {"acc": base + 0.25},
            "custom|arc:easy|0": {"acc_norm": 0.75},
            "custom|piqa|0": {"acc": 1.0},
            "all": {"acc": 0.0},
        }
        general = {"config": {"general": {"step": step, "consumed_train_samples": step * 4}}}
        (d / "results_0.json").write_text(json.dumps({"results": results, "config_general": general}))
    (tmp_path / "15000").mkdir()  # no file: reported and skipped
    (tmp_path / "notes").mkdir()  # not a step
    rows = []
    assert mod.replay(str(tmp_path), rows.append) == 2
    assert [r["iteration_step"] for r in rows] == [5000, 10000]
    first = rows[0]
    assert first["consumed_train_samples"] == 20000
    assert first["custom|mmlu:anatomy|0_acc"] == 0.25 and first["custom|arc:easy|0_acc"] == 0.75
    assert abs(first["mmlu:average_acc"] - 0.375) < 1e-12 and first["arc:average_acc"] == 0.75
    assert abs(first["all:average_acc"] - (0.25 + 0.5 + 0.75 + 1.0) / 4) < 1e-12
    out = tmp_path / "curve.jsonl"
    assert mod.main(["--eval-path", str(tmp_path), "--jsonl", str(out)]) == 0
    assert len(out.read_text().splitlines()) == 2


def test_storage_warmup_and_status(tmp_path):
    mod = _load("scripts/weka.py", "weka_script")
    a, b = tmp_path / "a", tmp_path / "b"
    (a / "sub").mkdir(parents=True)
    b.mkdir()
    (a / "x.ds").write_bytes(b"1" * 1000)
    (a / "sub" / "y.ds").write_bytes(b"2" * 3000)
    assert mod.parse_paths(f"  - {a}/\n  - {b}\n# comment\n") == [str(a), str(b)]
    calls = []

    def fake_weka(cmd):
        calls.append(cmd[:4])
        if cmd[3] == "location":
            files = [c for c in cmd[4:] if not c.startswith("-") and c != "path,size,ssdRead"]
            return "\n".join(f"{p} {os.path.getsize(p)} B {os.path.getsize(p) // 2} B" for p in files)
        return ""

    status = mod.tier_status([str(a), str(b)], backend="weka", run=fake_weka)
    assert status == {str(a): 50.0, str(b): 0.0}
    fetched = mod.warmup([str(a)], backend="weka", workers=2, run=fake_weka)
    assert fetched == {str(a): 2} and ["weka", "fs", "tier", "fetch"] in calls
    # no tooling: files are read through, the status is unknown
    assert mod.warmup([str(a)], backend="read", workers=2) == {str(a): 2}
    assert mod.tier_status([str(a)], backend="read") == {str(a): -1.0}
    cfg = tmp_path / "cfg.yaml"
    cfg.write_text(f"data_stages:\n- name: s\n  data:\n    dataset:\n      dataset_folder:\n      - {a}\n      - {b}/\n- name: t\n  data:\n    dataset: null\n")
    assert mod.folders_of_config(str(cfg)) == [str(a), str(b)]
    assert mod.main(["status", "--backend", "read", str(a)]) == 0


def test_slurm_launcher_writes_config_and_script(tmp_path, monkeypatch):
    import sys

    mod = _load("slurm_launcher.py", "slurm_launcher_mod")
    monkeypatch.chdir(tmp_path)
    ck = tmp_path / "ck"
    argv = ["--run", "r1", "--model", "8b", "--dp", "2", "--tp", "4", "--pp", "2", "--seq", "4096", "--mbs", "1", "--acc", "8", "--steps", "100", "--dry-run",
            "--requeue", "--email", "a@b.c", "--extra-env", "A=1,B=two", "--pre-launch-commands", "module load cuda", "--checkpoints-path", str(ck), "--account", "acct"]
    mod.main(argv)
    script = (tmp_path / "logs/slurm_scripts/r1.slurm").read_text()
    assert "#SBATCH --nodes=2" in script and "#SBATCH --gpus-per-node=8" in script and "#SBATCH --account=acct" in script
    assert "#SBATCH --signal=B:USR1@300" in script and "#SBATCH --requeue" in script and "--mail-user=a@b.c" in script
    assert "export A=1" in script and "export B=two" in script and "module load cuda" in script and "export WANDB_MODE=disabled" in script
    assert f"export NANOTRON_KILL_SWITCH={ck}/r1/STOP" in script and "touch \"$NANOTRON_KILL_SWITCH\"" in script and "scontrol requeue $SLURM_JOB_ID" in script
    assert "--nproc_per_node 8" in script and "--max_restarts 0" in script and "run_train.py --config-file" in script
    # the config is loadable and says what was asked for; no latest.txt yet, so no resume
    from nanotron_b200.config import get_config_from_file

    cfg = get_config_from_file(str(tmp_path / "logs/configs/r1.yaml"))
    assert (cfg.parallelism.dp, cfg.parallelism.tp, cfg.parallelism.pp) == (2, 4, 2) and cfg.model.model_config.hidden_size == 4096
    assert cfg.checkpoints.resume_checkpoint_path is None and cfg.tokens.batch_accumulation_per_replica == 8
    # a second launch of the same run finds the checkpoint of the first and resumes from it
    (ck / "r1").mkdir(parents=True)
    (ck / "r1" / "latest.txt").write_text("50")
    mod.main(argv)
    cfg = get_config_from_file(str(tmp_path / "logs/configs/r1.yaml"))
    assert str(cfg.checkpoints.resume_checkpoint_path) == str(ck / "r1")
    # a chain of dependent jobs
    calls = []

    class Out:
        returncode, stderr = 0, ""

        def __init__(self, n):
            self.stdout = f"Submitted batch job {n}"

    def fake_run(cmd, **kw):
        calls.append(cmd)
        return Out(100 + len(calls))

    first = mod.submit("x.slurm", run=fake_run)
    second = mod.submit("x.slurm", dependency=first, run=fake_run)
    assert (first, second) == ("101", "102") and calls[1] == ["sbatch", "--dependency=afterany:101", "x.slurm"]
    assert mod.parse_extra_env("A=1, B=2 C=x=y") == {"A": "1", "B": "2", "C": "x=y"}
    # fewer GPUs than a node: one node with that many GPUs
    a = mod.parse_args(["--dp", "2", "--tp", "2", "--dry-run"])
    assert (a.nodes, a.gpus_per_node) == (1, 4)
