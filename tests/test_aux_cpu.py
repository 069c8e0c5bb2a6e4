"""Auxiliary subsystems on CPU: timers, per-layer metrics, the block-local logging mixin, the decoding store, the evaluation
job launcher, result collection for wandb, and the maintenance / preprocessing scripts."""
import importlib.util
import json
import os
import sys
import time

import numpy as np
import pytest
import torch
from torch import nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_timers_as_context_manager_decorator_and_registry():
    from nanotron_b200.logging.timers import Timers, TimerType

    timers = Timers()
    timers.configure(timer_type=TimerType.CPU, enabled=True)
    with timers("block"):
        time.sleep(0.02)
    with timers("block"):
        time.sleep(0.02)
    assert "block" in timers and timers["block"].call_count == 2
    assert 0.03 < timers["block"].total_time < 1.0 and timers["block"].average_time == pytest.approx(timers["block"].total_time / 2)

    @timers("decorated")
    def work(n):
        time.sleep(0.01)
        return n + 1

    assert work(1) == 2 and timers["decorated"].call_count == 1

    @timers
    def bare():
        return 7

    assert bare() == 7 and "bare" in timers
    assert set(timers.get_all_elapsed()) == {"block", "decorated", "bare"}
    timers.reset("block")
    assert timers["block"].call_count == 0
    # disabled timers cost nothing and record nothing
    timers.disable()
    with timers("off"):
        pass
    assert timers["off"].call_count == 0 and "off" not in timers.get_all_elapsed()


def test_tensor_statistics_and_per_layer_metric_names():
    from nanotron_b200.metrics_logging import STAT_NAMES, MetricsLogger, compute_tensor_stats

    x = torch.tensor([0.0, 1.0, -1.0, 2.0])
    stats = dict(zip(STAT_NAMES, compute_tensor_stats(x).tolist()))
    assert stats["mean"] == pytest.approx(0.5) and stats["min"] == -1 and stats["max"] == 2
    assert stats["l1"] == pytest.approx(4.0) and stats["l2"] == pytest.approx(6**0.5) and stats["zero_frac"] == pytest.approx(0.25)
    assert compute_tensor_stats(torch.empty(0)).tolist() == [0.0] * len(STAT_NAMES)

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv_proj, self.o_proj = nn.Linear(4, 12, bias=False), nn.Linear(4, 4, bias=False)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn, self.input_layernorm = Attn(), nn.LayerNorm(4)

    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.decoder = nn.ModuleList([Block(), Block()])
            self.lm_head = nn.Linear(4, 8, bias=False)

    class Cfg:
        class metrics_logging:
            log_level, log_detail_interval = 1, 5

    model = Tiny()
    for p in model.parameters():
        p.grad = torch.ones_like(p)
    ml = MetricsLogger(Cfg)
    detailed = ml.collect_all_metrics(model, iteration_step=10)
    assert "global/weights_l2" in detailed
    assert "weights/layer_1/attn/qkv_proj/std" in detailed and "grads/layer_0/attn/o_proj/l2" in detailed and "weights/lm_head/mean" in detailed
    assert float(detailed["grads/layer_0/attn/o_proj/l2"]) == pytest.approx(4.0)  # 16 ones
    assert set(ml.collect_all_metrics(model, iteration_step=11)) == {"global/weights_l2"}  # off the detail interval


def test_block_local_logging_is_collected_from_the_model_tree():
    from nanotron_b200.logging.logmixin import LoggingCollectorMixin, LogMixin

    class Leaf(nn.Module, LogMixin):
        def forward(self, x):
            self.tbi_logger({"act_norm": x.norm()})
            return x

    class Model(nn.Module, LoggingCollectorMixin):
        def __init__(self):
            super().__init__()
            self.a, self.b = Leaf(), Leaf()

    m = Model()
    m.a(torch.ones(4))
    m.b(torch.full((4,), 2.0))
    logs = m.get_tbi_logs()
    assert {k.split(":")[0] if ":" in k else k for k in logs}  # something was collected
    assert sorted(float(v) for v in logs.values()) == [2.0, 4.0]
    m.clear_all_tbi_logs()
    assert m.get_tbi_logs() == {}


def test_decoding_store_attaches_per_module_state():
    from nanotron_b200.generation.generate_store import AttachableStore, Store, attach_store

    class Layer(nn.Module, AttachableStore):
        def forward(self, x):
            store = self.get_local_store()
            if store is not None:
                store["calls"] = store.get("calls", 0) + 1
            return x

    model = nn.Sequential(Layer(), Layer())
    model(torch.zeros(1))  # no store attached: nothing is kept
    store = Store()
    with attach_store(model, store):
        model(torch.zeros(1))
        model(torch.zeros(1))
        assert [s["calls"] for s in store.values()] == [2, 2]
    assert model[0].get_local_store() is None
    store.flush()
    assert len(store) == 0


def test_evaluation_job_script_is_rendered_from_the_upload_log(tmp_path):
    from nanotron_b200.config import Config, GeneralArgs, LightEvalConfig, ParallelismArgs
    from nanotron_b200.eval.one_job_runner import LightEvalRunner

    cfg = Config.create_empty()
    cfg.general = GeneralArgs(project="p", run="run7")
    cfg.lighteval = LightEvalConfig(slurm_script_dir=tmp_path / "scripts", logs_path=tmp_path / "logs", local_checkpoint_dir=tmp_path / "ckpt", parallelism=ParallelismArgs(dp=1, pp=1, tp=2),
                                    s3_save_path="s3://bucket/evals", upload_to_wandb=True, wandb_project="evals", eval_interval=100)
    runner = LightEvalRunner(cfg)
    log = '{"operation":"cp","success":true,"source":"/tmp/x","destination":"s3://bucket/ckpts/run7/200/model/model/lm_head/pp_block/model_weight.safetensors"}\n'
    assert runner._checkpoint_from_upload_log(log) == "s3://bucket/ckpts/run7/200" and runner._step_from_path("s3://bucket/ckpts/run7/200") == 200
    assert runner._checkpoint_from_upload_log("nothing useful") is None
    script, out_log = runner.render_slurm_script("s3://bucket/ckpts/run7/200", 200)
    text = open(script).read()
    assert "#SBATCH --gpus-per-node=2" in text and "s5cmd cp --exclude 'optimizer/*'" in text and "run_evals.py --checkpoint-config-path" in text
    assert "s3://bucket/evals/run7/200/" in text and "upload_to_wandb --wandb_project evals" in text and out_log.endswith(".out")
    # a step off the evaluation interval launches nothing
    assert runner.eval_single_checkpoint(log.replace("/200/", "/250/")) == (None, None)


def test_result_files_are_flattened_for_wandb(tmp_path):
    from nanotron_b200.eval.upload_to_wandb import collect_results

    (tmp_path / "a").mkdir()
    (tmp_path / "a" / "results_1.json").write_text(json.dumps({"results": {"arc:easy": {"acc": 0.5, "acc_stderr": 0.1, "note": "x"}, "piqa": {"acc_norm": 0.75}}}))
    assert collect_results(str(tmp_path)) == {"arc:easy/acc": 0.5, "arc:easy/acc_stderr": 0.1, "piqa/acc_norm": 0.75}


def test_badly_named_shards_get_their_extension_back(tmp_path, monkeypatch):
    fix = _load("scripts/fix_checkpoint_bad_naming.py", "fix_naming")
    assert fix.fixed_name("model_weight.safetensors_pp-rank-0-of-1_tp-rank-0-of-2") == "model_weight_pp-rank-0-of-1_tp-rank-0-of-2.safetensors"
    assert fix.fixed_name("model_weight_pp-rank-0-of-1_tp-rank-0-of-2.safetensors") is None and fix.fixed_name("config.yaml") is None
    d = tmp_path / "10" / "model"
    d.mkdir(parents=True)
    (d / "model_weight.safetensors_pp-rank-0-of-1_tp-rank-1-of-2").write_bytes(b"x")
    (d / "model_bias_pp-rank-0-of-1_tp-rank-1-of-2.safetensors").write_bytes(b"y")
    monkeypatch.setattr(sys, "argv", ["fix", str(tmp_path / "10")])
    fix.main()
    assert sorted(os.listdir(d)) == ["model_bias_pp-rank-0-of-1_tp-rank-1-of-2.safetensors", "model_weight_pp-rank-0-of-1_tp-rank-1-of-2.safetensors"]


def test_preprocessed_token_shards_are_readable_by_the_dataset(tmp_path):
    """tools/preprocess_data.py's writer produces the token file + index + metadata that the Nanoset reader opens."""
    prep = _load("tools/preprocess_data.py", "preprocess_data_tool")
    docs = [[5, 6, 7, 2], [8, 9, 2], [10, 11, 12, 13, 2]]
    path = str(tmp_path / "part_000.ds")
    assert prep.write_token_shard(path, docs, token_size=2, tokenizer_name="gpt2") == 12
    assert np.fromfile(path, dtype=np.uint16).tolist() == [t for d in docs for t in d]
    assert np.fromfile(path + ".index", dtype=np.uint64).tolist() == [4, 7, 12]
    assert open(path + ".metadata").read().splitlines() == ["gpt2|2", "12"]
    from nanotron_b200.data.tokenized_bytes import TokenizedBytesFileDataset

    ds = TokenizedBytesFileDataset(path, seq_len=3, dtype=np.uint16)
    assert len(ds) == 3  # 12 tokens in samples of seq_len + 1
    first = ds[0]
    tokens = first["input_ids"] if isinstance(first, dict) else first
    assert torch.as_tensor(tokens).reshape(-1).tolist()[:4] == [5, 6, 7, 2]


def test_scaling_sweep_generates_configs_and_job_scripts(tmp_path, monkeypatch):
    import csv

    sb = _load("scripts/scaling_benchmarks.py", "scaling_benchmarks_script")
    assert sb.parse_layout("dp2tp4") == {"dp": 2, "tp": 4, "pp": 1}
    assert set(sb.default_layouts(4)) >= {"dp4tp1pp1", "dp1tp4pp1", "dp1tp2pp2"}
    layouts = sb.layouts_for(8)
    assert all(dp * tp * pp == 8 for dp, tp, pp in layouts) and (1, 8, 1) in layouts and (8, 1, 1) in layouts
    n = sb.estimate_num_params(layers=32, hidden=4096, heads=32, kv_heads=8, ffn=14336, vocab=128256, tie_word_embeddings=False)
    assert 7.9e9 < n < 8.2e9
    # generate mode: one config + one job script per experiment, and the experiment table
    monkeypatch.setattr(sys, "argv", ["scaling_benchmarks.py", "generate", "--sizes", "8B", "--nodes", "1", "--limit", "3", "--configs-dir", str(tmp_path / "cfg"),
                                      "--scripts-dir", str(tmp_path / "sh"), "--logs-dir", str(tmp_path / "logs"), "--benchmark-csv", str(tmp_path / "res.csv")])
    sb.main()
    rows = list(csv.DictReader(open(tmp_path / "cfg" / "experiments.csv")))
    assert len(rows) == 3 and len(os.listdir(tmp_path / "sh")) == 3
    from nanotron_b200.config import get_config_from_file

    for row in rows:
        cfg = get_config_from_file(row["config"])
        assert cfg.parallelism.dp * cfg.parallelism.tp * cfg.parallelism.pp == 8
        assert "run_train.py" in open(row["script"]).read() and "#SBATCH --nodes=1" in open(row["script"]).read()


def _metrics_run(out_dir):
    import json

    import nanotron_b200.config as c
    import nanotron_b200.distributed as dist
    from helpers import dummy_dataloader, make_config, tiny_qwen_config
    from nanotron_b200.trainer import DistributedTrainer

    os.environ["NANOTRON_METRICS_JSONL"] = os.path.join(out_dir, "metrics.jsonl")
    os.environ["DEBUG_CPU"] = "1"
    cfg = make_config(tiny_qwen_config(log_attn_probs=True), tp=2, seq=16, steps=4, tp_mode="reduce_scatter")
    cfg.metrics_logging = c.MetricsLoggingArgs(log_level=1, log_detail_interval=2)
    cfg.logging.iteration_step_info_interval = 3  # console steps 1 and 4, detailed steps 2 and 4
    cfg.checkpoints.checkpoints_path = os.path.join(out_dir, "ckpt")
    t = DistributedTrainer(cfg)
    t.train(dummy_dataloader(t))
    dist.barrier()
    t.parallel_context.destroy()


def test_detailed_metrics_attention_statistics_and_diagnostics_reach_the_metric_file(tmp_path):
    import json

    from helpers import run_distributed

    run_distributed(_metrics_run, 2, out_dir=str(tmp_path))
    files = sorted(f for f in os.listdir(tmp_path) if f.startswith("metrics.jsonl"))
    assert files == ["metrics.jsonl.pp0_tp0", "metrics.jsonl.pp0_tp1"]  # one stream per model shard
    rows = {f: [json.loads(line) for line in open(tmp_path / f)] for f in files}
    logger, other = rows["metrics.jsonl.pp0_tp0"], rows["metrics.jsonl.pp0_tp1"]
    assert [r["iteration_step"] for r in logger] == [1, 2, 4] and [r["iteration_step"] for r in other] == [2, 4]
    first, detailed, both = logger
    assert "lm_loss" in first and "tokens_per_sec" in first and "weights/layer_0/attn/qkv_proj/mean" not in first
    # attention statistics of every layer and head (two local heads per tensor-parallel rank), host memory
    assert "tbi_logs/model.decoder.0.pp_block.attn/attn_probs_mean" in first and "tbi_logs/model.decoder.1.pp_block.attn/attn_probs/head_1_max" in first
    assert "tbi_logs/model.decoder.0.pp_block.attn/attn_probs/head_2_max" not in first
    assert first["cpu_memory/process_rss"] > 0
    # a detailed step that is not a console step carries the per-layer statistics only; step 4 carries both
    assert "lm_loss" not in detailed and "weights/layer_0/attn/qkv_proj/l2" in detailed and "grads/layer_1/mlp/down_proj/l2" in detailed
    assert "lm_loss" in both and "weights/layer_1/mlp/gate_up_proj/std" in both and both["hd_total_memory"] > 0
    assert detailed["tp_rank"] == 0 and other[0]["tp_rank"] == 1 and other[0]["tp_group_size"] == 2
    # the two tensor-parallel ranks see different shards of a sharded matrix and the same replicated norm weight
    assert other[0]["weights/layer_0/attn/qkv_proj/l2"] != detailed["weights/layer_0/attn/qkv_proj/l2"]
    assert other[0]["weights/layer_0/input_layernorm/mean"] == detailed["weights/layer_0/input_layernorm/mean"]


def test_benchmark_mode_appends_one_row_and_stops_after_four_steps(tmp_path, monkeypatch):
    """``NANOTRON_BENCHMARK=1``: the throughput table is printed and appended to ``general.benchmark_csv_path`` at step 4, then the
    run ends (a second run appends under the same header)."""
    import csv

    from helpers import dummy_dataloader, make_config, single_process_env, tiny_llama_config
    from nanotron_b200.trainer import DistributedTrainer

    monkeypatch.setenv("NANOTRON_BENCHMARK", "1")
    monkeypatch.setenv("SLURM_JOB_ID", "4242")
    path = tmp_path / "bench.csv"
    for run in range(2):
        single_process_env()
        cfg = make_config(tiny_llama_config(), seq=16, steps=10)
        cfg.general.benchmark_csv_path = str(path)
        cfg.logging.iteration_step_info_interval = 1
        t = DistributedTrainer(cfg)
        with pytest.raises(SystemExit) as stop:
            t.train(dummy_dataloader(t))
        assert stop.value.code == 0 and t.iteration_step == 4
        t.parallel_context.destroy()
    rows = list(csv.DictReader(open(path)))
    assert len(rows) == 2 and rows[0]["job_id"] == "4242" and rows[0]["seq_len"] == "16" and rows[0]["dp"] == rows[0]["tp"] == "1"
    assert float(rows[0]["tok/s/gpu"]) > 0 and rows[0]["pp_engine"] == "AllForwardAllBackwardPipelineEngine" and rows[0]["Total Params"] == rows[0]["Local Params"]


def test_profiler_section_writes_a_trace_with_the_named_regions(tmp_path):
    import glob
    import gzip
    import json

    import nanotron_b200.config as c
    from helpers import dummy_dataloader, make_config, single_process_env, tiny_llama_config
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    cfg = make_config(tiny_llama_config(), seq=16, steps=6)
    cfg.profiler = c.ProfilerArgs(profiler_export_path=tmp_path / "traces", wait=1, warmup=1, active=1, repeat=1, skip_first=1)
    t = DistributedTrainer(cfg)
    t.train(dummy_dataloader(t))
    t.parallel_context.destroy()
    traces = glob.glob(str(tmp_path / "traces" / "*" / "*.json*"))
    assert len(traces) == 1, traces  # one active window of one step
    opener = gzip.open if traces[0].endswith(".gz") else open
    with opener(traces[0], "rt") as f:
        names = {e.get("name") for e in json.load(f)["traceEvents"]}
    assert {"train_batch_iter", "micro_batch_forward", "micro_batch_backward", "optimizer_step"} <= names
    # a schedule that does not fit into the run is rejected when the configuration is built
    cfg.profiler = c.ProfilerArgs(profiler_export_path=tmp_path / "traces", wait=3, warmup=3, active=3, repeat=1, skip_first=3)
    with pytest.raises((AssertionError, ValueError)):
        c.Config(**{f.name: getattr(cfg, f.name) for f in __import__("dataclasses").fields(cfg)})


def test_wandb_receives_one_record_per_logged_step(monkeypatch):
    """With ``WANDB_MODE`` set, the logger rank opens one run named after the configuration and logs every console step (the
    package is replaced by a recorder here)."""
    import sys
    import types

    from helpers import dummy_dataloader, make_config, single_process_env, tiny_llama_config
    from nanotron_b200.trainer import DistributedTrainer

    calls = {"init": [], "log": []}
    fake = types.ModuleType("wandb")
    fake.init = lambda **kw: calls["init"].append(kw)
    fake.log = lambda record, **kw: calls["log"].append(record)
    monkeypatch.setitem(sys.modules, "wandb", fake)
    monkeypatch.setenv("WANDB_MODE", "offline")
    single_process_env()
    cfg = make_config(tiny_llama_config(), seq=16, steps=5)
    cfg.logging.iteration_step_info_interval = 2  # steps 1, 3, 5
    t = DistributedTrainer(cfg)
    t.train(dummy_dataloader(t))
    t.parallel_context.destroy()
    assert len(calls["init"]) == 1 and calls["init"][0]["project"] == "test" and calls["init"][0]["name"] == "t" and "nanotron_config" in calls["init"][0]["config"]
    assert [r["iteration_step"] for r in calls["log"]] == [1, 3, 5]
    assert all({"lm_loss", "tokens_per_sec", "lr", "consumed_tokens", "model_tflops_per_gpu"} <= set(r) for r in calls["log"])
