"""``run_train.py`` end to end on CPU (2 gloo ranks started by torchrun): pre-tokenised files written by the preprocessing tool,
two data stages that read different folders, periodic checkpoints, and a resume in the middle of the second stage that must
continue the interrupted run step for step (weights, optimizer, learning-rate schedule, and the position inside the data)."""
import importlib.util
import os
import re
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import _free_port as pick

    return pick()


def _write_datasets(tmp_path):
    spec = importlib.util.spec_from_file_location("preprocess_data_tool_e2e", os.path.join(ROOT, "tools", "preprocess_data.py"))
    prep = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(prep)
    rng = np.random.default_rng(0)
    folders = []
    for name, lo, hi in (("first", 3, 120), ("second", 130, 250)):  # disjoint token ranges: the stages cannot be confused
        d = tmp_path / name
        d.mkdir()
        docs = [list(rng.integers(lo, hi, size=int(rng.integers(20, 60)))) + [2] for _ in range(120)]
        prep.write_token_shard(str(d / "part_000.ds"), docs, token_size=2, tokenizer_name="none")
        folders.append(str(d))
    return folders


def _config(tmp_path, folders, resume=None, streamed=False):
    sys.path.insert(0, ROOT)
    import nanotron_b200.config as c

    model = c.Qwen2Config(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=256, max_position_embeddings=32,
                          rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2)

    def stage(name, start, folder):
        return c.DatasetStageArgs(name=name, start_training_step=start, data=c.DataArgs(dataset=c.NanosetDatasetsArgs(dataset_folder=folder, token_size_in_bytes=2, use_old_brrr_dataloader=streamed), seed=7, num_loading_workers=0))

    cfg = c.Config(
        general=c.GeneralArgs(project="e2e", run="e2e", seed=3),
        checkpoints=c.CheckpointsArgs(checkpoints_path=str(tmp_path / "ckpt"), checkpoint_interval=4, save_final_state=True, resume_checkpoint_path=resume),
        parallelism=c.ParallelismArgs(dp=2, pp=1, tp=1, pp_engine="1f1b", tp_mode="ALL_REDUCE", tp_linear_async_communication=False),
        model=c.ModelArgs(model_config=model, init_method=c.RandomInit(std=0.05), dtype="float32"),
        tokenizer=c.TokenizerArgs(tokenizer_name_or_path=None),
        optimizer=c.OptimizerArgs(
            optimizer_factory=c.AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=False), zero_stage=1, weight_decay=0.01, clip_grad=1.0,
            accumulate_grad_in_fp32=True,
            learning_rate_scheduler=c.LRSchedulerArgs(learning_rate=5e-3, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=5e-4),
        ),
        logging=c.LoggingArgs(log_level="info", log_level_replica="error", iteration_step_info_interval=1),
        tokens=c.TokensArgs(sequence_length=32, train_steps=7, micro_batch_size=2, batch_accumulation_per_replica=2),
        data_stages=[stage("first", 1, folders[0]), stage("second", 4, folders[1])],
    )
    path = str(tmp_path / ("resume.yaml" if resume else "config.yaml"))
    cfg.save_as_yaml(path)
    return path


def _train(config_path, extra=()):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "run_train.py"), "--config-file", config_path, *extra]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    text = out.stdout + out.stderr
    losses = {int(m.group(1)): float(m.group(2)) for m in re.finditer(r"iteration: (\d+) / \d+.*?lm_loss: ([\d.]+)", text)}
    return losses, text


import pytest  # noqa: E402


@pytest.mark.parametrize("streamed", [False, True], ids=["nanoset", "streamed_token_files"])
def test_run_train_with_data_stages_and_resume(tmp_path, streamed):
    folders = _write_datasets(tmp_path)
    full, log = _train(_config(tmp_path, folders, streamed=streamed))
    assert sorted(full) == list(range(1, 8)), (sorted(full), log[-2000:])
    assert "second" in log  # the stage switch was announced
    assert sorted(d for d in os.listdir(tmp_path / "ckpt") if d.isdigit()) == ["4", "7"]
    # the checkpoint knows how many tokens came from which folder, job-wide (2 ranks x 2 micro-batches x 2 sequences x 32 tokens per step)
    import json

    meta = json.load(open(tmp_path / "ckpt" / "4" / "checkpoint_metadata.json"))["metas"]
    per_stage = [sum(s["consumed_tokens_per_dataset_folder"].values()) for s in meta["data_stages"]]
    assert per_stage == [3 * 256, 1 * 256] and meta["consumed_tokens_total"] == 4 * 256, meta
    # resume from step 4 (one step into the second stage): steps 5..7 must repeat the interrupted run
    (tmp_path / "ckpt" / "latest.txt").write_text("4")
    resumed, log2 = _train(_config(tmp_path, folders, resume=str(tmp_path / "ckpt"), streamed=streamed))
    assert sorted(resumed) == [5, 6, 7], (sorted(resumed), log2[-2000:])
    for step in (5, 6, 7):
        assert abs(resumed[step] - full[step]) < 2e-3 * max(1.0, full[step]), (step, resumed, full)
    if not streamed:
        # the same checkpoint (written by 2 data-parallel ranks) decodes under tensor parallelism 2 through run_generate.py
        env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
               os.path.join(ROOT, "run_generate.py"), "--ckpt-path", str(tmp_path / "ckpt" / "7"), "--tp", "2", "--max-new-tokens", "4"]
        out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
        assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
        assert "generat" in (out.stdout + out.stderr).lower()


def _write_text_datasets(tmp_path):
    """A word-level tokenizer saved in the Hugging Face format, a folder of raw text and a folder of prompt / completion pairs
    (both learnable: words count upwards)."""
    import json

    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2, "<unk>": 3, **{f"w{i}": i + 4 for i in range(200)}}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", unk_token="<unk>", pad_token="<pad>").save_pretrained(str(tmp_path / "tok"))
    rng = np.random.default_rng(0)
    (tmp_path / "text").mkdir()
    (tmp_path / "sft").mkdir()
    with open(tmp_path / "text" / "train.jsonl", "w") as f:
        for _ in range(400):
            start, stride = int(rng.integers(0, 200)), int(rng.integers(1, 4))
            f.write(json.dumps({"text": " ".join(f"w{(start + stride * j) % 200}" for j in range(int(rng.integers(20, 60))))}) + "\n")
    with open(tmp_path / "sft" / "train.jsonl", "w") as f:
        for _ in range(300):
            start = int(rng.integers(0, 200))
            f.write(json.dumps({"prompt": " ".join(f"w{(start + j) % 200}" for j in range(6)), "completion": " ".join(f"w{(start + 6 + j) % 200}" for j in range(8))}) + "\n")


@pytest.mark.parametrize("kind", ["text", "sft"])
def test_run_train_on_raw_text_and_on_prompt_completion_pairs(tmp_path, kind):
    """``PretrainDatasetsArgs`` (tokenise + pack on the fly, Llama with masks) and ``SFTDatasetsArgs`` (loss on the completion only,
    Qwen2 with position ids) through ``run_train.py``: the datasets load from local folders, the loss falls."""
    sys.path.insert(0, ROOT)
    import nanotron_b200.config as c

    _write_text_datasets(tmp_path)
    steps = 40 if kind == "text" else 20
    shape = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=256, max_position_embeddings=64, rms_norm_eps=1e-5, tie_word_embeddings=False)
    if kind == "text":
        model, dataset = c.LlamaConfig(**shape), c.PretrainDatasetsArgs(hf_dataset_or_datasets=str(tmp_path / "text"), text_column_name="text")
    else:
        model, dataset = c.Qwen2Config(**shape), c.SFTDatasetsArgs(hf_dataset_or_datasets=str(tmp_path / "sft"))
    cfg = c.Config(
        general=c.GeneralArgs(project="e2e", run=kind, seed=3),
        checkpoints=c.CheckpointsArgs(checkpoints_path=str(tmp_path / "ckpt"), checkpoint_interval=1000, save_final_state=kind == "text"),
        # raw text: two data-parallel replicas; prompt / completion pairs: two pipeline stages (the collator hands pointers to the stage
        # that does not consume a key, and the metric line comes from the last stage although replicas only log errors)
        parallelism=c.ParallelismArgs(dp=2, pp=1, tp=1) if kind == "text" else c.ParallelismArgs(dp=1, pp=2, tp=1, pp_engine="1f1b"),
        model=c.ModelArgs(model_config=model, init_method=c.RandomInit(std=0.05), dtype="float32"),
        tokenizer=c.TokenizerArgs(tokenizer_name_or_path=str(tmp_path / "tok")),
        optimizer=c.OptimizerArgs(
            optimizer_factory=c.AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=False), zero_stage=0, weight_decay=0.01, clip_grad=1.0,
            accumulate_grad_in_fp32=True, learning_rate_scheduler=c.LRSchedulerArgs(learning_rate=1e-2, lr_warmup_steps=2, lr_decay_style="cosine", min_decay_lr=1e-3),
        ),
        logging=c.LoggingArgs(log_level="info", log_level_replica="error", iteration_step_info_interval=1),
        tokens=c.TokensArgs(sequence_length=32, train_steps=steps, micro_batch_size=4, batch_accumulation_per_replica=1 if kind == "text" else 2),
        data_stages=[c.DatasetStageArgs(name="only", start_training_step=1, data=c.DataArgs(dataset=dataset, seed=7, num_loading_workers=0))],
    )
    path = str(tmp_path / f"{kind}.yaml")
    cfg.save_as_yaml(path)
    os.environ["HF_DATASETS_CACHE"] = str(tmp_path / "hf_cache")
    os.environ["HF_HUB_OFFLINE"] = "1"
    try:
        losses, text = _train(path, extra=("--sanity-check-dataloader-interval", "15") if kind == "text" else ())
        generations = []
        if kind == "text":
            # the checkpoint names its tokenizer: run_generate.py decodes text prompts, with and without the key / value cache
            for extra in ([], ["--use-cache"]):
                cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
                       os.path.join(ROOT, "run_generate.py"), "--ckpt-path", str(tmp_path / "ckpt" / str(steps)), "--tp", "2", "--max-new-tokens", "5", "--prompt", "w3 w4 w5 w6", "--prompt", "w10 w12 w14"] + extra
                out = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1"), cwd=ROOT, timeout=600)
                assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
                generations.append(re.findall(r"generation: (.*)", out.stdout + out.stderr))
            # ... and run_evals.py scores a multiple-choice task from local files: the right continuation keeps counting
            import json

            rng = np.random.default_rng(1)
            (tmp_path / "eval").mkdir()
            with open(tmp_path / "eval" / "arc:easy.test.jsonl", "w") as f:
                for i in range(24):
                    start, pos = int(rng.integers(0, 150)), int(rng.integers(0, 4))
                    wrong = [" ".join(f"w{int(x)}" for x in rng.integers(0, 200, size=3)) for _ in range(3)]
                    texts = wrong[:pos] + [" ".join(f"w{start + 8 + j}" for j in range(3))] + wrong[pos:]
                    f.write(json.dumps({"id": str(i), "question": " ".join(f"w{start + j}" for j in range(8)), "choices": {"text": texts, "label": list("ABCD")}, "answerKey": "ABCD"[pos]}) + "\n")
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
                   os.path.join(ROOT, "run_evals.py"), "--checkpoint-config-path", str(tmp_path / "ckpt" / str(steps) / "config.yaml"), "--tasks", "arc_cf:easy", "--data-dir", str(tmp_path / "eval"),
                   "--tp", "2", "--max-length", "64", "--output", str(tmp_path / "eval" / "results.json")]
            out = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1"), cwd=ROOT, timeout=600)
            assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
            scores = json.load(open(tmp_path / "eval" / "results.json"))["results"]["arc_cf:easy|test"]
            assert scores["num_samples"] == 24 and scores["acc_token"] >= 0.6, scores  # chance is 0.25
    finally:
        os.environ.pop("HF_DATASETS_CACHE")
        os.environ.pop("HF_HUB_OFFLINE")
    assert sorted(losses) == list(range(1, steps + 1)), text[-2000:]
    assert losses[20] < losses[1] - 1.0, losses
    if kind == "text":
        # micro-batches 0, 15, 30 of rank 0 were described, decoded with the run's tokenizer
        assert text.count("[dataloader sample] stage 'only'") == 3 and "first row: 'w" in text and "labels that count: 128 of 128" in text
        assert len(generations[0]) == 2 and all(len(g.split()) == 5 and all(w.startswith("w") for w in g.split()) for g in generations[0]), generations
        assert generations[0] == generations[1]
