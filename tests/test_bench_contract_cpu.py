"""The benchmark's command-line contract that can be checked without a GPU: which parallel layout each GPU count gets, the
presets of the target configurations, and the labels written into the result line."""
import argparse
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_module"] = mod
    spec.loader.exec_module(mod)
    return mod


def _args(**kw):
    base = dict(layout=None, tp=None, pp=None, cp=None, ep=None, model="llama3-8b", config="llama3-8b")
    base.update(kw)
    return argparse.Namespace(**base)


def test_default_layout_per_gpu_count_matches_the_target_configuration():
    b = _bench()
    # (tp, pp, dp): 1 GPU none, 2 -> tp2, 4 -> tp4, 8 -> tp4 x pp2; the global batch does not grow with the GPU count
    assert b.resolve_layout(_args(layout="model"), 1) == (1, 1, 1)
    assert b.resolve_layout(_args(layout="model"), 2) == (2, 1, 1)
    assert b.resolve_layout(_args(layout="model"), 4) == (4, 1, 1)
    assert b.resolve_layout(_args(layout="model"), 8) == (4, 2, 1)
    # data-parallel layout on request, explicit sizes override both
    assert b.resolve_layout(_args(layout="dp"), 8) == (1, 1, 8)
    assert b.resolve_layout(_args(layout="model", tp=2, pp=2), 8) == (2, 2, 2)
    assert b.resolve_layout(_args(layout="model", tp=8), 8) == (8, 1, 1)


def test_layout_labels_name_what_runs():
    b = _bench()
    assert b.layout_label(1, 1, 1, 0) == "dp1"
    assert "tp4" in b.layout_label(4, 2, 1, 0) and "pp2" in b.layout_label(4, 2, 1, 0)
    assert "zero1" in b.layout_label(1, 1, 8, 1)


def test_presets_cover_the_target_configurations():
    b = _bench()
    assert set(b.CONFIGS) >= {"llama3-8b", "llama3.2-1b-dp8", "qwen-moe-ep8", "llama3-8b-cp8-64k"}
    one_b = b.CONFIGS["llama3.2-1b-dp8"]
    assert one_b["mbs"] == 4 and one_b["accum"] == 1 and one_b["layout"] == "dp"
    cp = b.CONFIGS["llama3-8b-cp8-64k"]
    assert cp["seq"] == 65536 and cp["recompute"] and cp["cp"] == -1
    m = b.MODELS["llama3-8b"]
    assert (m["hidden_size"], m["num_hidden_layers"], m["num_attention_heads"], m["num_key_value_heads"], m["vocab_size"]) == (4096, 32, 32, 8, 128256)
    assert b.QWEN_MOE["num_key_value_heads"] == 4 and b.QWEN_MOE["hidden_size"] == 2048
