"""Multi-GPU checks: each spawns ``torchrun`` on the GPUs of this machine and is skipped when there are fewer than two."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, nproc, port, timeout=600, args=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port), script, *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_data_parallel_step_matches_nccl():
    r = _torchrun("tests/multigpu/check_fused_dp.py", 2, 29731)
    assert r.returncode == 0 and "FUSED_DP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tensor_parallel_linears_match_nccl():
    r = _torchrun("tests/multigpu/check_fused_tp.py", 2, 29732)
    assert r.returncode == 0 and "FUSED_TP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_expert_parallel_moe_matches_nccl():
    r = _torchrun("tests/multigpu/check_fused_ep.py", 2, 29733)
    assert r.returncode == 0 and "FUSED_EP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_context_parallel_attention_matches_full_attention():
    r = _torchrun("tests/multigpu/check_fused_cp.py", 2, 29734)
    assert r.returncode == 0 and "FUSED_CP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_default_context_parallel_attention_matches_full_attention():
    r = _torchrun("tests/multigpu/check_cp_default.py", 2, 29735)
    assert r.returncode == 0 and "CP_DEFAULT_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_and_tensor_parallel_layouts_track_one_gpu(tmp_path):
    """pp 2 (both engines), tp 2 with the fused linears and, on four GPUs, tp 2 x pp 2: same loss curve as one GPU."""
    base = str(tmp_path / "base.pt")
    r = _torchrun("tests/multigpu/check_train_layout.py", 1, 29736, args=["--out", base])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    layouts = [(2, ["--pp", "2"]), (2, ["--pp", "2", "--engine", "afab"]), (2, ["--tp", "2"])]
    if torch.cuda.device_count() >= 4:
        layouts.append((4, ["--tp", "2", "--pp", "2"]))
    for i, (n, extra) in enumerate(layouts):
        r = _torchrun("tests/multigpu/check_train_layout.py", n, 29737 + i, args=[*extra, "--expect", base])
        assert r.returncode == 0 and "LAYOUT_OK" in r.stdout, str(extra) + r.stdout[-3000:] + r.stderr[-3000:]
