#!/bin/bash
# Four gloo ranks on CPU.  NANOTRON_DEBUG_RANK=<r> stops rank r at start-up (SIGSTOP) so a debugger can attach: kill -CONT <pid> resumes it.
set -e
cd "$(dirname "$0")/../.."
python examples/contributor_guide/debug_config_tiny_llama.py
export CUDA_VISIBLE_DEVICES=""
torchrun --nproc-per-node 4 --master-addr 127.0.0.1 run_train.py --config-file examples/contributor_guide/debug_config_tiny_llama.yaml
