#!/bin/bash
# The smallest complete run: writes the tiny Llama configuration and trains it on dummy data with dp2 x tp2 x pp2.
# On a machine without GPUs the same command runs on CPU (gloo) with --nproc-per-node 8.
set -e
cd "$(dirname "$0")/.."
python examples/config_tiny_llama.py
export CUDA_DEVICE_MAX_CONNECTIONS=1
torchrun --nproc-per-node 8 --master-addr 127.0.0.1 run_train.py --config-file examples/config_tiny_llama.yaml
