# Convenience targets; everything they run is a plain command that also works by hand.
PYTHON ?= python

.PHONY: build test test-gpu bench clean

build:            ## compile the sm_100a kernels and the C++ dataset helpers in-tree
	$(PYTHON) -m nanotron_b200.ops.build

test:             ## CPU suite (gloo ranks stand in for GPUs)
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu:         ## kernels against their fp32 oracles, trainer on the native path (needs a B200)
	$(PYTHON) -m pytest tests -x -q -m gpu

bench:            ## Llama-3-8B training step on one GPU
	$(PYTHON) bench.py --gpus 1

clean:
	rm -f nanotron_b200/ops/libntb_kernels.so nanotron_b200/data/libntb_dataidx.so
