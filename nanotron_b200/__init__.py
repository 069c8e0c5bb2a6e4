"""nanotron_b200: a Blackwell-first LLM pretraining framework.

Public surface mirrors huggingface/nanotron (``Config``, ``ParallelContext``,
``DistributedTrainer``, sharded safetensors checkpoints, Llama / Qwen2(+MoE) /
Starcoder2 models) while every hot op is a hand-written sm_100a kernel living
under :mod:`nanotron_b200.ops`.  The same code also runs on CPU with the gloo
backend, which is what the numerical oracles and the multi-rank logic tests use.
"""

__version__ = "0.2.0"
