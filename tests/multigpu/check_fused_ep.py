"""Run with torchrun on 2+ GPUs: expert-parallel mixture-of-experts training with the in-kernel NVLink dispatch / combine
and the tcgen05 grouped GEMMs must follow the loss curve of the NCCL all-to-all + library grouped-GEMM path.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_fused_ep.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from helpers import dummy_dataloader, make_config, tiny_qwen_config  # noqa: E402


def train(fused: bool, steps=5):
    import nanotron_b200.config as c
    from nanotron_b200.nn import moe
    from nanotron_b200.ops import moe_fused
    from nanotron_b200.trainer import DistributedTrainer

    moe.FUSED_EXPERTS = fused
    world = int(os.environ["WORLD_SIZE"])
    mc = tiny_qwen_config(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, vocab_size=1024,
                          moe_config=c.MoEConfig(num_experts=16, top_k=2, moe_intermediate_size=128, shared_expert_intermediate_size=256, enable_shared_expert=True, router_aux_loss_coef=0.01))
    cfg = make_config(mc, dp=world, ep=world, seq=256, mbs=2, steps=steps, dtype="bfloat16", lr=1e-3)
    torch.manual_seed(0)
    t = DistributedTrainer(cfg)
    t.prepare_training()
    dl = dummy_dataloader(t)
    losses = []
    for _ in range(steps):
        _, loss, _ = t.training_step(dl)
        t.iteration_step += 1
        losses.append(float(loss))
    if fused:
        ctxs = [c_ for c_ in moe_fused._CONTEXTS.values() if c_.world == world]
        assert ctxs and all(c_.epoch > 0 for c_ in ctxs), "training did not go through the fused expert-parallel kernels"
        for c_ in ctxs:
            c_.check()
    return losses


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    base = train(False)
    fused = train(True)
    if rank == 0:
        print("nccl  losses", ["%.4f" % l for l in base])
        print("fused losses", ["%.4f" % l for l in fused])
    assert all(abs(a - b) < 5e-2 for a, b in zip(base, fused)), (base, fused)
    if rank == 0:
        print("FUSED_EP_OK")
    import torch.distributed as tdist

    tdist.barrier()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
