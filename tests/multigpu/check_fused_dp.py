"""Run with torchrun on N >= 2 GPUs: the in-kernel NVLink data-parallel step (reduce-scatter + AdamW + all-gather over peer
memory) must give the same loss curve and the same parameters as the NCCL path, with ZeRO-1 and with a replicated optimizer.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_fused_dp.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from helpers import dummy_dataloader, make_config, tiny_llama_config  # noqa: E402


def run(fused: bool, zero: int, steps: int = 5, overlap: bool = True, accum: int = 1):
    import nanotron_b200.distributed as dist
    from nanotron_b200.trainer import DistributedTrainer

    world = int(os.environ["WORLD_SIZE"])
    mc = tiny_llama_config(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, vocab_size=1024)
    cfg = make_config(mc, dp=world, seq=128, mbs=2, accum=accum, steps=steps, dtype="bfloat16", zero=zero, lr=1e-3)
    cfg.optimizer.fused_zero_comm = None if fused else False
    cfg.optimizer.overlap_grad_reduce = overlap
    torch.manual_seed(0)
    t = DistributedTrainer(cfg)
    assert (t.fused_dp is not None) == fused, f"fused path active={t.fused_dp is not None}, expected {fused}"
    t.prepare_training()
    dl = dummy_dataloader(t)
    losses = []
    for _ in range(steps):
        _, loss, _ = t.training_step(dl)
        t.iteration_step += 1
        losses.append(float(loss))
    if t.fused_dp is not None:
        t.fused_dp.alloc.check()
        early = t.fused_dp.overlapped_elems
        assert (early > 0) == overlap, f"elements reduced during the backward: {early}, overlap requested: {overlap}"
    params = torch.cat([p.detach().float().reshape(-1) for _, p in sorted(t.unwrapped_model.named_parameters())])
    # replicas agree bit for bit
    ref = params.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, params), "data-parallel replicas diverged"
    norm = float(t.grad_norm_unclipped) if t.grad_norm_unclipped is not None else None
    return losses, params, norm


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    for zero in (1, 0):
        base_losses, base_params, base_norm = run(fused=False, zero=zero)
        fused_losses, fused_params, fused_norm = run(fused=True, zero=zero)
        diff = (base_params - fused_params).abs().max().item()
        if rank == 0:
            print(f"zero={zero} nccl   losses {['%.4f' % l for l in base_losses]} grad_norm {base_norm}")
            print(f"zero={zero} fused  losses {['%.4f' % l for l in fused_losses]} grad_norm {fused_norm}")
            print(f"zero={zero} max |param diff| = {diff:.3e}")
        assert all(abs(a - b) < 2e-2 for a, b in zip(base_losses, fused_losses)), (base_losses, fused_losses)
        assert diff < 2e-2, diff
        assert abs(base_norm - fused_norm) < 1e-2 * max(1.0, base_norm), (base_norm, fused_norm)
        # the same step without starting the reduce-scatter during the backward, and with several micro-batches per step
        # (only the last backward may launch buckets)
        for accum in (1, 3):
            nccl_losses, nccl_params, nccl_norm = run(fused=False, zero=zero, accum=accum)
            late_losses, late_params, late_norm = run(fused=True, zero=zero, overlap=False, accum=accum)
            early_losses, early_params, early_norm = run(fused=True, zero=zero, overlap=True, accum=accum)
            d_late = (late_params - nccl_params).abs().max().item()
            d_early = (early_params - nccl_params).abs().max().item()
            if rank == 0:
                print(f"zero={zero} accum={accum} nccl        losses {['%.4f' % l for l in nccl_losses]} grad_norm {nccl_norm}")
                print(f"zero={zero} accum={accum} fused       losses {['%.4f' % l for l in late_losses]} grad_norm {late_norm}  max |param diff| vs nccl {d_late:.3e}")
                print(f"zero={zero} accum={accum} fused+early losses {['%.4f' % l for l in early_losses]} grad_norm {early_norm}  max |param diff| vs nccl {d_early:.3e}")
            # bf16 parameters: one rounding step at magnitude 1 is 7.8e-3
            assert d_late < 1e-2 and d_early < 1e-2, (d_late, d_early)
            assert abs(early_norm - nccl_norm) < 1e-3 * max(1.0, nccl_norm) and abs(late_norm - nccl_norm) < 1e-3 * max(1.0, nccl_norm), (nccl_norm, late_norm, early_norm)
    if rank == 0:
        print("FUSED_DP_OK")
    import torch.distributed as tdist

    if tdist.is_initialized():
        tdist.destroy_process_group()


if __name__ == "__main__":
    main()
