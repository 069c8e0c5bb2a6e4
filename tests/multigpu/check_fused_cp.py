"""Run with torchrun on 2+ GPUs: context-parallel attention with the K / V exchange inside the tcgen05 attention kernels (forward reads
peer tiles by TMA, backward reduces dK / dV into the owners' accumulators) against full-sequence attention computed in fp32.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_fused_cp.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def zigzag(x, rank, cp, dim):
    chunks = x.chunk(2 * cp, dim=dim)
    return torch.cat([chunks[rank], chunks[2 * cp - 1 - rank]], dim=dim)


def main():
    import torch.distributed as tdist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    tdist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from nanotron_b200.parallel.context_parallel import fused_ring

    group = tdist.group.WORLD
    B, Hq, Hkv, D = 2, 8, 2, 128
    for chunk in (128, 384):
        S = 2 * world * chunk
        torch.manual_seed(0)  # same full tensors on every rank
        q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
        g = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
        # oracle: full causal attention in fp32
        qf, kf, vf = (t.float().transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True, enable_gqa=True)
        ref.backward(g.float().transpose(1, 2))
        ref_o = ref.transpose(1, 2)
        ref_dq, ref_dk, ref_dv = (t.grad.transpose(1, 2) for t in (qf, kf, vf))
        # local shards in zig-zag order, flattened [B * s_local, H, D]
        loc = lambda t: zigzag(t, rank, world, 1).reshape(B * 2 * chunk, t.shape[2], D).contiguous()
        ql, kl, vl = (loc(t).detach().requires_grad_(True) for t in (q, k, v))
        assert fused_ring.supported(ql, kl, group, chunk)
        out = fused_ring.fused_ring_attention(ql, kl, vl, group, batch=B)
        out.backward(loc(g))
        torch.cuda.synchronize()
        fused_ring.get_context(group, B * 2 * chunk, Hkv).alloc.check()
        checks = {"out": (out, loc(ref_o)), "dq": (ql.grad, loc(ref_dq)), "dk": (kl.grad, loc(ref_dk)), "dv": (vl.grad, loc(ref_dv))}
        for name, (got, exp) in checks.items():
            err = ((got.float() - exp.float()).abs().max() / exp.float().abs().max()).item()
            if rank == 0:
                print(f"chunk {chunk:4d} {name:3s} rel err vs fp32 full attention = {err:.3e}")
            assert err < 3e-2, (chunk, name, err)
    if rank == 0:
        print("FUSED_CP_OK")
    tdist.barrier()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
