"""Run with torchrun on 2+ GPUs: the context-parallel attention variants "allgather" (default) and "ring" (K / V blocks sent
around the group, partial results merged by log-sum-exp).  The default context-parallel attention (differentiable NCCL all-gather of K / V, then the
variable-length attention kernel on each zig-zag query chunk against the key prefix that ends with it) against full-sequence causal
attention computed in fp32 -- forward output and the gradients of q, k and v.  Both attention selections are checked: the in-tree
kernels (default) and the library kernel with its explicit bottom-right aligned mask.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_cp_default.py
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
    from nanotron_b200 import ops
    from nanotron_b200.parallel.context_parallel.ring_attention import ring_attention

    group = tdist.group.WORLD
    B, Hq, Hkv, D = 2, 8, 2, 128
    for mode in ("auto", "sdpa"):
        ops.set_attention(mode)
        for chunk in (128, 320):
            S = 2 * world * chunk
            torch.manual_seed(0)  # same full tensors on every rank
            q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
            k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
            v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
            g = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
            qf, kf, vf = (t.float().transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v))
            ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True, enable_gqa=True)
            ref.backward(g.float().transpose(1, 2))
            ref_o = ref.transpose(1, 2)
            ref_dq, ref_dk, ref_dv = (t.grad.transpose(1, 2) for t in (qf, kf, vf))
            loc = lambda t: zigzag(t, rank, world, 1).reshape(B * 2 * chunk, t.shape[2], D).contiguous()
            ql, kl, vl = (loc(t).detach().requires_grad_(True) for t in (q, k, v))
            pos = torch.zeros(B, 2 * chunk, dtype=torch.long, device="cuda")  # only its shape is read
            for variant in ("allgather", "ring"):
                ql.grad = kl.grad = vl.grad = None
                out = ring_attention(ql, kl, vl, cp_pg=group, causal=True, variant=variant, position_ids=pos)
                out.backward(loc(g))
                torch.cuda.synchronize()
                checks = {"out": (out, loc(ref_o)), "dq": (ql.grad, loc(ref_dq)), "dk": (kl.grad, loc(ref_dk)), "dv": (vl.grad, loc(ref_dv))}
                for name, (got, exp) in checks.items():
                    err = ((got.float() - exp.float()).abs().max() / exp.float().abs().max()).item()
                    if rank == 0:
                        print(f"attention={mode:5s} {variant:9s} chunk {chunk:4d} {name:3s} rel err vs fp32 full attention = {err:.3e}")
                    assert err < 3e-2, (mode, variant, chunk, name, err)
    ops.set_attention("auto")
    if rank == 0:
        print("CP_DEFAULT_OK")
    tdist.barrier()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
