"""Pipeline-parallel runtime on gloo ranks with hand-built block graphs (the models' own tests cover Llama / Qwen2 end to end):
both engines against a single-process replica of the same network, tensors that carry no gradient, an activation consumed by
two stages (diamond), and block-to-block traffic without any engine."""
import pytest
import torch
from torch import nn

from helpers import run_distributed


class _Layer(nn.Module):
    def __init__(self, idx: int, width: int = 8):
        super().__init__()
        g = torch.Generator().manual_seed(100 + idx)
        self.lin = nn.Linear(width, width)
        with torch.no_grad():
            self.lin.weight.copy_(torch.randn(width, width, generator=g) * 0.4)
            self.lin.bias.copy_(torch.randn(width, generator=g) * 0.1)

    def forward(self, x, keep=None):
        out = {"x": torch.tanh(self.lin(x))}
        if keep is not None:
            out["keep"] = keep  # a tensor that is only passed along (no gradient)
        return out


class _Loss(nn.Module):
    def forward(self, x, keep=None):
        loss = (x * x).mean() if keep is None else (x * x * keep).mean()
        return {"loss": loss}


def _chain(p2p, n_layers, with_keep):
    from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

    keys = {"x", "keep"} if with_keep else {"x"}
    layers = nn.ModuleList([PipelineBlock(p2p=p2p, module_builder=_Layer, module_kwargs={"idx": i}, module_input_keys=keys, module_output_keys=keys) for i in range(n_layers)])
    loss = PipelineBlock(p2p=p2p, module_builder=_Loss, module_kwargs={}, module_input_keys=keys, module_output_keys={"loss"})
    return layers, loss


class _ChainModel(nn.Module):
    def __init__(self, p2p, n_layers, with_keep):
        super().__init__()
        self.layers, self.loss = _chain(p2p, n_layers, with_keep)
        self.with_keep = with_keep

    def forward(self, x, keep=None):
        state = {"x": x}
        if self.with_keep:
            state["keep"] = keep
        for layer in self.layers:
            state = layer(**state)
        return self.loss(**state)


def _reference_grads(n_layers, batches, with_keep):
    """The same network on one process: gradient of the mean over micro-batches of the loss."""
    layers = [_Layer(i) for i in range(n_layers)]
    total = 0.0
    for mb in batches:
        x = mb["x"]
        for layer in layers:
            x = layer(x)["x"]
        loss = (x * x).mean() if not with_keep else (x * x * mb["keep"]).mean()
        (loss / len(batches)).backward()
        total += float(loss) / len(batches)
    return [{n: p.grad.clone() for n, p in layer.named_parameters()} for layer in layers], total


def _run_chain(engine_name, pp, n_mb, with_keep):
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.pipeline_parallel.engine import AllForwardAllBackwardPipelineEngine, OneForwardOneBackwardPipelineEngine
    from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
    from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

    ctx = ParallelContext(1, pp, 1)
    rank = dist.get_rank(ctx.pp_pg)
    p2p = P2P(ctx.pp_pg, device=torch.device("cpu"))
    n_layers = 2 * pp - 1  # uneven: the last stage holds one layer and the loss
    model = _ChainModel(p2p, n_layers, with_keep)
    owner = lambda i: min(i // 2, pp - 1)
    for i, blk in enumerate(model.layers):
        blk.build_and_set_rank(owner(i))
    model.loss.build_and_set_rank(pp - 1)
    g = torch.Generator().manual_seed(7)
    full = [{"x": torch.randn(3, 8, generator=g), "keep": (torch.rand(3, 8, generator=g) > 0.3).float()} for _ in range(n_mb)]
    feed = []
    for mb in full:
        item = {"x": mb["x"] if rank == 0 else TensorPointer(group_rank=0)}
        if with_keep:
            item["keep"] = mb["keep"] if rank == 0 else TensorPointer(group_rank=0)
        feed.append(item)
    engine = AllForwardAllBackwardPipelineEngine() if engine_name == "afab" else OneForwardOneBackwardPipelineEngine()
    for step in range(2):  # the second batch replays the shapes learnt in the first
        for p in model.parameters():
            p.grad = None
        outputs = engine.train_batch_iter(model=model, pg=ctx.pp_pg, batch=iter(feed), nb_microbatches=n_mb)
        ref, ref_loss = _reference_grads(n_layers, full, with_keep)
        for i, blk in enumerate(model.layers):
            if owner(i) != rank:
                continue
            for n, p in blk.pp_block.named_parameters():
                torch.testing.assert_close(p.grad, ref[i][n], atol=1e-6, rtol=1e-5)
        if rank == pp - 1:
            total = sum(float(o["loss"]) for o in outputs)  # every micro-batch's loss is already divided by their number
            assert abs(total - ref_loss) < 1e-6
        else:
            assert all(isinstance(o["loss"], TensorPointer) for o in outputs)
    ctx.destroy()


@pytest.mark.parametrize("engine,pp,n_mb", [("afab", 2, 3), ("1f1b", 2, 1), ("1f1b", 2, 4), ("1f1b", 4, 3), ("1f1b", 4, 6), ("afab", 4, 2)])
def test_engines_match_a_single_process_replica(engine, pp, n_mb):
    run_distributed(_run_chain, pp, engine_name=engine, pp=pp, n_mb=n_mb, with_keep=False)


@pytest.mark.parametrize("engine", ["afab", "1f1b"])
def test_tensors_without_gradient_travel_with_the_activations(engine):
    """A mask produced on the first stage is handed from block to block and used by the loss on the last one."""
    run_distributed(_run_chain, 3, engine_name=engine, pp=3, n_mb=4, with_keep=True)


class _Join(nn.Module):
    def forward(self, a, b):
        return {"loss": (a * b).pow(2).mean()}


class _Diamond(nn.Module):
    """rank 0: h = L0(x);  rank 1: a = L1(h);  rank 2: b = L2(h);  rank 3: loss(a, b).  h feeds two stages."""

    def __init__(self, p2p):
        super().__init__()
        from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

        self.l0, self.l1, self.l2 = (PipelineBlock(p2p=p2p, module_builder=_Layer, module_kwargs={"idx": i}, module_input_keys={"x"}, module_output_keys={"x"}) for i in range(3))
        self.join = PipelineBlock(p2p=p2p, module_builder=_Join, module_kwargs={}, module_input_keys={"a", "b"}, module_output_keys={"loss"})

    def forward(self, x):
        h = self.l0(x=x)["x"]
        a = self.l1(x=h)["x"]
        b = self.l2(x=h)["x"]
        return self.join(a=a, b=b)


def _run_diamond(engine_name):
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.pipeline_parallel.engine import AllForwardAllBackwardPipelineEngine, OneForwardOneBackwardPipelineEngine
    from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
    from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

    ctx = ParallelContext(1, 4, 1)
    rank = dist.get_rank(ctx.pp_pg)
    model = _Diamond(P2P(ctx.pp_pg, device=torch.device("cpu")))
    for r, blk in enumerate((model.l0, model.l1, model.l2, model.join)):
        blk.build_and_set_rank(r)
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(2, 8, generator=g) for _ in range(4)]
    feed = [{"x": x if rank == 0 else TensorPointer(group_rank=0)} for x in xs]
    engine = AllForwardAllBackwardPipelineEngine() if engine_name == "afab" else OneForwardOneBackwardPipelineEngine()
    engine.train_batch_iter(model=model, pg=ctx.pp_pg, batch=iter(feed), nb_microbatches=len(xs))
    # single-process replica
    ref = [_Layer(i) for i in range(3)]
    for x in xs:
        h = ref[0](x)["x"]
        loss = (ref[1](h)["x"] * ref[2](h)["x"]).pow(2).mean() / len(xs)
        loss.backward()
    if rank < 3:
        mine = (model.l0, model.l1, model.l2)[rank].pp_block
        for n, p in mine.named_parameters():
            torch.testing.assert_close(p.grad, dict(ref[rank].named_parameters())[n].grad, atol=1e-6, rtol=1e-5)
    ctx.destroy()


@pytest.mark.parametrize("engine", ["afab", "1f1b"])
def test_an_activation_consumed_by_two_stages_gets_both_gradients(engine):
    run_distributed(_run_diamond, 4, engine_name=engine)


def _run_without_engine():
    """Blocks called directly, no pipeline state: tensors that need no gradient are exchanged on the spot."""
    import nanotron_b200.distributed as dist
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
    from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

    ctx = ParallelContext(1, 2, 1)
    rank = dist.get_rank(ctx.pp_pg)
    model = _ChainModel(P2P(ctx.pp_pg, device=torch.device("cpu")), 2, with_keep=False)
    model.layers[0].build_and_set_rank(0)
    model.layers[1].build_and_set_rank(1)
    model.loss.build_and_set_rank(1)
    x = torch.randn(3, 8, generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        out = model(x=x if rank == 0 else TensorPointer(group_rank=0))
    if rank == 1:
        h = x
        for i in range(2):
            h = _Layer(i)(h)["x"]
        torch.testing.assert_close(out["loss"], (h * h).mean())
    else:
        assert isinstance(out["loss"], TensorPointer) and out["loss"].group_rank == 1
    ctx.destroy()


def test_blocks_exchange_tensors_without_an_engine():
    run_distributed(_run_without_engine, 2)
