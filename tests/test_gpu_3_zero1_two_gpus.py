"""ZeRO-1 Lion step on two GPUs (skipped on a single-GPU box): the NCCL all-gather path and the
fused path (step kernel storing into the peer's buffer) must both reproduce, on every rank, the
single-process oracle result for every parameter."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fused, reduce, ret):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import oracle
    from fast_ops_b200.lion import Lion

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        gen = torch.Generator().manual_seed(42)
        shapes = [(333, 70), (100001,), (5,), (640, 640), (3,), (4096,)]
        init = [(torch.randn(s, generator=gen) * 0.02).bfloat16() for s in shapes]
        params = [t.clone().to(dev).requires_grad_(True) for t in init]
        opt = Lion(params, lr=1e-3, betas=(0.9, 0.99), weight_decay=0.1, process_group=dist.group.WORLD,
                   fused_gather=fused, reduce_gradients=reduce)
        ref_p = [t.clone() for t in init]
        ref_m = [torch.zeros_like(t) for t in init]
        for step in range(3):
            grads = [(torch.randn(s, generator=gen) * 1e-3).bfloat16() for s in shapes]
            for p, g in zip(params, grads):
                # with reduce_gradients the ranks hold g/2 and 3g/2 (3g/2 rounded to bf16): the average need
                # not be g bit for bit, but it has g's sign and Lion's parameter update uses only that;
                # the momentum is therefore not compared in this mode
                p.grad.copy_((g * (1.0 if not reduce else (0.5 if rank == 0 else 1.5))).to(dev))
            opt.step()
            for rp, g, rm in zip(ref_p, grads, ref_m):
                oracle.lion_step(rp.view(-1), g.view(-1), rm.view(-1), 1e-3, (0.9, 0.99), 0.1)
            torch.cuda.synchronize()
            for i, (p, rp) in enumerate(zip(params, ref_p)):
                assert torch.equal(p.data.cpu(), rp), f"rank {rank} step {step} param {i}: differs from the oracle"
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused,reduce", [(False, False), (True, False), (False, True)],
                         ids=["nccl_all_gather", "fused_peer_stores", "reduce_scatter_then_all_gather"])
def test_zero1_two_gpus(fused, reduce):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), fused, reduce, ret), nprocs=2, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}
