"""Host logic of the ZeRO-1 Lion path on CPU: flat layout arithmetic, and a world-size-2 gloo run
in which the device step is replaced by the oracle (the C-ABI call itself needs a GPU)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fast_ops_b200.lion.zero1 import FlatLayout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_flat_layout_alignment_and_cover():
    numels = [5, 8, 0, 13, 4096, 1]
    for world in (1, 2, 3, 8):
        lay = FlatLayout.build(numels, world)
        assert lay.total % (8 * world) == 0
        assert all(o % 8 == 0 for o in lay.offsets)
        for a, b, n in zip(lay.offsets, lay.offsets[1:], numels):
            assert b >= a + n  # no overlap
        covered = [0] * len(numels)
        for r in range(world):
            b, e = lay.shard_range(r)
            assert (e - b) == lay.shard_size and b % 8 == 0
            for i in range(len(numels)):
                t0, s0, n = lay.tensor_slice_in_shard(i, r)
                assert 0 <= s0 and s0 + n <= lay.shard_size and t0 + n <= numels[i]
                covered[i] += n
        assert covered == numels  # every element belongs to exactly one rank
    with pytest.raises(ValueError):
        FlatLayout.build([4], 0)
    with pytest.raises(ValueError):
        FlatLayout.build([4], 2).shard_range(2)


def test_llama7b_shard_sizes_match_the_plan():
    shapes = [32000 * 4096] * 2
    for _ in range(32):
        shapes += [4096 * 4096] * 4 + [11008 * 4096] * 3 + [4096] * 2
    lay = FlatLayout.build(shapes, 8)
    assert sum(shapes) == 6738411520
    assert lay.total == 6738411520 and lay.shard_size == 842301440


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import oracle
    from fast_ops_b200.lion import Lion

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(42)  # same parameters and (already reduced) grads on all ranks
        shapes = [(33, 7), (1000,), (5,), (64, 64), (3,)]
        init = [(torch.randn(s, generator=gen) * 0.02).bfloat16() for s in shapes]
        params = [t.clone().requires_grad_(True) for t in init]
        opt = Lion(params, lr=1e-3, betas=(0.9, 0.99), weight_decay=0.1, process_group=dist.group.WORLD)
        zero = opt._zero

        def cpu_flat_step(p, g, m_shard, begin, end, lr, betas, wd):
            pp, gg = p[begin:end].clone(), g[begin:end].clone()
            oracle.lion_step(pp, gg, m_shard, lr, betas, wd)
            p[begin:end] = pp

        zero.flat_step_fn = cpu_flat_step  # stands in for the C-ABI call, which needs a GPU
        ref_p = [t.clone() for t in init]
        ref_m = [torch.zeros_like(t) for t in init]
        for step in range(3):
            grads = [(torch.randn(s, generator=gen) * 1e-3).bfloat16() for s in shapes]
            for i, (p, g) in enumerate(zip(params, grads)):
                if step == 1 and i == 0:
                    p.grad = g.clone()          # a caller that assigns a fresh tensor: copied in
                else:
                    p.grad.copy_(g)             # the fast path: write into the flat view
            opt.step()
            for rp, g, rm in zip(ref_p, grads, ref_m):
                oracle.lion_step(rp.view(-1), g.view(-1), rm.view(-1), 1e-3, (0.9, 0.99), 0.1)
            for p, rp in zip(params, ref_p):
                assert torch.equal(p.data, rp), f"rank {rank} step {step}: params differ after the all-gather"
        # momentum exists only for this rank's slice, and matches the reference there
        b, e = zero.begin, zero.end
        assert zero.m_shard.numel() == e - b == zero.layout.shard_size
        for i, (p, rm) in enumerate(zip(params, ref_m)):
            t0, s0, n = zero.layout.tensor_slice_in_shard(i, rank)
            assert torch.equal(opt.state[p]["exp_avg"], rm.view(-1)[t0:t0 + n])
        assert all(p.data.data_ptr() >= zero.flat_p.data_ptr() for p in params)

        # state_dict round trip: a fresh optimizer over the same parameters adopts the saved shard
        sd = opt.state_dict()
        opt2 = Lion(params, lr=1e-3, betas=(0.9, 0.99), weight_decay=0.1, process_group=dist.group.WORLD)
        opt2.load_state_dict(sd)
        assert torch.equal(opt2._zero.m_shard, zero.m_shard)
        assert all(opt2.state[p]["exp_avg"].data_ptr() >= opt2._zero.m_shard.data_ptr() for p in params
                   if opt2.state[p]["exp_avg"].numel())

        # reduce_gradients: ranks hold g*(rank+1); the average over two ranks is 1.5*g, taken
        # here with g scaled so that every value stays exactly representable
        opt3 = Lion(params, lr=1e-3, betas=(0.9, 0.99), weight_decay=0.1, process_group=dist.group.WORLD,
                    reduce_gradients=True)
        opt3._zero.flat_step_fn = cpu_flat_step
        base = [(torch.randn(s, generator=gen) * 1e-3).bfloat16() for s in shapes]
        ref_p3 = [p.data.clone() for p in params]
        ref_m3 = [torch.zeros_like(t) for t in init]
        for p, g in zip(params, base):
            p.grad.copy_(g * (2.0 if rank == 0 else 6.0))  # average = 4*g, exact in bf16
        opt3.step()
        for rp, g, rm in zip(ref_p3, base, ref_m3):
            oracle.lion_step(rp.view(-1), (g * 4.0).view(-1), rm.view(-1), 1e-3, (0.9, 0.99), 0.1)
        for p, rp in zip(params, ref_p3):
            assert torch.equal(p.data, rp), f"rank {rank}: reduce_gradients step differs"
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_zero1_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}
