"""Fused Lion step on the GPU against the reference's vectors and against the CPU oracle."""
import numpy as np
import pytest
import torch

import fast_ops_b200._lib as L
import oracle
from fast_ops_b200.lion import Lion, lion_update
from helpers import DT, bf16_ulp_distance, from_bits, golden_files, to_bits, ulp_distance

pytestmark = pytest.mark.gpu


def assert_parity(got: torch.Tensor, want: torch.Tensor, what: str):
    """The stated bar: within 1 bf16 ulp.  The kernel mirrors the oracle's roundings, so the
    stricter check (bit-exact) is made as well and reported separately."""
    got, want = got.detach().cpu(), want.detach().cpu()
    d = bf16_ulp_distance(got, want)
    assert int(d.max()) <= 1, f"{what}: {int((d > 1).sum())} elements off by more than 1 bf16 ulp"
    exact = ulp_distance(got, want)
    assert int(exact.max()) == 0, f"{what}: {int((exact > 0).sum())} of {got.numel()} elements not bit-exact"


@pytest.mark.parametrize("path", golden_files("lion"), ids=lambda p: p.split("lion_")[-1][:-4])
def test_lion_kernel_matches_reference_vectors(cuda_device, path):
    z = np.load(path)
    pd, md = DT[str(z["p_dtype"])], DT[str(z["m_dtype"])]
    lr, betas, wd = float(z["lr"]), tuple(float(b) for b in z["betas"]), float(z["weight_decay"])
    p = from_bits(z["p0"], pd).to(cuda_device)
    m = torch.zeros(p.numel(), dtype=md, device=cuda_device)
    for s in range(z["grads"].shape[0]):
        g = from_bits(z["grads"][s], pd).to(cuda_device)
        lion_update(p, g, m, lr, betas[0], betas[1], wd)
        assert np.array_equal(to_bits(p), z["params"][s]), f"param differs from the reference at step {s}"
        assert np.array_equal(to_bits(m), z["exp_avgs"][s]), f"exp_avg differs from the reference at step {s}"
        # exact sign agreement of the applied update: p moved the same way
    assert L.device_status(cuda_device.index) == 0


def _mini_model_shapes():
    """A small list with the flavour of the GPT-2 / Llama parameter lists: a few large
    matrices, many small vectors, sizes that are not multiples of the 4096-element chunk or
    of the 8-element vector."""
    shapes = [(50257, 16), (1024, 48)]
    for _ in range(3):
        shapes += [(256, 768), (768,), (256, 256), (256,), (256, 1024), (1024,), (1024, 256), (256,), (256,), (256,)]
    shapes += [(7,), (1,), (4095,), (4097,), (8191,)]
    return shapes


@pytest.mark.parametrize("pd,md", [("f32", "bf16"), ("bf16", "bf16"), ("f16", "f16"), ("f32", "f32"), ("bf16", "f32")])
def test_lion_optimizer_matches_oracle_over_steps(cuda_device, pd, md):
    gen = torch.Generator().manual_seed(7)
    shapes = _mini_model_shapes()
    cpu_p = [(torch.randn(s, generator=gen) * 0.02).to(DT[pd]) for s in shapes]
    cpu_m = [torch.zeros(s, dtype=DT[md]) for s in shapes]
    params = [t.clone().to(cuda_device).requires_grad_(True) for t in cpu_p]
    lr, betas, wd = 1e-4, (0.9, 0.99), 0.1
    opt = Lion(params, lr=lr, betas=betas, weight_decay=wd, momentum_dtype=DT[md])
    launches0 = L.load().fo_launch_count()
    for step in range(3):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(DT[pd]) for s in shapes]
        for p, g in zip(params, grads):
            p.grad = g.to(cuda_device)
        opt.step()
        for cp, g, cm in zip(cpu_p, grads, cpu_m):
            oracle.lion_step(cp, g, cm, lr, betas, wd)
        for i, (p, cp, cm) in enumerate(zip(params, cpu_p, cpu_m)):
            assert_parity(p.data, cp, f"step {step} param {i} {shapes[i]}")
            assert_parity(opt.state[p]["exp_avg"], cm, f"step {step} exp_avg {i} {shapes[i]}")
    # one launch per step for the whole list
    assert L.load().fo_launch_count() - launches0 == 3
    assert L.device_status(cuda_device.index) == 0


def test_lion_signs_zero_and_cancellation(cuda_device):
    n = 4096
    m0 = (torch.randn(n, generator=torch.Generator().manual_seed(3)) * 1e-3).bfloat16()
    g = (-(m0.float() * 0.9) / (1 - 0.9)).bfloat16()  # beta1*m + (1-beta1)*g is zero or one rounding away
    g[:64] = 0
    m0[:64] = 0
    p0 = torch.full((n,), 0.25).bfloat16()
    cp, cm = p0.clone(), m0.clone()
    oracle.lion_step(cp, g, cm, 1e-2, (0.9, 0.99), 0.0)
    p, m = p0.to(cuda_device), m0.to(cuda_device)
    lion_update(p, g.to(cuda_device), m, 1e-2, 0.9, 0.99, 0.0)
    # the parameter moves by -lr*sign(u): identical movement means identical sign, zeros included
    assert torch.equal(p.cpu(), cp)
    assert torch.equal(p.cpu()[:64], p0[:64]), "sign(0) must be 0"
    assert torch.equal(m.cpu(), cm)
    moved = (cp.float() - p0.float())
    assert (moved > 0).any() and (moved < 0).any()


def test_lion_unaligned_views_and_flat_ranges(cuda_device):
    gen = torch.Generator().manual_seed(5)
    n = 3 * 4096 + 5
    base_p = (torch.randn(n + 3, generator=gen) * 0.02).bfloat16()
    base_g = (torch.randn(n + 3, generator=gen) * 1e-3).bfloat16()
    base_m = (torch.randn(n + 3, generator=gen) * 1e-3).bfloat16()
    # views that start 2 bytes off a 16-byte boundary
    cp, cg, cm = base_p[1:1 + n].clone(), base_g[1:1 + n].clone(), base_m[1:1 + n].clone()
    dp, dg, dm = base_p.to(cuda_device)[1:1 + n], base_g.to(cuda_device)[1:1 + n], base_m.to(cuda_device)[1:1 + n]
    oracle.lion_step(cp, cg, cm, 3e-5, (0.9, 0.99), 0.1)
    lion_update(dp, dg, dm, 3e-5, 0.9, 0.99, 0.1)
    assert torch.equal(dp.cpu(), cp) and torch.equal(dm.cpu(), cm)

    # shard [begin, end) of flat buffers; everything outside stays untouched
    lib = L.load()
    fp, fg = base_p.clone().to(cuda_device), base_g.clone().to(cuda_device)
    begin, end = 1000, 9192
    ms = base_m[begin:end].clone().to(cuda_device)
    L.check(lib.fo_lion_flat_step(fp.data_ptr(), fg.data_ptr(), ms.data_ptr(), begin, end, L.FO_BF16, L.FO_BF16,
                                  L.FO_BF16, 3e-5, 0.9, 0.99, 0.1, cuda_device.index,
                                  L.current_stream_ptr(cuda_device)))
    op, om = base_p[begin:end].clone(), base_m[begin:end].clone()
    oracle.lion_step(op, base_g[begin:end].clone(), om, 3e-5, (0.9, 0.99), 0.1)
    got = fp.cpu()
    assert torch.equal(got[begin:end], op) and torch.equal(ms.cpu(), om)
    assert torch.equal(got[:begin], base_p[:begin]) and torch.equal(got[end:], base_p[end:])


def test_lion_interface_and_errors(cuda_device):
    with pytest.raises(RuntimeError):
        Lion([torch.zeros(8, device=cuda_device, requires_grad=True)], lr=0.0)
    with pytest.raises(RuntimeError):
        Lion([torch.zeros(8, device=cuda_device, requires_grad=True)], betas=(1.5, 0.9))
    p = torch.zeros(16, device=cuda_device, dtype=torch.bfloat16, requires_grad=True)
    q = torch.zeros(0, device=cuda_device, dtype=torch.bfloat16, requires_grad=True)  # empty tensor
    r = torch.ones(16, device=cuda_device, dtype=torch.bfloat16, requires_grad=True)  # no grad: skipped
    opt = Lion([p, q, r], lr=1e-2)
    assert opt.defaults == {"lr": 1e-2, "betas": (0.9, 0.99), "weight_decay": 0.0}
    p.grad = torch.ones_like(p)
    q.grad = torch.ones_like(q)
    opt.step()
    assert torch.equal(p.detach().cpu().float(), torch.full((16,), -1e-2).bfloat16().float())
    assert torch.equal(r.detach().cpu().float(), torch.ones(16))
    assert opt.state[p]["exp_avg"].dtype == torch.bfloat16 and "exp_avg" not in opt.state[r]
    sd = opt.state_dict()
    opt2 = Lion([p, q, r], lr=1e-2)
    opt2.load_state_dict(sd)
    assert torch.equal(opt2.state[p]["exp_avg"], opt.state[p]["exp_avg"])
    with pytest.raises(RuntimeError):  # dtype mismatch between param and grad
        lion_update(p.data, torch.ones(16, device=cuda_device), opt.state[p]["exp_avg"], 1e-2, 0.9, 0.99, 0.0)
    with pytest.raises(RuntimeError):  # no CPU path
        lion_update(torch.zeros(8), torch.zeros(8), torch.zeros(8), 1e-2, 0.9, 0.99, 0.0)
    with pytest.raises(RuntimeError):  # non-dense
        big = torch.zeros(32, device=cuda_device, dtype=torch.bfloat16)
        lion_update(big[::2], big[::2], big[::2], 1e-2, 0.9, 0.99, 0.0)


def test_lion_step_replays_from_a_cuda_graph(cuda_device):
    """The multi-tensor step allocates nothing once its table is cached, so it can be captured."""
    gen = torch.Generator().manual_seed(9)
    shapes = [(300, 40), (5000,), (17,)]
    cpu_p = [(torch.randn(s, generator=gen) * 0.02).bfloat16() for s in shapes]
    cpu_m = [torch.zeros(s, dtype=torch.bfloat16) for s in shapes]
    params = [t.clone().to(cuda_device).requires_grad_(True) for t in cpu_p]
    for p in params:
        p.grad = torch.zeros_like(p)
    opt = Lion(params, lr=1e-3, weight_decay=0.1)
    grads = [[(torch.randn(s, generator=gen) * 1e-3).bfloat16() for s in shapes] for _ in range(3)]

    def load(step):
        for p, g in zip(params, grads[step]):
            p.grad.copy_(g.to(cuda_device))

    load(0)
    opt.step()  # eager: builds and caches the device table
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):  # recorded, not run
        opt.step()
    for step in (1, 2):
        load(step)
        graph.replay()
    torch.cuda.synchronize()
    for step in range(3):
        for cp, g, cm in zip(cpu_p, grads[step], cpu_m):
            oracle.lion_step(cp, g, cm, 1e-3, (0.9, 0.99), 0.1)
    for p, cp, cm in zip(params, cpu_p, cpu_m):
        assert torch.equal(p.detach().cpu(), cp) and torch.equal(opt.state[p]["exp_avg"].cpu(), cm)


def _gpt2_medium_shapes():
    """The GPT-2-medium parameter list of the fused-Lion benchmark configuration: 290 tensors,
    354 821 120 parameters (wte, wpe, 24 blocks of 4 weight/bias pairs and 2 LayerNorm pairs)."""
    shapes = [(50257, 1024), (1024, 1024)]
    for _ in range(24):
        shapes += [(1024, 3072), (3072,), (1024, 1024), (1024,), (1024, 4096), (4096,), (4096, 1024), (1024,),
                   (1024,), (1024,), (1024,), (1024,)]
    return shapes


def test_lion_full_gpt2_medium_list_bit_exact(cuda_device):
    """The whole 290-tensor list in one launch per step (43 313 chunks, a 51 M-element first tensor,
    many 1024-element vectors that fill an eighth of a chunk), fp32 p/g with bf16 momentum, the
    benchmark's hyper-parameters, three steps, every element compared with the oracle."""
    gen = torch.Generator().manual_seed(355)
    shapes = _gpt2_medium_shapes()
    assert len(shapes) == 290 and sum(int(np.prod(s)) for s in shapes) == 354_821_120
    cpu_p = [torch.randn(s, generator=gen) * 0.02 for s in shapes]
    cpu_m = [torch.zeros(s, dtype=torch.bfloat16) for s in shapes]
    params = [t.clone().to(cuda_device).requires_grad_(True) for t in cpu_p]
    lr, betas, wd = 1e-4, (0.9, 0.99), 0.1
    opt = Lion(params, lr=lr, betas=betas, weight_decay=wd, momentum_dtype=torch.bfloat16)
    launches0 = L.load().fo_launch_count()
    for step in range(3):
        grads = [torch.randn(s, generator=gen) * 1e-3 for s in shapes]
        for p, g in zip(params, grads):
            p.grad = g.to(cuda_device)
        opt.step()
        for cp, g, cm in zip(cpu_p, grads, cpu_m):
            oracle.lion_step(cp, g, cm, lr, betas, wd)
    assert L.load().fo_launch_count() - launches0 == 3
    for i, (p, cp, cm) in enumerate(zip(params, cpu_p, cpu_m)):
        assert torch.equal(p.detach().cpu(), cp), f"param {i} {shapes[i]} differs from the oracle"
        assert torch.equal(opt.state[p]["exp_avg"].cpu(), cm), f"exp_avg {i} {shapes[i]} differs from the oracle"
    assert L.device_status(cuda_device.index) == 0


def test_lion_flat_step_on_the_last_shard_of_a_llama7b_sized_buffer(cuda_device):
    """ZeRO-1 shard 7 of 8 of a flat bf16 buffer of 6 738 411 520 elements: `begin` lies beyond
    2^31 elements (and beyond 2^32 bytes), which the small flat-range tests never reach.  Windows of
    2^20 elements at the shard's start, middle and end are compared with the oracle; the elements
    just outside the shard must stay untouched."""
    free, _ = torch.cuda.mem_get_info(cuda_device)
    total = 6_738_411_520
    if free < 2 * 2 * total + (8 << 30):
        pytest.skip("needs about 30 GB of free device memory")
    assert total % 64 == 0
    shard = total // 8
    begin, end = 7 * shard, total
    assert begin > 2 ** 31
    flat_p = torch.empty(total, device=cuda_device, dtype=torch.bfloat16)
    flat_g = torch.empty(total, device=cuda_device, dtype=torch.bfloat16)
    gen = torch.Generator(device=cuda_device).manual_seed(70)
    # only the shard and a margin before it need defined values
    lo = begin - (1 << 20)
    piece = 1 << 27
    for off in range(lo, total, piece):
        n = min(piece, total - off)
        flat_p[off:off + n] = (torch.randn(n, generator=gen, device=cuda_device) * 0.02).bfloat16()
        flat_g[off:off + n] = (torch.randn(n, generator=gen, device=cuda_device) * 1e-3).bfloat16()
    m_shard = (torch.randn(shard, generator=gen, device=cuda_device) * 1e-3).bfloat16()
    w = 1 << 20
    windows = [begin, begin + (shard // 2) // 8 * 8 + 3, end - w]  # one of them off the 16-byte grid
    before = [(flat_p[a:a + w].cpu(), flat_g[a:a + w].cpu(), m_shard[a - begin:a - begin + w].cpu()) for a in windows]
    margin = flat_p[lo:begin].clone()
    lib = L.load()
    hyper = (3e-5, 0.9, 0.99, 0.1)
    L.check(lib.fo_lion_flat_step(flat_p.data_ptr(), flat_g.data_ptr(), m_shard.data_ptr(), begin, end, L.FO_BF16,
                                  L.FO_BF16, L.FO_BF16, *hyper, cuda_device.index, L.current_stream_ptr(cuda_device)))
    torch.cuda.synchronize()
    for a, (p0, g0, m0) in zip(windows, before):
        oracle.lion_step(p0, g0, m0, hyper[0], (hyper[1], hyper[2]), hyper[3])
        assert torch.equal(flat_p[a:a + w].cpu(), p0), f"window at {a}: parameters differ from the oracle"
        assert torch.equal(m_shard[a - begin:a - begin + w].cpu(), m0), f"window at {a}: momentum differs"
    assert torch.equal(flat_p[lo:begin], margin), "elements before the shard were modified"
    assert L.device_status(cuda_device.index) == 0


@pytest.mark.parametrize("peer_offset", [0, 1], ids=["aligned_peer", "unaligned_peer"])
def test_flat_step_push_takes_any_peer_alignment(cuda_device, peer_offset):
    """fo_lion_flat_step_push with a second buffer of the same device standing in for a peer: the
    updated slice lands in both buffers, also when the peer's buffer starts off the 16-byte grid
    (the 16-byte stores are then not usable; the kernel must fall back, not fault)."""
    import ctypes

    n, begin, end = 40000, 8192, 8192 + 24576 + 5
    gen = torch.Generator().manual_seed(17)
    p0 = (torch.randn(n, generator=gen) * 0.02).bfloat16()
    g = (torch.randn(n, generator=gen) * 1e-3).bfloat16()
    m0 = (torch.randn(end - begin, generator=gen) * 1e-3).bfloat16()
    local = p0.clone().to(cuda_device)
    peer_store = torch.zeros(n + 8, device=cuda_device, dtype=torch.bfloat16)
    peer = peer_store[peer_offset:peer_offset + n]
    m = m0.clone().to(cuda_device)
    lib = L.load()
    arr = (ctypes.c_void_p * 1)(peer.data_ptr())
    L.check(lib.fo_lion_flat_step_push(local.data_ptr(), g.to(cuda_device).data_ptr(), m.data_ptr(), begin, end, arr, 1,
                                       L.FO_BF16, L.FO_BF16, L.FO_BF16, 1e-3, 0.9, 0.99, 0.1, cuda_device.index,
                                       L.current_stream_ptr(cuda_device)))
    torch.cuda.synchronize()
    want_p, want_m = p0[begin:end].clone(), m0.clone()
    oracle.lion_step(want_p, g[begin:end].clone(), want_m, 1e-3, (0.9, 0.99), 0.1)
    assert torch.equal(local[begin:end].cpu(), want_p) and torch.equal(m.cpu(), want_m)
    assert torch.equal(peer[begin:end].cpu(), want_p), "the peer's copy of the slice differs"
    assert torch.count_nonzero(peer[:begin]) == 0 and torch.count_nonzero(peer[end:]) == 0
    assert torch.equal(local[:begin].cpu(), p0[:begin]) and torch.equal(local[end:].cpu(), p0[end:])
