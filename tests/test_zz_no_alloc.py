"""fo_lion_multi_tensor_step_noalloc against fo_lion_multi_tensor_step, through the C ABI.

The allocation-free entry point serves callers that cannot call cudaMalloc inside their step
loop (all device memory already belongs to their own pool, or an allocation's device-wide
synchronisation is not acceptable); it keeps its tensor table in a fixed array inside the
library.  It must produce exactly what the allocating entry point produces, on every call: the
array is shared between calls, so two different lists are run back to back.

This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

import fast_ops_b200._lib as L
import oracle

pytestmark = pytest.mark.gpu


def _arrays(ps, gs, ms):
    n = len(ps)
    return ((ctypes.c_void_p * n)(*[t.data_ptr() for t in ps]), (ctypes.c_void_p * n)(*[t.data_ptr() for t in gs]),
            (ctypes.c_void_p * n)(*[t.data_ptr() for t in ms]), (ctypes.c_int64 * n)(*[t.numel() for t in ps]), n)


def _make(shapes, pd, md, seed, device):
    gen = torch.Generator().manual_seed(seed)
    p = [(torch.randn(s, generator=gen) * 0.02).to(pd).to(device) for s in shapes]
    g = [(torch.randn(s, generator=gen) * 1e-3).to(pd).to(device) for s in shapes]
    m = [(torch.randn(s, generator=gen) * 1e-3).to(md).to(device) for s in shapes]
    return p, g, m


def _run(entry, p, g, m, pd, md, hyper, device):
    ap, ag, am, an, n = _arrays(p, g, m)
    L.check(entry(ap, ag, am, an, n, L.dtype_code(pd), L.dtype_code(pd), L.dtype_code(md), *hyper, device.index,
                  L.current_stream_ptr(device)))


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(cuda_device):
    lib = L.load()
    calls = [
        # a long ragged list, then a short one with other dtypes: the second call must not see
        # anything the first left in the shared table
        ([(4097,), (3, 5), (0,), (50000,), (8,), (12345,)] + [(257,)] * 40, torch.float32, torch.bfloat16,
         (1e-4, 0.9, 0.99, 0.1)),
        ([(70000,), (1,), (4096,)], torch.bfloat16, torch.bfloat16, (3e-5, 0.95, 0.98, 0.0)),
    ]
    for i, (shapes, pd, md, hyper) in enumerate(calls):
        p1, g1, m1 = _make(shapes, pd, md, 100 + i, cuda_device)
        p2, m2 = [t.clone() for t in p1], [t.clone() for t in m1]
        p3, g3, m3 = ([t.cpu().reshape(-1).clone() for t in ts] for ts in (p1, g1, m1))  # the CPU oracle's copy
        for _ in range(2):  # two steps each, so the momentum written by step 1 feeds step 2
            _run(lib.fo_lion_multi_tensor_step, p1, g1, m1, pd, md, hyper, cuda_device)
            _run(lib.fo_lion_multi_tensor_step_noalloc, p2, g1, m2, pd, md, hyper, cuda_device)
        torch.cuda.synchronize()
        for a, b in zip(p1, p2):
            assert torch.equal(a, b), f"call {i}: parameters differ"
        for a, b in zip(m1, m2):
            assert torch.equal(a, b), f"call {i}: momentum differs"
        # and against the reference arithmetic itself, not only against the other entry point
        for _ in range(2):
            for cp, cg, cm in zip(p3, g3, m3):
                if cp.numel():
                    oracle.lion_step(cp, cg, cm, hyper[0], (hyper[1], hyper[2]), hyper[3])
        for a, cp, b, cm in zip(p2, p3, m2, m3):
            assert torch.equal(a.cpu().reshape(-1), cp), f"call {i}: parameters differ from the oracle"
            assert torch.equal(b.cpu().reshape(-1), cm), f"call {i}: momentum differs from the oracle"


def test_noalloc_rejects_lists_beyond_its_maximum(cuda_device):
    lib = L.load()
    n = 1025
    t = torch.zeros(8, device=cuda_device, dtype=torch.bfloat16)
    ptrs = (ctypes.c_void_p * n)(*([t.data_ptr()] * n))
    numels = (ctypes.c_int64 * n)(*([8] * n))
    rc = lib.fo_lion_multi_tensor_step_noalloc(ptrs, ptrs, ptrs, numels, n, L.FO_BF16, L.FO_BF16, L.FO_BF16,
                                               1e-4, 0.9, 0.99, 0.0, cuda_device.index, None)
    assert rc == -1 and b"at most 1024 tensors" in lib.fo_last_error()
    torch.cuda.synchronize()
    assert torch.equal(t.cpu(), torch.zeros(8, dtype=torch.bfloat16)), "a rejected call must not launch"


def test_noalloc_refuses_a_capturing_stream(cuda_device):
    """Captured into a CUDA graph, the table upload would become a node that re-reads the
    library's single host-side table image at every replay, when it describes whichever list was
    passed last; the entry point refuses instead of replaying the wrong list."""
    lib = L.load()
    shapes = [(4096,), (100,)]
    p, g, m = _make(shapes, torch.bfloat16, torch.bfloat16, 7, cuda_device)
    hyper = (1e-4, 0.9, 0.99, 0.1)
    _run(lib.fo_lion_multi_tensor_step_noalloc, p, g, m, torch.bfloat16, torch.bfloat16, hyper, cuda_device)  # set-up call
    torch.cuda.synchronize()
    before = [t.clone() for t in p]
    ap, ag, am, an, n = _arrays(p, g, m)
    stream = torch.cuda.Stream(cuda_device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        graph.capture_begin()
        try:
            rc = lib.fo_lion_multi_tensor_step_noalloc(ap, ag, am, an, n, L.FO_BF16, L.FO_BF16, L.FO_BF16, *hyper,
                                                       cuda_device.index, stream.cuda_stream)
            message = lib.fo_last_error()
        finally:
            graph.capture_end()
    assert rc == -3 and b"capturing" in message  # FO_ERR_UNSUPPORTED
    torch.cuda.synchronize()
    for a, b in zip(p, before):
        assert torch.equal(a, b), "a refused call must not change anything"
