"""One-tile checks of the tensor-core building blocks (TMA box layout, shared-memory and
instruction descriptors, packed operands in tensor memory) against a plain matmul."""
import pytest
import torch

import fast_ops_b200._lib as L

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("N,K", [(128, 64), (128, 128), (64, 128), (64, 64)])
@pytest.mark.parametrize("mode", [0, 1], ids=["qk_smem_smem", "pv_tmem_smem"])
def test_umma_tile(cuda_device, dtype, N, K, mode):
    gen = torch.Generator().manual_seed(100 * N + K + mode)
    a = torch.randn(128, K, generator=gen).to(dtype)
    b = (torch.randn(N, K, generator=gen) if mode == 0 else torch.randn(K, N, generator=gen)).to(dtype)
    ref = a.float() @ (b.float().t() if mode == 0 else b.float())
    ad, bd = a.to(cuda_device), b.to(cuda_device)
    c = torch.full((128, N), float("nan"), device=cuda_device)
    lib = L.load()
    L.check(lib.fo_debug_umma_tile(ad.data_ptr(), bd.data_ptr(), c.data_ptr(), N, K, L.dtype_code(dtype), mode,
                                   cuda_device.index, L.current_stream_ptr(cuda_device)))
    torch.cuda.synchronize()
    assert L.device_status(cuda_device.index) == 0
    # products of 16-bit inputs are exact in fp32; only the summation order differs
    assert torch.allclose(c.cpu(), ref, atol=1e-3, rtol=1e-4), (c.cpu() - ref).abs().max()


def test_bounded_wait_runs_out_and_reports(cuda_device):
    """The attention kernels' device-side waits have a budget; when it runs out the wait records a
    code in the device status word and the kernel goes on to its normal end.  Here one warp waits
    20 ms on a barrier that nothing ever completes: the launch must come back by itself, the
    status word must carry the code until it is reset, and the device must be usable afterwards."""
    import time

    from fast_ops_b200.flash_attention import flash_attention_forward

    lib = L.load()
    assert L.device_status(cuda_device.index, reset=True) in (0, 0x10)
    assert L.device_status(cuda_device.index) == 0
    returned = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    L.check(lib.fo_debug_wait_timeout(20_000, returned.data_ptr(), cuda_device.index,
                                      L.current_stream_ptr(cuda_device)))
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert 0.015 < elapsed < 1.0, f"the wait took {elapsed:.3f} s for a 20 ms budget"
    assert returned.item() == 2, "the kernel did not come back through the give-up path"
    assert L.device_status(cuda_device.index) == 0x10
    assert L.device_status(cuda_device.index, reset=True) == 0x10  # reported once more, then cleared
    assert L.device_status(cuda_device.index) == 0
    # an ordinary attention call afterwards runs and is correct
    q = torch.randn(1, 1, 256, 64, device=cuda_device).half()
    out = flash_attention_forward(q, q, q, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), q.float(), q.float(), is_causal=True)
    torch.cuda.synchronize()
    assert L.device_status(cuda_device.index) == 0
    assert (out.float() - ref).abs().max().item() <= 2e-3
    rc = lib.fo_debug_wait_timeout(0, None, cuda_device.index, None)
    assert rc == -1 and b"budget_us" in lib.fo_last_error()
