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
