"""The tcgen05 building blocks: a 128 x N x Kc bf16 GEMM for every operand-major combination,
against torch, so that the shared-memory and instruction descriptor encodings are pinned."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("N,Kc", [(128, 128), (256, 128), (128, 256), (32, 64), (64, 16), (256, 256)])
def test_umma_gemm_matches_torch(a_mn, b_mn, N, Kc):
    from deltanet_b200 import _lib as L
    lib = L.lib()
    gen = torch.Generator().manual_seed(N * 7 + Kc + a_mn * 2 + b_mn)
    A = torch.randn(128, Kc, generator=gen).to(torch.bfloat16).cuda()
    B = torch.randn(N, Kc, generator=gen).to(torch.bfloat16).cuda()
    ref = A.float() @ B.float().T
    a_src = A.T.contiguous() if a_mn else A.contiguous()
    b_src = B.T.contiguous() if b_mn else B.contiguous()
    D = torch.full((128, N), float("nan"), device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.check(lib.dn_selftest_umma(a_mn, b_mn, N, Kc, a_src.data_ptr(), b_src.data_ptr(), D.data_ptr(),
                                 err.data_ptr(), torch.cuda.current_stream().cuda_stream), "dn_selftest_umma")
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "a bounded wait inside the kernel gave up"
    rel = float((D - ref).norm() / ref.norm())
    assert rel < 1e-5, rel
