"""tcgen05 GEMM against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(BF16)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 512, 4096), (200, 300, 520), (16, 2112, 4096),
                                   (4096, 768, 1536), (1000, 4096, 512), (64, 96, 72)])
def test_gemm_matches_fp32_reference(M, N, K):
    from ironpangu_b200.ops.gemm import gemm
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    a, b = rnd(M, K), rnd(N, K, scale=0.05)
    ref = a.float() @ b.float().T
    c32 = gemm(a, b, out_f32=True, status_ptr=fab.desc.status)
    torch.testing.assert_close(c32, ref, rtol=1e-3, atol=1e-3 * K ** 0.5 * 0.05)
    res = rnd(M, N)
    c = gemm(a, b, residual=res, status_ptr=fab.desc.status)
    torch.testing.assert_close(c.float(), ref.to(BF16).float() + res.float(), rtol=2e-2, atol=2e-2)
    assert fab.status() == 0
    fab.close()


def test_gemm_strided_views():
    """A and the output may be column slices of wider buffers (row stride > width)."""
    from ironpangu_b200.ops.gemm import gemm

    wide = rnd(256, 2112)
    a = wide[:, :1536]
    b = rnd(768, 1536, scale=0.05)
    outw = torch.zeros(256, 1024, dtype=BF16, device="cuda")
    gemm(a, b, out=outw[:, 128:128 + 768])
    torch.testing.assert_close(outw[:, 128:896].float(), a.float() @ b.float().T, rtol=2e-2, atol=2e-2)
    assert float(outw[:, :128].abs().max()) == 0 and float(outw[:, 896:].abs().max()) == 0
