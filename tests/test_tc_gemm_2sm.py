"""The CTA-pair tcgen05 GEMM (tcgen05.mma cta_group::2, 256 x 256 tiles) against a plain PyTorch fp32 product: one tile per
pair, and the persistent form (several tiles per pair, two accumulators in tensor memory; 4096 x 5120 gives 320 tiles on 74 pairs)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.mark.parametrize("persistent", [False, True])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 512, 200), (512, 256, 1024), (1024, 768, 4096), (4096, 5120, 512), (300, 2112, 520), (513, 288, 64), (1000, 4128, 1536)])
def test_two_sm_gemm_matches_fp32(M, N, K, persistent):
    from ironpangu_b200.ops.gemm import gemm, gemm_2sm

    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g, device="cuda").to(BF16)
    b = torch.randn(N, K, generator=g, device="cuda").to(BF16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = gemm_2sm(a, b, status_ptr=st.data_ptr(), persistent=persistent)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = a.float() @ b.float().T
    torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-1)
    assert torch.equal(c, gemm(a, b))                              # same accumulation order as the one-CTA kernel
    res = torch.randn(M, N, generator=g, device="cuda").to(BF16)
    cf = gemm_2sm(a, b, residual=res, out_f32=True, status_ptr=st.data_ptr(), persistent=persistent)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    torch.testing.assert_close(cf, ref.to(BF16).float() + res.float(), rtol=2e-2, atol=2e-1)


def test_two_sm_gemm_refuses_other_shapes():
    from ironpangu_b200.ops.gemm import gemm_2sm

    a = torch.zeros(128, 64, dtype=BF16, device="cuda")
    b = torch.zeros(250, 64, dtype=BF16, device="cuda")          # N must be a multiple of 32
    with pytest.raises(RuntimeError):
        gemm_2sm(a, b)


@pytest.mark.parametrize("M,F,K", [(256, 128, 64), (512, 6144, 2048), (300, 160, 520), (1024, 1536, 4096)])
def test_two_sm_swiglu_projection(M, F, K):
    """Packed gate | up projection with its activation on CTA pairs: equal to the one-CTA grouped kernel's SwiGLU mode (same
    accumulation order, same rounding points) and close to the fp32 product."""
    from ironpangu_b200.ops import prefill as P
    from ironpangu_b200.ops.gemm import gemm_swiglu

    g = torch.Generator(device="cuda").manual_seed(M + F + K)
    a = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(BF16)
    b = (torch.randn(2 * F, K, generator=g, device="cuda") * 0.05).to(BF16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = gemm_swiglu(a, b, status_ptr=st.data_ptr())
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    gu = a.float() @ b.float().T
    gate, up = gu[:, :F].to(BF16).float(), gu[:, F:].to(BF16).float()
    ref = torch.nn.functional.silu(gate) * up
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    nt = (M + 127) // 128
    tiles = torch.zeros(nt, 4, dtype=torch.int32)
    for i in range(nt):
        tiles[i, 1], tiles[i, 2] = i * 128, min(128, M - i * 128)
    ap = torch.zeros(nt * 128, K, dtype=BF16, device="cuda")
    ap[:M] = a
    one = torch.empty(nt * 128, F, dtype=BF16, device="cuda")
    P.grouped_gemm(ap, b.unsqueeze(0), tiles.cuda(), torch.tensor([nt], dtype=torch.int32, device="cuda"), one, swiglu=True)
    assert torch.equal(out, one[:M])
