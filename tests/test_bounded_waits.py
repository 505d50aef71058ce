"""Failure detection on the device without faulting one: peers that never arrive.

``Fabric(silent_peers=True)`` maps the other ranks to blocks on this GPU that nothing writes, with a small poll limit. Every
fused collective must give up after its bounded wait, record PEER_TIMEOUT in the sticky status word and return; the context
stays usable, and after the status is cleared a one-rank fabric computes correct results on the same device."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _status_bits():
    from ironpangu_b200.parallel import fabric as F

    return {"PEER_TIMEOUT": F.STATUS_PEER_TIMEOUT}


def test_decode_collectives_time_out_and_report():
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    bits = _status_bits()
    fab = Fabric(0, 2, silent_peers=True, spin_limit=2000)
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(1, 512, generator=g, device="cuda").to(BF16)
    w = (torch.randn(256, 512, generator=g, device="cuda") * 0.05).to(BF16)
    assert fab.status() == 0
    K.gemv_allreduce(x, w, fab)                     # the peer's partial sums never come
    torch.cuda.synchronize()
    assert fab.status() & bits["PEER_TIMEOUT"]
    fab.clear_status()
    head = (torch.randn(1024, 512, generator=g, device="cuda") * 0.05).to(BF16)
    K.lm_head_argmax(x, head, fab)                  # the peer's (value, index) candidates never come
    torch.cuda.synchronize()
    assert fab.status() & bits["PEER_TIMEOUT"]
    fab.close()
    # the device is fine: a one-rank fabric computes the same GEMV correctly afterwards
    solo = Fabric(0, 1)
    y = K.gemv_allreduce(x, w, solo)
    torch.testing.assert_close(y.float(), (x.float() @ w.float().T), rtol=2e-2, atol=2e-2)
    assert solo.status() == 0
    solo.close()


def test_bulk_gemm_allreduce_times_out_and_frees_its_tensor_memory():
    from ironpangu_b200.ops.gemm import gemm, gemm_allreduce
    from ironpangu_b200.parallel.fabric import Fabric

    bits = _status_bits()
    fab = Fabric(0, 2, silent_peers=True, spin_limit=2000, data_half_bytes=8 << 20)
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(256, 256, generator=g, device="cuda").to(BF16)
    b = (torch.randn(512, 256, generator=g, device="cuda") * 0.05).to(BF16)

    class Sym:                                        # both "ranks" publish into buffers on this device
        def __init__(self):
            import ctypes as C
            self.tensor = torch.zeros(256, 512, dtype=BF16, device="cuda")
            self.other = torch.zeros(256, 512, dtype=BF16, device="cuda")
            self.peer_ptrs = (C.c_void_p * 8)(self.tensor.data_ptr(), self.other.data_ptr())

    sym = Sym()
    gemm_allreduce(a, b, fab, sym)
    torch.cuda.synchronize()
    assert fab.status() & bits["PEER_TIMEOUT"]
    fab.close()
    # tensor memory was released on the way out: a plain tcgen05 GEMM still gets its allocation and is correct
    c = gemm(a, b)
    torch.testing.assert_close(c.float(), a.float() @ b.float().T, rtol=2e-2, atol=2e-2)
