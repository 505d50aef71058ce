"""MoME, mHC, gated delta rule and the sparse-attention indexer against plain PyTorch restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _r(t):
    return t.to(BF16).float()


def test_mome_chunked_equals_token_by_token_reference():
    from ironpangu_b200.ops import hc

    g = torch.Generator(device="cuda").manual_seed(0)
    C, taps, n = 300, 3, 11
    w = torch.randn(C + 20, taps, generator=g, device="cuda") * 0.5
    xs = torch.randn(n, C, generator=g, device="cuda").to(BF16)
    ref = []
    hist = torch.zeros(taps - 1, C, device="cuda")
    for t in range(n):
        x = xs[t].float()
        conv = x * w[20:, taps - 1] + sum(hist[k] * w[20:, k] for k in range(taps - 1))
        ref.append(_r(x + (conv if t + 1 >= taps else 0)))
        hist = torch.cat([hist[1:], x[None]])
    ref = torch.stack(ref)
    state = torch.zeros(2, taps - 1, C, dtype=BF16, device="cuda")
    got = []
    for s in range(0, n, 4):          # chunks of 4 rows of sequence slot 1
        m = min(4, n - s)
        pos = torch.arange(s, s + m, dtype=torch.int32, device="cuda")
        got.append(hc.mome(xs[s:s + m], w, state, pos, torch.ones(m, dtype=torch.int32, device="cuda"), c_offset=20))
    torch.testing.assert_close(torch.cat(got).float(), ref, rtol=1e-2, atol=1e-2)
    assert float(state[0].float().abs().max()) == 0.0                      # the other slot is untouched


def _mhc_ref(X, phi, gamma, alpha, beta, iters, eps):
    T, S, W = X.shape
    Xf = X.float().reshape(T, S * W)
    inv = torch.rsqrt(Xf.pow(2).mean(-1, keepdim=True) + eps)
    m = inv * ((Xf * gamma) @ phi.T)
    pre = torch.sigmoid(m[:, :S] * alpha[0] + beta[:S]) + 1e-6
    post = 2 * torch.sigmoid(m[:, S:2 * S] * alpha[1] + beta[S:2 * S])
    R = (m[:, 2 * S:] * alpha[2] + beta[2 * S:]).view(T, S, S)
    R = torch.softmax(R, -1) + 1e-6
    R = R / (R.sum(1, keepdim=True) + 1e-6)
    for _ in range(1, iters):
        R = R / (R.sum(2, keepdim=True) + 1e-6)
        R = R / (R.sum(1, keepdim=True) + 1e-6)
    y = _r(torch.einsum("ts,tsw->tw", pre, X.float()))
    return y, post, R


def test_mhc_pre_and_post():
    from ironpangu_b200.ops import hc

    g = torch.Generator(device="cuda").manual_seed(1)
    T, S, W = 5, 4, 320
    X = torch.randn(T, S, W, generator=g, device="cuda").to(BF16)
    M = S * S + 2 * S
    phi = torch.randn(M, S * W, generator=g, device="cuda") * 0.05
    gamma = 1 + 0.1 * torch.randn(S * W, generator=g, device="cuda")
    alpha = torch.tensor([0.7, 1.1, 0.9], device="cuda")
    beta = torch.randn(M, generator=g, device="cuda") * 0.3
    y, post, comb = hc.mhc_pre(X, phi, gamma, alpha, beta, sinkhorn=20, eps=1e-6)
    ry, rpost, rcomb = _mhc_ref(X, phi, gamma, alpha, beta, 20, 1e-6)
    # the one-launch form (last CTA of a token runs the tail) gives the same bits, twice in a row (the tickets reset themselves)
    tickets = torch.zeros(8, dtype=torch.int32, device="cuda")
    for _ in range(2):
        y1, post1, comb1 = hc.mhc_pre(X, phi, gamma, alpha, beta, sinkhorn=20, eps=1e-6, tickets_ptr=tickets.data_ptr())
        assert torch.equal(y1, y) and torch.equal(post1, post) and torch.equal(comb1, comb)
    assert int(tickets.abs().sum()) == 0
    torch.testing.assert_close(post, rpost, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(comb, rcomb, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(comb.sum(1), torch.ones(T, S, device="cuda"), rtol=1e-3, atol=1e-3)   # doubly stochastic
    torch.testing.assert_close(y.float(), ry, rtol=1e-2, atol=1e-2)
    branch = torch.randn(T, W, generator=g, device="cuda").to(BF16)
    Y = hc.mhc_post(X, branch, post, comb)
    want = _r(rpost[:, :, None] * branch.float()[:, None, :] + torch.einsum("tki,tkw->tiw", rcomb, X.float()))
    torch.testing.assert_close(Y.float(), want, rtol=1e-2, atol=1e-2)
    # the branch norm folded into the same launch equals the stand-alone norm followed by the plain kernel, bit for bit or a rounding apart
    from ironpangu_b200.ops import decode as K

    gain = (1 + 0.1 * torch.randn(W, generator=g, device="cuda")).to(BF16)
    wide = torch.randn(T, W + 64, generator=g, device="cuda").to(BF16)[:, 32:32 + W]          # a row-strided branch
    fused = hc.mhc_post(X, wide, post, comb, norm_w=gain, eps=1e-5)
    two = hc.mhc_post(X, K.rmsnorm(wide, gain, 1e-5), post, comb)
    torch.testing.assert_close(fused.float(), two.float(), rtol=1e-2, atol=1e-2)
    assert (fused != two).float().mean() < 0.02


def test_delta_rule_matches_recurrence():
    from ironpangu_b200.ops import hc

    g = torch.Generator(device="cuda").manual_seed(2)
    H, dk, dv, steps = 3, 64, 96, 6
    state = torch.zeros(2, H, dk, dv, device="cuda")
    S = torch.zeros(H, dk, dv, device="cuda")
    slot = torch.ones(1, dtype=torch.int32, device="cuda")
    for _ in range(steps):
        q = torch.randn(1, H, dk, generator=g, device="cuda").to(BF16)
        k = torch.nn.functional.normalize(torch.randn(1, H, dk, generator=g, device="cuda"), dim=-1).to(BF16)
        v = torch.randn(1, H, dv, generator=g, device="cuda").to(BF16)
        gate = -torch.rand(1, H, generator=g, device="cuda")
        beta = torch.rand(1, H, generator=g, device="cuda")
        out = hc.delta_rule_decode(q, k, v, gate, beta, state, slot)
        S = S * torch.exp(gate[0])[:, None, None]
        r = v[0].float() - torch.einsum("hk,hkv->hv", k[0].float(), S)
        S = S + torch.einsum("hk,hv->hkv", k[0].float(), beta[0][:, None] * r)
        want = torch.einsum("hk,hkv->hv", q[0].float() / dk ** 0.5, S)
        torch.testing.assert_close(out[0].float(), _r(want), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(state[1], S, rtol=1e-4, atol=1e-4)
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("topk", [8, 64])
def test_sparse_index_selects_the_top_scores(topk):
    from ironpangu_b200.ops import hc

    g = torch.Generator(device="cuda").manual_seed(3)
    T, Hi, dim, pt, pages, ctx = 3, 6, 128, 16, 8, 100
    keys = torch.randn(pages, pt, dim, generator=g, device="cuda").to(BF16)
    q = torch.randn(T, Hi, dim, generator=g, device="cuda").to(BF16)
    w = torch.rand(T, Hi, generator=g, device="cuda")
    table = torch.tensor([[3, 0, 7, 1, 5, 2, 6, 4]], dtype=torch.int32, device="cuda")
    pos = torch.tensor([99, 5, 40], dtype=torch.int32, device="cuda")
    slots = torch.zeros(T, dtype=torch.int32, device="cuda")
    out = hc.sparse_index(q, w, keys, pos, slots, table, ctx=ctx, topk=topk)
    rows = torch.tensor([int(table[0, s // pt]) * pt + s % pt for s in range(ctx)], device="cuda")
    kk = keys.view(-1, dim)[rows].float()
    score = torch.einsum("th,ths->ts", w, torch.relu(torch.einsum("thd,sd->ths", q.float(), kk)))
    for t in range(T):
        n = int(pos[t]) + 1
        got = [i for i in out[t].tolist() if i >= 0]
        assert got == sorted(got) and len(got) == min(n, topk) and all(i < n for i in got)
        if n > topk:
            kth = score[t, :n].topk(topk).values[-1]
            assert float(score[t, got].min()) >= float(kth) - 1e-3 * abs(float(kth)) - 1e-4
