"""Router kernels next to the expert path (logits matvec, sigmoid top-k) against the oracle's restatement of the
benchmark's router definition.  The reference's own router kernels are binaries without source: parity with them is
not pinned; what is pinned here is the definition (top-k by score, ties to the lower id, renormalised weights)."""
import numpy as np
import pytest

from conftest import TOL

pytestmark = pytest.mark.gpu

H, I, E, S = 2048, 1536, 64, 5


@pytest.mark.parametrize("rows,experts,k", [(1, 64, 4), (16, 64, 4), (300, 65, 4), (4096, 64, 4), (7, 288, 8), (3, 5, 5)])
def test_topk_equals_oracle(pkg, oracle, cuda, rows, experts, k):
    import torch
    g = np.random.default_rng(1234 + rows)
    logits = g.standard_normal((rows, experts)).astype(np.float32)
    if rows >= 7:
        logits[1, :] = 0.25                        # all tied: the lowest ids win, in ascending order
        logits[2, 3] = logits[2, 40 % experts] = 9.0   # a tie at the top
        logits[3, :] = np.float32(-50.0)           # scores underflow towards 0: the weights stay finite and sum to 1
    want_p, want_w = oracle.topk(logits, rows, experts, k)
    ld = torch.from_numpy(logits).to(cuda)
    picks = torch.full((rows, k + 1), -7, dtype=torch.int32, device=cuda)
    weights = torch.zeros((rows, k + 1), dtype=torch.float32, device=cuda)
    pkg.topk(ld, picks, weights, pdl=0)
    torch.cuda.synchronize()
    assert np.array_equal(picks.cpu().numpy(), want_p)
    got_w = weights.cpu().numpy()
    assert np.allclose(got_w, want_w, rtol=2e-6, atol=1e-7)
    assert np.allclose(got_w[:, :k].sum(1), 1.0, atol=1e-5) and (got_w[:, k] == 1.0).all()


@pytest.mark.parametrize("rows,experts", [(1, 64), (16, 64), (513, 65)])
def test_router_logits(pkg, oracle, synth, cuda, rows, experts):
    import torch
    x = synth.activations_bf16(77, rows, H)                                   # uint16 bit patterns
    g = np.random.default_rng(5)
    wr = torch.from_numpy((g.standard_normal((experts, H)) / np.sqrt(H)).astype(np.float32)).to(torch.bfloat16)
    wr_bits = wr.view(torch.int16).numpy().view(np.uint16)
    want = oracle.router_logits(x, wr_bits, rows, H, experts)
    xd = torch.from_numpy(x.view(np.int16)).to(cuda).view(torch.bfloat16)
    logits = torch.empty((rows, experts), dtype=torch.float32, device=cuda)
    pkg.router_logits(xd, wr.to(cuda), logits, pdl=0)
    torch.cuda.synchronize()
    got = logits.cpu().numpy()
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())    # fp32 accumulation against double


def test_router_feeds_the_layer(pkg, oracle, synth, cuda):
    """router -> top-k -> Moe on the device, chained with programmatic dependent launch, equals the layer run on the
    table the oracle derives from the same logits."""
    import torch
    rows = 8
    bank = synth.device_bank(901, H, I, E, cuda)
    x = synth.activations_bf16(902, rows, H)
    xd = torch.from_numpy(x.view(np.int16)).to(cuda).view(torch.bfloat16)
    gen = torch.Generator(device=cuda).manual_seed(3)
    wr = (torch.randn((E, H), generator=gen, device=cuda) / H ** 0.5).to(torch.bfloat16)
    logits = torch.empty((rows, E), dtype=torch.float32, device=cuda)
    picks = torch.empty((rows, S), dtype=torch.int32, device=cuda)
    weights = torch.empty((rows, S), dtype=torch.float32, device=cuda)
    moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=16))
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        pkg.route(xd, wr, logits, picks, weights, stream=st)          # one launch (<= 16 rows)
        moe.run(bank, xd, picks, weights, rows, stream=st)
    st.synchronize()
    # the one-launch form and the two kernels give the same logits bits, hence the same table
    l2, p2, w2 = torch.empty_like(logits), torch.empty_like(picks), torch.empty_like(weights)
    pkg.router_logits(xd, wr, l2, pdl=0)
    pkg.topk(l2, p2, w2, pdl=0)
    torch.cuda.synchronize()
    assert torch.equal(l2, logits) and torch.equal(p2, picks) and torch.equal(w2, weights)
    got = moe.output[:rows].clone()
    want_p, want_w = oracle.topk(logits.cpu().numpy(), rows, E, S - 1)
    assert np.array_equal(picks.cpu().numpy(), want_p)
    moe2 = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=16, pdl=0))
    moe2.run(bank, xd, torch.from_numpy(want_p).to(cuda), torch.from_numpy(want_w).to(cuda), rows)
    torch.cuda.synchronize()
    ref = moe2.output[:rows]
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6 * float(ref.abs().max()))
