"""GPU parity of the one-launch layer kernel for windows of 1..16 rows (glmflash_moe_run / glmflash_moe_run_ep):
against the CPU oracle, against the three-launch pipeline it replaces, row independence, graph
replays, expert windows, and the cross-GPU exchange emulated on one GPU without a fault (reference probes
src/window_experts_probe.rs:66-183, src/experts.rs:284-327)."""
import os

import numpy as np
import pytest

from conftest import TOL, rel_err

pytestmark = pytest.mark.gpu

H, I, E, S = 2048, 1536, 64, 5


def _bf16_dev(x_bits, cuda):
    import torch
    return torch.from_numpy(x_bits.view(np.int16)).to(cuda).view(torch.bfloat16)


def _moe(pkg, launches=1, **kw):
    """A layer owner; launches = 1: the one-launch layer kernel, 3: gate/up + down + combine (read at construction)."""
    old = os.environ.get("GLMFLASH_LAYER_KERNELS")
    os.environ["GLMFLASH_LAYER_KERNELS"] = str(launches)
    try:
        return pkg.Moe(pkg.make_config(**kw))
    finally:
        if old is None:
            os.environ.pop("GLMFLASH_LAYER_KERNELS", None)
        else:
            os.environ["GLMFLASH_LAYER_KERNELS"] = old


@pytest.fixture(scope="module")
def banks(synth, cuda):
    b = {"benchmark": synth.expert_bank(1000, H, I, E), "scaled": synth.expert_bank(1001, H, I, E, svh_scale=True)}
    return b, {k: synth.to_device(v, cuda) for k, v in b.items()}


def _run(moe, wd, x, picks, rw, rows, cuda):
    import torch
    moe.run(wd, _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda), rows)
    torch.cuda.synchronize()
    assert int(moe.status.cpu()[0]) == 0
    return moe.output[:rows].cpu().numpy().copy()


@pytest.mark.parametrize("which", ["benchmark", "scaled"])
@pytest.mark.parametrize("rows", [1, 2, 3, 5, 8, 9, 16])
def test_one_launch_vs_three_launch_and_oracle(pkg, oracle, synth, cuda, banks, which, rows):
    host, dev = banks
    x = synth.activations_bf16(2100 + rows, rows, H)
    picks, rw = synth.route(3100 + rows, rows, E, S - 1, shared_bias=rows > 1)
    one = _moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=16)
    three = _moe(pkg, 3, hidden=H, inter=I, experts=E, slots=S, max_rows=16)
    got = _run(one, dev[which], x, picks, rw, rows, cuda)
    old = _run(three, dev[which], x, picks, rw, rows, cuda)
    assert np.isfinite(got).all()
    # the two pipelines cut K differently (128-k and 256-k splits), so they agree up to fp32 re-association and the
    # occasional bf16 rounding that flips with it: far inside the oracle tolerance
    assert rel_err(got, old)[1] < 5e-4 and rel_err(got, old)[0] < TOL, rel_err(got, old)
    import torch
    from glmflash_b200 import _view, lib
    pairs = lambda m: _view(lib().glmflash_moe_pairs(m._h), (16 * S, H), torch.float32)[: rows * S].cpu().numpy()
    assert rel_err(pairs(one), pairs(three))[1] < 5e-4
    want = oracle.combine(oracle.experts_run_rows(host[which], H, I, E + 1, S, x, picks, mode=1), rw, rows, S, H)
    emax, erms = rel_err(got, want)
    assert emax < TOL and erms < TOL, (which, rows, emax, erms)


def test_rows_of_a_window_have_the_bytes_of_their_own_call(pkg, synth, cuda, banks):
    # reference src/window_experts_probe.rs:114-135 on the whole layer: window sizes 1..16 x overlapping routing
    _, dev = banks
    x = synth.activations_bf16(61, 16, H)
    picks, rw = synth.route(62, 16, E, S - 1, shared_bias=True)
    moe = _moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=16)
    singles = np.concatenate([_run(moe, dev["benchmark"], x[r:r + 1], picks[r:r + 1], rw[r:r + 1], 1, cuda) for r in range(16)])
    for rows in (2, 3, 7, 8, 9, 15, 16):
        got = _run(moe, dev["benchmark"], x[:rows], picks[:rows], rw[:rows], rows, cuda)
        assert (got.view(np.uint32) == singles[:rows].view(np.uint32)).all(), rows


def test_graph_replays_and_back_to_back_layers(pkg, synth, cuda, banks):
    """Three different windows chained in one stream (the next kernel's CTAs start while the previous one drains), captured
    and replayed: every replay has the bytes of the eager run (counters and epochs reset themselves in the stream)."""
    import torch
    _, dev = banks
    moe = _moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=16)
    cases = []
    for k, rows in enumerate((1, 11, 4)):
        x = synth.activations_bf16(500 + k, rows, H)
        picks, rw = synth.route(510 + k, rows, E, S - 1, shared_bias=True)
        cases.append((rows, _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda),
                      _run(moe, dev["benchmark" if k != 1 else "scaled"], x, picks, rw, rows, cuda)))
    outs = [torch.empty((16, H), dtype=torch.float32, device=cuda) for _ in cases]

    def chain():
        for k, (rows, x, p, w, _) in enumerate(cases):
            moe.run(dev["benchmark" if k != 1 else "scaled"], x, p, w, rows)
            outs[k][:rows].copy_(moe.output[:rows])
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        chain()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            chain()
    for _ in range(4):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert int(moe.status.cpu()[0]) == 0
        for k, (rows, _, _, _, eager) in enumerate(cases):
            assert (outs[k][:rows].cpu().numpy().view(np.uint32) == eager.view(np.uint32)).all(), k


def test_expert_windows_sum_to_the_layer(pkg, synth, cuda, banks):
    """Two expert windows (the partials of two ranks) add up to the layer; a row whose pairs all live on the other
    rank is a row of zeros, and ids above E name nothing."""
    _, dev = banks
    rows = 6
    x = synth.activations_bf16(51, rows, H)
    picks, rw = synth.route(52, rows, E, S - 1)
    picks[2, :4] = [40, 41, 50, 63]                             # row 2: nothing in the low window
    full = _run(_moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=8), dev["scaled"], x, picks, rw, rows, cuda)
    lo = _run(_moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=8, expert_lo=0, expert_hi=32, shared_exl3=0),
              dev["scaled"], x, picks, rw, rows, cuda)
    hi = _run(_moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=8, expert_lo=32, expert_hi=64, shared_exl3=1),
              dev["scaled"], x, picks, rw, rows, cuda)
    assert (lo[2] == 0).all()
    assert rel_err(lo + hi, full)[0] < 1e-5


@pytest.mark.parametrize("launches", [3, 1])
@pytest.mark.parametrize("rows", [1, 7, 16])
def test_eight_expert_windows_sum_to_the_layer(pkg, synth, cuda, banks, launches, rows):
    """The partials of eight ranks (eight routed experts each, the shared expert on rank `rows % 8`) add up to the layer.
    A rank launches clusters for its own experts only, so its kernels must number the window's experts among ITS experts."""
    _, dev = banks
    x = synth.activations_bf16(71 + rows, rows, H)
    picks, rw = synth.route(72 + rows, rows, E, S - 1, shared_bias=rows > 1)
    full = _run(_moe(pkg, launches, hidden=H, inter=I, experts=E, slots=S, max_rows=16), dev["scaled"], x, picks, rw, rows, cuda)
    total = np.zeros_like(full)
    for r in range(8):
        part = _run(_moe(pkg, launches, hidden=H, inter=I, experts=E, slots=S, max_rows=16, expert_lo=8 * r, expert_hi=8 * r + 8,
                         shared_exl3=int(r == rows % 8)), dev["scaled"], x, picks, rw, rows, cuda)
        total += part
    assert rel_err(total, full)[0] < 1e-5


@pytest.mark.parametrize("rows", [1, 2, 7, 16])
def test_shared_expert_owner_decided_per_window(pkg, synth, cuda, banks, rows):
    """shared_exl3 = 2: of eight ranks the one whose expert window holds the fewest distinct routed experts of the window's
    routing table (ties: the lowest rank) computes the shared expert.  Exactly that rank's partial contains it, the
    partials add up to the layer, and the rank's local combine (the NCCL-baseline path) agrees with its expert kernels."""
    _, dev = banks
    x = synth.activations_bf16(171 + rows, rows, H)
    picks, rw = synth.route(172 + rows, rows, E, S - 1, shared_bias=rows > 1)
    full = _run(_moe(pkg, 3, hidden=H, inter=I, experts=E, slots=S, max_rows=16), dev["scaled"], x, picks, rw, rows, cuda)
    loads = [len({int(e) for e in picks[:, :S - 1].ravel() if 8 * r <= e < 8 * r + 8}) for r in range(8)]
    owner = min(range(8), key=lambda r: (loads[r], r))
    total = np.zeros_like(full)
    for r in range(8):
        kw = dict(hidden=H, inter=I, experts=E, slots=S, max_rows=16, expert_lo=8 * r, expert_hi=8 * r + 8)
        dyn = _run(_moe(pkg, 3, shared_exl3=2, **kw), dev["scaled"], x, picks, rw, rows, cuda)
        fixed = _run(_moe(pkg, 3, shared_exl3=int(r == owner), **kw), dev["scaled"], x, picks, rw, rows, cuda)
        assert (dyn.view(np.uint32) == fixed.view(np.uint32)).all(), (r, owner, loads)
        total += dyn
    assert rel_err(total, full)[0] < 1e-5


def test_exchange_with_the_owner_decided_per_window_on_one_gpu(pkg, synth, cuda, banks):
    """The three-launch pipeline + the flag-in-data exchange with shared_here = 2, two ranks emulated on one GPU as in the
    test below: the expert kernels and the exchange kernel of a rank take the same decision, so the sum is the layer."""
    import torch
    _, dev = banks
    for rows in (1, 6, 16):
        x = synth.activations_bf16(191 + rows, rows, H)
        picks, rw = synth.route(192 + rows, rows, E, S - 1, shared_bias=rows > 1)
        full = _run(_moe(pkg, 3, hidden=H, inter=I, experts=E, slots=S, max_rows=16), dev["scaled"], x, picks, rw, rows, cuda)
        kw = lambda r: dict(hidden=H, inter=I, experts=E, slots=S, max_rows=16, expert_lo=r * 32, expert_hi=(r + 1) * 32, shared_exl3=2)
        moes = [_moe(pkg, 3, **kw(r)) for r in (0, 1)]
        eps = [pkg.EpCombine(pkg.make_config(**kw(r)), r, 2, None) for r in (0, 1)]
        for e_ in eps:
            e_.connect_ptrs([q.local_base for q in eps])
        xd, pd, wd = _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda)
        eps[1].set_wait_limit(20000)
        moes[1].run_ep(eps[1], dev["scaled"], xd, pd, wd, rows, shared_here=2)
        torch.cuda.synchronize()
        assert int(eps[1].status.cpu()[0]) == 4                 # rank 1 gave up waiting for rank 0: nothing hung
        got = moes[0].run_ep(eps[0], dev["scaled"], xd, pd, wd, rows)          # -1: as the layer owner's config says (2)
        torch.cuda.synchronize()
        assert int(eps[0].status.cpu()[0]) == 0 and int(moes[0].status.cpu()[0]) == 0 and int(moes[1].status.cpu()[0]) == 0
        assert rel_err(got.cpu().numpy(), full)[0] < 1e-5, rows
        with pytest.raises(RuntimeError, match="decided per window"):
            moes[0].run_ep(eps[0], dev["scaled"], xd, pd, wd, rows, shared_here=1)


def test_small_and_odd_shapes_vs_oracle(pkg, oracle, synth, cuda):
    """Shapes other than the benchmark's: one split per projection, and a hidden size (2304) that is not a power of
    two times 256 (nine splits in the layer kernel, 6 x 24 k-tiles in the table-driven kernels)."""
    import torch
    for (h, i, e, s, rows) in ((512, 256, 4, 3, 2), (2304, 512, 6, 4, 5), (256, 256, 3, 3, 16)):
        bank = synth.expert_bank(77, h, i, e, svh_scale=True)
        wd = synth.to_device(bank, cuda)
        x = synth.activations_bf16(78, rows, h)
        picks, rw = synth.route(79, rows, e, s - 1)
        want_y = oracle.experts_run_rows(bank, h, i, e + 1, s, x, picks, mode=1)
        want = oracle.combine(want_y, rw, rows, s, h)
        got = _run(_moe(pkg, 1, hidden=h, inter=i, experts=e, slots=s, max_rows=16), wd, x, picks, rw, rows, cuda)
        emax, erms = rel_err(got, want)
        assert emax < TOL and erms < TOL, (h, i, emax, erms)
        # the table-driven surface (ExpertGpu::run_rows) on the same shape
        ex = pkg.ExpertGpu(pkg.make_config(h, i, e, s, max_rows=16))
        ids, count, members = oracle.grouping(picks, rows, s, e + 1, 16)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
        ex.run_rows(wd, _bf16_dev(x, cuda), t(picks), t(ids), t(np.array([count], np.int32)), t(members), rows, 16)
        torch.cuda.synchronize()
        assert int(ex.status.cpu()[0]) == 0
        emax, erms = rel_err(ex.y[: rows * s].cpu().numpy(), want_y)
        assert emax < TOL and erms < TOL, ("run_rows", h, i, emax, erms)


def test_exchange_of_two_ranks_on_one_gpu(pkg, synth, cuda, banks):
    """The fused exchange without a second GPU and without a fault: two layer owners (expert windows of ranks 0 and 1) and
    two exchange owners live on ONE GPU, connected by pointers.  Rank 1 runs first with a short wait limit: it pushes its
    blocks into both receive areas, its own wait for rank 0 runs out (status PEER_TIMEOUT, context intact).  Rank 0 then
    finds rank 1's blocks already there and finishes: its output is the rank-ordered sum = the layer."""
    import torch
    _, dev = banks
    rows = 5
    x = synth.activations_bf16(91, rows, H)
    picks, rw = synth.route(92, rows, E, S - 1, shared_bias=True)
    full = _run(_moe(pkg, 1, hidden=H, inter=I, experts=E, slots=S, max_rows=16), dev["scaled"], x, picks, rw, rows, cuda)
    kw = lambda r: dict(hidden=H, inter=I, experts=E, slots=S, max_rows=16, expert_lo=r * 32, expert_hi=(r + 1) * 32, shared_exl3=0)
    moes = [_moe(pkg, 1, **kw(r)) for r in (0, 1)]
    eps = [pkg.EpCombine(pkg.make_config(**kw(r)), r, 2, None) for r in (0, 1)]
    for e_ in eps:
        e_.connect_ptrs([q.local_base for q in eps])
    xd, pd, wd = _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda)
    for step in range(3):                                       # three exchanges: the receive buffers alternate
        eps[1].set_wait_limit(20000)
        eps[0].set_wait_limit(2000000)
        moes[1].run_ep(eps[1], dev["scaled"], xd, pd, wd, rows, shared_here=step % 2)
        torch.cuda.synchronize()
        assert int(eps[1].status.cpu()[0]) == 4                 # rank 1 gave up waiting for rank 0: nothing hung
        eps[1].clear_status()
        got = moes[0].run_ep(eps[0], dev["scaled"], xd, pd, wd, rows, shared_here=1 - step % 2)
        torch.cuda.synchronize()
        assert int(eps[0].status.cpu()[0]) == 0 and int(moes[0].status.cpu()[0]) == 0 and int(moes[1].status.cpu()[0]) == 0
        assert rel_err(got.cpu().numpy(), full)[0] < 1e-5, step
