"""GPU parity of the prefill path (FastExperts: tcgen05 grouped GEMM) through the C ABI: against the CPU oracle,
against the upstream kernels compiled unmodified, row independence, shared vs separate rotation, graph replay
(reference probe src/fast_experts.rs:217-423)."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, TOL, rel_err

pytestmark = pytest.mark.gpu

H, I, E, S = 2048, 1536, 64, 5


def _bf16_dev(x_bits, cuda):
    import torch
    return torch.from_numpy(x_bits.view(np.int16)).to(cuda).view(torch.bfloat16)


@pytest.fixture(scope="module")
def bank(synth):
    return synth.expert_bank(1001, H, I, E, svh_scale=True)      # unit-variance pre-activations: nothing saturates


@pytest.fixture(scope="module")
def dbank(bank, synth, cuda):
    return synth.to_device(bank, cuda)


@pytest.fixture(scope="module")
def bank_bench(synth):
    return synth.expert_bank(1000, H, I, E)                      # the benchmark's distribution (SwiGLU mostly clamped)


@pytest.fixture(scope="module")
def dbank_bench(bank_bench, synth, cuda):
    return synth.to_device(bank_bench, cuda)


def probe_picks(rows, spread=16):
    # the reference probe's routing (src/fast_experts.rs:255-266): experts (r*7 + slot) % 16, shared last
    return np.array([[(r * 7 + s) % spread for s in range(S - 1)] + [E] for r in range(rows)], dtype=np.int32)


def run_fast(pkg, oracle, cuda, wd, x_bits, picks, rows, max_rows, shared_x=False, fe=None, **cfg_kw):
    import torch
    if fe is None:
        fe = pkg.FastExperts(pkg.make_config(H, I, E, S, max_rows=max_rows, **cfg_kw))
    ids, count, members = oracle.grouping(picks, rows, S, E + 1, max_rows)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    fe.output.fill_(float("nan"))
    args = (wd, _bf16_dev(x_bits, cuda), t(picks), t(ids), t(np.array([count], np.int32)), t(members), rows, max_rows)
    fe.run(*args, shared_x=shared_x)
    torch.cuda.synchronize()
    assert int(fe.status.cpu()[0]) == 0, "a bounded wait inside the kernel gave up"
    return fe.output[: rows * S].cpu().numpy().copy(), fe, args


# the reference probe's row counts and member strides (src/fast_experts.rs:247-254), a mid-size chunk, and the owner's
# largest capacity (src/fast_experts.rs:44-47), on both scale distributions
@pytest.mark.parametrize("which", ["scaled", "benchmark"])
@pytest.mark.parametrize("rows,max_rows", [(1, 129), (63, 129), (64, 129), (65, 129), (129, 129), (300, 512), (4097, 4097), (500, 8192)])
def test_fast_vs_oracle(pkg, oracle, synth, cuda, bank, dbank, bank_bench, dbank_bench, rows, max_rows, which):
    if which == "benchmark":
        bank, dbank = bank_bench, dbank_bench
    x = synth.activations_bf16(100 + rows, rows, H)
    picks = probe_picks(rows)
    y, fe, _ = run_fast(pkg, oracle, cuda, dbank, x, picks, rows, max_rows)
    assert np.isfinite(y).all()
    # the oracle on a bounded sample of rows (every expert of the sample is unpacked once)
    sample = sorted(set([0, rows - 1, rows // 2] + list(np.random.default_rng(rows).integers(0, rows, 3))))
    want = oracle.experts_run_rows(bank, H, I, E + 1, S, x[sample], picks[sample], mode=1)
    got = y.reshape(rows, S, H)[sample].reshape(-1, H)
    emax, erms = rel_err(got, want)
    assert emax < TOL and erms < TOL, (rows, emax, erms)
    # grouped intermediate: plan counts and the pair map are a permutation of the pairs
    plan = fe.plan.cpu().numpy()
    assert plan[1] == rows * S
    assert sorted(fe.row_pairs[: rows * S].cpu().numpy().tolist()) == list(range(rows * S))


def test_fast_matches_decode_path_and_upstream(pkg, oracle, synth, cuda, bank, dbank):
    """129 rows: the prefill result agrees with this library's decode path (row by row), and with upstream's
    prefill kernels and upstream's decode kernels, all within the tolerance."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_gpu
    rows, max_rows = 129, 129
    x = synth.activations_bf16(777, rows, H)
    picks = probe_picks(rows)
    y, fe, _ = run_fast(pkg, oracle, cuda, dbank, x, picks, rows, max_rows)
    # decode path, 16 rows at a time
    ex = pkg.ExpertGpu(pkg.make_config(H, I, E, S, max_rows=16))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    for r0 in range(0, 32, 16):
        n = 16
        ids, count, members = oracle.grouping(picks[r0:r0 + n], n, S, E + 1, 16)
        ex.run_rows(dbank, _bf16_dev(x[r0:r0 + n], cuda), t(picks[r0:r0 + n]), t(ids), t(np.array([count], np.int32)), t(members), n, 16)
        torch.cuda.synchronize()
        yd = ex.y[: n * S].cpu().numpy()
        assert rel_err(y[r0 * S:(r0 + n) * S], yd)[0] < TOL
    if not ref_gpu.available():
        pytest.skip("upstream cubins not built")
    S6 = S + 1
    picks6 = np.concatenate([picks, np.full((rows, 1), E + 1, np.int32)], 1)
    ids, count, members = oracle.grouping(picks, rows, S, E + 1, max_rows)
    for shared_x in (False,):
        ry, _ = ref_gpu.fast_experts_run(dbank, _bf16_dev(x, cuda), t(picks6), t(ids), t(np.array([count], np.int32)), t(members),
                                         rows, max_rows, H, I, E + 1, S6, shared_x=shared_x)
        torch.cuda.synchronize()
        ry = ry.cpu().numpy().reshape(rows, S6, H)[:, :S].reshape(rows * S, H)
        emax, erms = rel_err(y, ry)
        assert emax < TOL and erms < TOL, ("upstream prefill", emax, erms)


def test_fast_row_independence_and_replay(pkg, oracle, synth, cuda, dbank):
    """A row's bytes do not depend on the rows it shares a chunk with; shared_x == separate when suh_g == suh_u;
    graph replays are byte-equal (reference src/fast_experts.rs:366-412)."""
    import torch
    rows = 200
    x = synth.activations_bf16(555, rows, H)
    picks = probe_picks(rows)
    full, fe, args = run_fast(pkg, oracle, cuda, dbank, x, picks, rows, 256)
    part, _, _ = run_fast(pkg, oracle, cuda, dbank, x[:70], picks[:70], 70, 256, fe=fe)
    assert (part.view(np.uint32) == full[: 70 * S].view(np.uint32)).all()
    # same rotation vector for gate and up: one rotated copy must give the bytes of two
    wd2 = dict(dbank)
    wd2["suh_u"] = wd2["suh_g"]
    sep, _, args2 = run_fast(pkg, oracle, cuda, wd2, x, picks, rows, 256, shared_x=False, fe=fe)
    shr, _, _ = run_fast(pkg, oracle, cuda, wd2, x, picks, rows, 256, shared_x=True, fe=fe)
    assert (sep.view(np.uint32) == shr.view(np.uint32)).all()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fe.run(*args)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fe.run(*args)
    for _ in range(3):
        fe.output.fill_(0)
        graph.replay()
        torch.cuda.synchronize()
        assert (fe.output[: rows * S].cpu().numpy().view(np.uint32) == full.view(np.uint32)).all()


@pytest.mark.parametrize("which", ["scaled", "benchmark"])
def test_prefill_config4_vs_upstream(pkg, oracle, synth, cuda, bank, dbank, bank_bench, dbank_bench, which):
    """Benchmark config 4: 4096 tokens, uniform random top-4 routing (about 256 tokens per expert)."""
    import torch
    if which == "benchmark":
        bank, dbank = bank_bench, dbank_bench
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_gpu
    rows = 4096
    x = synth.activations_bf16(4096, rows, H)
    picks, rw = synth.route(4097, rows, E, S - 1, uniform=True)
    y, fe, _ = run_fast(pkg, oracle, cuda, dbank, x, picks, rows, rows)
    assert np.isfinite(y).all()
    sample = [0, 1, 2047, 4095]
    want = oracle.experts_run_rows(bank, H, I, E + 1, S, x[sample], picks[sample], mode=1)
    got = y.reshape(rows, S, H)[sample].reshape(-1, H)
    emax, erms = rel_err(got, want)
    assert emax < TOL and erms < TOL, (emax, erms)
    if ref_gpu.available():
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
        S6 = S + 1
        picks6 = np.concatenate([picks, np.full((rows, 1), E + 1, np.int32)], 1)
        ids, count, members = oracle.grouping(picks, rows, S, E + 1, rows)
        ry, _ = ref_gpu.fast_experts_run(dbank, _bf16_dev(x, cuda), t(picks6), t(ids), t(np.array([count], np.int32)), t(members),
                                         rows, rows, H, I, E + 1, S6)
        torch.cuda.synchronize()
        ry = ry.cpu().numpy().reshape(rows, S6, H)[:, :S].reshape(rows * S, H)
        emax, erms = rel_err(y, ry)
        assert emax < TOL and erms < TOL, ("upstream prefill", emax, erms)
    # the whole layer through Moe (grouping -> prefill experts -> combine)
    moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=rows))
    moe.run(dbank, _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda), rows)
    torch.cuda.synchronize()
    out = moe.output[:rows].cpu().numpy()
    want_out = oracle.combine(y, rw, rows, S, H)
    assert rel_err(out, want_out)[0] < 1e-5


def test_shared_expert_row_window(pkg, synth, cuda, dbank):
    """Expert-parallel prefill splits the shared expert by rows: a handle with shared_rows = (lo, hi) computes the shared
    pair only for window rows in [lo, hi); every other pair is untouched.  Checked against the layer without a row
    window: out_window[r] = out_full[r] - Y_shared[r] outside the window (same fp32 order: the shared pair is the last
    term of the sum), identical inside."""
    import torch
    rows, lo, hi = 300, 100, 171
    x = _bf16_dev(synth.activations_bf16(41, rows, H), cuda)
    picks, rw = synth.route(42, rows, E, S - 1, uniform=True)
    pd, wd = torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda)
    full = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=rows))
    full.run(dbank, x, pd, wd, rows)
    torch.cuda.synchronize()
    pairs = pkg._view(full.pairs_ptr.value, (rows, S, H), torch.float32).clone()
    out_full = full.output[:rows].clone()
    win = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=rows, shared_rows=(lo, hi)))
    for _ in range(2):
        win.run(dbank, x, pd, wd, rows)
    torch.cuda.synchronize()
    got = win.output[:rows]
    inside = torch.zeros(rows, dtype=torch.bool, device=cuda)
    inside[lo:hi] = True
    assert torch.equal(got[inside], out_full[inside])
    routed_only = out_full - pairs[:, S - 1, :]                 # not bit-exact: (a + s) - s; compare with a tolerance
    assert torch.allclose(got[~inside], routed_only[~inside], rtol=1e-5, atol=1e-5 * float(out_full.abs().max()))
    # exact form: routed-only sum in the combine's order
    want = torch.zeros((rows, H), dtype=torch.float32, device=cuda)
    for s in range(S - 1):
        want = torch.addcmul(want, wd[:, s, None], pairs[:, s, :])
    assert torch.allclose(got[~inside], want[~inside], rtol=2e-6, atol=1e-6 * float(out_full.abs().max()))
    with pytest.raises(pkg.GlmFlashError):
        pkg.Moe(pkg.make_config(H, I, E, S, max_rows=16, shared_rows=(0, 8)))   # only handles for more than 16 rows
