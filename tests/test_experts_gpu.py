"""GPU parity of the decode / verify expert path (ExpertGpu, Moe) through the C ABI: against the CPU oracle,
against the upstream kernels compiled unmodified, row independence and graph replay (reference probes
src/experts.rs:284-327, src/window_experts_probe.rs:66-183)."""
import numpy as np
import pytest

from conftest import TOL, rel_err

pytestmark = pytest.mark.gpu

H, I, E, S = 2048, 1536, 64, 5


def _bf16_dev(x_bits, cuda):
    import torch
    return torch.from_numpy(x_bits.view(np.int16)).to(cuda).view(torch.bfloat16)


@pytest.fixture(scope="module")
def bank(synth):
    return synth.expert_bank(1000, H, I, E)                 # the benchmark's distribution (SwiGLU mostly clamped)


@pytest.fixture(scope="module")
def bank_scaled(synth):
    return synth.expert_bank(1001, H, I, E, svh_scale=True)  # unit-variance pre-activations: nothing saturates


@pytest.fixture(scope="module")
def dbank(bank, synth, cuda):
    return synth.to_device(bank, cuda)


@pytest.fixture(scope="module")
def dbank_scaled(bank_scaled, synth, cuda):
    return synth.to_device(bank_scaled, cuda)


def run_experts(pkg, oracle, cuda, wd, x_bits, picks, rows, max_rows, **cfg_kw):
    import torch
    cfg = pkg.make_config(H, I, E, S, max_rows=max_rows, **cfg_kw)
    ex = pkg.ExpertGpu(cfg)
    ids, count, members = oracle.grouping(picks, rows, S, E + 1, max_rows)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    ex.y.fill_(float("nan"))
    ex.run_rows(wd, _bf16_dev(x_bits, cuda), t(picks), t(ids), t(np.array([count], np.int32)), t(members), rows, max_rows)
    torch.cuda.synchronize()
    assert int(ex.status.cpu()[0]) == 0
    return ex.y[: rows * S].cpu().numpy().copy(), ex.xd[: rows * S].cpu().numpy().copy(), ex


@pytest.mark.parametrize("which", ["benchmark", "scaled"])
@pytest.mark.parametrize("rows,bias", [(1, False), (8, True), (16, True)])
def test_experts_vs_oracle(pkg, oracle, synth, cuda, bank, bank_scaled, dbank, dbank_scaled, which, rows, bias):
    # configs 2 and 3: 1 token; 8 and 16 tokens with a shared router bias (about half the experts overlap)
    b, wd = (bank, dbank) if which == "benchmark" else (bank_scaled, dbank_scaled)
    x = synth.activations_bf16(2000 + rows, rows, H)
    picks, _ = synth.route(3000 + rows, rows, E, S - 1, shared_bias=bias)
    y, xd, _ = run_experts(pkg, oracle, cuda, wd, x, picks, rows, max(rows, 1))
    want, want_xd = oracle.experts_run_rows(b, H, I, E + 1, S, x, picks, mode=1, want_xd=True)
    assert np.isfinite(y).all()
    emax, erms = rel_err(y, want)
    assert emax < TOL and erms < TOL, (which, rows, emax, erms)
    assert rel_err(xd.astype(np.float32), want_xd)[1] < 2e-3       # fp16-rounded intermediate (1 ulp = 1e-3)


def test_upstream_skip_shared(pkg, oracle, synth, cuda, bank, dbank):
    # shared_exl3 = 0 reproduces upstream: ids >= E are not computed and their Y rows stay untouched
    rows = 3
    x = synth.activations_bf16(41, rows, H)
    picks, _ = synth.route(42, rows, E, S - 1)
    y, _, _ = run_experts(pkg, oracle, cuda, dbank, x, picks, rows, 4, shared_exl3=0)
    y = y.reshape(rows, S, H)
    assert np.isnan(y[:, S - 1]).all() and np.isfinite(y[:, : S - 1]).all()
    want = oracle.experts_run_rows(bank, H, I, E + 1, S, x, picks, skip_ge=E, mode=1).reshape(rows, S, H)
    assert rel_err(y[:, : S - 1], want[:, : S - 1])[0] < TOL


def test_expert_window(pkg, oracle, synth, cuda, bank, dbank):
    # expert-parallel window: only routed ids in [lo, hi) are computed (the shared expert follows shared_exl3);
    # the union of two windows is the whole result
    rows = 5
    x = synth.activations_bf16(51, rows, H)
    picks, _ = synth.route(52, rows, E, S - 1)
    full, _, _ = run_experts(pkg, oracle, cuda, dbank, x, picks, rows, 8)
    lo, _, _ = run_experts(pkg, oracle, cuda, dbank, x, picks, rows, 8, expert_lo=0, expert_hi=32, shared_exl3=0)
    hi, _, _ = run_experts(pkg, oracle, cuda, dbank, x, picks, rows, 8, expert_lo=32, expert_hi=64, shared_exl3=1)
    in_lo = np.repeat((picks.reshape(-1) < 32)[:, None], H, 1)
    assert np.isnan(lo[~in_lo]).all() and np.isnan(hi[in_lo]).all()
    merged = np.where(in_lo, lo, hi)
    assert (merged.view(np.uint32) == full.view(np.uint32)).all()


@pytest.mark.parametrize("pattern", ["identical", "partial", "disjoint"])
def test_row_independence(pkg, oracle, synth, cuda, dbank, pattern):
    # reference src/window_experts_probe.rs:66-135: every row of a window has the bytes of its 1-row call
    import torch
    x = synth.activations_bf16(61, 16, H)
    base, _ = synth.route(62, 16, E, S - 1)
    if pattern == "identical":
        picks_all = np.repeat(base[:1], 16, 0)
    elif pattern == "partial":
        picks_all = base.copy()
        picks_all[:, :2] = base[0, :2]                     # two experts shared by every row
        for r in range(16):                                # keep the routed ids of a row distinct
            used = set(picks_all[r, :2])
            k = 0
            for s in range(2, S - 1):
                while (r * 3 + k + 2) % E in used:
                    k += 1
                picks_all[r, s] = (r * 3 + k + 2) % E
                used.add(picks_all[r, s])
    else:
        picks_all = np.stack([np.concatenate([(np.arange(S - 1) + r * (S - 1)) % E, [E]]) for r in range(16)]).astype(np.int32)
    singles = []
    for r in range(16):
        y, _, _ = run_experts(pkg, oracle, cuda, dbank, x[r:r + 1], picks_all[r:r + 1], 1, 1)
        singles.append(y)
    singles = np.concatenate(singles)
    for rows in (1, 2, 3, 7, 8, 9, 15, 16):
        y, _, _ = run_experts(pkg, oracle, cuda, dbank, x[:rows], picks_all[:rows], rows, 16)
        assert (y.view(np.uint32) == singles[: rows * S].view(np.uint32)).all(), (pattern, rows)


def test_graph_replay_is_byte_equal(pkg, oracle, synth, cuda, dbank):
    # reference src/experts.rs:309-316: captured graph == eager, replay after replay (tickets reset in-stream)
    import torch
    rows = 9
    x = synth.activations_bf16(71, rows, H)
    picks, _ = synth.route(72, rows, E, S - 1, shared_bias=True)
    eager, _, ex = run_experts(pkg, oracle, cuda, dbank, x, picks, rows, 16)
    ids, count, members = oracle.grouping(picks, rows, S, E + 1, 16)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    args = (dbank, _bf16_dev(x, cuda), t(picks), t(ids), t(np.array([count], np.int32)), t(members), rows, 16)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ex.run_rows(*args)                                  # warm-up on the capture stream
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ex.run_rows(*args)
    for _ in range(5):
        ex.y.fill_(0)
        graph.replay()
        torch.cuda.synchronize()
        assert (ex.y[: rows * S].cpu().numpy().view(np.uint32) == eager.view(np.uint32)).all()


def test_pdl_chain_equals_plain_launches(pkg, oracle, synth, cuda, dbank):
    """Programmatic dependent launch only moves prologues earlier: bytes are those of plain launches, also when the
    layer is replayed back to back (the next layer's grouping overlaps this layer's combine)."""
    import torch
    rows = 7
    outs = {}
    for pdl in (0, 1):
        moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=8, pdl=pdl))
        res = []
        for it in range(3):
            x = synth.activations_bf16(400 + it, rows, H)
            picks, rw = synth.route(410 + it, rows, E, S - 1, shared_bias=True)
            args = (dbank, _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda), rows)
            for _ in range(3):                                  # back to back: kernels of consecutive runs overlap
                moe.run(*args)
            torch.cuda.synchronize()
            res.append(moe.output[:rows].cpu().numpy().copy())
        outs[pdl] = np.stack(res)
    assert np.isfinite(outs[1]).all()
    assert (outs[0].view(np.uint32) == outs[1].view(np.uint32)).all()


def test_vs_upstream_kernels(pkg, oracle, synth, cuda, bank_scaled, dbank_scaled):
    """The upstream CUDA kernels, compiled unmodified for sm_100a, on the same tensors: Xd and Y agree within
    the tolerance, and the oracle agrees with upstream's GPU result (this pins the oracle to the reference)."""
    import os, sys, torch
    from conftest import ROOT
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_gpu
    if not ref_gpu.available():
        pytest.skip("upstream cubins not built")
    rows = 6
    x = synth.activations_bf16(81, rows, H)
    picks, _ = synth.route(82, rows, E, S - 1, shared_bias=True)
    y, xd, _ = run_experts(pkg, oracle, cuda, dbank_scaled, x, picks, rows, 8)
    # upstream skips the last slot of a row: give it one extra unused slot so that the shared expert is computed
    S6 = S + 1
    picks6 = np.concatenate([picks, np.full((rows, 1), E + 1, np.int32)], 1)
    ids, count, members = oracle.grouping(picks, rows, S, E + 1, 16)      # member codes row*32+slot are slot-count free
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    for grouped in ("exl3_grouped_8_4", "exl3_load_nc_8_1"):
        ry, rxd = ref_gpu.experts_run_rows(dbank_scaled, _bf16_dev(x, cuda), t(picks6), t(ids), t(np.array([count], np.int32)),
                                           t(members), rows, 16, H, I, E + 1, S6, grouped=grouped)
        torch.cuda.synchronize()
        ry = ry.cpu().numpy().reshape(rows, S6, H)[:, :S].reshape(rows * S, H)
        rxd = rxd.cpu().numpy().reshape(rows, S6, I)[:, :S].reshape(rows * S, I)
        emax, erms = rel_err(y, ry)
        assert emax < TOL and erms < TOL, (grouped, emax, erms)
        assert rel_err(xd.astype(np.float32), rxd.astype(np.float32))[1] < 2e-3
    want = oracle.experts_run_rows(bank_scaled, H, I, E + 1, S, x, picks, mode=0, sk_gu=4, sk_dn=1)
    assert rel_err(ry, want)[1] < TOL          # upstream's own gate: relative RMS < 1e-3 (src/experts.rs:304-308)


@pytest.mark.parametrize("rows", [1, 4, 16])
def test_moe_layer(pkg, oracle, synth, cuda, bank_scaled, dbank_scaled, rows):
    import torch
    x = synth.activations_bf16(91, rows, H)
    picks, rw = synth.route(92, rows, E, S - 1, shared_bias=rows > 1)
    moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=16))
    moe.run(dbank_scaled, _bf16_dev(x, cuda), torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda), rows)
    torch.cuda.synchronize()
    got = moe.output[:rows].cpu().numpy()
    want = oracle.combine(oracle.experts_run_rows(bank_scaled, H, I, E + 1, S, x, picks, mode=1), rw, rows, S, H)
    emax, erms = rel_err(got, want)
    assert emax < TOL and erms < TOL, (emax, erms)
    # host-buffer entry point: pinned in, pinned out
    xh = torch.from_numpy(x.view(np.int16)).pin_memory()
    ph, wh = torch.from_numpy(picks).pin_memory(), torch.from_numpy(rw).pin_memory()
    oh = torch.empty((rows, H), dtype=torch.float32).pin_memory()
    moe.run_host(dbank_scaled, xh, ph, wh, rows, oh)
    assert (oh.numpy().view(np.uint32) == got.view(np.uint32)).all()
