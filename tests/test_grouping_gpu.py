"""GPU grouping against the host-built expectation (reference probe src/grouping.rs:123-215): capacities
8192 and 16, the probe's row counts, concentrated and spread routing, poisoned outputs, graph replays."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def probe_picks(rows, E, slots, concentrated, seed):
    # the probe's generator: xorshift start, experts (start + slot*37) % E, shared last
    p = np.empty((rows, slots), np.int32)
    for r in range(rows):
        seed ^= (seed << 13) & 0xFFFFFFFFFFFFFFFF
        seed ^= seed >> 7
        seed ^= (seed << 17) & 0xFFFFFFFFFFFFFFFF
        start = 0 if concentrated else seed % E
        for s in range(slots - 1):
            p[r, s] = (start + s * 37) % E
        p[r, slots - 1] = E
    return p, seed


@pytest.mark.parametrize("E,slots", [(288, 9), (64, 5)])
@pytest.mark.parametrize("capacity,row_counts", [(8192, [8192, 1, 2, 31, 32, 33, 63, 64, 65, 129, 1024, 4097, 8191]),
                                                 (16, [1, 2, 3, 8, 15, 16])])
def test_grouping_matches_host(pkg, oracle, cuda, E, slots, capacity, row_counts):
    import torch
    cfg = pkg.make_config(experts=E, slots=slots, max_rows=capacity)
    g = pkg.Grouping(cfg)
    seed = 0x0123456789ABCDEF
    for rows in row_counts:
        for concentrated in (True, False):
            picks, seed = probe_picks(rows, E, slots, concentrated, seed)
            ids, count, members = oracle.grouping(picks, rows, slots, E + 1, capacity)
            pd = torch.from_numpy(picks).to(cuda)
            g.ids.fill_(-77)                       # poison: stale ids / counts / tails must not survive
            g.members.fill_(12345)
            g.run(pd, rows)
            torch.cuda.synchronize()

            def check():
                assert int(g.count.cpu()[0]) == count
                assert (g.ids[:count].cpu().numpy() == ids[:count]).all(), "stable expert order"
                assert (g.members.cpu().numpy() == members).all(), f"member order or stale tail at {rows}"
            check()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g.run(pd, rows)
            for _ in range(3):
                g.members.fill_(777)
                graph.replay()
                torch.cuda.synchronize()
                check()


def test_grouping_matches_upstream_kernels(pkg, cuda):
    """Same picks through the upstream grouping kernels (compiled unmodified) and through this library."""
    import sys, os
    from conftest import ROOT
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_gpu
    if not ref_gpu.available():
        pytest.skip("upstream cubins not built")
    import torch
    E, slots = 288, 9
    seed = 0xABCDEF
    for capacity, rows in [(16, 1), (16, 16), (32, 32), (8192, 33), (8192, 4097)]:
        g = pkg.Grouping(pkg.make_config(experts=E, slots=slots, max_rows=capacity))
        picks, seed = probe_picks(rows, E, slots, False, seed)
        pd = torch.from_numpy(picks).to(cuda)
        g.run(pd, rows)
        rid, rcount, rmem = ref_gpu.grouping_run(pd, rows, capacity)
        torch.cuda.synchronize()
        n = int(rcount.cpu()[0])
        assert int(g.count.cpu()[0]) == n
        assert torch.equal(g.ids[:n], rid[:n]) and torch.equal(g.members, rmem)
