"""Verify-window graph cache: the reference's retention policy (its unit tests, src/verifier_graph_cache.rs:216-309, on
the C-ABI restatement) and, on a GPU, capture / replay of shared verify windows with bytes equal to eager runs
(src/multi_decode.rs:470-537: two to four requests, four-token windows, one <= 16-row expert call)."""
import numpy as np
import pytest


def small(pkg, entries, nodes):
    return pkg.GraphCache(pkg.GraphPolicy(1, entries, nodes, 4, 2))


def capture(pkg, cache, key, nodes):
    assert cache.action(key) == pkg.EAGER
    assert cache.action(key) == pkg.CAPTURE
    assert cache.insert(key, nodes) == 0


def test_default_keeps_clear_all_behaviour_and_candidate_captures_first(pkg):
    old = pkg.GraphCache(bounded=False)
    for key in range(32):
        assert old.action(key) == pkg.CAPTURE
        assert old.insert(key, 3) == 0
    assert old.action(31) == pkg.REPLAY
    assert old.action(32) == pkg.CAPTURE
    assert old.stats()["retained_graphs"] == 0
    new = pkg.GraphCache(bounded=True)
    assert new.action(1) == pkg.CAPTURE
    assert new.insert(1, 3) == 0
    assert new.action(1) == pkg.REPLAY
    assert new.stats()["eager"] == 0
    assert (old.policy.entries, old.policy.bounded) != (new.policy.entries, new.policy.bounded)


def test_cold_shape_scan_does_not_destroy_hot_graphs_or_grow_sightings(pkg):
    cache = small(pkg, 2, 12)
    capture(pkg, cache, 1, 4)
    capture(pkg, cache, 2, 4)
    for key in range(3, 100):
        assert cache.action(1) == pkg.REPLAY
        assert cache.action(key) == pkg.EAGER
    st = cache.stats()
    assert st["retained_graphs"] == 2 and st["evictions"] == 0 and st["tracked_sightings"] == 4
    capture(pkg, cache, 101, 4)
    assert cache.action(1) == pkg.REPLAY
    assert cache.action(2) == pkg.EAGER
    assert cache.stats()["evictions"] == 1


def test_node_budget_evicts_only_enough_and_oversized_graph_is_returned(pkg):
    cache = small(pkg, 5, 10)
    capture(pkg, cache, 1, 4)
    capture(pkg, cache, 2, 4)
    assert cache.action(1) == pkg.REPLAY
    capture(pkg, cache, 3, 5)
    st = cache.stats()
    assert st["retained_nodes"] == 9 and st["retained_graphs"] == 2
    assert cache.action(1) == pkg.REPLAY                        # key 1 survived, key 2 went
    assert cache.insert(4, 11) == 1                             # handed back
    st = cache.stats()
    assert st["retained_nodes"] == 9 and st["oversized"] == 1 and st["peak_nodes"] <= 10


def test_repeated_four_slot_shapes_fit_without_warm_recapture(pkg):
    cache = pkg.GraphCache(bounded=True)
    for _ in range(9):
        for slot in range(4):
            for parity in range(2):
                for rows in range(1, 17):
                    key = rows | parity << 8 | slot << 16
                    if cache.action(key) == pkg.CAPTURE:
                        assert cache.insert(key, 2048) == 0
    st = cache.stats()
    assert st["captures"] == 128 and st["hits"] == 128 * 8 and st["evictions"] == 0 and st["retained_nodes"] == 262144


def test_bad_policy_is_rejected(pkg):
    with pytest.raises(pkg.GlmFlashError):
        pkg.GraphCache(pkg.GraphPolicy(1, 0, 10, 4, 1))


@pytest.mark.gpu
def test_shared_verify_windows_replay_with_eager_bytes(pkg, synth, cuda):
    import torch
    H, I, E, S = 2048, 1536, 64, 5
    wd = synth.to_device(synth.expert_bank(1001, H, I, E, svh_scale=True), cuda)
    moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=16))
    cache = pkg.GraphCache(pkg.GraphPolicy(1, 8, 1 << 20, 16, 2))          # capture at the second sighting
    x_all = synth.activations_bf16(31, 16, H)
    picks_all, rw_all = synth.route(32, 16, E, S - 1, shared_bias=True)
    xd = torch.from_numpy(x_all.view(np.int16)).to(cuda).view(torch.bfloat16)
    pd, wdv = torch.from_numpy(picks_all).to(cuda), torch.from_numpy(rw_all).to(cuda)
    out = torch.empty((16, H), dtype=torch.float32, device=cuda)
    eager = {}
    for requests in (2, 3, 4):                                  # requests x 4-token windows share one expert call
        rows = 4 * requests
        moe.run(wd, xd, pd, wdv, rows)
        torch.cuda.synchronize()
        eager[rows] = moe.output[:rows].cpu().numpy().copy()
    side = torch.cuda.Stream()
    for rnd in range(4):
        for requests in (2, 3, 4):
            rows = 4 * requests

            def window(rows=rows):
                moe.run(wd, xd, pd, wdv, rows)
                out[:rows].copy_(moe.output[:rows])
            out.zero_()
            cache.run(rows, window, stream=side)
            side.synchronize()
            assert (out[:rows].cpu().numpy().view(np.uint32) == eager[rows].view(np.uint32)).all(), (rnd, rows)
    st = cache.stats()
    assert st["eager"] == 3 and st["captures"] == 3 and st["hits"] == 6 and st["retained_graphs"] == 3
    assert int(moe.status.cpu()[0]) == 0
