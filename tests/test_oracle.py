"""The CPU oracle against the reference's own known-answer tests and an independent numpy restatement."""
import numpy as np

from conftest import rel_err


def test_hadamard_involution(oracle):
    # reference src/experts.rs:569-576: H(H(x)) == 128 x exactly
    x = np.arange(128, dtype=np.float32) - 64.0
    z = oracle.had128(oracle.had128(x))
    assert (z == x * 128.0).all()


def test_codebook_finite(oracle):
    # reference src/experts.rs:577-582
    cb = oracle.codebook_all().view(np.float16).astype(np.float32)
    assert np.isfinite(cb).all()
    # the codebook's published shape: 10 746 distinct values within +-3.95, std 1.244
    assert len(np.unique(cb)) == 10746 and abs(cb.std() - 1.2441) < 1e-3 and np.abs(cb).max() < 3.96


def test_codebook_matches_numpy(oracle):
    s = np.arange(65536, dtype=np.uint32)
    x = ((s * np.uint32(0xCBAC1FED)) & np.uint32(0x8FFF8FFF)) ^ np.uint32(0x3B603B60)
    lo = (x & 0xFFFF).astype(np.uint16).view(np.float16)
    hi = (x >> 16).astype(np.uint16).view(np.float16)
    assert ((lo + hi).view(np.uint16) == oracle.codebook_all()).all()


def numpy_decode(words):
    """Independent restatement of the tile format: 1024-bit MSB-first circular stream, weight p <- bits [4p-12, 4p+4)."""
    words = words.reshape(-1, 32)
    bits = ((words[:, :, None] >> (31 - np.arange(32, dtype=np.uint32))) & 1).reshape(-1, 1024)
    p = np.arange(256)
    idx = (4 * p[:, None] - 12 + np.arange(16)[None, :]) % 1024
    states = (bits[:, idx] << (15 - np.arange(16, dtype=np.uint32))).sum(-1).astype(np.uint32)
    x = ((states * np.uint32(0xCBAC1FED)) & np.uint32(0x8FFF8FFF)) ^ np.uint32(0x3B603B60)
    w = (x & 0xFFFF).astype(np.uint16).view(np.float16) + (x >> 16).astype(np.uint16).view(np.float16)
    lane, j = p // 8, p % 8
    row = 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1)
    col = lane // 4 + 8 * (j >> 2)
    out = np.empty((words.shape[0], 16, 16), np.float16)
    out[:, row, col] = w
    return out, states


def test_tile_forms_agree(oracle):
    rng = np.random.default_rng(1)
    w = rng.integers(0, 1 << 32, size=(200, 32), dtype=np.uint64).astype(np.uint32)
    w[0] = 0
    w[1] = 0xFFFFFFFF
    a = oracle.decode_tiles(w, "stream")      # src/experts.rs:47-74
    b = oracle.decode_tiles(w, "lanes")       # native/exl3.cu:33-40
    c, states = numpy_decode(w)
    assert (a.view(np.uint16) == b.view(np.uint16)).all()
    assert (a.view(np.uint16) == c.view(np.uint16)).all()
    assert (oracle.tile_states(w) == states).all()


def test_rounding_helpers(oracle):
    rng = np.random.default_rng(2)
    v = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-9, 6, 2000), [0.0, -0.0, 65504.0, 65519.9, 65520.0,
                        6.1e-5, 5.96e-8, 2.98e-8, 1e-9]]).astype(np.float32)
    L = oracle.lib()
    with np.errstate(over="ignore"):
        want_h = v.astype(np.float16).view(np.uint16)
    got_h = np.array([L.gfo_f32_to_f16(float(f)) for f in v], dtype=np.uint16)
    assert (got_h == want_h).all()
    import torch
    want_b = torch.from_numpy(v).to(torch.bfloat16).to(torch.float32).numpy()
    got_b = np.array([L.gfo_bf(float(f)) for f in v], dtype=np.float32)
    assert (got_b == want_b).all()


def test_unpack_and_matmul_orders(oracle):
    rng = np.random.default_rng(3)
    K, N = 256, 128
    words = rng.integers(0, 1 << 32, size=(K // 16, N // 16, 32), dtype=np.uint64).astype(np.uint32)
    w = oracle.unpack(words, K, N).astype(np.float32)
    tiles, _ = numpy_decode(words)
    ref = tiles.reshape(K // 16, N // 16, 16, 16).transpose(0, 2, 1, 3).reshape(K, N).astype(np.float32)
    assert (w == ref).all()
    x = rng.standard_normal(K).astype(np.float32)
    exact = (x.astype(np.float64) @ w.astype(np.float64))
    for sk in (1, 4):
        y = oracle.matmul(x, w, sk=sk, mode=0)        # the reference's split/warp order, fp32
        assert rel_err(y, exact)[0] < 1e-5
    assert rel_err(oracle.matmul(x, w, mode=1), exact)[0] < 1e-6


def test_grouping_contract(oracle):
    # reference src/grouping.rs:143-192: expected ids / members built on the host
    rng = np.random.default_rng(4)
    E1, slots, rows, maxm = 17, 5, 23, 32
    picks = np.stack([np.concatenate([rng.permutation(E1 - 1)[: slots - 1], [E1 - 1]]) for _ in range(rows)]).astype(np.int32)
    ids, count, members = oracle.grouping(picks, rows, slots, E1, maxm)
    exp = {e: [r * 32 + s for r in range(rows) for s in range(slots) if picks[r, s] == e] for e in range(E1)}
    used = [e for e in range(E1) if exp[e]]
    assert count == len(used) and list(ids[:count]) == used
    for u, e in enumerate(used):
        assert list(members[u, : len(exp[e])]) == exp[e] and (members[u, len(exp[e]):] == -1).all()
    assert (members[count:] == -1).all()


def test_expert_pipeline_modes_agree(oracle, synth):
    # the fp32 reference-order pipeline (src/experts.rs:76-135) and the binary64-accumulation variant agree to 1e-3
    H, I, E, S = 256, 256, 2, 3
    bank = synth.expert_bank(5, H, I, E, svh_scale=True)
    x = synth.activations_bf16(6, 2, H)
    picks, rw = synth.route(7, 2, E, S - 1)
    y0 = oracle.experts_run_rows(bank, H, I, E + 1, S, x, picks, mode=0, threads=1)
    y1 = oracle.experts_run_rows(bank, H, I, E + 1, S, x, picks, mode=1)
    assert np.isfinite(y0).all() and rel_err(y0, y1)[1] < 1e-3
    out = oracle.combine(y1, rw, 2, S, H)
    want = (rw[:, : S - 1, None] * y1.reshape(2, S, H)[:, : S - 1]).sum(1) + y1.reshape(2, S, H)[:, S - 1]
    assert rel_err(out, want)[0] < 1e-6


def test_topk_matches_the_route_generator(oracle):
    """The oracle's sigmoid top-k against the numpy definition that generates the benchmark's routing tables
    (glm-flash-rs_b200/synth.py: sigmoid scores, top-4, ties to the lower id, renormalised weights)."""
    g = np.random.default_rng(99)
    rows, E, k = 64, 64, 4
    logits = g.standard_normal((rows, E)).astype(np.float32)
    logits[5, :] = 1.5                                           # all tied
    scores = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    order = np.argsort(-scores, axis=1, kind="stable")[:, :k]
    top = np.take_along_axis(scores, order, axis=1)
    want_w = top / top.sum(axis=1, keepdims=True)
    picks, weights = oracle.topk(logits, rows, E, k)
    assert np.array_equal(picks[:, :k], order) and (picks[:, k] == E).all()
    assert np.allclose(weights[:, :k], want_w, rtol=1e-6, atol=1e-7) and (weights[:, k] == 1.0).all()


def test_router_logits_small(oracle):
    g = np.random.default_rng(3)
    rows, Hs, E = 3, 64, 5
    xf = g.standard_normal((rows, Hs)).astype(np.float32)
    wf = g.standard_normal((E, Hs)).astype(np.float32)
    xb = (xf.view(np.uint32) >> 16).astype(np.uint16)            # truncated to bf16 bit patterns (exact inputs)
    wb = (wf.view(np.uint32) >> 16).astype(np.uint16)
    x32 = (xb.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    w32 = (wb.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    want = (x32 @ w32.T).astype(np.float32)
    got = oracle.router_logits(xb, wb, rows, Hs, E)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
