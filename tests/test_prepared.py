"""Prepared-weights loader (reference src/prepared.rs): manifest validation, chunk hashes, tensor paths -- on the CPU --
and, on a GPU, a synthetic bank written as four tensor-parallel shards, loaded, re-assembled into whole experts and run
through the layer: the bytes of the layer on the original bank."""
import json
import os

import numpy as np
import pytest

from prepared_fixture import tp_shards, write_prepared


def small_tree(rng):
    return {"cfg": {"hidden": 512, "layers": 2},
            "layers": [{"moe": {"experts": {"gt": rng.integers(0, 1 << 31, (3, 2, 2, 32), dtype=np.int64).astype(np.int32),
                                             "suh_g": rng.standard_normal((3, 32)).astype(np.float16)}}},
                       {"norm": rng.standard_normal(64).astype(np.float32)}],
            "tables": ("dict", [("a", rng.standard_normal(16).astype(np.float32)), (7, np.arange(5, dtype=np.uint8))])}


def test_open_walks_the_tree_and_verifies(pkg, tmp_path):
    rng = np.random.default_rng(0)
    tree = small_tree(rng)
    mp = write_prepared(tmp_path / "m", tree, {"rank": 2, "world": 4, "model": "synthetic"}, chunk=1000)
    p = pkg.Prepared(mp)
    assert p.names() == sorted(['weights.layers[0].moe.experts.gt', 'weights.layers[0].moe.experts.suh_g', 'weights.layers[1].norm',
                                'weights.tables["a"]', 'weights.tables[7]'])
    assert p.key_int("rank") == 2 and p.key_int("world") == 4
    t = p.tensor("weights.layers[0].moe.experts.gt")
    assert t["dtype"] == "int32" and t["shape"] == [3, 2, 2, 32] and t["contiguous"] and t["on_device"] and t["ptr"] is None
    assert t["nbytes"] == 3 * 2 * 2 * 32 * 4
    p.verify()                                                  # every chunk matches its SHA-256
    with pytest.raises(pkg.GlmFlashError, match="missing tensor"):
        p.tensor("weights.layers[0].moe.experts.ut")
    with pytest.raises(pkg.GlmFlashError, match="no integer"):
        p.key_int("model")


def test_corrupted_chunk_is_named(pkg, tmp_path):
    rng = np.random.default_rng(1)
    mp = write_prepared(tmp_path / "m", small_tree(rng), {"rank": 0, "world": 4}, chunk=512)
    data = bytearray(open(tmp_path / "m" / "data.bin", "rb").read())
    data[1300] ^= 0x40                                          # chunk 2
    open(tmp_path / "m" / "data.bin", "wb").write(bytes(data))
    p = pkg.Prepared(mp)                                        # the manifest itself is intact
    with pytest.raises(pkg.GlmFlashError, match="weight hash mismatch in chunk 2"):
        p.verify()


def test_truncated_payload_and_bad_manifests_are_rejected(pkg, tmp_path):
    rng = np.random.default_rng(2)
    mp = write_prepared(tmp_path / "m", small_tree(rng), {"rank": 0, "world": 4}, chunk=512)
    data = open(tmp_path / "m" / "data.bin", "rb").read()
    open(tmp_path / "m" / "data.bin", "wb").write(data[:-1])
    with pytest.raises(pkg.GlmFlashError, match="data file size mismatch"):
        pkg.Prepared(mp)
    open(tmp_path / "m" / "data.bin", "wb").write(data)
    good = json.load(open(mp))

    def broken(change, match):
        m = json.loads(json.dumps(good))
        change(m)
        json.dump(m, open(mp, "w"))
        with pytest.raises(pkg.GlmFlashError, match=match):
            pkg.Prepared(mp)
    broken(lambda m: m.update(format=2), "unsupported prepared format")
    broken(lambda m: m.update(chunk=129 * 1024 * 1024), "invalid chunk size")
    broken(lambda m: m["chunk_sha256"].pop(), "chunk hash count")
    broken(lambda m: m["storages"][1].update(offset=0), "out-of-order storage")
    broken(lambda m: m["storages"][-1].update(nbytes=10 ** 9), "storage outside data file")
    broken(lambda m: m["tree"]["f"]["layers"]["L"][1]["f"]["norm"].update(shape=[65]), "escapes storage")
    broken(lambda m: m["tree"]["f"]["layers"]["L"][1]["f"]["norm"].update(dev="cpu"), "changes device")
    broken(lambda m: m["tree"]["f"]["layers"]["L"][1]["f"]["norm"].update(stride=[1, 1]), "rank mismatch")
    broken(lambda m: m["tree"]["f"]["layers"]["L"][1]["f"].update(arr={"N": 1}), "NumPy storage is unsupported")
    open(mp, "w").write("{ not json")
    with pytest.raises(pkg.GlmFlashError, match="not valid JSON"):
        pkg.Prepared(mp)


def test_strided_extent_rules(pkg, tmp_path):
    # the reference's unit tests (src/prepared.rs:382-413): a strided view's extent includes its offset and holes
    rng = np.random.default_rng(3)
    mp = write_prepared(tmp_path / "m", {"t": rng.standard_normal(32).astype(np.float16)}, {"rank": 0})
    m = json.load(open(mp))
    m["tree"]["f"]["t"].update(dtype="bfloat16", shape=[2, 3], stride=[8, 1], off=4)      # extent 30 bytes of the 64
    json.dump(m, open(mp, "w"))
    t = pkg.Prepared(mp).tensor("weights.t")
    assert t["nbytes"] == 30 - 8 and not t["contiguous"]
    m["tree"]["f"]["t"].update(stride=[2 ** 63, 1])
    json.dump(m, open(mp, "w"))
    with pytest.raises(pkg.GlmFlashError, match="overflow"):
        pkg.Prepared(mp)


@pytest.mark.gpu
def test_tp_shards_reassemble_into_the_bank(pkg, synth, cuda, tmp_path):
    import torch
    H, I, E, S, rows = 512, 1024, 8, 4, 5
    bank = synth.expert_bank(21, H, I, E, svh_scale=True)
    shards = []
    for r, sh in enumerate(tp_shards(bank, 4, E)):
        mp = write_prepared(tmp_path / f"rank{r}", {"layers": [{"moe": {"experts": sh}}]}, {"rank": r, "world": 4}, chunk=1 << 20)
        p = pkg.Prepared(mp)
        assert p.key_int("rank") == r
        p.load(["weights.layers[0].moe.experts"])
        shards.append(p)
    assert shards[0].tensor("weights.layers[0].moe.experts.gt")["ptr"]
    x = synth.activations_bf16(22, rows, H)
    picks, rw = synth.route(23, rows, E, S - 1)
    xd = torch.from_numpy(x.view(np.int16)).to(cuda).view(torch.bfloat16)
    pd, wd = torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda)
    want = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=8, shared_exl3=0))
    want.run(synth.to_device(bank, cuda), xd, pd, wd, rows)
    torch.cuda.synchronize()
    ref = want.output[:rows].cpu().numpy().copy()
    total = np.zeros_like(ref)
    for lo, hi in ((0, 3), (3, 8)):                             # two expert-parallel windows of whole experts
        eb = pkg.ExpertBank(shards, "weights.layers[0].moe.experts", lo, hi)
        assert (eb.hidden, eb.inter) == (H, I)
        moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=8, shared_exl3=0, expert_lo=lo, expert_hi=hi))
        moe.run(eb.weights, xd, pd, wd, rows)
        torch.cuda.synchronize()
        assert int(moe.status.cpu()[0]) == 0
        total += moe.output[:rows].cpu().numpy()
    assert np.abs(total - ref).max() <= 1e-5 * np.abs(ref).max()
    one = pkg.ExpertBank(shards, "weights.layers[0].moe.experts", 0, E)
    moe = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=8, shared_exl3=0))
    moe.run(one.weights, xd, pd, wd, rows)
    torch.cuda.synchronize()
    assert (moe.output[:rows].cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()
