"""Golden vectors produced by the REFERENCE's own CUDA kernels on a B200 (tests/golden/make_golden.py): the CPU
oracle must reproduce them here, without a GPU (this pins the oracle to the reference), and the library must
reproduce them on the GPU (-m gpu)."""
import importlib.util
import os

import numpy as np
import pytest

from conftest import ROOT, TOL, rel_err

GOLD = os.path.join(ROOT, "tests", "golden", "ref_sm100.npz")


def _mk():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


@pytest.fixture(scope="module")
def mk(pkg):
    return _mk()


def test_oracle_decode_equals_reference_device_decode(oracle, gold, mk):
    # bit-exact: the reference's decoded weights (through its own GEMV kernel on one-hot rows) vs the oracle's unpack
    _, _, _, _, words, _ = mk.inputs()
    w = oracle.unpack(words, 256, 128)
    assert (w.view(np.uint16) == gold["decode_w"].view(np.uint16)).all()


def test_oracle_pipeline_matches_reference_kernels(oracle, gold, mk):
    bank, x, picks, rw, _, _ = mk.inputs()
    Y, xd = oracle.experts_run_rows(bank, mk.H, mk.I, mk.E + 1, mk.S, x, picks, mode=0, sk_gu=4, sk_dn=1, want_xd=True)
    emax, erms = rel_err(Y, gold["y"])
    assert emax < TOL and erms < TOL, (emax, erms)             # the reference's own gate is relative RMS < 1e-3
    assert rel_err(xd, gold["xd"].astype(np.float32))[1] < 2e-3
    assert rel_err(Y, gold["y_prefill"])[1] < TOL              # its prefill kernels agree with its decode kernels too


def test_oracle_grouping_equals_reference_kernels(oracle, gold, mk):
    _, _, _, _, _, gp = mk.inputs()
    ids, count, members = oracle.grouping(gp, gp.shape[0], 9, 289, 64)
    assert count == int(gold["group_count"][0])
    assert (ids[:count] == gold["group_ids"]).all() and (members == gold["group_members"]).all()


@pytest.mark.gpu
def test_library_matches_reference_golden(pkg, oracle, synth, cuda, gold, mk):
    import torch
    bank, x, picks, rw, words, gp = mk.inputs()
    dec = pkg.exl3_decode(torch.from_numpy(words.view(np.int32)).to(cuda)).cpu().numpy()          # [tiles][16][16]
    w = dec.reshape(16, 8, 16, 16).transpose(0, 2, 1, 3).reshape(256, 128)
    assert (w.view(np.uint16) == gold["decode_w"].view(np.uint16)).all()
    wd = synth.to_device(bank, cuda)
    xb = torch.from_numpy(x.view(np.int16)).to(cuda).view(torch.bfloat16)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    for rows_cap, owner in ((16, pkg.ExpertGpu), (64, pkg.FastExperts)):
        o = owner(pkg.make_config(mk.H, mk.I, mk.E, mk.S, max_rows=rows_cap))
        ids, count, members = oracle.grouping(picks, mk.ROWS, mk.S, mk.E + 1, rows_cap)
        args = (wd, xb, t(picks), t(ids), t(np.array([count], np.int32)), t(members), mk.ROWS, rows_cap)
        if owner is pkg.ExpertGpu:
            o.run_rows(*args)
            y = o.y
        else:
            o.run(*args)
            y = o.output
        torch.cuda.synchronize()
        emax, erms = rel_err(y[: mk.ROWS * mk.S].cpu().numpy(), gold["y"])
        assert emax < TOL and erms < TOL, (owner.__name__, emax, erms)
    g = pkg.Grouping(pkg.make_config(experts=288, slots=9, max_rows=64))
    g.run(t(gp), gp.shape[0])
    torch.cuda.synchronize()
    n = int(g.count.cpu()[0])
    assert n == int(gold["group_count"][0]) and (g.ids[:n].cpu().numpy() == gold["group_ids"]).all()
    assert (g.members.cpu().numpy() == gold["group_members"]).all()
