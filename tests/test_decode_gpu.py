"""GPU parity of the trellis decode and the single EXL3 linear (benchmark config 1), through the C ABI."""
import numpy as np
import pytest

from conftest import TOL, rel_err

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)).to(cuda)


def test_decode_all_states_bit_exact(pkg, oracle, cuda):
    # tile i carries state i in the low half of word 0: weight (k = 9, n = 8) of the tile is codebook(i)
    rng = np.random.default_rng(10)
    words = rng.integers(0, 1 << 32, size=(65536, 32), dtype=np.uint64).astype(np.uint32)
    words[:, 0] = (words[:, 0] & np.uint32(0xFFFF0000)) | np.arange(65536, dtype=np.uint32)
    got = pkg.exl3_decode(_dev(words, cuda)).cpu().numpy()
    assert (got[:, 9, 8].view(np.uint16) == oracle.codebook_all()).all()
    want = oracle.decode_tiles(words[:4096])
    assert (got[:4096].view(np.uint16) == want.view(np.uint16)).all()          # bit-exact, whole tiles


def test_decode_edge_tiles(pkg, oracle, cuda):
    words = np.zeros((3, 32), np.uint32)
    words[1] = 0xFFFFFFFF
    words[2] = np.arange(32, dtype=np.uint32) * np.uint32(0x01010101)
    got = pkg.exl3_decode(_dev(words, cuda)).cpu().numpy()
    assert (got.view(np.uint16) == oracle.decode_tiles(words).view(np.uint16)).all()
    import torch
    assert pkg.exl3_decode(torch.empty((0, 32), dtype=torch.int32, device=cuda)).shape[0] == 0    # empty input


@pytest.mark.parametrize("rows", [1, 7, 16])
def test_single_linear_config1(pkg, oracle, synth, cuda, rows):
    # benchmark config 1: fp16 x[rows,2048] ~ N(0,1) times an EXL3 K=4 weight 2048 -> 1536, seed 0
    K, N = 2048, 1536
    g = synth.rng(0)
    x = g.standard_normal((rows, K)).astype(np.float16)
    words = g.integers(0, 1 << 32, size=(K // 16, N // 16, 32), dtype=np.uint64).astype(np.uint32)
    suh = synth.scales(g, 1, K)[0]
    svh = synth.scales(g, 1, N)[0]
    y = pkg.exl3_linear(_dev(x, cuda), _dev(words, cuda), _dev(suh, cuda), _dev(svh, cuda), K, N).cpu().numpy()
    want16, want32 = oracle.linear_f16(x, words, suh, svh, K, N, mode=1)
    emax, erms = rel_err(y.astype(np.float32), want32)
    assert np.isfinite(y).all() and emax < TOL and erms < TOL, (emax, erms)
    # and against the reference's own fp32 summation order
    _, ref32 = oracle.linear_f16(x, words, suh, svh, K, N, sk=4, mode=0)
    assert rel_err(y.astype(np.float32), ref32)[1] < TOL
    if rows > 1:      # a row does not depend on the rows it shares the call with
        y1 = pkg.exl3_linear(_dev(x[:1], cuda), _dev(words, cuda), _dev(suh, cuda), _dev(svh, cuda), K, N).cpu().numpy()
        assert (y1.view(np.uint16) == y[:1].view(np.uint16)).all()
